"""Slot manager and request scheduler over the native step function of seq.SeqModel.

Continuous batching in the simplest form that keeps the weights read once per step: waiting requests are admitted into free
slots; a step carries the next prompt portion of every request that is still prefilling (at most `chunk` tokens each, `budget`
rows in total) TOGETHER with one row of every request that is decoding; when nothing is prefilling or waiting, the decoding
slots run `burst` greedy steps on the device without a host round trip.  Sampling: greedy (argmax on the device) or top-k with
temperature (the k candidates are selected on the device, the draw happens here with the request's generator)."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np


class SlotManager:
    """Which sequence owns which slot.  acquire() resets the slot's state on the device; release() only frees the number."""

    def __init__(self, model):
        self.model = model
        self.free = list(range(model.n_slots))[::-1]
        self.owner = {}

    def acquire(self, key) -> int:
        if key in self.owner:
            return self.owner[key]
        if not self.free:
            raise RuntimeError("no free slot")
        s = self.free.pop()
        self.model.reset(s)
        self.owner[key] = s
        return s

    def release(self, key):
        s = self.owner.pop(key, None)
        if s is not None:
            self.free.append(s)

    def slot(self, key) -> int:
        return self.owner[key]


@dataclass
class Request:
    rid: int
    prompt: np.ndarray
    max_new: int
    top_k: int = 0
    temperature: float = 1.0
    seed: int = 0
    fed: int = 0                       # prompt tokens already in the slot
    out: list = field(default_factory=list)
    done: bool = False
    rng: np.random.Generator | None = None


class Scheduler:
    def __init__(self, model, chunk: int = 512, budget: int = 2048, burst: int = 16, eos_id: int = -1):
        self.model, self.chunk, self.budget, self.burst, self.eos = model, chunk, budget, burst, eos_id
        self.slots = SlotManager(model)
        self.waiting: deque[Request] = deque()
        self.active: list[Request] = []
        self.finished: dict[int, Request] = {}
        self._next = 0

    def submit(self, prompt, max_new: int, top_k: int = 0, temperature: float = 1.0, seed: int = 0) -> int:
        prompt = np.asarray(prompt, np.int32)
        if prompt.size == 0:
            raise ValueError("empty prompt")
        if prompt.size + max_new > self.model.max_ctx:
            raise ValueError(f"{prompt.size} + {max_new} tokens exceed the slot capacity {self.model.max_ctx}")
        r = Request(self._next, prompt, max_new, top_k, temperature, seed, rng=np.random.default_rng(seed))
        self._next += 1
        self.waiting.append(r)
        return r.rid

    def _pick(self, r: Request, seg: int, greedy_tok: int) -> int:
        if r.top_k <= 1:
            return int(greedy_tok)
        v, ids = self.model.topk(seg, min(r.top_k, self.model.vocab))
        z = (v.astype(np.float64) - v[0]) / max(r.temperature, 1e-6)
        p = np.exp(z)
        return int(ids[r.rng.choice(len(ids), p=p / p.sum())])

    def _finish(self, r: Request):
        r.done = True
        self.slots.release(r.rid)
        self.active.remove(r)
        self.finished[r.rid] = r

    def step(self) -> bool:
        """One scheduling decision; False when nothing is left to do."""
        while self.waiting and self.slots.free:
            r = self.waiting.popleft()
            self.slots.acquire(r.rid)
            self.active.append(r)
        if not self.active:
            return False
        prefilling = [r for r in self.active if r.fed < r.prompt.size]
        decoding = [r for r in self.active if r.fed >= r.prompt.size]
        if not prefilling and not self.waiting and decoding and all(r.top_k <= 1 for r in decoding):
            n = min(self.burst, min(r.max_new - len(r.out) for r in decoding))
            toks = self.model.decode([self.slots.slot(r.rid) for r in decoding], n, self.eos)
            for r, row in zip(decoding, toks):
                for t in row:
                    r.out.append(int(t))
                    if int(t) == self.eos:
                        break
            for r in decoding:
                if len(r.out) >= r.max_new or (r.out and r.out[-1] == self.eos):
                    self._finish(r)
            return True
        segs, who, room = [], [], self.budget - len(decoding)
        for r in decoding:                       # one row each: the token sampled last
            segs.append((self.slots.slot(r.rid), [r.out[-1]]))
            who.append(r)
        for r in prefilling:
            n = min(self.chunk, r.prompt.size - r.fed, room)
            if n <= 0:
                continue
            segs.append((self.slots.slot(r.rid), r.prompt[r.fed:r.fed + n]))
            who.append(r)
            r.fed += n
            room -= n
        nxt = self.model.step_greedy(segs)
        for i, r in enumerate(who):
            if r.fed < r.prompt.size:
                continue                          # a portion in the middle of a prompt: its sample is not used
            r.out.append(self._pick(r, i, nxt[i]))
        for r in list(who):
            if r.fed >= r.prompt.size and (len(r.out) >= r.max_new or r.out[-1] == self.eos):
                self._finish(r)
        return True

    def run(self) -> dict:
        while self.step():
            pass
        return {rid: np.asarray(r.out, np.int32) for rid, r in sorted(self.finished.items())}


def generate(model, prompts, max_new: int, **kw) -> list:
    """Greedy (or top-k) continuation of each prompt through the scheduler; returns the new tokens per prompt."""
    sch = Scheduler(model, **{k: v for k, v in kw.items() if k in ("chunk", "budget", "burst", "eos_id")})
    ids = [sch.submit(p, max_new, **{k: v for k, v in kw.items() if k in ("top_k", "temperature", "seed")}) for p in prompts]
    out = sch.run()
    return [out[i] for i in ids]
