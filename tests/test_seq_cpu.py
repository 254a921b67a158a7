"""CPU-side pieces of the layer-list sequence models: container IO, the Reninex config reader, the registry, the scheduler's
batching logic (over a fake model), the oracle's own building blocks, and the C header against the binding."""
import json
import re
from pathlib import Path

import numpy as np
import pytest

from oracle import seq_ref as R
from tinyllama_cpp_b200 import registry, reninex, safetensors_io as st
from tinyllama_cpp_b200.scheduler import Scheduler, SlotManager, generate

ROOT = Path(__file__).resolve().parent.parent


def test_safetensors_round_trip(tmp_path):
    rng = np.random.default_rng(0)
    a = rng.standard_normal((5, 7)).astype(np.float32)
    t = {"a": ("BF16", st.f32_to_bf16_bits(a)), "s": ("BF16", st.f32_to_bf16_bits(np.float32(1.5)).reshape(())), "i": ("I32", np.arange(6, dtype=np.int32).reshape(2, 3))}
    st.write(tmp_path / "m.safetensors", t)
    back = st.read(tmp_path / "m.safetensors")
    assert set(back) == set(t)
    for k in t:
        assert back[k][0] == t[k][0] and back[k][1].shape == t[k][1].shape and np.array_equal(back[k][1], t[k][1])
    assert np.abs(st.bf16_bits_to_f32(back["a"][1]) - a).max() <= np.abs(a).max() * 2.0 ** -8


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8, -2.5, 3.0e38], np.float32)
    got = st.bf16_bits_to_f32(st.f32_to_bf16_bits(x))
    assert got.tolist()[:4] == [1.0, 1.0, 1.0 + 2.0 ** -6, -2.5]


def test_describe_reads_every_constant():
    cfg = reninex.make_config(vocab=55, width=40, n_layers=3, ff=24, taps=5, l_heads=6, l_kv=3, l_dim=4, l_vdim=12, r_heads=2, r_dim=10, r_vdim=6,
                              rot_dims=6, rot_base=500.0, loop=(1, 3, 4), bigram=(17, 2, 9), left_scale=0.3, right_scale=1.7, eps=3e-4, no_mlp=(1,))
    d = reninex.describe(cfg)
    assert (d["vocab"], d["width"], d["taps"], d["eps"]) == (55, 40, 5, 3e-4)
    assert d["bigram"] == {"buckets": 17, "mul_prev": 2, "mul_cur": 9} and d["loop"] == {"start": 1, "stop": 3, "times": 4}
    le, ri = d["layers"][0]["branches"]
    assert (le["heads"], le["kv_heads"], le["dim"], le["vdim"], le["out_scale"]) == (6, 3, 4, 12, 0.3)
    assert (ri["heads"], ri["dim"], ri["vdim"], ri["rot_dims"], ri["rot_base"], ri["out_scale"]) == (2, 10, 6, 6, 500.0, 1.7)
    assert abs(ri["scale"] - 10 ** -0.5) < 1e-12 and len(ri["decay"]) == 2
    assert [l["ff"] for l in d["layers"]] == [24, 0, 24]
    shapes = reninex.tensor_shapes(d)
    assert shapes["l0.mix.left.q"] == (24, 40) and shapes["l0.mix.left.k"] == (12, 40) and shapes["l0.mix.left.v"] == (36, 40)
    assert shapes["l0.mix.right.g"] == (12, 40) and shapes["l0.mix.right.o"] == (40, 12) and shapes["loop.step"] == (4, 40)
    assert "l1.mlp.gate" not in shapes and "l1.canon2" not in shapes and shapes["bigram"] == (18, 40) and shapes["l2.norm1"] == ()
    with pytest.raises(ValueError):
        reninex.describe(dict(cfg, architecture="Other"))
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["type"] = "serial"
    with pytest.raises(ValueError):
        reninex.describe(bad)


def test_optional_sections_may_be_absent():
    cfg = reninex.make_config(taps=0, bigram=None, loop=None, rot_dims=0)
    d = reninex.describe(cfg)
    assert d["taps"] == 0 and d["bigram"] is None and d["loop"] is None and d["layers"][0]["branches"][1]["rot_dims"] == 0
    assert "bigram" not in reninex.tensor_shapes(d) and "loop.in" not in reninex.tensor_shapes(d)


def test_registry_and_checkpoint_folder(tmp_path):
    cfg = reninex.make_config()
    t = reninex.synth_tensors(reninex.describe(cfg), 1)
    reninex.write_checkpoint(tmp_path / "m", cfg, t)
    assert registry.family_of(tmp_path / "m") == "Reninex"
    desc, back = reninex.read_checkpoint(tmp_path / "m")
    assert set(back) == set(reninex.tensor_shapes(desc)) and all(np.array_equal(back[k], t[k]) for k in t)
    (tmp_path / "x.gten").write_bytes(b"")
    assert registry.family_of(tmp_path / "x.gten") == "TinyLlama"
    (tmp_path / "u").mkdir()
    (tmp_path / "u" / "config.json").write_text('{"architecture": "Unknown"}')
    with pytest.raises(ValueError):
        registry.family_of(tmp_path / "u")


def test_header_and_binding_agree():
    from tinyllama_cpp_b200 import seq
    header = (ROOT / "include" / "gten_b200_seq.h").read_text()
    declared = set(re.findall(r"\b(gtb_seq_[a-z0-9_]+)\s*\(", header))
    assert declared == set(seq.SYMBOLS), declared ^ set(seq.SYMBOLS)
    if seq.LIB_PATH.exists():
        L = seq.lib()
        for s in seq.SYMBOLS + ["gtb_init", "gtb_last_error", "gtb_launch_count"]:
            assert hasattr(L, s), s


# ---- oracle building blocks
def test_oracle_conv_and_rotation_and_retention_closed_forms():
    rng = np.random.default_rng(1)
    h, w = rng.standard_normal((6, 3)), rng.standard_normal((3, 4))
    c = R.causal_conv(h, w)
    assert np.allclose(c[0], w[:, 3] * h[0]) and np.allclose(c[2], w[:, 3] * h[2] + w[:, 2] * h[1] + w[:, 1] * h[0])
    x = rng.standard_normal((5, 2, 6))
    y = R.rotate(x, np.arange(5), 4, 100.0)
    assert np.allclose(y[..., 4:], x[..., 4:]) and np.allclose(y[0], x[0])
    assert np.allclose(np.hypot(y[..., 0], y[..., 2]), np.hypot(x[..., 0], x[..., 2]))     # pairs (0, 2) and (1, 3) turn rigidly
    a = 3 * 100.0 ** (-2 * 1 / 4)
    assert np.allclose(y[3, 0, 1], x[3, 0, 1] * np.cos(a) - x[3, 0, 3] * np.sin(a))
    # retention = decayed sum over the past: o_t = sum_s decay^(t-s) (q_t.k_s) v_s
    T, W_, d, dv = 7, 5, 4, 3
    hh = rng.standard_normal((T, W_))
    wq, wk, wv, wg, wo = (rng.standard_normal(s) for s in ((d, W_), (d, W_), (dv, W_), (dv, W_), (W_, dv)))
    got = R.retention(hh, wq, wk, wv, wg, wo, 1, d, dv, [0.8], 0, 1.0, 1e-6)
    q, k, v, g = hh @ wq.T, hh @ wk.T * d ** -0.5, hh @ wv.T, hh @ wg.T
    o = np.stack([sum(0.8 ** (t - s) * (q[t] @ k[s]) * v[s] for s in range(t + 1)) for t in range(T)])
    assert np.allclose(got, (R.unit_rms(o, 1e-6) * g / (1 + np.exp(-g))) @ wo.T)
    assert R.bigram_rows([4, 4, 9], 11, 3, 5).tolist() == [11, (4 * 3 + 4 * 5) % 11, (4 * 3 + 9 * 5) % 11]


# ---- scheduler over a fake model: next token = hash of everything the slot has seen
class FakeModel:
    vocab, max_ctx = 50, 4096

    def __init__(self, n_slots):
        self.n_slots, self.hist, self.pending, self.calls = n_slots, [[] for _ in range(n_slots)], [0] * n_slots, []

    def reset(self, s):
        self.hist[s] = []

    def _next(self, s):
        return (sum((i + 1) * t for i, t in enumerate(self.hist[s])) * 7 + 3) % self.vocab

    def step_greedy(self, segs):
        self.calls.append([(s, len(t)) for s, t in segs])
        out = []
        for s, t in segs:
            self.hist[s] += [int(x) for x in t]
            self.pending[s] = self._next(s)
            out.append(self.pending[s])
        return np.asarray(out, np.int32)

    def decode(self, slots, n, eos=-1):
        self.calls.append([("decode", len(slots), n)])
        out = np.zeros((len(slots), n), np.int32)
        for k in range(n):
            for i, s in enumerate(slots):
                self.hist[s].append(self.pending[s])
                self.pending[s] = self._next(s)
                out[i, k] = self.pending[s]
        return out


def fake_alone(prompt, n_new):
    m = FakeModel(1)
    cur, out = int(m.step_greedy([(0, prompt)])[0]), []
    out.append(cur)
    while len(out) < n_new:
        cur = int(m.step_greedy([(0, [cur])])[0])
        out.append(cur)
    return out


def test_scheduler_batches_chunks_and_refills_slots():
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, 50, n) for n in (70, 3, 29, 1, 40)]
    m = FakeModel(2)
    outs = generate(m, prompts, 9, chunk=16, budget=24, burst=4)
    for p, o in zip(prompts, outs):
        assert o.tolist() == fake_alone(p, 9)
    flat = [c for c in m.calls if c[0][0] != "decode"]
    assert max(sum(n for _, n in c) for c in flat) <= 24 and max(n for c in flat for _, n in c) <= 16
    assert any(len(c) == 2 and {n for _, n in c} != {1} and 1 in {n for _, n in c} for c in flat)    # a prompt portion next to a decode row
    assert any(c[0][0] == "decode" for c in m.calls)


def test_slot_manager():
    m = FakeModel(2)
    sm = SlotManager(m)
    a, b = sm.acquire("a"), sm.acquire("b")
    assert {a, b} == {0, 1} and sm.acquire("a") == a
    with pytest.raises(RuntimeError):
        sm.acquire("c")
    sm.release("a")
    assert sm.acquire("c") == a
