"""Reninex: reader of the family's config.json, its tensor inventory, synthetic weights.

A Reninex model is a list of parallel blocks.  Each block normalises the stream once (RMS norm with a single gain), feeds the
result through a short causal per-channel convolution (one filter in front of the mixer, one in front of the feed-forward) and
adds mixer + feed-forward to the stream.  The mixer is the weighted sum of two branches that read the same input:
"left", causal attention with unit-RMS queries and keys, grouped key/value heads, no positions and a per-head sigmoid instead of
a softmax; "right", retention: a per-head linear recurrence with a fixed decay, rotary positions on queries and keys, a unit-RMS
output per head and a SiLU gate.  A range of layers may be run several times with shared weights (each pass enters through a
projection of [stream | embedding output] plus a per-pass vector and keeps its own state), and the embedding adds a hashed
bigram row.  This module turns config.json into the flat description the native library takes (seq.SeqModel).
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from . import safetensors_io as st
from .seq import MIX_RETENTION, MIX_SIGMOID_ATTN

ARCHITECTURE = "Reninex"


def describe(cfg: dict) -> dict:
    """config.json (parsed) -> description for seq.SeqModel.  Every size and constant comes from cfg."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: {cfg.get('architecture')!r}")
    d = {"vocab": int(cfg["vocab"]), "width": int(cfg["width"]), "eps": float(cfg["norm"]["eps"]), "layers": []}
    canon = cfg.get("canon")
    d["taps"] = int(canon["taps"]) if canon else 0
    bg = (cfg.get("embedding") or {}).get("bigram")
    d["bigram"] = {k: int(bg[k]) for k in ("buckets", "mul_prev", "mul_cur")} if bg else None
    lp = cfg.get("loop")
    d["loop"] = {k: int(lp[k]) for k in ("start", "stop", "times")} if lp and int(lp.get("times", 0)) > 0 and int(lp["stop"]) > int(lp["start"]) else None
    for i, l in enumerate(cfg["layers"]):
        if l.get("type") != "parallel":
            raise ValueError(f"layer {i}: unknown type {l.get('type')!r}")
        m, branches = l["mixer"], []
        le, ri = m["left"], m["right"]
        branches.append({"kind": MIX_SIGMOID_ATTN, "name": "left", "heads": int(le["heads"]), "kv_heads": int(le["kv_heads"]),
                         "dim": int(le["dim"]), "vdim": int(le["vdim"]), "scale": float(le["scale"]), "qk_norm": 1,
                         "out_scale": float(m["left_scale"])})
        rot = ri.get("rot")
        if len(ri["decay"]) != int(ri["heads"]):
            raise ValueError(f"layer {i}: {len(ri['decay'])} decays for {ri['heads']} heads")
        branches.append({"kind": MIX_RETENTION, "name": "right", "heads": int(ri["heads"]), "dim": int(ri["dim"]), "vdim": int(ri["vdim"]),
                         "scale": float(int(ri["dim"]) ** -0.5), "rot_dims": int(rot["dims"]) if rot else 0,
                         "rot_base": float(rot["base"]) if rot else 1.0, "out_norm": 1, "gated": 1,
                         "decay": [float(x) for x in ri["decay"]], "out_scale": float(m["right_scale"])})
        mlp = l.get("mlp")
        if mlp is not None and mlp.get("kind") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        d["layers"].append({"branches": branches, "ff": int(mlp["ff"]) if mlp else 0})
    return d


def tensor_shapes(desc: dict) -> dict:
    """name -> shape of every tensor of a checkpoint of this description (all bfloat16)."""
    W, out = desc["width"], {}
    out["embed"] = (desc["vocab"], W)
    if desc["bigram"]:
        out["bigram"] = (desc["bigram"]["buckets"] + 1, W)
    if desc["loop"]:
        out["loop.in"] = (W, 2 * W)
        out["loop.step"] = (desc["loop"]["times"], W)
    for i, l in enumerate(desc["layers"]):
        p = f"l{i}."
        out[p + "norm1"] = ()
        for b in l["branches"]:
            bp = p + "mix." + b["name"] + "."
            kvh = b.get("kv_heads", b["heads"])
            out[bp + "q"] = (b["heads"] * b["dim"], W)
            out[bp + "k"] = (kvh * b["dim"], W)
            out[bp + "v"] = (kvh * b["vdim"], W)
            if b["kind"] == MIX_SIGMOID_ATTN:
                out[bp + "pb"] = (b["heads"],)
            if b.get("gated"):
                out[bp + "g"] = (b["heads"] * b["vdim"], W)
            out[bp + "o"] = (W, b["heads"] * b["vdim"])
        if l["ff"]:
            out[p + "mlp.gate"] = (l["ff"], W)
            out[p + "mlp.up"] = (l["ff"], W)
            out[p + "mlp.down"] = (W, l["ff"])
        if desc["taps"]:
            out[p + "canon1"] = (W, desc["taps"])
            if l["ff"]:
                out[p + "canon2"] = (W, desc["taps"])
    out["final.norm"] = ()
    out["head"] = (desc["vocab"], W)
    return out


def synth_tensors(desc: dict, seed: int = 0, gain: float = 1.0) -> dict:
    """Random weights (bfloat16 bit patterns) with unit-scale activations: matrices ~ N(0, gain^2 / fan_in), gains near 1."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(desc).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm"):
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif leaf == "pb":
            a = rng.standard_normal(shape) - 1.0
        elif leaf in ("canon1", "canon2"):
            a = 0.3 * rng.standard_normal(shape)
        elif leaf == "step":
            a = 0.1 * rng.standard_normal(shape)
        elif name in ("embed", "bigram"):
            a = rng.standard_normal(shape) * (0.7 if desc["bigram"] else 1.0)
        else:
            a = rng.standard_normal(shape) * gain / np.sqrt(shape[-1])
        out[name] = st.f32_to_bf16_bits(np.asarray(a, np.float32))
    return out


def read_checkpoint(model_dir) -> tuple[dict, dict]:
    """(description, name -> bfloat16 bit patterns) of a folder with config.json and model.safetensors."""
    model_dir = Path(model_dir)
    desc = describe(json.loads((model_dir / "config.json").read_text()))
    return desc, st.read_as_bf16(model_dir / "model.safetensors", tensor_shapes(desc), ARCHITECTURE)


def write_checkpoint(model_dir, cfg: dict, tensors: dict) -> None:
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    (model_dir / "config.json").write_text(json.dumps(cfg, indent=1))
    st.write(model_dir / "model.safetensors", {k: ("BF16", v) for k, v in tensors.items()})


def make_config(vocab=96, width=64, n_layers=2, ff=96, taps=3, l_heads=4, l_kv=2, l_dim=16, l_vdim=16, r_heads=2, r_dim=16, r_vdim=32,
                rot_dims=8, rot_base=10000.0, loop=None, bigram=(61, 7, 3), left_scale=0.7, right_scale=0.4, eps=1e-5, no_mlp=()) -> dict:
    """A config.json dictionary for tests, benchmarks and examples."""
    decay = [float(1.0 - 2.0 ** (-3 - 1.5 * h)) for h in range(r_heads)]
    layer = lambda i: {"type": "parallel", "mixer": {
        "left": {"heads": l_heads, "kv_heads": l_kv, "dim": l_dim, "vdim": l_vdim, "scale": float(l_dim ** -0.5)}, "left_scale": left_scale,
        "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": decay, "rot": {"dims": rot_dims, "base": rot_base} if rot_dims else None},
        "right_scale": right_scale}, "mlp": None if i in no_mlp else {"kind": "dense", "ff": ff}}
    cfg = {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": [layer(i) for i in range(n_layers)]}
    if taps:
        cfg["canon"] = {"taps": taps}
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg
