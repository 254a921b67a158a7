"""Robopel: reader of the family's config.json, its tensor inventory, synthetic weights.

A Robopel model is a list of post-norm layers: x += norm1(mixer(x)), then x += norm2(ff(x)), where both sublayers read the stream
itself and the norms (RMS, weight stored around zero) sit on the sublayers' OUTPUT.  config.json lists the layers; each names its
mixer -- "mingru", an element-wise gated recurrence whose gates read only the current token, or "attention", softmax attention over
a sliding window plus one mean key/value per block of tokens that has left the window, with a learned sink in the denominator,
soft-capped scores, weighted per-head q/k norm, interleaved rotary pairs with long-wavelength frequency rescaling, a sigmoid output
gate, and optionally the keys and values of an earlier layer ("kv_from") -- and its feed-forward: dense with a PolyNorm activation,
routed experts (squared-ReLU experts plus identity experts, softmax router with a choice correction, unnormalised weights), or none.
The embedding is scaled by a constant.  This module turns config.json into the flat description the native library takes
(seq.SeqModel); every size and constant comes from the config."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from . import safetensors_io as st
from .seq import BLOCK_POSTNORM, FF_EXPERTS, FF_POLYNORM, MIX_MINGRU, MIX_SOFTMAX_ATTN, ROT_INTERLEAVED

ARCHITECTURE = "Robopel"


def _attention(i: int, m: dict, n_layers: int) -> dict:
    b = {"kind": MIX_SOFTMAX_ATTN, "name": "", "heads": int(m["heads"]), "kv_heads": int(m.get("kv_heads", m["heads"])), "dim": int(m["dim"]),
         "vdim": int(m.get("vdim", m["dim"])), "scale": float(m["scale"]), "qk_norm": 2, "sink": 1, "gated": 2,
         "softcap": float(m.get("softcap") or 0.0), "kv_from": -1}
    if b["heads"] % b["kv_heads"]:
        raise ValueError(f"layer {i}: {b['heads']} query heads do not divide into {b['kv_heads']} key/value heads")
    rot = m.get("rot")
    if rot:
        b.update(rot_dims=int(rot["dims"]), rot_base=float(rot["base"]), rot_layout=ROT_INTERLEAVED)
        sc = rot.get("scaling")
        if sc:
            b.update(rot_factor=float(sc["factor"]), rot_low=float(sc["low"]), rot_high=float(sc["high"]), rot_original=float(sc["original"]))
    mask = m.get("mask")
    if mask:
        b.update(window=int(mask.get("size") or 0), pool=int(mask.get("pool") or 0))
    if m.get("kv_from") is not None:
        b["kv_from"] = int(m["kv_from"])
        if not 0 <= b["kv_from"] < i:
            raise ValueError(f"layer {i}: kv_from {b['kv_from']} is not an earlier layer")
    return b


def describe(cfg: dict) -> dict:
    """config.json (parsed) -> description for seq.SeqModel."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: {cfg.get('architecture')!r}")
    d = {"vocab": int(cfg["vocab"]), "width": int(cfg["width"]), "eps": float(cfg["norm"]["eps"]), "final_norm": 1,
         "embed_scale": float((cfg.get("embedding") or {}).get("scale", 1.0)), "layers": []}
    for i, l in enumerate(cfg["layers"]):
        m = l["mixer"]
        if l.get("type") == "mingru":
            br = {"kind": MIX_MINGRU, "name": "", "heads": 1, "dim": int(m["width"]), "vdim": int(m["width"]), "scale": 1.0}
        elif l.get("type") == "attention":
            br = _attention(i, m, len(cfg["layers"]))
        else:
            raise ValueError(f"layer {i}: unknown type {l.get('type')!r}")
        lay = {"style": BLOCK_POSTNORM, "branches": [br], "ff": 0}
        mlp = l.get("mlp")
        if mlp:
            if mlp.get("kind") == "dense":
                lay.update(ff=int(mlp["ff"]), ff_kind=FF_POLYNORM)
            elif mlp.get("kind") == "moe":
                r = mlp["router"]
                lay.update(ff=int(mlp["expert"]["ff"]), ff_kind=FF_EXPERTS, experts=int(r["experts"]), identity=int(r.get("identity") or 0), top=int(r["top"]))
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        d["layers"].append(lay)
    for i, lay in enumerate(d["layers"]):            # a shared cache must fit the layer that reads it
        b = lay["branches"][0]
        if b.get("kv_from", -1) >= 0:
            src = d["layers"][b["kv_from"]]["branches"][0]
            if src["kind"] != MIX_SOFTMAX_ATTN or src.get("kv_from", -1) >= 0:
                raise ValueError(f"layer {i}: kv_from {b['kv_from']} is not an attention layer with keys and values of its own")
            if (src["kv_heads"], src["dim"], src["vdim"]) != (b["kv_heads"], b["dim"], b["vdim"]):
                raise ValueError(f"layer {i}: head sizes differ from those of layer {b['kv_from']}, whose cache it reads")
    return d


def tensor_shapes(desc: dict) -> dict:
    """name -> shape of every tensor of a checkpoint of this description (all bfloat16)."""
    W, out = desc["width"], {}
    out["embed"] = (desc["vocab"], W)
    for i, l in enumerate(desc["layers"]):
        p, b = f"l{i}.", l["branches"][0]
        out[p + "norm1"] = (W,)
        if b["kind"] == MIX_MINGRU:
            n = b["dim"]
            out.update({p + "mix.z": (n, W), p + "mix.z.b": (n,), p + "mix.x": (n, W), p + "mix.x.b": (n,), p + "mix.g": (n, W), p + "mix.o": (W, n)})
        else:
            out[p + "mix.q"] = (b["heads"] * b["dim"], W)
            out[p + "mix.q.norm"] = (b["dim"],)
            if b["kv_from"] < 0:
                out[p + "mix.k"] = (b["kv_heads"] * b["dim"], W)
                out[p + "mix.v"] = (b["kv_heads"] * b["vdim"], W)
                out[p + "mix.k.norm"] = (b["dim"],)
            out[p + "mix.sink"] = (b["heads"],)
            out[p + "mix.g"] = (b["heads"] * b["vdim"], W)
            out[p + "mix.o"] = (W, b["heads"] * b["vdim"])
        if l["ff"]:
            out[p + "norm2"] = (W,)
            if l["ff_kind"] == FF_POLYNORM:
                out.update({p + "mlp.up": (l["ff"], W), p + "mlp.down": (W, l["ff"]), p + "mlp.act": (4,)})
            else:
                n_out = l["experts"] + l["identity"]
                out.update({p + "mlp.router": (n_out, W), p + "mlp.correction": (n_out,)})
                for e in range(l["experts"]):
                    out[f"{p}mlp.e{e}.up"] = (l["ff"], W)
                    out[f"{p}mlp.e{e}.down"] = (W, l["ff"])
    out["final.norm"] = (W,)
    out["head"] = (desc["vocab"], W)
    return out


def synth_tensors(desc: dict, seed: int = 0, gain: float = 1.0) -> dict:
    """Random weights (bfloat16 bit patterns): matrices ~ N(0, gain^2 / fan_in), norm weights near zero, an embedding whose scaled
    rows have unit-order entries."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(desc).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            a = 0.1 * rng.standard_normal(shape)
        elif name.endswith("q.norm") or name.endswith("k.norm"):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf == "sink":
            a = rng.standard_normal(shape)
        elif leaf == "b":
            a = 0.5 * rng.standard_normal(shape)
        elif leaf == "act":
            a = np.array([0.6, 0.3, 0.2, 0.05]) + 0.1 * rng.standard_normal(shape)
        elif leaf == "correction":
            a = 0.05 * rng.standard_normal(shape)
        elif name == "embed":
            a = rng.standard_normal(shape) / max(desc.get("embed_scale", 1.0), 1e-6)
        elif leaf == "router":
            a = rng.standard_normal(shape) * 2.0 * gain / np.sqrt(shape[-1])
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


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, window=24, pool=4, rot_dims=8, rot_base=10000.0, scaling=(8.0, 1.0, 4.0, 64), scale=None,
                    softcap=30.0, kv_from=None, mlp=None) -> dict:
    """One "attention" entry of config["layers"]; scaling = (factor, low, high, original) or None."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(dim ** -0.5 if scale is None else scale)}
    if softcap:
        m["softcap"] = float(softcap)
    if window:
        m["mask"] = {"size": window, "pool": pool} if pool else {"size": window}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": rot_base}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def mingru_layer(width=48, mlp=None) -> dict:
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def dense_mlp(ff=80) -> dict:
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts=6, identity=1, top=2, ff=24) -> dict:
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


def make_config(vocab=96, width=64, layers=None, embed_scale=8.0, eps=1e-5) -> dict:
    """A config.json dictionary for tests, benchmarks and examples."""
    if layers is None:
        layers = [mingru_layer(mlp=dense_mlp()), attention_layer(mlp=moe_mlp()), mingru_layer(mlp=moe_mlp()), attention_layer(kv_from=1, mlp=dense_mlp())]
    return {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "layers": layers}
