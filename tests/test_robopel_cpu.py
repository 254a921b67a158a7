"""CPU-side pieces of the Robopel family: the config reader on every constant and on absent sections, the tensor inventory, the
registry and checkpoint folder, and closed forms of the oracle's own building blocks (oracle/robopel_ref.py)."""
import json

import numpy as np
import pytest

from oracle import robopel_ref as R
from tinyllama_cpp_b200 import registry, robopel as RP, seq


def test_describe_reads_every_constant():
    layers = [RP.mingru_layer(width=36, mlp=RP.moe_mlp(experts=5, identity=3, top=4, ff=28)),
              RP.attention_layer(heads=6, kv_heads=3, dim=10, vdim=14, window=19, pool=6, rot_dims=6, rot_base=777.0, scaling=(3.0, 2.0, 5.0, 123), scale=0.21, softcap=7.5,
                                 mlp=RP.dense_mlp(44)),
              RP.attention_layer(heads=9, kv_heads=3, dim=10, vdim=14, window=5, pool=0, rot_dims=0, softcap=0, kv_from=1)]
    cfg = RP.make_config(vocab=55, width=40, layers=layers, embed_scale=3.5, eps=3e-4)
    d = RP.describe(cfg)
    assert (d["vocab"], d["width"], d["eps"], d["embed_scale"], d["final_norm"]) == (55, 40, 3e-4, 3.5, 1)
    g, a, s = (l["branches"][0] for l in d["layers"])
    assert (g["kind"], g["dim"]) == (seq.MIX_MINGRU, 36)
    l0 = d["layers"][0]
    assert (l0["style"], l0["ff_kind"], l0["ff"], l0["experts"], l0["identity"], l0["top"]) == (seq.BLOCK_POSTNORM, seq.FF_EXPERTS, 28, 5, 3, 4)
    assert (a["kind"], a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["window"], a["pool"]) == (seq.MIX_SOFTMAX_ATTN, 6, 3, 10, 14, 19, 6)
    assert (a["rot_dims"], a["rot_base"], a["rot_layout"], a["rot_factor"], a["rot_low"], a["rot_high"], a["rot_original"]) == (6, 777.0, seq.ROT_INTERLEAVED, 3.0, 2.0, 5.0, 123.0)
    assert (a["scale"], a["softcap"], a["kv_from"], a["qk_norm"], a["sink"], a["gated"]) == (0.21, 7.5, -1, 2, 1, 2)
    assert (d["layers"][1]["ff_kind"], d["layers"][1]["ff"]) == (seq.FF_POLYNORM, 44)
    assert (s["kv_from"], s["heads"], s["window"], s.get("pool", 0), s.get("rot_dims", 0), s["softcap"]) == (1, 9, 5, 0, 0, 0.0) and d["layers"][2]["ff"] == 0
    sh = RP.tensor_shapes(d)
    assert sh["l0.mix.z"] == (36, 40) and sh["l0.mix.x.b"] == (36,) and sh["l0.mix.o"] == (40, 36) and sh["l0.mlp.router"] == (8, 40) and sh["l0.mlp.correction"] == (8,)
    assert sh["l0.mlp.e4.up"] == (28, 40) and sh["l0.mlp.e4.down"] == (40, 28) and "l0.mlp.e5.up" not in sh
    assert sh["l1.mix.q"] == (60, 40) and sh["l1.mix.k"] == (30, 40) and sh["l1.mix.v"] == (42, 40) and sh["l1.mix.g"] == (84, 40) and sh["l1.mix.o"] == (40, 84)
    assert sh["l1.mix.q.norm"] == (10,) and sh["l1.mix.sink"] == (6,) and sh["l1.mlp.act"] == (4,) and sh["l1.norm2"] == (40,)
    assert "l2.mix.k" not in sh and "l2.mix.v" not in sh and "l2.mix.k.norm" not in sh and sh["l2.mix.q"] == (90, 40) and "l2.norm2" not in sh
    assert sh["final.norm"] == (40,)
    with pytest.raises(ValueError):
        RP.describe(dict(cfg, architecture="Other"))
    for path, value in ((("layers", 0, "type"), "conv"), (("layers", 1, "mlp", "kind"), "gated"), (("layers", 2, "mixer", "kv_from"), 2),
                        (("layers", 2, "mixer", "kv_from"), 0), (("layers", 2, "mixer", "dim"), 12), (("layers", 1, "mixer", "kv_heads"), 4)):
        bad = json.loads(json.dumps(cfg))
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ValueError):
            RP.describe(bad)


def test_optional_sections_may_be_absent():
    cfg = RP.make_config(layers=[RP.attention_layer(window=0, pool=0, rot_dims=0, softcap=0), RP.attention_layer(pool=0, scaling=None)])
    del cfg["embedding"]
    d = RP.describe(cfg)
    a, b = (l["branches"][0] for l in d["layers"])
    assert d["embed_scale"] == 1.0 and a.get("window", 0) == 0 and a.get("rot_dims", 0) == 0 and a["softcap"] == 0.0
    assert b["window"] == 24 and b["pool"] == 0 and b.get("rot_factor", 0.0) == 0.0 and b["rot_dims"] == 8


def test_registry_and_checkpoint_folder(tmp_path):
    cfg = RP.make_config()
    t = RP.synth_tensors(RP.describe(cfg), 1)
    RP.write_checkpoint(tmp_path / "m", cfg, t)
    assert registry.family_of(tmp_path / "m") == "Robopel" and "Robopel" in registry.STEPWISE
    desc, back = RP.read_checkpoint(tmp_path / "m")
    assert set(back) == set(RP.tensor_shapes(desc)) and all(np.array_equal(back[k], t[k]) for k in t)


def test_oracle_mingru_closed_forms():
    u = np.array([-30.0, -1.0, -1e-9, 0.0, 1e-9, 2.0])
    c = R.mingru_candidate(u)
    assert np.all(c > 0) and np.allclose(c[2:5], 0.5, atol=1e-8) and c[5] == 2.5 and np.isclose(c[1], 1 / (1 + np.e))
    # the recurrence is a convex combination: S_t = sum_s z_s c_s prod_{r > s} (1 - z_r)
    rng = np.random.default_rng(0)
    T, W_, n = 6, 5, 3
    h = rng.standard_normal((T, W_))
    wz, wx, wg, wo = (rng.standard_normal(s) for s in ((n, W_), (n, W_), (n, W_), (W_, n)))
    bz, bx = rng.standard_normal(n), rng.standard_normal(n)
    z, cand, g = R.logistic(h @ wz.T + bz), R.mingru_candidate(h @ wx.T + bx), h @ wg.T
    S = np.stack([sum(z[s] * cand[s] * np.prod(1 - z[s + 1:t + 1], axis=0) for s in range(t + 1)) for t in range(T)])
    assert np.allclose(R.mingru(h, wz, bz, wx, bx, wg, wo), (S * g / (1 + np.exp(-g))) @ wo.T)


def test_oracle_rotation_and_frequency_scaling():
    f = R.rotary_frequencies(8, 100.0)
    assert np.allclose(f, [1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75])
    # original 40, low 1, high 4: wavelengths below 10 keep their frequency, above 40 are slowed down, between are blended
    fs = R.rotary_frequencies(8, 100.0, {"factor": 5.0, "low": 1.0, "high": 4.0, "original": 40})
    wl = 2 * np.pi / f
    assert wl[0] < 10 and fs[0] == f[0] and wl[3] > 40 and np.isclose(fs[3], f[3] / 5)
    assert 10 < wl[1] < 40 and f[1] / 5 < fs[1] < f[1]
    s = (40 / wl[1] - 1.0) / 3.0
    assert np.isclose(fs[1], (1 - s) * f[1] / 5 + s * f[1])
    x = np.random.default_rng(1).standard_normal((5, 2, 10))
    y = R.rotate_interleaved(x, np.arange(5), f)
    assert np.allclose(y[..., 8:], x[..., 8:]) and np.allclose(y[0], x[0])
    assert np.allclose(np.hypot(y[..., 2], y[..., 3]), np.hypot(x[..., 2], x[..., 3]))        # pair (2, 3) turns rigidly
    a = 3 * f[1]
    assert np.allclose(y[3, 0, 2], x[3, 0, 2] * np.cos(a) - x[3, 0, 3] * np.sin(a)) and np.allclose(y[3, 0, 3], x[3, 0, 3] * np.cos(a) + x[3, 0, 2] * np.sin(a))


def test_oracle_polynorm_and_router():
    z = np.array([[1.0, -2.0, 3.0, 0.5]])
    got = R.polynorm(z, [2.0, 3.0, 5.0, 7.0], 0.0)
    want = 2 * z / np.sqrt((z ** 2).mean()) + 3 * z ** 2 / np.sqrt((z ** 4).mean()) + 5 * z ** 3 / np.sqrt((z ** 6).mean()) + 7
    assert np.allclose(got, want)
    h = np.eye(3)
    wr = np.array([[0.0, 0, 0], [1.0, 0, 0], [2.0, 0, 0], [0.5, 0, 0]])         # token 0 scores outputs 2 > 1 > 3 > 0
    pick, w = R.route(h[:1], wr, np.zeros(4), 2)
    s = np.exp([0, 1, 2, 0.5]) / np.exp([0, 1, 2, 0.5]).sum()
    assert pick.tolist() == [[2, 1]] and np.allclose(w, [[s[2], s[1]]]) and w.sum() < 1                 # weights are not renormalised
    pick, w = R.route(h[:1], wr, np.array([5.0, 0, 0, 0]), 2)
    assert pick.tolist() == [[0, 2]] and np.allclose(w, [[s[0], s[2]]])                                 # the correction picks, the score weighs
    ups, downs = [np.ones((2, 3))] * 2, [np.ones((3, 2))] * 2                                           # two experts; router output 2 is an identity expert
    pick, w = R.route(np.array([[0.0, 0.0, 1.0]]), np.array([[9.0, 0, 0], [0, 0, 0], [0.0, 0, 9]]), np.zeros(3), 1)
    assert pick.tolist() == [[2]]
    y = R.moe_ff(np.array([[0.0, 0.0, 1.0]]), np.array([[9.0, 0, 0], [0, 0, 0], [0.0, 0, 9]]), np.zeros(3), ups, downs, 1)
    assert np.allclose(y, w[0, 0] * np.array([[0.0, 0.0, 1.0]]))                                        # identity: the input itself times the weight
    y = R.moe_ff(np.array([[1.0, 0.0, 0.0]]), np.array([[9.0, 0, 0], [0, 0, 0], [0.0, 0, 9]]), np.zeros(3), ups, downs, 1)
    s0 = np.exp(9) / (np.exp(9) + 2)
    assert np.allclose(y, s0 * 2.0)                                                                     # relu(1)^2 summed over ff = 2, on every output


def test_oracle_layer_is_post_norm():
    """x + norm(sublayer(x)): scaling a sublayer's out projection by any positive number leaves the layer's output unchanged."""
    cfg = RP.make_config(vocab=30, width=16, layers=[RP.mingru_layer(width=8, mlp=RP.dense_mlp(12))], eps=0.0)
    t = RP.synth_tensors(RP.describe(cfg), 3)
    W = {k: R.bf16_to_float(v) for k, v in t.items()}
    a = R.forward(cfg, W, [1, 2, 3, 4])[0]
    W2 = dict(W)
    W2["l0.mix.o"] = 4.0 * W["l0.mix.o"]
    W2["l0.mlp.down"] = 0.25 * W["l0.mlp.down"]
    assert np.allclose(a, R.forward(cfg, W2, [1, 2, 3, 4])[0])
