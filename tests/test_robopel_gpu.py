"""The Robopel family on the layer-list library (libgten_b200_seq.so) against the plain numpy restatement in oracle/robopel_ref.py.

Every test makes its own small configuration and random weights.  float32 mode is held to rounding (1e-4 of the logits' spread);
bfloat16 mode to a loose bound that a wrong key, window edge, state or expert still breaks by orders of magnitude.  Where random
weights would hide a fault (one far key among hundreds, a window's edge, a pooled block) the test plants a key that the last query
matches and lets the oracle confirm that this key carries the query's attention."""
import json

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle import robopel_ref as R  # noqa: E402
from tinyllama_cpp_b200 import robopel as RP  # noqa: E402
from tinyllama_cpp_b200 import safetensors_io as st  # noqa: E402


@pytest.fixture(scope="module")
def lib():
    from tinyllama_cpp_b200 import build, seq
    build.build(target="seq")
    seq.init(0)
    return seq


def make(lib, cfg, mode="float32", seed=0, n_slots=3, max_ctx=512, max_rows=0, tweak=None, **synth):
    desc = RP.describe(cfg)
    t = RP.synth_tensors(desc, seed, **synth)
    if tweak:
        tweak(t)
    m = lib.SeqModel(desc, lib.MODE_BY_NAME[mode], n_slots, max_ctx, max_rows).load(t)
    return m, {k: R.bf16_to_float(v) for k, v in t.items()}


def rel(got, want):
    """rms of the difference after removing each row's mean, over the rms spread of the expected rows."""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float(np.sqrt((d * d).mean(-1)).max() / np.sqrt((w * w).mean()))


TOL = {"float32": 1e-4, "bfloat16": 6e-2}


def close(got, want, mode, cfg=None):
    """Within TOL on every row -- except bfloat16 runs of models with routed experts: operand rounding may flip a close choice between two
    experts at a few tokens (a flipped token is then off by its whole expert, and colours the rows after it), so there nine rows in ten
    are held to TOL and the rest only to being of the logits' own size."""
    routed = cfg is not None and any((l.get("mlp") or {}).get("kind") == "moe" for l in cfg["layers"])
    if mode != "bfloat16" or not routed:
        return rel(got, want) < TOL[mode]
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    rows = np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean())
    return float(np.mean(rows < TOL[mode])) >= 0.9 and float(rows.max()) < 2.0


def toks(seed, n, vocab, lo=0):
    return np.random.default_rng(1000 + seed).integers(lo, vocab, n).astype(np.int32)


A, G, D, E = RP.attention_layer, RP.mingru_layer, RP.dense_mlp, RP.moe_mlp


# ------------------------------------------------------------------ each mechanism alone
VARIANTS = {
    "mingru": [G(width=40)],
    "mingru_dense": [G(width=72, mlp=D(88))],
    "attention_plain": [A(heads=2, kv_heads=2, dim=12, vdim=20, window=0, pool=0, rot_dims=0, softcap=0)],
    "attention_window": [A(heads=3, kv_heads=1, dim=16, vdim=8, window=9, pool=0, rot_dims=0, softcap=0)],
    "attention_pool": [A(heads=4, kv_heads=2, dim=8, vdim=8, window=7, pool=3, rot_dims=0, softcap=0)],
    "attention_rot": [A(window=0, pool=0, rot_dims=16, scaling=None, softcap=0)],
    "attention_rot_scaled_partial": [A(window=0, pool=0, rot_dims=10, rot_base=300.0, scaling=(6.0, 1.0, 3.0, 40), softcap=0)],
    "attention_softcap": [A(window=0, pool=0, rot_dims=0, softcap=1.5, scale=0.9)],
    "attention_all": [A(heads=6, kv_heads=3, dim=12, vdim=20, window=11, pool=4, rot_dims=8, softcap=4.0, mlp=D(40))],
    "experts": [G(width=32, mlp=E(experts=5, identity=0, top=2, ff=24))],
    "experts_identity": [G(width=32, mlp=E(experts=4, identity=3, top=3, ff=20))],
    "experts_top1": [G(width=32, mlp=E(experts=7, identity=1, top=1, ff=8))],
    "shared_cache": [A(window=10, pool=2, mlp=D(48)), G(width=24), A(heads=8, kv_heads=2, window=5, pool=3, rot_dims=4, kv_from=0, softcap=0, mlp=E())],
    "all": None,
}


@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", list(VARIANTS))
def test_mechanisms_one_at_a_time(lib, mode, variant):
    cfg = RP.make_config(vocab=101, width=72, layers=VARIANTS[variant], embed_scale=5.0)
    m, W = make(lib, cfg, mode, seed=3)
    m.set_option("capture", 1)
    t = toks(1, 41, cfg["vocab"])
    got = m.step([(0, t)], range(len(t)))
    want, trace = R.forward(cfg, W, t)
    assert m.n_runs == trace.shape[0]
    for u in range(m.n_runs):            # the stream after every layer, first and last row
        for r in (0, len(t) - 1):
            assert rel(m.read_capture(u, r)[None], trace[u, r][None]) < TOL[mode] * (4 if mode == "bfloat16" else 1), (u, r)
    assert rel(got, want) < TOL[mode]


def test_oracle_attention_is_a_softmax_with_a_sink_over_window_and_blocks():
    """Guards the oracle: its weights are positive, sum to less than one by the sink's share, and cover exactly the window's tokens
    and the blocks that lie wholly before it."""
    rng = np.random.default_rng(0)
    T, W_, H, Gk, d, dv, win, P = 23, 10, 4, 2, 6, 5, 6, 4
    h = rng.standard_normal((T, W_))
    wq, wk, wv = rng.standard_normal((H * d, W_)), rng.standard_normal((Gk * d, W_)), rng.standard_normal((Gk * dv, W_))
    k, v = R.keys_and_values(h, wk, wv, None, Gk, d, dv, None, 1e-6)
    sink = rng.standard_normal(H)
    _, book = R.softmax_attention(h, wq, None, k, v, sink, None, rng.standard_normal((W_, H * dv)), H, d, dv, 0.4, None, win, P, None, 1e-6, return_weights=True)
    for i, hd, blocks, tk, w in book:
        assert tk == list(range(max(0, i - win + 1), i + 1))
        assert blocks == [b for b in range(T) if b * P + P - 1 <= i - win]
        assert np.all(w > 0) and len(w) == len(blocks) + len(tk)
        s = np.concatenate([[k[b * P:(b + 1) * P, hd // 2].mean(0) @ (h[i] @ wq.T).reshape(H, d)[hd] for b in blocks],
                            [k[j, hd // 2] @ (h[i] @ wq.T).reshape(H, d)[hd] for j in tk]]) * 0.4
        assert np.isclose(w.sum(), np.exp(s).sum() / (np.exp(s).sum() + np.exp(sink[hd])))
    assert R.visible(13, 6, 4) == ([8, 9, 10, 11, 12, 13], [0, 1]) and R.visible(10, 6, 4) == ([5, 6, 7, 8, 9, 10], [0])
    assert R.visible(5, 6, 4) == ([0, 1, 2, 3, 4, 5], [])


# ------------------------------------------------------------------ prefill = decode = portions
@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
def test_prefill_against_token_by_token(lib, mode):
    cfg = RP.make_config(vocab=90, width=64)
    m, W = make(lib, cfg, mode, seed=5)
    t = toks(2, 70, cfg["vocab"])
    whole = m.step([(0, t)], range(len(t)))
    one = np.concatenate([m.step([(1, t[i:i + 1])], [0]) for i in range(len(t))])
    want, _ = R.forward(cfg, W, t)
    assert rel(whole, want) < TOL[mode] and rel(one, want) < TOL[mode]
    assert rel(one, whole) < TOL[mode]


@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 50, 2, 7, 1, 1, 30], [33, 1, 64, 2], [97, 3], [1] * 5 + [95], [70, 30]])
def test_portions_of_any_size(lib, sizes):
    layers = [A(heads=4, kv_heads=1, dim=8, vdim=24, window=13, pool=5, rot_dims=4, mlp=E(experts=5, identity=2, top=2, ff=12)), G(width=40, mlp=D(56)),
              A(heads=2, kv_heads=1, dim=8, vdim=24, window=29, pool=2, rot_dims=8, kv_from=0)]
    cfg = RP.make_config(vocab=77, width=48, layers=layers)
    m, W = make(lib, cfg, "float32", seed=7)
    n = sum(sizes)
    t = toks(3, n, cfg["vocab"])
    want, _ = R.forward(cfg, W, t)
    at, rows = 0, []
    for s in sizes:
        rows.append(m.step([(2, t[at:at + s])], range(s)))
        at += s
    assert m.position(2) == n
    assert rel(np.concatenate(rows), want) < TOL["float32"]


def test_passes_inside_a_step_cut_anywhere(lib):
    """max_rows smaller than a step: the library cuts the step into passes; same logits."""
    cfg = RP.make_config(vocab=64, width=64)
    t = toks(4, 70, 64)
    m1, W = make(lib, cfg, "float32", seed=9, max_rows=16)
    m2, _ = make(lib, cfg, "float32", seed=9)
    a = m1.step([(0, t), (1, t[:23])], range(93))
    b = m2.step([(0, t), (1, t[:23])], range(93))
    want, _ = R.forward(cfg, W, t)
    assert rel(a[:70], want) < TOL["float32"] and rel(a, b) < 1e-5


# ------------------------------------------------------------------ batches, slots
@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
def test_batch_of_unequal_requests_equals_each_alone(lib, mode):
    cfg = RP.make_config(vocab=80, width=64)
    m, W = make(lib, cfg, mode, seed=11, n_slots=4)
    seqs = [toks(10 + i, n, 80) for i, n in enumerate((67, 5, 94, 1))]
    first = [s[: max(1, len(s) // 2)] for s in seqs]
    out1 = m.step([(i, f) for i, f in enumerate(first)], range(sum(len(f) for f in first)))
    rest = [(i, s[len(f):]) for i, (s, f) in enumerate(zip(seqs, first)) if len(s) > len(f)]
    out2 = m.step(rest, range(sum(len(r) for _, r in rest)))
    at1, at2 = 0, 0
    for i, (s, f) in enumerate(zip(seqs, first)):
        want, _ = R.forward(cfg, W, s)
        got = out1[at1:at1 + len(f)]
        at1 += len(f)
        if len(s) > len(f):
            got = np.concatenate([got, out2[at2:at2 + len(s) - len(f)]])
            at2 += len(s) - len(f)
        assert rel(got, want) < TOL[mode], i


def test_slot_freed_and_used_again(lib):
    from tinyllama_cpp_b200.scheduler import SlotManager
    cfg = RP.make_config(vocab=70, width=64)
    m, W = make(lib, cfg, "float32", seed=13, n_slots=2)
    sm = SlotManager(m)
    a, b, c = toks(20, 60, 70), toks(21, 9, 70), toks(22, 45, 70)
    sa = sm.acquire("a")
    m.step([(sa, a)])
    sb = sm.acquire("b")
    m.step([(sb, b[:4])])
    sm.release("a")
    sc = sm.acquire("c")                 # takes a's slot: a's cache, pooled blocks and recurrent state must not show
    assert sc == sa
    got_c = m.step([(sc, c), (sb, b[4:])], range(len(c) + len(b) - 4))
    assert rel(got_c[: len(c)], R.forward(cfg, W, c)[0]) < TOL["float32"]
    assert rel(got_c[len(c):], R.forward(cfg, W, b)[0][4:]) < TOL["float32"]
    with pytest.raises(RuntimeError):
        sm.acquire("d")


# ------------------------------------------------------------------ planted keys: window edges, pooled blocks, far keys
NEEDLE, QUERY = 1, 2


def planted(lib, window, pool, mode="float32", heads=2, kv_heads=1, dim=16, rot_dims=0, max_ctx=600):
    """One attention layer without a feed-forward.  Token QUERY's query points at token NEEDLE's key (the needle's embedding is solved
    for: W_k e_needle = W_q[head 0] e_query up to the norm, plus a part outside W_k's row space that makes its VALUE distinct); a large
    score scale makes the match carry the softmax.  Filler tokens are 3 .. vocab-1."""
    cfg = RP.make_config(vocab=60, width=64, embed_scale=4.0,
                         layers=[A(heads=heads, kv_heads=kv_heads, dim=dim, vdim=16, window=window, pool=pool, rot_dims=rot_dims, scaling=None, scale=1.2, softcap=0)])

    def tweak(t):
        emb = st.bf16_bits_to_f32(t["embed"]).astype(np.float64)
        wq, wk = (st.bf16_bits_to_f32(t["l0.mix." + n]).astype(np.float64) for n in ("q", "k"))
        target = wq[:dim] @ emb[QUERY] / (st.bf16_bits_to_f32(t["l0.mix.q.norm"]) / st.bf16_bits_to_f32(t["l0.mix.k.norm"]))
        e = np.linalg.pinv(wk[:dim]) @ target
        null = np.random.default_rng(5).standard_normal(64)
        null -= np.linalg.pinv(wk[:dim]) @ (wk[:dim] @ null)
        emb[NEEDLE] = e + 2.0 * null * np.linalg.norm(e) / np.linalg.norm(null)
        t["embed"] = st.f32_to_bf16_bits(emb.astype(np.float32))
        t["l0.mix.sink"] = st.f32_to_bf16_bits(np.full(heads, -4.0, np.float32))
    return cfg, make(lib, cfg, mode, seed=17, max_ctx=max_ctx, tweak=tweak)


def needle_weight(cfg, W, t):
    """Share of the last query's attention (head 0) that lands on keys made of needle tokens, by the oracle."""
    m = cfg["layers"][0]["mixer"]
    x = W["embed"][t] * cfg["embedding"]["scale"]
    fr = R.layer_freqs(m)
    mask = m.get("mask") or {}
    k, v = R.keys_and_values(x, W["l0.mix.k"], W["l0.mix.v"], W["l0.mix.k.norm"], m["kv_heads"], m["dim"], m["vdim"], fr, cfg["norm"]["eps"])
    _, book = R.softmax_attention(x, W["l0.mix.q"], W["l0.mix.q.norm"], k, v, W["l0.mix.sink"], W["l0.mix.g"], W["l0.mix.o"], m["heads"], m["dim"], m["vdim"],
                                  m["scale"], m.get("softcap"), mask.get("size"), mask.get("pool"), fr, cfg["norm"]["eps"], return_weights=True)
    i, hd, blocks, tk, w = [b for b in book if b[0] == len(t) - 1 and b[1] == 0][0]
    P = mask.get("pool") or 1
    share = sum(w[n] for n, b in enumerate(blocks) if np.all(t[b * P:(b + 1) * P] == NEEDLE))
    return share + sum(w[len(blocks) + n] for n, j in enumerate(tk) if t[j] == NEEDLE)


def run_three_ways(m, t):
    """The last token's logits: whole prompt, decoded alone after the rest, and in portions of changing size."""
    n = len(t)
    whole = m.step([(0, t)], [n - 1])
    m.step([(1, t[:-1])])
    dec = m.step([(1, t[-1:])], [0])
    at, sizes = 0, [2, 37, 3, 64, 2, 5]
    while at < n - 1:
        s = min(sizes[0], n - 1 - at)
        sizes = sizes[1:] + sizes[:1]
        m.step([(2, t[at:at + s])])
        at += s
    por = m.step([(2, t[-1:])], [0])
    for s in range(3):
        m.reset(s)
    return whole, dec, por


@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
def test_window_edge_in_prompt_and_decode(lib, mode):
    """A needle exactly `window - 1` tokens back is seen, one token further it is not (no pooled blocks here)."""
    window, n = 21, 90
    cfg, (m, W) = planted(lib, window, 0, mode)
    seen = {}
    for back in (window - 1, window):
        t = toks(30, n, 60, lo=3)
        t[-1], t[n - 1 - back] = QUERY, NEEDLE
        share = needle_weight(cfg, W, t)
        seen[back] = share
        want = R.forward(cfg, W, t)[0][-1:]
        for got in run_three_ways(m, t):
            assert rel(got, want) < TOL[mode], back
    assert seen[window - 1] > 0.5 and seen[window] == 0.0


@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,pool", [(16, 4), (10, 7), (33, 2)])
def test_pooled_block_just_seen_and_not_yet(lib, mode, window, pool):
    """A block of needles that ends exactly at i - window is seen as one pooled key, and so is one far back.  A block that ends one
    token later is not seen: its last token is the window's oldest and its other tokens are seen by nobody -- needles planted there
    must not reach the query (a block that is pooled one token early would show them)."""
    n = 130
    cfg, (m, W) = planted(lib, window, pool, mode)
    for end_gap, hidden in ((window, False), (window + pool * 9, False), (window - 1, True)):       # i - (last position of the block)
        t = toks(31, n, 60, lo=3)
        t = t[: n - (n - end_gap) % pool]                # shorten the sequence until a block ends exactly end_gap before the query
        t[-1] = QUERY
        i = len(t) - 1
        b = (i - end_gap) // pool
        assert b * pool + pool - 1 == i - end_gap
        t[b * pool:(b + 1) * pool - (1 if hidden else 0)] = NEEDLE
        share = needle_weight(cfg, W, t)
        want = R.forward(cfg, W, t)[0][-1:]
        for got in run_three_ways(m, t):
            assert rel(got, want) < TOL[mode], end_gap
        if hidden:
            plain = t.copy()
            plain[t == NEEDLE] = 9
            assert share == 0.0 and rel(R.forward(cfg, W, plain)[0][-1:], want) < 1e-9
        else:
            assert share > 0.4


def test_far_key_among_hundreds(lib):
    """A single needle block hundreds of tokens back among ~140 pooled blocks carries the last query; without it the answer moves."""
    window, pool, n = 24, 4, 590
    cfg, (m, W) = planted(lib, window, pool, "float32", heads=4, kv_heads=2, rot_dims=0, max_ctx=600)
    t = toks(32, n, 60, lo=3)
    t[-1] = QUERY
    t[8:12] = NEEDLE
    assert needle_weight(cfg, W, t) > 0.4
    want = R.forward(cfg, W, t)[0][-1:]
    for got in run_three_ways(m, t):
        assert rel(got, want) < TOL["float32"]
    t2 = t.copy()
    t2[8:12] = 7
    assert rel(R.forward(cfg, W, t2)[0][-1:], want) > 50 * TOL["float32"]


@pytest.mark.parametrize("n", [127, 128, 129, 257])
def test_key_tile_borders_in_prompt_and_decode(lib, n):
    cfg = RP.make_config(vocab=64, width=64, layers=[A(heads=2, kv_heads=2, window=0, pool=0), A(heads=2, kv_heads=1, window=150, pool=8, mlp=D(32))])
    m, W = make(lib, cfg, "float32", seed=19)
    t = toks(30, n + 2, 64)
    want, _ = R.forward(cfg, W, t)
    got = m.step([(0, t[:n])], [n - 2, n - 1])
    got = np.concatenate([got, m.step([(0, t[n:n + 1])], [0]), m.step([(0, t[n + 1:])], [0])])
    assert rel(got, want[n - 2:]) < TOL["float32"]


def test_first_tokens(lib):
    """Positions 0 .. a few: an empty recurrent state, a window that is not yet full, no pooled block, the sink alone beside one key."""
    cfg = RP.make_config(vocab=50, width=64, layers=[G(mlp=E()), A(window=4, pool=2, mlp=D()), A(window=3, pool=1, kv_from=1)])
    m, W = make(lib, cfg, "float32", seed=23)
    t = toks(40, 11, 50)
    want, _ = R.forward(cfg, W, t)
    assert rel(m.step([(0, t)], range(11)), want) < TOL["float32"]
    got = np.concatenate([m.step([(1, t[i:i + 1])], [0]) for i in range(11)])
    assert rel(got, want) < TOL["float32"]


# ------------------------------------------------------------------ long decoding, other sizes
@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
def test_long_decoding(lib, mode):
    """The window and the pooled blocks move over decoded tokens; the recurrent state is carried 250 steps."""
    cfg = RP.make_config(vocab=64, width=64, layers=[G(mlp=D()), A(window=40, pool=8, mlp=E()), A(window=17, pool=3, kv_from=1), G(width=24)])
    m, W = make(lib, cfg, mode, seed=29)
    t = toks(50, 260, 64)
    want, _ = R.forward(cfg, W, t)
    m.step([(0, t[:10])])
    got = np.concatenate([m.step([(0, t[i:i + 1])], [0]) for i in range(10, 260)])
    assert rel(got, want[10:]) < TOL[mode]
    assert rel(got[-5:], want[-5:]) < TOL[mode]


@pytest.mark.parametrize("layers,vocab,width", [
    ([G(width=9, mlp=D(24)), A(heads=1, kv_heads=1, dim=40, vdim=8, window=5, pool=5, rot_dims=2), A(heads=3, kv_heads=1, dim=40, vdim=8, window=50, pool=1, rot_dims=40, kv_from=1, mlp=E(3, 0, 3, 8))], 33, 40),
    ([A(heads=8, kv_heads=8, dim=8, vdim=24, window=6, pool=6, rot_dims=8, mlp=E(9, 4, 4, 40)), G(width=200, mlp=E(2, 1, 1, 72))], 130, 136),
    ([A(heads=2, kv_heads=1, dim=136, vdim=200, window=12, pool=3, rot_dims=64, mlp=D(32))], 64, 64),                      # heads beyond the tiled kernels' sizes
    ([A(heads=4, kv_heads=2, dim=20, vdim=12, window=1, pool=2), A(heads=2, kv_heads=2, dim=20, vdim=12, window=64, pool=64, kv_from=0)], 64, 64),   # a window of one token
    ([A(heads=2, kv_heads=2, dim=16, vdim=16, window=8, pool=0), G(width=64)], 64, 64),                                       # a window without pooled blocks
    ([G(width=25, mlp=E(3, 1, 2, 10)), A(heads=3, kv_heads=1, dim=20, vdim=10, window=9, pool=4, rot_dims=10, mlp=D(30))], 37, 50),  # rows that are no multiple of four
])
def test_other_sizes(lib, layers, vocab, width):
    cfg = RP.make_config(vocab=vocab, width=width, layers=layers, embed_scale=1.0, eps=3e-4)
    m, W = make(lib, cfg, "float32", seed=31)
    t = toks(60, 85, vocab)
    want, _ = R.forward(cfg, W, t)
    got = np.concatenate([m.step([(0, t[:20])], range(20)), m.step([(0, t[20:22])], range(2)), m.step([(0, t[22:])], range(63))])
    assert rel(got, want) < TOL["float32"]


@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
@pytest.mark.parametrize("layers", [
    [A(heads=4, kv_heads=2, dim=16, vdim=16, window=40, pool=8, rot_dims=16, mlp=E(6, 2, 2, 32)), G(width=48, mlp=D(64))],
    [A(heads=2, kv_heads=1, dim=48, vdim=40, window=100, pool=16, rot_dims=24), A(heads=4, kv_heads=1, dim=48, vdim=40, window=70, pool=5, rot_dims=48, kv_from=0, mlp=E(3, 1, 2, 24))],
    [A(heads=3, kv_heads=3, dim=20, vdim=12, window=64, pool=64, rot_dims=8), G(width=136, mlp=E(12, 3, 2, 80))],
    [A(heads=2, kv_heads=2, dim=128, vdim=128, window=0, pool=0, rot_dims=128, softcap=0), A(heads=2, kv_heads=2, dim=64, vdim=64, window=128, pool=32, mlp=D(128))],
])
def test_tiled_kernels_on_portions(lib, mode, layers):
    """Prompt portions run the tiled kernels (chunked minGRU, tensor-core attention and grouped expert products in bfloat16 mode):
    portions that start in the middle of a sequence, end inside a tile or chunk, passes of several segments -- against the oracle and
    against the row kernels (options fused_attn = 0, grouped_experts = 0)."""
    cfg = RP.make_config(vocab=64, width=64, layers=layers)
    m, W = make(lib, cfg, mode, seed=61, n_slots=4, max_ctx=400)
    a, b = toks(110, 300, 64), toks(111, 170, 64)
    wa, wb = R.forward(cfg, W, a)[0], R.forward(cfg, W, b)[0]
    outs = {}
    for fused in (1, 0):
        m.set_option("fused_attn", fused)
        m.set_option("grouped_experts", fused)
        sa, sb = (0, 1) if fused else (2, 3)
        g1 = m.step([(sa, a[:70])], range(70))
        g2 = m.step([(sa, a[70:199]), (sb, b[:33])], range(129 + 33))
        g3 = m.step([(sb, b[33:170]), (sa, a[199:300])], range(137 + 101))
        ga = np.concatenate([g1, g2[:129], g3[137:]])
        gb = np.concatenate([g2[129:], g3[:137]])
        assert close(ga, wa, mode, cfg) and close(gb, wb, mode, cfg), (fused, rel(ga, wa), rel(gb, wb))
        outs[fused] = (ga, gb)
    assert close(outs[1][0], outs[0][0], mode, cfg) and close(outs[1][1], outs[0][1], mode, cfg)
    nxt = m.step([(0, [5])], [0])            # decoding continues from the state the tiled kernels left
    assert rel(nxt, R.forward(cfg, W, np.append(a, 5))[0][-1:]) < (TOL[mode] if mode == "float32" else 2.0)


@pytest.mark.parametrize("width,layers", [
    (72, [G(width=50, mlp=E(5, 1, 2, 12)), A(heads=6, kv_heads=2, dim=12, vdim=20, window=31, pool=3, rot_dims=6, mlp=D(88))]),
    (50, [A(heads=3, kv_heads=3, dim=20, vdim=10, window=40, pool=7, rot_dims=10, mlp=D(30)), G(width=25, mlp=D(90)), A(heads=6, kv_heads=3, dim=20, vdim=10, window=0, pool=0, kv_from=0)]),
])
def test_tensor_core_path_with_awkward_sizes(lib, width, layers):
    """bfloat16 mode, portions of 64 rows and more: the tcgen05 products and the tiled kernels with sizes that are multiples of nothing."""
    cfg = RP.make_config(vocab=101, width=width, layers=layers)
    m, W = make(lib, cfg, "bfloat16", seed=67)
    t = toks(120, 150, cfg["vocab"])
    want, _ = R.forward(cfg, W, t)
    got = np.concatenate([m.step([(0, t[:70])], range(70)), m.step([(0, t[70:])], range(80))])
    assert close(got, want, "bfloat16", cfg)
    m.set_option("tensor", 0)
    simt = np.concatenate([m.step([(1, t[:70])], range(70)), m.step([(1, t[70:])], range(80))])
    assert close(got, simt, "bfloat16", cfg)


def test_router_choice_uses_the_correction_and_weights_do_not(lib):
    """A large correction on one expert forces its choice although its score is small; its weight stays the small score."""
    cfg = RP.make_config(vocab=40, width=32, layers=[G(width=16, mlp=E(experts=4, identity=1, top=2, ff=16))])

    def tweak(t):
        c = np.zeros(5, np.float32)
        c[3] = 10.0
        t["l0.mlp.correction"] = st.f32_to_bf16_bits(c)
    m, W = make(lib, cfg, "float32", seed=71, tweak=tweak)
    t = toks(7, 30, 40)
    pick, w = R.route(np.random.default_rng(0).standard_normal((6, 32)), W["l0.mlp.router"], W["l0.mlp.correction"], 2)
    assert np.all(pick[:, 0] == 3) and np.all(w[:, 0] < 0.9)          # the restatement: expert 3 always comes first, with a score of its own size
    want = R.forward(cfg, W, t)[0]
    assert rel(m.step([(0, t)], range(30)), want) < TOL["float32"]                                             # whole prompt: router product + routing kernel
    assert rel(np.concatenate([m.step([(1, t[i:i + 1])], [0]) for i in range(30)]), want) < TOL["float32"]      # row by row: routing inside the residual update
    plain = dict(W)
    plain["l0.mlp.correction"] = np.zeros(5)
    assert rel(R.forward(cfg, plain, t)[0], want) > 50 * TOL["float32"]                                        # and the correction matters


# ------------------------------------------------------------------ generation through the scheduler, command line
def oracle_greedy(cfg, W, prompt, n_new):
    t = list(prompt)
    margins = []
    for _ in range(n_new):
        lg = R.forward(cfg, W, t)[0][-1]
        o = np.argsort(lg)
        margins.append(lg[o[-1]] - lg[o[-2]])
        t.append(int(o[-1]))
    return np.asarray(t[len(prompt):]), np.asarray(margins)


def test_greedy_generation_through_the_scheduler(lib):
    from tinyllama_cpp_b200.scheduler import generate
    cfg = RP.make_config(vocab=64, width=64)
    m, W = make(lib, cfg, "float32", seed=41, n_slots=2, gain=2.0)
    prompts = [toks(80 + i, n, 64) for i, n in enumerate((19, 3, 40))]     # three requests, two slots: one waits
    outs = generate(m, prompts, 12, chunk=8, burst=5)
    for p, o in zip(prompts, outs):
        want, margin = oracle_greedy(cfg, W, p, 12)
        assert len(o) == 12
        k = int(np.argmax(o != want)) if np.any(o != want) else 12
        assert k == 12 or margin[k] < 1e-3, (o, want, margin)


def test_device_decode_loop_equals_host_fed_steps(lib):
    cfg = RP.make_config(vocab=64, width=64)
    m, _ = make(lib, cfg, "float32", seed=43, n_slots=3, gain=2.0)
    p0, p1 = toks(90, 11, 64), toks(91, 30, 64)
    nxt = m.step_greedy([(0, p0), (1, p1)])
    dev = m.decode([0, 1], 9)
    m.set_option("graph", 0)
    m.reset(0), m.reset(1)
    assert np.array_equal(nxt, m.step_greedy([(0, p0), (1, p1)]))
    assert np.array_equal(dev, m.decode([0, 1], 9))
    m.reset(2)
    cur, host = int(m.step_greedy([(2, p1)])[0]), []
    for _ in range(9):
        cur = int(m.step_greedy([(2, [cur])])[0])
        host.append(cur)
    assert host == dev[1].tolist()
    assert m.position(1) == 30 + 9


def test_missing_and_misshapen_tensors_are_named(lib):
    cfg = RP.make_config(vocab=64, width=64)
    d = RP.describe(cfg)
    t = RP.synth_tensors(d, 0)
    t.pop("l1.mix.sink")
    with pytest.raises(lib.SeqError, match="l1.mix.sink"):
        lib.SeqModel(d, lib.F32, 1, 16).load(t)
    t = RP.synth_tensors(d, 0)
    t["l3.mix.k"] = t["l1.mix.k"]                      # a layer that reads another layer's cache has no keys of its own
    with pytest.raises(lib.SeqError, match="l3.mix.k"):
        lib.SeqModel(d, lib.F32, 1, 16).load(t)


def test_command_line_generation_and_trace_replay(lib, tmp_path):
    """bin/generate and bin/trace_run on a checkpoint folder written by the family's own writer."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cfg = RP.make_config(vocab=64, width=64)
    t = RP.synth_tensors(RP.describe(cfg), 71, gain=2.0)
    RP.write_checkpoint(tmp_path / "m", cfg, t)
    W = {k: R.bf16_to_float(v) for k, v in t.items()}
    p = toks(130, 37, 64)
    out = subprocess.run([sys.executable, str(root / "bin" / "generate"), "--model", str(tmp_path / "m"), "--dtype", "float32", "--prompt",
                          ",".join(map(str, p)), "--max-new", "6", "--chunk", "8"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    got = np.array([int(x) for x in out.stdout.strip().splitlines()[-1].split(",")])
    want, margin = oracle_greedy(cfg, W, p, 6)
    k = int(np.argmax(got != want)) if np.any(got != want) else 6
    assert k == 6 or margin[k] < 1e-3
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": p[:29].tolist(), "want": [28, 2]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": p[29:].tolist(), "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [9], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": p[:3].tolist(), "want": [2]}], "end": ["b"]}]
    tr = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "bfloat16", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                        input="\n".join(json.dumps(x) for x in steps) + "\n", capture_output=True, text=True, timeout=300)
    assert tr.returncode == 0, tr.stderr[-2000:]
    assert [l for l in tr.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    lg = R.forward(cfg, W, np.append(p, 9))[0]
    assert rel(np.fromfile(tmp_path / "o" / "0.f32", "<f4").reshape(2, 64), lg[[28, 2]]) < TOL["bfloat16"]      # in the order asked for
    assert not (tmp_path / "o" / "1.f32").exists()
    assert rel(np.fromfile(tmp_path / "o" / "2.f32", "<f4").reshape(1, 64), lg[37:38]) < TOL["bfloat16"]
    assert rel(np.fromfile(tmp_path / "o" / "3.f32", "<f4").reshape(1, 64), lg[2:3]) < TOL["bfloat16"]
