"""Layer-list sequence models (libgten_b200_seq.so) against the plain numpy restatement in oracle/seq_ref.py.

Every test makes its own small configuration and random weights.  float32 mode is held to rounding (1e-4 of the logits'
spread); bfloat16 mode to a loose bound that a wrong key, position or state still breaks by orders of magnitude."""
import json

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle import seq_ref as R  # noqa: E402


@pytest.fixture(scope="module")
def lib():
    from tinyllama_cpp_b200 import build, seq
    build.build(target="seq")
    seq.init(0)
    return seq


def make(lib, cfg, mode="float32", seed=0, n_slots=3, max_ctx=512, max_rows=0, tweak=None, **synth):
    from tinyllama_cpp_b200 import reninex
    desc = reninex.describe(cfg)
    t = reninex.synth_tensors(desc, seed, **synth)
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


def toks(seed, n, vocab):
    return np.random.default_rng(1000 + seed).integers(0, vocab, n).astype(np.int32)


def small(**kw):
    from tinyllama_cpp_b200 import reninex
    return reninex.make_config(**kw)


# ------------------------------------------------------------------ each mechanism alone, against its own oracle function
@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", ["left_only", "right_only", "no_mlp", "no_conv", "no_bigram", "loop", "all"])
def test_mechanisms_one_at_a_time(lib, mode, variant):
    kw = dict(vocab=101, width=72, n_layers=3, ff=88, taps=3, l_heads=6, l_kv=2, l_dim=12, l_vdim=20, r_heads=3, r_dim=24, r_vdim=16,
              rot_dims=12, bigram=(37, 5, 11))
    if variant == "left_only":
        kw.update(right_scale=0.0, left_scale=1.0)
    if variant == "right_only":
        kw.update(left_scale=0.0, right_scale=1.0)
    if variant == "no_mlp":
        kw.update(no_mlp=(0, 1, 2))
    if variant == "no_conv":
        kw.update(taps=0)
    if variant == "no_bigram":
        kw.update(bigram=None)
    if variant in ("loop", "all"):
        kw.update(loop=(1, 3, 2))
    cfg = small(**kw)
    m, W = make(lib, cfg, mode, seed=3)
    m.set_option("capture", 1)
    t = toks(1, 41, cfg["vocab"])
    got = m.step([(0, t)], range(len(t)))
    want, trace = R.forward(cfg, W, t)
    assert m.n_runs == trace.shape[0]
    for u in range(m.n_runs):            # the stream after every layer run, first and last row
        for r in (0, len(t) - 1):
            assert rel(m.read_capture(u, r)[None], trace[u, r][None]) < TOL[mode] * (4 if mode == "bfloat16" else 1), (u, r)
    assert rel(got, want) < TOL[mode]


def test_sigmoid_attention_function_matches_direct_sum():
    """The oracle's own attention against a direct double loop (guards the oracle)."""
    rng = np.random.default_rng(0)
    T, W_, H, G, d, dv = 9, 10, 4, 2, 6, 5
    h = rng.standard_normal((T, W_))
    wq, wk, wv = rng.standard_normal((H * d, W_)), rng.standard_normal((G * d, W_)), rng.standard_normal((G * dv, W_))
    wo, pb = rng.standard_normal((W_, H * dv)), rng.standard_normal(H)
    y, w = R.sigmoid_attention(h, wq, wk, wv, wo, pb, H, G, d, dv, 0.3, 1e-5, return_weights=True)
    assert np.all(w[:, np.triu_indices(T, 1)[0], np.triu_indices(T, 1)[1]] == 0)
    assert np.all((w[:, np.tril_indices(T)[0], np.tril_indices(T)[1]] > 0))
    assert not np.allclose(w.sum(-1), 1.0)          # weights are not normalised over keys


# ------------------------------------------------------------------ prefill = decode = portions
@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
def test_prefill_against_token_by_token(lib, mode):
    cfg = small(vocab=90, width=64, n_layers=2, loop=(0, 2, 2), taps=4)
    m, W = make(lib, cfg, mode, seed=5)
    t = toks(2, 60, cfg["vocab"])
    whole = m.step([(0, t)], range(len(t)))
    one = np.concatenate([m.step([(1, t[i:i + 1])], [0]) for i in range(len(t))])
    want, _ = R.forward(cfg, W, t)
    assert rel(whole, want) < TOL[mode] and rel(one, want) < TOL[mode]
    assert rel(one, whole) < TOL[mode]


@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 50, 2, 7, 1, 1, 30], [33, 1, 64, 2], [97, 3], [1] * 5 + [95]])
def test_portions_of_any_size(lib, sizes):
    cfg = small(vocab=77, width=48, n_layers=2, taps=5, l_dim=8, l_vdim=24, r_dim=8, r_vdim=8, rot_dims=4, loop=(1, 2, 3))
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
    cfg = small(vocab=64, width=64, n_layers=2)
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
    cfg = small(vocab=80, width=64, n_layers=2, loop=(0, 1, 2))
    m, W = make(lib, cfg, mode, seed=11, n_slots=4)
    seqs = [toks(10 + i, n, 80) for i, n in enumerate((37, 5, 64, 1))]
    # step 1: a portion of every request at once; step 2: the rest of two of them and single rows of the others
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
    cfg = small(vocab=70, width=64, n_layers=2, loop=(0, 2, 2))
    m, W = make(lib, cfg, "float32", seed=13, n_slots=2)
    sm = SlotManager(m)
    a, b, c = toks(20, 50, 70), toks(21, 9, 70), toks(22, 31, 70)
    sa = sm.acquire("a")
    m.step([(sa, a)])
    sb = sm.acquire("b")
    m.step([(sb, b[:4])])
    sm.release("a")
    sc = sm.acquire("c")                 # takes a's slot: every trace of a (cache, state, history, previous token) must be gone
    assert sc == sa
    got_c = m.step([(sc, c), (sb, b[4:])], range(len(c) + len(b) - 4))
    assert rel(got_c[: len(c)], R.forward(cfg, W, c)[0]) < TOL["float32"]
    assert rel(got_c[len(c):], R.forward(cfg, W, b)[0][4:]) < TOL["float32"]
    with pytest.raises(RuntimeError):
        sm.acquire("d")


# ------------------------------------------------------------------ far keys, tile borders, first tokens
def test_far_key_dominates_and_is_found(lib):
    """Bias far below zero and a large score scale: a handful of keys carry each query's attention.  The oracle tells which key
    dominates the last query of some head; sequences are searched until that key lies in the first tokens, hundreds of keys back."""
    from tinyllama_cpp_b200 import reninex
    cfg = small(vocab=60, width=64, n_layers=1, taps=2, l_heads=2, l_kv=1, l_dim=16, l_vdim=16, right_scale=0.05, left_scale=1.0, no_mlp=(0,))
    cfg["layers"][0]["mixer"]["left"]["scale"] = 2.5

    def tweak(t):
        from tinyllama_cpp_b200 import safetensors_io as st
        t["l0.mix.left.pb"] = st.f32_to_bf16_bits(np.full(2, -9.0, np.float32))
    m, W = make(lib, cfg, "float32", seed=17, max_ctx=400, tweak=tweak)
    n, found = 300, None
    for s in range(40):
        t = toks(100 + s, n, 60)
        h = R.gain_norm(W["embed"][t] + W["bigram"][R.bigram_rows(t, 61, 7, 3)], W["l0.norm1"], cfg["norm"]["eps"])
        hm = h + R.causal_conv(h, W["l0.canon1"])
        _, w = R.sigmoid_attention(hm, W["l0.mix.left.q"], W["l0.mix.left.k"], W["l0.mix.left.v"], W["l0.mix.left.o"], W["l0.mix.left.pb"], 2, 1, 16, 16, 2.5, cfg["norm"]["eps"], True)
        best = w[:, -1].argmax(-1)
        if best.min() < 8 and w[:, -1].max() > 20 * np.median(w[:, -1]):
            found = t
            break
    assert found is not None
    want, _ = R.forward(cfg, W, found)
    whole = m.step([(0, found)], [n - 1])
    assert rel(whole, want[-1:]) < TOL["float32"]
    m.step([(1, found[:-1])])
    dec = m.step([(1, found[-1:])], [0])             # the same query decoded alone
    assert rel(dec, want[-1:]) < TOL["float32"]
    # and the check has teeth: without the far keys the answer is far off
    near, _ = R.forward(cfg, W, found[8:])
    assert rel(near[-1:], want[-1:]) > 50 * TOL["float32"]


@pytest.mark.parametrize("n", [127, 128, 129, 257])
def test_key_tile_borders_in_prompt_and_decode(lib, n):
    cfg = small(vocab=64, width=64, n_layers=1, l_heads=2, l_kv=2, r_heads=1, r_dim=8, r_vdim=8, rot_dims=8)
    m, W = make(lib, cfg, "float32", seed=19)
    t = toks(30, n + 2, 64)
    want, _ = R.forward(cfg, W, t)
    got = m.step([(0, t[:n])], [n - 2, n - 1])
    got = np.concatenate([got, m.step([(0, t[n:n + 1])], [0]), m.step([(0, t[n + 1:])], [0])])
    assert rel(got, want[n - 2:]) < TOL["float32"]


def test_first_tokens(lib):
    """Position 0 uses the bigram table's last row and sees zeros in the convolution; rows 1..taps see part of them."""
    cfg = small(vocab=50, width=64, n_layers=2, taps=6, bigram=(13, 3, 2))
    m, W = make(lib, cfg, "float32", seed=23)
    t = toks(40, 9, 50)
    want, _ = R.forward(cfg, W, t)
    assert rel(m.step([(0, t)], range(9)), want) < TOL["float32"]
    got = np.concatenate([m.step([(1, t[i:i + 1])], [0]) for i in range(9)])
    assert rel(got, want) < TOL["float32"]
    # a sequence that starts with the same token twice: the first-token row is not the hashed row of (token, token)
    tt = np.array([7, 7, 7], np.int32)
    assert rel(m.step([(2, tt)], range(3)), R.forward(cfg, W, tt)[0]) < TOL["float32"]


# ------------------------------------------------------------------ long decoding, other sizes
@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
def test_long_decoding(lib, mode):
    cfg = small(vocab=64, width=64, n_layers=2, r_heads=3, loop=(1, 2, 2))
    m, W = make(lib, cfg, mode, seed=29)
    t = toks(50, 260, 64)
    want, _ = R.forward(cfg, W, t)
    m.step([(0, t[:10])])
    got = np.concatenate([m.step([(0, t[i:i + 1])], [0]) for i in range(10, 260)])
    assert rel(got, want[10:]) < TOL[mode]
    assert rel(got[-5:], want[-5:]) < TOL[mode]


@pytest.mark.parametrize("kw", [
    dict(vocab=33, width=40, ff=24, l_heads=1, l_kv=1, l_dim=40, l_vdim=8, r_heads=1, r_dim=4, r_vdim=40, rot_dims=2, taps=1),
    dict(vocab=130, width=136, ff=200, l_heads=8, l_kv=8, l_dim=8, l_vdim=24, r_heads=5, r_dim=32, r_vdim=8, rot_dims=32, taps=2, loop=(0, 1, 1)),
    dict(vocab=64, width=64, ff=64, l_heads=4, l_kv=1, l_dim=32, l_vdim=16, r_heads=2, r_dim=16, r_vdim=72, rot_dims=0, taps=7, n_layers=4, loop=(1, 4, 2), no_mlp=(2,)),
    dict(vocab=64, width=64, ff=32, l_heads=2, l_kv=1, l_dim=136, l_vdim=200, r_heads=1, r_dim=520, r_vdim=72, rot_dims=40, n_layers=1),   # heads beyond the tiled kernels' sizes
])
def test_other_sizes(lib, kw):
    cfg = small(**kw)
    m, W = make(lib, cfg, "float32", seed=31)
    t = toks(60, 45, cfg["vocab"])
    want, _ = R.forward(cfg, W, t)
    got = np.concatenate([m.step([(0, t[:20])], range(20)), m.step([(0, t[20:22])], range(2)), m.step([(0, t[22:])], range(23))])
    assert rel(got, want) < TOL["float32"]


def test_tensor_core_products_match_simt(lib):
    """bfloat16 mode: the tcgen05 product against the SIMT product on the same operands (same rounding points)."""
    cfg = small(vocab=96, width=128, ff=192, n_layers=2, l_dim=32, l_vdim=32, r_dim=32, r_vdim=32, rot_dims=16)
    m, W = make(lib, cfg, "bfloat16", seed=37)
    t = toks(70, 200, 96)
    a = m.step([(0, t)], range(200))
    m.set_option("tensor", 0)
    b = m.step([(1, t)], range(200))
    assert rel(a, b) < 1e-2
    assert rel(a, R.forward(cfg, W, t)[0]) < TOL["bfloat16"]


@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
@pytest.mark.parametrize("kw", [
    dict(l_heads=4, l_kv=2, l_dim=16, l_vdim=16, r_heads=2, r_dim=16, r_vdim=32, rot_dims=8),
    dict(l_heads=2, l_kv=1, l_dim=48, l_vdim=40, r_heads=3, r_dim=24, r_vdim=72, rot_dims=24),          # padded head sizes, two value slices
    dict(l_heads=3, l_kv=3, l_dim=20, l_vdim=12, r_heads=1, r_dim=136, r_vdim=8, rot_dims=64),           # unaligned rows; 32-row chunks
    dict(l_heads=2, l_kv=2, l_dim=128, l_vdim=128, r_heads=2, r_dim=128, r_vdim=128, rot_dims=128, width=128),
])
def test_tiled_mixer_kernels_on_portions(lib, mode, kw):
    """Prompt portions run the tiled kernels (tensor-core sigmoid attention in bfloat16 mode, chunked retention): portions that
    start in the middle of a sequence, end inside a tile or chunk, and passes of several segments -- against the oracle and
    against the simple kernels (option fused_attn = 0)."""
    cfg = small(vocab=64, **{"width": 64, "n_layers": 2, "loop": (1, 2, 2), **kw})
    m, W = make(lib, cfg, mode, seed=61, n_slots=4, max_ctx=400)
    a, b = toks(110, 300, 64), toks(111, 170, 64)
    wa, wb = R.forward(cfg, W, a)[0], R.forward(cfg, W, b)[0]
    outs = {}
    for fused in (1, 0):
        m.set_option("fused_attn", fused)
        sa, sb = (0, 1) if fused else (2, 3)
        g1 = m.step([(sa, a[:70])], range(70))                                   # one tile + 6 rows
        g2 = m.step([(sa, a[70:199]), (sb, b[:33])], range(129 + 33))            # starts at 70, two segments
        g3 = m.step([(sb, b[33:170]), (sa, a[199:300])], range(137 + 101))
        ga = np.concatenate([g1, g2[:129], g3[137:]])
        gb = np.concatenate([g2[129:], g3[:137]])
        assert rel(ga, wa) < TOL[mode] and rel(gb, wb) < TOL[mode], fused
        outs[fused] = (ga, gb)
    assert rel(outs[1][0], outs[0][0]) < TOL[mode] and rel(outs[1][1], outs[0][1]) < TOL[mode]
    # decoding continues from the state the tiled kernels left
    nxt = m.step([(0, [5])], [0])
    assert rel(nxt, R.forward(cfg, W, np.append(a, 5))[0][-1:]) < TOL[mode]


@pytest.mark.parametrize("kw", [
    dict(vocab=101, width=72, ff=88, l_heads=6, l_kv=2, l_dim=12, l_vdim=20, r_heads=3, r_dim=24, r_vdim=16, rot_dims=12, taps=3),     # nothing a multiple of 32
    dict(vocab=33, width=40, ff=24, l_heads=1, l_kv=1, l_dim=40, l_vdim=8, r_heads=1, r_dim=4, r_vdim=40, rot_dims=2, taps=9, n_layers=1),  # fewer outputs than a tile, long filter
])
def test_tensor_core_path_with_awkward_sizes(lib, kw):
    """bfloat16 mode, portions of 64 rows and more (tcgen05 products, their row / column guards and unaligned epilogue stores)."""
    cfg = small(**kw)
    m, W = make(lib, cfg, "bfloat16", seed=67)
    t = toks(120, 150, cfg["vocab"])
    want, _ = R.forward(cfg, W, t)
    got = np.concatenate([m.step([(0, t[:70])], range(70)), m.step([(0, t[70:])], range(80))])
    assert rel(got, want) < TOL["bfloat16"]
    m.set_option("tensor", 0)
    simt = np.concatenate([m.step([(1, t[:70])], range(70)), m.step([(1, t[70:])], range(80))])
    assert rel(got, simt) < 2e-2


# ------------------------------------------------------------------ generation through the scheduler
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
    cfg = small(vocab=64, width=64, n_layers=2, loop=(0, 2, 2))
    m, W = make(lib, cfg, "float32", seed=41, n_slots=2, gain=2.0)
    prompts = [toks(80 + i, n, 64) for i, n in enumerate((19, 3, 40))]     # three requests, two slots: one waits
    outs = generate(m, prompts, 12, chunk=8, burst=5)
    for p, o in zip(prompts, outs):
        want, margin = oracle_greedy(cfg, W, p, 12)
        assert len(o) == 12
        k = int(np.argmax(o != want)) if np.any(o != want) else 12
        assert k == 12 or margin[k] < 1e-3, (o, want, margin)


def test_device_decode_loop_equals_host_fed_steps(lib):
    cfg = small(vocab=64, width=64, n_layers=2)
    m, _ = make(lib, cfg, "float32", seed=43, n_slots=3, gain=2.0)
    p0, p1 = toks(90, 11, 64), toks(91, 30, 64)
    nxt = m.step_greedy([(0, p0), (1, p1)])
    dev = m.decode([0, 1], 9)
    for graph in (0,):
        m.set_option("graph", graph)
        m.reset(0), m.reset(1)
        n2 = m.step_greedy([(0, p0), (1, p1)])
        assert np.array_equal(nxt, n2)
        assert np.array_equal(dev, m.decode([0, 1], 9))
    # host-fed: each sampled token goes back in as a one-token segment
    m.reset(2)
    cur, host = int(m.step_greedy([(2, p1)])[0]), []
    for _ in range(9):
        cur = int(m.step_greedy([(2, [cur])])[0])
        host.append(cur)
    assert host == dev[1].tolist()
    assert m.position(1) == 30 + 9


def test_eos_stops_a_slot(lib):
    cfg = small(vocab=64, width=64, n_layers=1)
    m, _ = make(lib, cfg, "float32", seed=47, n_slots=2, gain=2.0)
    p = toks(95, 8, 64)
    m.step_greedy([(0, p)])
    free = m.decode([0], 8)[0]
    eos = int(free[3])
    first = int(np.argmax(free == eos))
    m.reset(0)
    m.step_greedy([(0, p)])
    out = m.decode([0], 8, eos_id=eos)[0]
    assert np.array_equal(out[: first + 1], free[: first + 1]) and np.all(out[first:] == eos)
    assert m.position(0) == 8 + first + 1        # the token that produced the end-of-sequence id is the last one the slot took in


def test_topk_candidates(lib):
    cfg = small(vocab=64, width=64, n_layers=1)
    m, W = make(lib, cfg, "float32", seed=53)
    p = toks(96, 12, 64)
    m.step_greedy([(0, p)])
    v, ids = m.topk(0, 5)
    lg = m.last_logits(0)
    o = np.argsort(-lg, kind="stable")[:5]
    assert np.array_equal(ids, o) and np.allclose(v, lg[o])
    assert rel(lg[None], R.forward(cfg, W, p)[0][-1:]) < TOL["float32"]


def test_errors(lib):
    cfg = small(vocab=64, width=64, n_layers=1)
    m, _ = make(lib, cfg, "float32", seed=59, n_slots=1, max_ctx=16)
    with pytest.raises(lib.SeqError):
        m.step([(0, list(range(17)))])           # past the slot's capacity
    with pytest.raises(lib.SeqError):
        m.step([(0, [64])])                      # token outside the vocabulary
    with pytest.raises(lib.SeqError):
        m.step([(1, [1])])                       # no such slot
    from tinyllama_cpp_b200 import reninex
    d = reninex.describe(cfg)
    t = reninex.synth_tensors(d, 0)
    t.pop("l0.mix.right.g")
    with pytest.raises(lib.SeqError, match="right.g"):
        lib.SeqModel(d, lib.F32, 1, 16).load(t)


def test_command_line_generation_and_trace_replay(lib, tmp_path):
    """bin/generate and bin/trace_run on a checkpoint folder written by the family's own writer."""
    import subprocess
    import sys
    from pathlib import Path
    from tinyllama_cpp_b200 import reninex
    root = Path(__file__).resolve().parent.parent
    cfg = small(vocab=64, width=64, n_layers=2, loop=(0, 1, 2))
    desc = reninex.describe(cfg)
    t = reninex.synth_tensors(desc, 71, gain=2.0)
    reninex.write_checkpoint(tmp_path / "m", cfg, t)
    W = {k: R.bf16_to_float(v) for k, v in t.items()}
    p = toks(130, 17, 64)
    out = subprocess.run([sys.executable, str(root / "bin" / "generate"), "--model", str(tmp_path / "m"), "--dtype", "float32", "--prompt",
                          ",".join(map(str, p)), "--max-new", "6", "--chunk", "8"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    got = np.array([int(x) for x in out.stdout.strip().splitlines()[-1].split(",")])
    want, margin = oracle_greedy(cfg, W, p, 6)
    k = int(np.argmax(got != want)) if np.any(got != want) else 6
    assert k == 6 or margin[k] < 1e-3
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": p[:9].tolist(), "want": [8, 2]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": p[9:].tolist(), "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": p[:3].tolist(), "want": [2]}], "end": ["a", "b"]}]
    # six more requests that are never ended, on four slots: the one idle longest gives way
    steps += [{"step": 3 + i, "entries": [{"id": f"c{i}", "tokens": p[:4 + i].tolist(), "want": [3 + i]}], "end": []} for i in range(6)]
    tr = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                        input="\n".join(json.dumps(x) for x in steps) + "\n", capture_output=True, text=True, timeout=300)
    assert tr.returncode == 0, tr.stderr[-2000:]
    assert [l for l in tr.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(9)]
    assert rel(np.fromfile(tmp_path / "o" / "8.f32", "<f4").reshape(1, 64), R.forward(cfg, W, p[:9])[0][8:9]) < TOL["float32"]
    lg = R.forward(cfg, W, p)[0]
    a0 = np.fromfile(tmp_path / "o" / "0.f32", "<f4").reshape(2, 64)
    assert rel(a0, lg[[8, 2]]) < TOL["float32"]                      # in the order asked for
    assert not (tmp_path / "o" / "1.f32").exists()
    assert rel(np.fromfile(tmp_path / "o" / "2.f32", "<f4").reshape(1, 64), lg[2:3]) < TOL["float32"]
