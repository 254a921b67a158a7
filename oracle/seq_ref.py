"""Plain, slow restatement of the Reninex equations in numpy float64: one function per mechanism, whole sequences only.

It shares nothing with the product path: it reads the config dictionary itself, has no cache and no state -- every call
recomputes a sequence from its first token -- so that stepwise, chunked and batched runs of the library can be held against it
position by position.  Tensors are given as float arrays (bfloat16 values are exactly representable)."""
from __future__ import annotations

import numpy as np


def bf16_to_float(bits) -> np.ndarray:
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def gain_norm(x, g, eps):
    """RMS norm whose weight is ONE number."""
    return unit_rms(x, eps) * float(np.asarray(g).reshape(-1)[0])


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def logistic(z):
    return 1.0 / (1.0 + np.exp(-z))


def causal_conv(h, w):
    """c_t = sum_j w[:, j] * h_(t - taps + 1 + j); rows before the sequence are zero.  h [T, C], w [C, taps]."""
    T, taps = h.shape[0], w.shape[1]
    out = np.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return np.asarray(rows)


def sigmoid_attention(h, wq, wk, wv, wo, pb, heads, kv_heads, dim, vdim, scale, eps, return_weights=False):
    """Causal attention without positions and without a softmax: weight(i, j) = logistic(scale * q_i.k_j + pb[head]), j <= i;
    q and k have unit RMS per head."""
    T = h.shape[0]
    q = unit_rms((h @ wq.T).reshape(T, heads, dim), eps)
    k = unit_rms((h @ wk.T).reshape(T, kv_heads, dim), eps)
    v = (h @ wv.T).reshape(T, kv_heads, vdim)
    out = np.zeros((T, heads, vdim))
    weights = np.zeros((heads, T, T))
    per_group = heads // kv_heads
    for hd in range(heads):
        g = hd // per_group
        for i in range(T):
            w = logistic(scale * (k[: i + 1, g] @ q[i, hd]) + pb[hd])
            weights[hd, i, : i + 1] = w
            out[i, hd] = w @ v[: i + 1, g]
    y = out.reshape(T, heads * vdim) @ wo.T
    return (y, weights) if return_weights else y


def rotate(x, positions, rot_dims, base):
    """Rotary positions on the first rot_dims entries of the last axis; entry i pairs with i + rot_dims/2."""
    if not rot_dims:
        return x
    half = rot_dims // 2
    freq = base ** (-2.0 * np.arange(half) / rot_dims)
    ang = np.asarray(positions, np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, w = x[..., :half], x[..., half:rot_dims]
    return np.concatenate([u * c - w * s, w * c + u * s, x[..., rot_dims:]], axis=-1)


def retention(h, wq, wk, wv, wg, wo, heads, dim, vdim, decay, rot_dims, rot_base, eps):
    """S_t = decay * S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head; k scaled by dim^-1/2 after rotation; o to unit RMS per head,
    times silu(W_g h), then the out projection."""
    T = h.shape[0]
    pos = np.arange(T)
    q = rotate((h @ wq.T).reshape(T, heads, dim), pos, rot_dims, rot_base)
    k = rotate((h @ wk.T).reshape(T, heads, dim), pos, rot_dims, rot_base) * dim ** -0.5
    v = (h @ wv.T).reshape(T, heads, vdim)
    o = np.zeros((T, heads, vdim))
    for hd in range(heads):
        S = np.zeros((dim, vdim))
        for t in range(T):
            S = decay[hd] * S + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    gate = h @ wg.T
    y = unit_rms(o, eps).reshape(T, heads * vdim) * (gate * logistic(gate))
    return y @ wo.T


def feed_forward(h, w_gate, w_up, w_down):
    return (gelu_tanh(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def block(x, cfg, W, i):
    """One parallel block: x + mixer(h + conv1(h)) + ff(h + conv2(h)), h = gain_norm(x)."""
    L, p, eps = cfg["layers"][i], f"l{i}.", cfg["norm"]["eps"]
    h = gain_norm(x, W[p + "norm1"], eps)
    taps = (cfg.get("canon") or {}).get("taps", 0)
    hm = h + causal_conv(h, W[p + "canon1"]) if taps else h
    m = L["mixer"]
    le, ri = m["left"], m["right"]
    a = sigmoid_attention(hm, W[p + "mix.left.q"], W[p + "mix.left.k"], W[p + "mix.left.v"], W[p + "mix.left.o"], W[p + "mix.left.pb"],
                          le["heads"], le["kv_heads"], le["dim"], le["vdim"], le["scale"], eps)
    rot = ri.get("rot") or {"dims": 0, "base": 1.0}
    r = retention(hm, W[p + "mix.right.q"], W[p + "mix.right.k"], W[p + "mix.right.v"], W[p + "mix.right.g"], W[p + "mix.right.o"],
                  ri["heads"], ri["dim"], ri["vdim"], ri["decay"], rot["dims"], rot["base"], eps)
    y = m["left_scale"] * a + m["right_scale"] * r
    if L.get("mlp"):
        hf = h + causal_conv(h, W[p + "canon2"]) if taps else h
        y = y + feed_forward(hf, W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"])
    return x + y


def forward(cfg, W, tokens):
    """logits [T, vocab] and the stream after every layer run [runs, T, width] of one whole sequence."""
    tokens = np.asarray(tokens)
    x = W["embed"][tokens]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + W["bigram"][bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])]
    x0, trace, n = x, [], len(cfg["layers"])
    lp = cfg.get("loop")
    if lp and lp["times"] > 0:
        order = [(i, None) for i in range(lp["start"])]
        order += [(i, t) for t in range(lp["times"]) for i in range(lp["start"], lp["stop"])]
        order += [(i, None) for i in range(lp["stop"], n)]
    else:
        order = [(i, None) for i in range(n)]
    for i, t in order:
        if t is not None and i == lp["start"]:
            x = np.concatenate([x, x0], axis=-1) @ W["loop.in"].T + W["loop.step"][t]
        x = block(x, cfg, W, i)
        trace.append(x)
    logits = gain_norm(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T
    return logits, np.stack(trace)
