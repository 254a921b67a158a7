"""Plain, slow restatement of the Robopel equations in numpy float64: one function per mechanism, whole sequences only.

Nothing here is shared with the product path: the functions read the config dictionary themselves, keep no cache and no state --
every call recomputes a sequence from its first token -- so that stepwise, portion-wise and batched runs of the library can be held
against them position by position.  Tensors are float arrays keyed by checkpoint name."""
from __future__ import annotations

import numpy as np


def bf16_to_float(bits) -> np.ndarray:
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def one_plus_norm(x, w, eps):
    """RMS norm whose stored weight sits around zero: unit_rms(x) * (1 + w)."""
    return unit_rms(x, eps) * (1.0 + w)


def logistic(z):
    return 1.0 / (1.0 + np.exp(-z))


# ------------------------------------------------------------------------------------------------ minGRU
def mingru_candidate(u):
    """u + 1/2 for u >= 0, logistic(u) below: continuous at 0, positive everywhere."""
    return np.where(u >= 0, u + 0.5, logistic(np.minimum(u, 0.0)))


def mingru(h, wz, bz, wx, bx, wg, wo):
    """S_t = (1 - z_t) S_(t-1) + z_t c_t element by element, S_(-1) = 0; z and c read only token t.  y_t = W_o (S_t * silu(W_g h_t))."""
    z = logistic(h @ wz.T + bz)
    c = mingru_candidate(h @ wx.T + bx)
    S, states = np.zeros(wz.shape[0]), []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        states.append(S)
    g = h @ wg.T
    return (np.stack(states) * g * logistic(g)) @ wo.T


# ------------------------------------------------------------------------------------------------ rotary positions
def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with `scaling` (factor, low, high, original) long wavelengths are slowed down by `factor`,
    short ones kept, and the band between original/high and original/low is blended linearly in original/wavelength."""
    f = base ** (-2.0 * np.arange(dims // 2) / dims)
    if not scaling:
        return f
    fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wl = 2.0 * np.pi / fi
        if wl < orig / hi:
            out[i] = fi
        elif wl > orig / lo:
            out[i] = fi / fac
        else:
            s = (orig / wl - lo) / (hi - lo)
            out[i] = (1.0 - s) * fi / fac + s * fi
    return out


def rotate_interleaved(x, positions, freqs):
    """Entries 2i and 2i+1 of the last axis turn by positions * freqs[i]; entries from 2 len(freqs) on pass.  x [T, heads, dim]."""
    out = np.array(x, dtype=np.float64)
    ang = np.asarray(positions, np.float64)[:, None] * freqs[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    n = 2 * len(freqs)
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ attention
def visible(i, window, pool):
    """(token positions, pooled block numbers) that query position i sees.  window None: every earlier token."""
    if not window:
        return list(range(i + 1)), []
    toks = [j for j in range(i + 1) if i - j < window]
    blocks = [b for b in range((i + 1) // pool + 1) if b * pool + pool - 1 <= i - window] if pool else []
    return toks, blocks


def keys_and_values(h, wk, wv, k_norm, kv_heads, dim, vdim, freqs, eps):
    """What a layer's cache holds: keys after the per-head norm and rotation, values as projected."""
    T = h.shape[0]
    k = (h @ wk.T).reshape(T, kv_heads, dim)
    if k_norm is not None:
        k = unit_rms(k, eps) * k_norm
    if freqs is not None:
        k = rotate_interleaved(k, np.arange(T), freqs)
    return k, (h @ wv.T).reshape(T, kv_heads, vdim)


def softmax_attention(h, wq, q_norm, k, v, sink, wg, wo, heads, dim, vdim, scale, softcap, window, pool, freqs, eps, return_weights=False):
    """Queries of this layer over given keys/values [T, kv_heads, .]: windowed tokens plus the mean key/value of every pooled block
    that lies wholly before the window, one softmax whose denominator also holds exp(sink[head]); sigmoid output gate."""
    T, kv_heads = h.shape[0], k.shape[1]
    q = (h @ wq.T).reshape(T, heads, dim)
    if q_norm is not None:
        q = unit_rms(q, eps) * q_norm
    if freqs is not None:
        q = rotate_interleaved(q, np.arange(T), freqs)
    per = heads // kv_heads
    out = np.zeros((T, heads, vdim))
    book = []
    for i in range(T):
        toks, blocks = visible(i, window, pool)
        for hd in range(heads):
            g = hd // per
            kk = [k[b * pool:(b + 1) * pool, g].mean(0) for b in blocks] + [k[j, g] for j in toks]
            vv = [v[b * pool:(b + 1) * pool, g].mean(0) for b in blocks] + [v[j, g] for j in toks]
            s = np.asarray(kk) @ q[i, hd] * scale
            if softcap:
                s = softcap * np.tanh(s / softcap)
            m = max(s.max(), sink[hd]) if sink is not None else s.max()
            e = np.exp(s - m)
            den = e.sum() + (np.exp(sink[hd] - m) if sink is not None else 0.0)
            w = e / den
            out[i, hd] = w @ np.asarray(vv)
            if return_weights:
                book.append((i, hd, blocks, toks, w))
    y = out.reshape(T, heads * vdim)
    if wg is not None:
        y = y * logistic(h @ wg.T)
    y = y @ wo.T
    return (y, book) if return_weights else y


# ------------------------------------------------------------------------------------------------ feed-forward
def polynorm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e with N = unit_rms over a token's vector; powers element by element."""
    a, b, c, e = (float(x) for x in coef)
    return a * unit_rms(z, eps) + b * unit_rms(z ** 2, eps) + c * unit_rms(z ** 3, eps) + e


def dense_ff(h, w_up, w_down, coef, eps):
    return polynorm(h @ w_up.T, coef, eps) @ w_down.T


def route(h, w_router, correction, top):
    """(chosen outputs [T, top], their weights [T, top]): softmax over all router outputs; the choice adds `correction`, the weight does not."""
    z = h @ w_router.T
    s = np.exp(z - z.max(-1, keepdims=True))
    s = s / s.sum(-1, keepdims=True)
    pick = np.argsort(-(s + correction), axis=-1, kind="stable")[:, :top]
    return pick, np.take_along_axis(s, pick, -1)


def moe_ff(h, w_router, correction, ups, downs, top):
    """Router outputs 0 .. len(ups)-1 are experts down(relu(up h)^2); the outputs after them return h itself."""
    pick, w = route(h, w_router, correction, top)
    y = np.zeros((h.shape[0], downs[0].shape[0] if downs else h.shape[1]))
    for t in range(h.shape[0]):
        for e, we in zip(pick[t], w[t]):
            y[t] += we * (h[t] if e >= len(ups) else downs[e] @ np.maximum(ups[e] @ h[t], 0.0) ** 2)
    return y


# ------------------------------------------------------------------------------------------------ the model
def layer_freqs(m):
    rot = m.get("rot")
    return rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot else None


def forward(cfg, W, tokens):
    """logits [T, vocab] and the stream after every layer [layers, T, width] of one whole sequence."""
    eps = cfg["norm"]["eps"]
    tokens = np.asarray(tokens)
    x = W["embed"][tokens] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    trace, kv = [], {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", L["mixer"]
        if L["type"] == "mingru":
            y = mingru(x, W[p + "z"], W[p + "z.b"], W[p + "x"], W[p + "x.b"], W[p + "g"], W[p + "o"])
        elif L["type"] == "attention":
            fr = layer_freqs(m)
            src = m.get("kv_from")
            if src is None:
                kv[i] = keys_and_values(x, W[p + "k"], W[p + "v"], W.get(p + "k.norm"), m["kv_heads"], m["dim"], m["vdim"], fr, eps)
                src = i
            k, v = kv[src]
            mask = m.get("mask") or {}
            y = softmax_attention(x, W[p + "q"], W.get(p + "q.norm"), k, v, W.get(p + "sink"), W.get(p + "g"), W[p + "o"], m["heads"], m["dim"], m["vdim"],
                                  m["scale"], m.get("softcap"), mask.get("size"), mask.get("pool"), fr, eps)
        else:
            raise ValueError(L["type"])
        x = x + one_plus_norm(y, W[f"l{i}.norm1"], eps)
        mlp = L.get("mlp")
        if mlp:
            q = f"l{i}.mlp."
            if mlp["kind"] == "dense":
                y = dense_ff(x, W[q + "up"], W[q + "down"], W[q + "act"], eps)
            else:
                n = mlp["router"]["experts"]
                y = moe_ff(x, W[q + "router"], W[q + "correction"], [W[f"{q}e{e}.up"] for e in range(n)], [W[f"{q}e{e}.down"] for e in range(n)], mlp["router"]["top"])
            x = x + one_plus_norm(y, W[f"l{i}.norm2"], eps)
        trace.append(x)
    return one_plus_norm(x, W["final.norm"], eps) @ W["head"].T, np.stack(trace)
