"""Plain Keralix forward: whole sequences, no cache, one function per mechanism.

Written from the design's equations alone; it shares no code with the engine (own config
reading, plain numpy arithmetic, a loop per token where the engine has kernels).  All
arithmetic runs in the numpy dtype given (float64 by default: a ground truth for judging
rounding).

The design in this file's notation (one sequence of T tokens, width W, n streams X[j]):

  e = embed[tokens] * embedding.scale;  X[j] = e for every stream j
  sublayer f with hyper-connection tensors (a: in [n], b: out [n], M: mix [n, n], indexed [from, to]):
          u = sum_j a[j] X[j];  y = f(rms(u) * norm);  X'[t] = sum_j M[j, t] X[j] + b[t] y   (all t from the old X)
  layer:  the mixer as sublayer 1 (norm1, hc1), the feed-forward as sublayer 2 (norm2, hc2; absent: skipped)
  mixer "attention": q = W_q h + b_q, k = W_k h + b_k; a causal convolution over time per channel of q and of k;
          v = k after the convolution; half-split rotation of the first rot.dims dimensions of q and k;
          score = cap * tanh(scale * q.k / cap); keys i - size < j <= i; softmax; W_o
  mixer "latent_attention": cq = rms(W_dq h) * dq.norm, q = W_uq cq; c = rms(W_dkv h) * dkv.norm;
          k = W_uk c, v = W_uv c per head; score = scale * q.k; causal; softmax whose denominator also counts
          exp(sink_h); heads * sigmoid(W_g h); W_o
  mixer "channel_delta": q, k, v projections, each a causal convolution then silu; q and k made unit vectors per
          head (q also times dim^-1/2); beta = sigmoid(W_b h); g = exp(-exp(A_log) * softplus(W_a2 W_a1 h + dt_bias));
          per head S = g * S (rows); u = beta (v - S^T k); S += k u^T; o = S^T q; o / rms(o) * norm * sigmoid(W_g2 W_g1 h); W_o
  ff:     W_down (silu(W_gate h) * (W_up h))
  out:    logits = embed (rms(sum_j X[j]) * final.norm)
"""
from __future__ import annotations

import numpy as np


# ----------------------------------------------------------------------------
# small pieces
# ----------------------------------------------------------------------------

def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.where(z > 30.0, z, np.log1p(np.exp(np.minimum(z, 30.0))))


def causal_conv(u, taps):
    """u [T, C], taps [C, n]: y_t = sum_j taps[:, j] * u_(t - n + 1 + j), zeros before the start (the last column
    weighs the current token)."""
    T, n = u.shape[0], taps.shape[1]
    y = np.zeros_like(u)
    for t in range(T):
        for j in range(n):
            s = t - n + 1 + j
            if s >= 0:
                y[t] += taps[:, j] * u[s]
    return y


def rotate_half_split(x, positions, base, dims):
    """x [T, heads, dim]: dimension i pairs with i + dims/2 for i < dims/2; the rest pass unchanged."""
    half = dims // 2
    out = x.copy()
    if half == 0:
        return out
    f = np.array([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    a = np.asarray(positions, dtype=x.dtype)[:, None] * f[None, :]          # [T, half]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ----------------------------------------------------------------------------
# mixers
# ----------------------------------------------------------------------------

def window_attention(h, W, p, m):
    """Grouped-query attention with convolved queries and keys, keys as values, capped scores and a sliding window."""
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = h @ W[p + "q"].T + W[p + "q.b"]
    k = h @ W[p + "k"].T + W[p + "k.b"]
    q = causal_conv(q, W[p + "q.conv"])
    k = causal_conv(k, W[p + "k.conv"])
    v = k.reshape(T, G, D)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    pos = np.arange(T)
    qh = rotate_half_split(q.reshape(T, H, D), pos, rot["base"], int(rot["dims"]))
    kh = rotate_half_split(k.reshape(T, G, D), pos, rot["base"], int(rot["dims"]))
    scale, cap = float(m["scale"]), m.get("softcap")
    size = int(m["mask"]["size"]) if m.get("mask") else None
    out = np.zeros((T, H, D), dtype=h.dtype)
    per = H // G
    for i in range(T):
        lo = 0 if size is None else max(0, i - size + 1)
        for a in range(H):
            g = a // per
            s = (kh[lo:i + 1, g] @ qh[i, a]) * scale
            if cap:
                s = cap * np.tanh(s / cap)
            w = np.exp(s - s.max())
            w = w / w.sum()
            out[i, a] = w @ v[lo:i + 1, g]
    return out.reshape(T, H * D) @ W[p + "o"].T


def latent_attention(h, W, p, m, eps):
    """Attention whose keys and values are made from one small latent per token; a sink in the softmax; an output gate."""
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cq = unit_rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).reshape(T, H, D)
    c = unit_rms(h @ W[p + "dkv"].T, eps) * W[p + "dkv.norm"]
    k = (c @ W[p + "uk"].T).reshape(T, H, D)
    v = (c @ W[p + "uv"].T).reshape(T, H, V)
    sink = W[p + "sink"]
    scale = float(m["scale"])
    out = np.zeros((T, H, V), dtype=h.dtype)
    for i in range(T):
        for a in range(H):
            s = (k[:i + 1, a] @ q[i, a]) * scale
            top = max(s.max(), sink[a])
            w = np.exp(s - top)
            out[i, a] = (w @ v[:i + 1, a]) / (w.sum() + np.exp(sink[a] - top))
    gate = sigmoid(h @ W[p + "g"].T)
    return (out.reshape(T, H * V) * gate) @ W[p + "o"].T


def delta_rule(q, k, v, beta, g):
    """One head group at a time: q, k [T, heads, dim] (already per value head), v [T, heads, vdim], beta [T, heads],
    g [T, heads, dim].  Returns o [T, heads, vdim] and the final states."""
    T, H, D = q.shape
    V = v.shape[2]
    S = np.zeros((H, D, V), dtype=q.dtype)
    o = np.zeros((T, H, V), dtype=q.dtype)
    for t in range(T):
        for a in range(H):
            S[a] = g[t, a][:, None] * S[a]
            u = beta[t, a] * (v[t, a] - S[a].T @ k[t, a])
            S[a] = S[a] + np.outer(k[t, a], u)
            o[t, a] = S[a].T @ q[t, a]
    return o, S


def channel_delta(h, W, p, m, eps):
    """Gated delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, V)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    per = H // G
    q = np.repeat(q, per, axis=1)
    k = np.repeat(k, per, axis=1)
    beta = sigmoid(h @ W[p + "b"].T)
    dt = softplus((h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).reshape(T, H, D)
    g = np.exp(-np.exp(W[p + "A_log"])[None, :, None] * dt)
    o, _ = delta_rule(q, k, v, beta, g)
    o = unit_rms(o, eps) * W[p + "norm"]
    gate = sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T)
    return (o.reshape(T, H * V) * gate) @ W[p + "o"].T


def feed_forward(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


MIXERS = {"attention": lambda h, W, p, m, eps: window_attention(h, W, p, m), "latent_attention": latent_attention,
          "channel_delta": channel_delta}


# ----------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------

def hyper_sublayer(X, W, p, norm_w, eps, f):
    """X [n, T, W] -> new X.  Without hyper-connection tensors (n == 1 and none stored): the plain residual add."""
    if p + "in" not in W:
        return X + f(unit_rms(X[0], eps) * norm_w)[None]
    a, b, M = W[p + "in"], W[p + "out"], W[p + "mix"]
    u = np.tensordot(a, X, axes=(0, 0))
    y = f(unit_rms(u, eps) * norm_w)
    return np.tensordot(M.T, X, axes=(1, 0)) + b[:, None, None] * y[None]


def forward(cfg, W, tokens, dtype=np.float64, layer_sums=None):
    """cfg: the config.json dictionary; W: name -> array; tokens: one sequence.  Returns logits [T, vocab].
    layer_sums: a list that receives the sum of the streams after every layer."""
    W = {k: np.asarray(v, dtype=dtype) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    n = int(cfg.get("streams") or 1)
    e = W["embed"][np.asarray(tokens)] * dtype((cfg.get("embedding") or {}).get("scale", 1.0))
    X = np.stack([e] * n)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        mixer = MIXERS[L["type"]]
        X = hyper_sublayer(X, W, p + "hc1.", W[p + "norm1"], eps, lambda h: mixer(h, W, p + "mix.", L["mixer"], eps))
        if L.get("mlp") is not None:
            X = hyper_sublayer(X, W, p + "hc2.", W[p + "norm2"], eps, lambda h: feed_forward(h, W, p + "mlp."))
        if layer_sums is not None:
            layer_sums.append(X.sum(axis=0))
    x = unit_rms(X.sum(axis=0), eps) * W["final.norm"]
    return x @ W["embed"].T
