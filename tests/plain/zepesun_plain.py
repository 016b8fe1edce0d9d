"""Plain Zepesun forward: whole sequences, no cache, one function per mechanism.

Written from the design's equations alone; it shares no code with the engine (own config
reading, plain numpy arithmetic, a loop per token where the engine has kernels).  All
arithmetic runs in the numpy dtype given (float64 by default: a ground truth for judging
rounding).

The design in this file's notation (one sequence of T tokens at positions 0..T-1, width W):

  x = embed[tokens] * embedding.scale + pos[positions]
  layer:  h = rms(x) * norm1;  x = x + mixer(h) + ff(h)        (ff absent: skipped)
  mixer "latent_attention": q = W_q h, per head [dim plain | rot_dim turned]; W_dkv h = [c_raw (kv_rank) | kr (rot_dim)];
          c = rms(c_raw) * dkv.norm; per head k = W_uk c, v = W_uv c; q's turned part and kr are rotated by position
          (pairs (i, i + n/2), angle p * base^(-2i/n)); score = scale * (q_plain . k + q_turned . kr); causal softmax;
          head outputs times sigmoid(W_g h)_head; W_o
  mixer "parallel": left_scale * left(h) + right_scale * right(h)
          left:  grouped-query attention with biases, no positions, score = scale * q.k, keys i - size < j <= i,
                 softmax; heads side by side times sigmoid(W_g h) element by element; W_o + b_o
          right: the matrix memory below
  mixer "mlstm": q = W_q h * dim^-1/2, k = W_k h, v = W_v h; per head a = cap * tanh((W_i h + b_i) / cap) and
          f = log sigmoid(cap * tanh((W_f h + b_f) / cap)); with m_0 = 0, S_0 = 0, n_0 = 0:
          m_t = max(f + m_(t-1), a);  S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(a - m_t) k v^T;  n_t the same with k alone;
          o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6);  rms(o) per head, times norm, times sigmoid(W_g h); W_o
  ff "dense": W_down (gelu_tanh(W_gate h + b) * (W_up h + b)) + b
  ff "moe":   s = softmax(W_router h); experts in groups.count equal groups of neighbours, a group's score its largest s,
          only the groups.keep best groups' experts may be chosen; the `top` largest s among them, weights s / (sum + 1e-20)
          * router.scale; expert: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit),
          W_down (g * sigmoid(1.702 g) * (u + 1)); plus the shared expert (same form) for every token
  out:    logits = head (rms(x) * final.norm)
"""
from __future__ import annotations

import numpy as np


# ----------------------------------------------------------------------------
# small pieces
# ----------------------------------------------------------------------------

def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def softmax_rows(s):
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def rotate_half_pairs(x, positions, base, n):
    """x [T, ..., D]: the first n dimensions turn, dimension i with i + n/2, by the angle p * base^(-2i/n)."""
    if not n:
        return x
    half = n // 2
    f = np.asarray(base, dtype=np.float64) ** (-2.0 * np.arange(half) / n)
    a = (np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]).astype(x.dtype)
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(a).reshape(shape), np.sin(a).reshape(shape)
    u, v = x[..., :half], x[..., half:n]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:n] = v * c + u * s
    return out


def masked_softmax_attention(q, k, v, scale, window=None):
    """q [T, H, D], k [T, H, D], v [T, H, V] (keys already spread over the query heads): position i sees j <= i, and with a
    window only i - j < window."""
    T = q.shape[0]
    out = np.zeros((T, q.shape[1], v.shape[2]), dtype=q.dtype)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        s = np.einsum("hd,jhd->hj", q[i], k[lo:i + 1]) * scale
        p = softmax_rows(s)
        out[i] = np.einsum("hj,jhv->hv", p, v[lo:i + 1])
    return out


# ----------------------------------------------------------------------------
# mixers
# ----------------------------------------------------------------------------

def latent_attention(h, W, p, m, eps, positions):
    T = h.shape[0]
    H, D, R, V, C = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    rot = m.get("rot") or {}
    q = (h @ W[p + "q"].T).reshape(T, H, D + R)
    down = h @ W[p + "dkv"].T
    c = unit_rms(down[:, :C], eps) * W[p + "dkv.norm"]
    kr = down[:, C:C + R]
    if R:
        qr = rotate_half_pairs(q[..., D:], positions, rot["base"], int(rot["dims"]))
        kr = rotate_half_pairs(kr, positions, rot["base"], int(rot["dims"]))
    else:
        qr = q[..., D:]
    k = (c @ W[p + "uk"].T).reshape(T, H, D)
    v = (c @ W[p + "uv"].T).reshape(T, H, V)
    qf = np.concatenate([q[..., :D], qr], axis=-1)
    kf = np.concatenate([k, np.repeat(kr[:, None, :], H, axis=1)], axis=-1)
    o = masked_softmax_attention(qf, kf, v, float(m["scale"]))
    gate = sigmoid(h @ W[p + "g"].T)                       # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * V) @ W[p + "o"].T


def window_attention(h, W, p, m):
    T = h.shape[0]
    H, D = int(m["heads"]), int(m["dim"])
    G, V = int(m.get("kv_heads", H)), int(m.get("vdim", D))
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, V)
    per = H // G
    k, v = np.repeat(k, per, axis=1), np.repeat(v, per, axis=1)        # query head j reads key head j // per
    window = int(m["mask"]["size"]) if m.get("mask") else None
    o = masked_softmax_attention(q, k, v, float(m["scale"]), window).reshape(T, H * V)
    o = o * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T + W[p + "o.b"]


def matrix_memory(q, k, v, a, f, state=None):
    """The recurrence alone.  q, k [T, H, D], v [T, H, V], a, f [T, H] (log input gate, log forget gate).
    Returns o [T, H, V] and the final (S, n, m)."""
    T, H, D = q.shape
    V = v.shape[2]
    if state is None:
        S, n, m = np.zeros((H, D, V), q.dtype), np.zeros((H, D), q.dtype), np.zeros((H,), q.dtype)
    else:
        S, n, m = (x.copy() for x in state)
    o = np.zeros((T, H, V), q.dtype)
    for t in range(T):
        m_new = np.maximum(f[t] + m, a[t])
        keep = np.exp(f[t] + m - m_new)
        put = np.exp(a[t] - m_new)
        S = keep[:, None, None] * S + put[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + put[:, None] * k[t]
        m = m_new
        num = np.einsum("hdv,hd->hv", S, q[t])
        den = np.maximum(np.abs(np.einsum("hd,hd->h", n, q[t])), np.exp(-m)) + 1e-6
        o[t] = num / den[:, None]
    return o, (S, n, m)


def mlstm(h, W, p, m, eps):
    T = h.shape[0]
    H, D, V, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (h @ W[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, V)
    a = cap * np.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)
    f = log_sigmoid(cap * np.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))
    o, _ = matrix_memory(q, k, v, a, f)
    o = unit_rms(o, eps).reshape(T, H * V) * W[p + "norm"]
    o = o * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps):
    left = window_attention(h, W, p + "left.", m["left"])
    right = mlstm(h, W, p + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ----------------------------------------------------------------------------
# feed-forwards
# ----------------------------------------------------------------------------

def dense_ff(h, W, p):
    g = h @ W[p + "gate"].T + W[p + "gate.b"]
    u = h @ W[p + "up"].T + W[p + "up.b"]
    return (gelu_tanh(g) * u) @ W[p + "down"].T + W[p + "down.b"]


def clamped_expert(h, W, p, limit):
    g = np.minimum(h @ W[p + "gate"].T, limit)
    u = np.clip(h @ W[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def route(z, top, groups, keep, scale, gaps=None):
    """z [T, E] router logits -> (ids [T, top], weights [T, top]).  gaps: a list that receives, per row, how far (in logits)
    the closest decision was from going the other way: the last kept group against the first one left out, the last chosen
    expert against the best candidate that was not chosen."""
    T, E = z.shape
    s = softmax_rows(z)
    allowed = np.ones_like(s, dtype=bool)
    gap = np.full(T, np.inf)
    if groups > 1 and keep < groups:
        per = E // groups
        gs = s.reshape(T, groups, per).max(axis=2)
        order = np.argsort(-gs, axis=1, kind="stable")
        ok = np.zeros((T, groups), dtype=bool)
        np.put_along_axis(ok, order[:, :keep], True, axis=1)
        allowed = np.repeat(ok, per, axis=1)
        zg = z.reshape(T, groups, per).max(axis=2)
        gap = np.take_along_axis(zg, order[:, keep - 1:keep], axis=1)[:, 0] - np.take_along_axis(zg, order[:, keep:keep + 1], axis=1)[:, 0]
    masked = np.where(allowed, s, -1.0)
    order = np.argsort(-masked, axis=1, kind="stable")
    ids = order[:, :top]
    if top < E:
        zm = np.where(allowed, z, -np.inf)
        nxt = np.take_along_axis(zm, order[:, top:top + 1], axis=1)[:, 0]
        gap = np.minimum(gap, np.take_along_axis(zm, order[:, top - 1:top], axis=1)[:, 0] - nxt)
    if gaps is not None:
        gaps.append(gap)
    w = np.take_along_axis(s, ids, axis=1)
    w = w / (w.sum(axis=1, keepdims=True) + 1e-20) * scale
    return ids, w


def moe_ff(h, W, p, mlp, gaps=None):
    T = h.shape[0]
    r = mlp["router"]
    groups = r.get("groups") or {}
    z = h @ W[p + "router"].T
    ids, w = route(z, int(r["top"]), int(groups.get("count", 1)), int(groups.get("keep", 1)), float(r.get("scale", 1.0)), gaps)
    limit = float(mlp["expert"]["limit"])
    out = np.zeros((T, W[p + "e0.down"].shape[0]), dtype=h.dtype)
    for t in range(T):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] += w[t, j].astype(h.dtype) * clamped_expert(h[t:t + 1], W, f"{p}e{e}.", limit)[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, W, p + "shared.", float(mlp["shared"]["limit"]))
    return out


# ----------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------

def layer_output(x, W, L, p, eps, positions, gaps=None):
    h = unit_rms(x, eps) * W[p + "norm1"]
    kind, m = L["type"], L["mixer"]
    if kind == "latent_attention":
        y = latent_attention(h, W, p + "mix.", m, eps, positions)
    elif kind == "parallel":
        y = parallel_mixer(h, W, p + "mix.", m, eps)
    elif kind == "mlstm":
        y = mlstm(h, W, p + "mix.", m, eps)
    else:
        raise ValueError(f"unknown layer type {kind!r}")
    mlp = L.get("mlp")
    if mlp is not None:
        y = y + (dense_ff(h, W, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, W, p + "mlp.", mlp, gaps))
    return x + y


def forward(cfg, W, tokens, dtype=np.float64, layer_outputs=None, gaps=None):
    """cfg: the config.json dictionary; W: name -> array; tokens: one sequence.  Returns logits [T, vocab].
    layer_outputs: a list that receives the stream after every layer; gaps: a list that receives every routed layer's
    per-row decision gaps (route)."""
    W = {k: np.asarray(v, dtype=dtype) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    tokens = np.asarray(tokens)
    positions = np.arange(len(tokens))
    x = W["embed"][tokens] * dtype((cfg.get("embedding") or {}).get("scale", 1.0)) + W["pos"][positions]
    for i, L in enumerate(cfg["layers"]):
        x = layer_output(x, W, L, f"l{i}.", eps, positions, gaps)
        if layer_outputs is not None:
            layer_outputs.append(x)
    x = unit_rms(x, eps) * W["final.norm"]
    return x @ W["head"].T
