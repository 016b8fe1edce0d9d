"""Made-up inputs for single Keralix mechanisms in which one far or edge element decides the output, with what the plain
implementation says about them.  Random weights and inputs would hide a lost far key, a sink that is left out or a window
that is one position off among hundreds of ordinary terms; here one score stands out by construction.  The builders run on
the CPU (tests/test_keralix_plain.py checks what they claim); the GPU tests feed the same inputs to the kernels."""
import numpy as np

from tests.plain import keralix_plain as P


def latent_rows_plain(m, eps, proj, W):
    """The plain latent attention fed with projections that pick the latents and the gate out of the row."""
    H, V, QR, R = m["heads"], m["vdim"], m["q_rank"], m["kv_rank"]
    eye = np.eye(proj.shape[1])
    Wp = dict(W, dq=eye[:QR], dkv=eye[QR:QR + R], g=eye[QR + R:], o=np.eye(H * V))
    return P.latent_attention(proj, Wp, "", m, eps)


def far_latent_case(far, seed, T=620, prompt=600, R=16, H=2):
    """One latent at position `far` whose key points along `direction`; every other latent is orthogonal to it.  A query
    along `direction` scores `top` = 12 on it and exactly 0 on all others, so that key outweighs the hundreds of others
    (e^12 against T) and an even head's output is its value; an odd head's sink equals `top`, so it takes exactly half of
    the weight (it counts once and is not scaled: the scale is 8 / R here).  A query along -direction finds nothing: all
    its scores are 0 or below, and the even heads' sink of 8 leaves the ordinary keys a small share.  Latent, query latent
    and head size are all R; H heads of value size 8.
    -> (m, W, proj rows [T, q latent | kv latent | gate], seekers, blind, v_far [heads, vdim], want [T, heads * vdim])"""
    rng = np.random.default_rng(seed)
    D, V, QR = R, 8, R
    m = {"heads": H, "dim": D, "vdim": V, "q_rank": QR, "kv_rank": R, "scale": 8.0 / R}
    W = {"uq": np.concatenate([np.eye(D, QR)] * H), "uk": np.concatenate([np.eye(D, R)] * H) * 1.5,
         "uv": rng.standard_normal((H * V, R)) / np.sqrt(R), "dq.norm": np.ones(QR), "dkv.norm": np.ones(R),
         "sink": np.array(([8.0, 12.0] * H)[:H])}
    direction = rng.standard_normal(R)
    direction /= np.sqrt(np.mean(direction ** 2))                       # rms 1: the norms leave it as it is
    proj = rng.standard_normal((T, QR + R + H * V))
    lat = proj[:, QR:QR + R]
    lat -= np.outer(lat @ direction, direction) / (direction @ direction)    # every ordinary latent is orthogonal to it
    proj[:, QR + R:] = 9.0                                              # gates open
    proj[far, QR:QR + R] = direction * 3.0                              # any length: the norm brings it to rms 1
    seekers = [t for t in (far + 1, 300, prompt - 1, prompt, T - 1) if t > far]
    blind = 301
    for t in seekers:
        proj[t, :QR] = direction * 0.3
    proj[blind, :QR] = -direction
    want = latent_rows_plain(m, 1e-5, proj, W)
    c_far = P.unit_rms(direction[None], 1e-5)[0]
    v_far = (W["uv"] @ c_far).reshape(H, V)
    return m, W, proj, seekers, blind, v_far, want


def window_rows_plain(m, rows, bias, taps_w):
    """The plain windowed attention fed with rows that already are the products [q | k] before biases."""
    nh, nkv, hd = m["heads"], m["kv_heads"], m["dim"]
    eye = np.eye(rows.shape[1])
    a = nh * hd
    W = {"q": eye[:a], "k": eye[a:], "q.b": bias[:a], "k.b": bias[a:], "q.conv": taps_w[:a], "k.conv": taps_w[a:], "o": np.eye(nh * hd)}
    return P.window_attention(rows, W, "", m)


def window_edge_case(window, hd, seed, T=260, marks=(0, 15, 16, 100, 127, 128, 200, 215, 216)):
    """Marked keys (three times a unit-rms `direction`) before, at and after page borders.  For each the query window - 1
    positions later (the last that sees it) and the next one (the first that does not) point along `direction` in head 0;
    the marked key then scores far above the ordinary ones, and since keys are values head 0 returns it whenever it is seen.
    -> (m, rows [T, q | k], bias, taps, direction, alone, want): `alone` are the marks with no other mark within reach of
    their two queries, where "seen" and "not seen" can be read off the output."""
    rng = np.random.default_rng(seed)
    nh, nkv = 2, 1
    m = {"heads": nh, "kv_heads": nkv, "dim": hd, "scale": 12.0 / hd, "softcap": 50.0, "mask": {"size": window}}
    C = (nh + nkv) * hd
    rows = rng.standard_normal((T, C))
    direction = rng.standard_normal(hd)
    direction /= np.sqrt(np.mean(direction ** 2))
    for p in marks:
        rows[p, nh * hd:] = direction * 3.0
    for p in marks:
        for t in (p + window - 1, p + window):
            if t < T:
                rows[t, :hd] = direction * 3.0
    taps_w, bias = np.ones((C, 1)), np.zeros(C)
    alone = [p for p in marks if p + window < T and not any(p < o <= p + window for o in marks)]
    return m, rows, bias, taps_w, direction, alone, window_rows_plain(m, rows, bias, taps_w)


def delta_inputs(rng, T, H, G, D, V, slow=False):
    q, k, v = rng.standard_normal((T, G * D)), rng.standard_normal((T, G * D)), rng.standard_normal((T, H * V))
    b = rng.standard_normal((T, H))
    a = rng.standard_normal((T, H * D)) * (0.2 if slow else 1.0) - (4.0 if slow else 0.0)
    return q, k, v, b, a


def delta_plain(q, k, v, b, a, A_log, dt_bias, H, G, D, V):
    """Unit norms, beta, decays and the recurrence of the plain implementation on rows that already are the convolved,
    activated q, k, v and the raw beta and decay projections.  -> (o [T, H, V], final states [H, D, V])"""
    T = len(q)
    qh, kh = q.reshape(T, G, D), k.reshape(T, G, D)
    qh = qh / np.sqrt(np.sum(qh * qh, axis=-1, keepdims=True) + 1e-6) * D ** -0.5
    kh = kh / np.sqrt(np.sum(kh * kh, axis=-1, keepdims=True) + 1e-6)
    qh, kh = np.repeat(qh, H // G, axis=1), np.repeat(kh, H // G, axis=1)
    g = np.exp(-np.exp(A_log)[None, :, None] * P.softplus(a + dt_bias).reshape(T, H, D))
    return P.delta_rule(qh, kh, v.reshape(T, H, V), P.sigmoid(b), g)


def far_delta_case(seed=3, T=420, prompt=400):
    """Decays near one and small step sizes for the ordinary tokens: the pair (k, v) that the first token writes whole
    (beta near one) is read back hundreds of tokens later by queries along k, shrunk only by what the decays and the other
    keys' small overwrites left.  -> (sizes (H, G, D, V), rows (q, k, v, b, a), A_log, dt_bias, seekers, want [T, H, V])"""
    rng = np.random.default_rng(seed)
    H, G, D, V = 2, 1, 64, 16
    q, k, v, b, a = delta_inputs(rng, T, H, G, D, V, slow=True)
    b -= 4.0
    mark = rng.standard_normal(D)
    k[0, :D] = mark * 4.0
    v[0] = 5.0
    b[0] = 9.0
    seekers = [1, 200, prompt - 1, prompt, T - 1]
    for t in seekers:
        q[t, :D] = mark * 4.0
    A_log, dt_bias = np.full(H, -2.0), np.zeros(H * D)
    want, _ = delta_plain(q, k, v, b, a, A_log, dt_bias, H, G, D, V)
    return (H, G, D, V), (q, k, v, b, a), A_log, dt_bias, seekers, want
