"""Made-up inputs for single Zepesun mechanisms in which one far or edge element decides the output, with what the plain
implementation says about them.  Random weights and inputs would hide a lost far key, a window that is one position off
or a state that was not carried among hundreds of ordinary terms; here one score stands out by construction.  The builders
run on the CPU (tests/test_zepesun_plain.py checks what they claim); the GPU tests feed the same inputs to the kernels."""
import numpy as np

from tests.plain import zepesun_plain as P


def latent_rows_plain(m, eps, proj, W, positions=None):
    """The plain latent attention fed with rows that already are the product [q | latent | key part | gate]."""
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    eye = np.eye(proj.shape[1])
    a, b = H * (D + R), H * (D + R) + C + R
    Wp = {"q": eye[:a], "dkv": eye[a:b], "g": eye[b:b + H], "dkv.norm": W["dkv.norm"], "uk": W["uk"], "uv": W["uv"], "o": np.eye(H * V)}
    return P.latent_attention(proj, Wp, "", m, eps, np.arange(len(proj)) if positions is None else positions)


def far_latent_case(far, seed, T=620, prompt=600, C=16, R=8, H=2, through="latent"):
    """One position `far` stands out for the queries that look for it, through the latent part of the score (its latent
    points along `direction`, every other latent is orthogonal to it) or through the rotated part (only it and the seeking
    queries carry a rotated part at all; the seekers' is turned back by their distance, so that after the rotation it lines
    up with the far key's).  Gates are open; every head returns the far position's value.
    -> (m, W, proj rows [T, q | latent | key part | gate], seekers, v_far [heads, vdim], want [T, heads * vdim])"""
    rng = np.random.default_rng(seed)
    D, V = C, 8
    m = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "kv_rank": C, "scale": 8.0 / C, "rot": {"base": 100.0, "dims": R}}
    W = {"uk": np.concatenate([np.eye(D, C)] * H) * 1.5, "uv": rng.standard_normal((H * V, C)) / np.sqrt(C), "dkv.norm": np.ones(C)}
    direction = rng.standard_normal(C)
    direction /= np.sqrt(np.mean(direction ** 2))
    a = H * (D + R)
    proj = rng.standard_normal((T, a + C + R + H))
    lat = proj[:, a:a + C]
    lat -= np.outer(lat @ direction, direction) / (direction @ direction)
    proj[:, a + C + R:] = 9.0                                    # gates open
    proj[:, a + C:a + C + R] = 0.0                               # no rotated key part ...
    q = proj[:, :a].reshape(T, H, D + R)
    q[:, :, D:] = 0.0                                            # ... and no rotated query part, but for the marked ones
    seekers = [t for t in (far + 1, 300, prompt - 1, prompt, T - 1) if t > far]
    if through == "latent":
        proj[far, a:a + C] = direction * 3.0
        for t in seekers:
            q[t, :, :D] = direction * 0.3 / 1.5 * 4.0
    else:
        key = rng.standard_normal(R)
        key /= np.sqrt(np.mean(key ** 2))
        proj[far, a + C:a + C + R] = key * 3.0
        for t in seekers:
            # the rotation is by position: a query part that equals the key part turned back by (t - far) meets it again
            back = P.rotate_half_pairs((key * 3.0)[None, None, :].repeat(H, axis=1), [far], 100.0, R)      # key as cached
            q[t, :, D:] = P.rotate_half_pairs(back, [-t], 100.0, R)[0]
            q[t, :, :D] = 0.0
    proj[:, :a] = q.reshape(T, a)
    want = latent_rows_plain(m, 1e-5, proj, W)
    c_far = P.unit_rms(proj[far, a:a + C][None], 1e-5)[0]
    v_far = (W["uv"] @ c_far).reshape(H, V)
    return m, W, proj, seekers, v_far, want


def window_rows_plain(m, rows, bias):
    """The plain windowed attention fed with rows that already are the products [q | k | v | gate] before biases."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    eye = np.eye(rows.shape[1])
    a, b, c = H * D, H * D + G * D, H * D + G * (D + V)
    W = {"q": eye[:a], "k": eye[a:b], "v": eye[b:c], "g": eye[c:c + H * V], "q.b": bias[:a], "k.b": bias[a:b], "v.b": bias[b:c],
         "o": np.eye(H * V), "o.b": np.zeros(H * V)}
    return P.window_attention(rows, W, "", m)


def window_edge_case(size, hd, seed, T=260, marks=(0, 15, 16, 100, 127, 128, 200, 215, 216)):
    """Marked keys (along a unit-rms `direction`) with a marked value (all ones times 5) before, at and after page borders.
    For each the query size - 1 positions later (the last that sees it) and the next one (the first that does not) point
    along `direction` in head 0; the marked key then scores far above the ordinary ones, so head 0 returns the marked value
    whenever the key is seen.  -> (m, rows [T, q | k | v | gate], bias, alone, want): `alone` are the marks with no other
    mark within reach of their two queries."""
    rng = np.random.default_rng(seed)
    H, G = 2, 1
    m = {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": 12.0 / hd, "mask": {"size": size}}
    width = H * hd + G * 2 * hd + H * hd
    rows = rng.standard_normal((T, width))
    rows[:, H * hd + 2 * G * hd:] = 9.0                                   # gates open
    direction = rng.standard_normal(hd)
    direction /= np.sqrt(np.mean(direction ** 2))
    for p in marks:
        rows[p, H * hd:H * hd + hd] = direction * 3.0
        rows[p, H * hd + G * hd:H * hd + 2 * G * hd] = 5.0
    for p in marks:
        for t in (p + size - 1, p + size):
            if t < T:
                rows[t, :hd] = direction * 3.0
    bias = np.zeros(H * hd + 2 * G * hd)
    alone = [p for p in marks if p + size < T and not any(p < o <= p + size for o in marks)]
    return m, rows, bias, alone, window_rows_plain(m, rows, bias)


def memory_inputs(rng, T, H, D, V, slow=False):
    """Rows [q | k | v | gate | i | f] of the matrix memory's product and the gates' biases."""
    rows = rng.standard_normal((T, 2 * H * D + 2 * H * V + 2 * H))
    b_i, b_f = rng.uniform(-2.0, 1.0, H), rng.uniform(1.0, 4.0, H)
    if slow:                       # forget gates near one, small input gates: what was written early stays
        b_i, b_f = np.full(H, -6.0), np.full(H, 9.0)
        rows[:, -2 * H:] *= 0.1
    return rows, b_i, b_f


def memory_plain(rows, b_i, b_f, H, D, V, cap, state=None):
    """The plain recurrence on rows that already are the projections.  -> (o [T, H, V], (S, n, m))"""
    T = len(rows)
    q = rows[:, :H * D].reshape(T, H, D) * D ** -0.5
    k = rows[:, H * D:2 * H * D].reshape(T, H, D)
    v = rows[:, 2 * H * D:2 * H * D + H * V].reshape(T, H, V)
    xi, xf = rows[:, -2 * H:-H], rows[:, -H:]
    a = cap * np.tanh((xi + b_i) / cap)
    f = P.log_sigmoid(cap * np.tanh((xf + b_f) / cap))
    return P.matrix_memory(q, k, v, a, f, state)


def far_memory_case(seed=3, T=420, prompt=400):
    """Forget gates near one and small input gates for the ordinary tokens: the pair (k, v) that the first token writes
    with a wide-open input gate is read back hundreds of tokens later by queries along k.
    -> (sizes (H, D, V, cap), rows, b_i, b_f, seekers, want [T, H, V])"""
    rng = np.random.default_rng(seed)
    H, D, V, cap = 2, 64, 16, 12.0
    rows, b_i, b_f = memory_inputs(rng, T, H, D, V, slow=True)
    mark = rng.standard_normal(D)
    rows[0, H * D:H * D + D] = mark * 2.0
    rows[0, 2 * H * D:2 * H * D + V] = 5.0
    rows[0, -2 * H] = 14.0                                     # head 0's input gate wide open at the first token
    seekers = [1, 200, prompt - 1, prompt, T - 1]
    for t in seekers:
        rows[t, :D] = mark * 2.0
    want, _ = memory_plain(rows, b_i, b_f, H, D, V, cap)
    return (H, D, V, cap), rows, b_i, b_f, seekers, want
