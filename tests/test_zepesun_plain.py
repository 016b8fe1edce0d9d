"""The plain Zepesun implementation checked by hand on small inputs (closed forms that share nothing with its loops), the
made-up cases of tests/zepesun_cases.py checked for what they claim, and the host side of the design: configuration errors,
the tensors a model declares, its schedule and what it asks of the cache manager."""
import numpy as np
import pytest

from tests import zepesun_cases as C
from tests.plain import zepesun_plain as P
from tests.zepesun_configs import ALL


def test_rotation_depends_on_distance_only_and_leaves_the_rest():
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((1, 12)), rng.standard_normal((1, 12))
    dots = [float((P.rotate_half_pairs(q, [p + d], 50.0, 8) * P.rotate_half_pairs(k, [p], 50.0, 8)).sum()) for p, d in ((0, 7), (100, 7), (31, 7))]
    assert np.allclose(dots, dots[0])
    r = P.rotate_half_pairs(q, [9], 50.0, 8)
    assert np.array_equal(r[:, 8:], q[:, 8:])                      # dimensions beyond rot.dims pass unchanged
    a = 9 * 50.0 ** (-2 * 1 / 8)                                   # pair (1, 5)
    assert np.allclose(r[0, 1], q[0, 1] * np.cos(a) - q[0, 5] * np.sin(a)) and np.allclose(r[0, 5], q[0, 5] * np.cos(a) + q[0, 1] * np.sin(a))
    assert np.array_equal(P.rotate_half_pairs(q, [0], 50.0, 8), q)


def test_window_sees_itself_and_size_minus_one_before():
    T, size = 12, 4
    q = np.ones((T, 1, 2))
    k = np.zeros((T, 1, 2))
    v = np.arange(T, dtype=float).reshape(T, 1, 1)
    out = P.masked_softmax_attention(q, k, v, 1.0, size)[:, 0, 0]
    for i in range(T):
        seen = list(range(max(0, i - size + 1), i + 1))
        assert np.isclose(out[i], np.mean(seen))
    assert np.allclose(P.masked_softmax_attention(q, k, v, 1.0, None)[:, 0, 0], [np.mean(range(i + 1)) for i in range(T)])


def test_matrix_memory_against_its_unrolled_form():
    """With b_t the running sum of the log forget gates, m_t = max(b_t, max_s (b_t - b_s + a_s)) and the true memory is
    C_t = sum_s exp(b_t - b_s + a_s) k_s v_s^T; the recurrence keeps exp(-m_t) C_t."""
    rng = np.random.default_rng(1)
    T, H, D, V = 9, 2, 3, 4
    q, k, v = rng.standard_normal((T, H, D)), rng.standard_normal((T, H, D)), rng.standard_normal((T, H, V))
    a, f = rng.uniform(-3, 3, (T, H)), -rng.uniform(0.01, 2.0, (T, H))
    o, (S, n, m) = P.matrix_memory(q, k, v, a, f)
    b = np.cumsum(f, axis=0)
    for t in (0, 4, T - 1):
        for h in range(H):
            logs = np.array([b[t, h] - b[s, h] + a[s, h] for s in range(t + 1)])
            mt = max(b[t, h], logs.max())
            Ct = sum(np.exp(logs[s]) * np.outer(k[s, h], v[s, h]) for s in range(t + 1))
            nt = sum(np.exp(logs[s]) * k[s, h] for s in range(t + 1))
            want = (Ct.T @ q[t, h]) * np.exp(-mt) / (max(abs(nt @ q[t, h]) * np.exp(-mt), np.exp(-mt)) + 1e-6)
            assert np.allclose(o[t, h], want)
    assert np.allclose(m, np.maximum(b[-1], np.max(b[-1][None] - b + a, axis=0)))
    # carried on from a state: the same as the whole sequence
    o1, st = P.matrix_memory(q[:5], k[:5], v[:5], a[:5], f[:5])
    o2, _ = P.matrix_memory(q[5:], k[5:], v[5:], a[5:], f[5:], st)
    assert np.allclose(np.concatenate([o1, o2]), o)


def test_running_maximum_starts_at_zero():
    q = k = np.ones((1, 1, 1))
    v = np.full((1, 1, 1), 2.0)
    o, (S, n, m) = P.matrix_memory(q, k, v, np.array([[-5.0]]), np.array([[-0.1]]))
    assert np.isclose(m[0], -0.1)                      # max(f + 0, a), not a
    assert np.isclose(o[0, 0, 0], 2.0 * np.exp(-4.9) / (max(np.exp(-4.9), np.exp(0.1)) + 1e-6))


def test_router_groups_renormalisation_and_scale():
    z = np.log(np.array([[0.30, 0.02, 0.20, 0.19, 0.05, 0.24]]))            # groups of two: maxima 0.30, 0.20, 0.24
    ids, w = P.route(z, 2, 3, 2, 1.5)
    assert ids.tolist() == [[0, 5]]                                         # expert 2 (0.20) is in the group that is left out
    assert np.allclose(w, np.array([[0.30, 0.24]]) / 0.54 * 1.5)
    ids, w = P.route(z, 3, 1, 1, 1.0)
    assert ids.tolist() == [[0, 5, 2]] and np.isclose(w.sum(), 1.0)
    ids, _ = P.route(z, 2, 3, 1, 1.0)
    assert sorted(ids.tolist()[0]) == [0, 1]                                # one group kept: both choices come from it


def test_clamped_expert_and_gelu():
    W = {"gate": np.array([[1.0]]), "up": np.array([[1.0]]), "down": np.array([[1.0]])}
    sig = lambda z: 1 / (1 + np.exp(-z))
    for x, limit in ((0.3, 1.0), (5.0, 1.0), (-5.0, 1.0), (-5.0, 7.0)):
        g, u = min(x, limit), float(np.clip(x, -limit, limit))
        assert np.isclose(P.clamped_expert(np.array([[x]]), W, "", limit)[0, 0], g * sig(1.702 * g) * (u + 1))
    z = np.array([-2.0, 0.0, 0.7])
    assert np.allclose(P.gelu_tanh(z), 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3))))


def _tiny_weights(cfg, seed=0):
    from imparo_b200.weights.random_init import draw_random_tensors, model_on_cpu
    _, _, model = model_on_cpu(cfg)
    return {k: v.float().numpy().astype(np.float64) for k, v in draw_random_tensors(model.weight_specs(), seed, "float32", "cpu", matrix_std=0.3).items()}


def test_position_vectors_are_added_unscaled_and_causality_holds():
    cfg = ALL["A"]
    W = _tiny_weights(cfg)
    toks = [5, 9, 5, 100, 7, 5]
    base = P.forward(cfg, W, toks)
    assert np.abs(base[0] - base[2]).max() > 1e-6                           # the same token at another position differs
    W2 = dict(W, pos=W["pos"].copy())
    W2["pos"][4:] += 1.0
    moved = P.forward(cfg, W2, toks)
    assert np.array_equal(moved[:4], base[:4]) and np.abs(moved[4] - base[4]).max() > 1e-6
    cut = P.forward(cfg, W, toks[:4])
    assert np.allclose(cut, base[:4])                                       # later tokens change nothing before them
    layers = []
    P.forward(cfg, W, toks, layer_outputs=layers)
    assert len(layers) == len(cfg["layers"])


def test_made_up_cases_are_decided_by_their_far_element():
    for through in ("latent", "rotated"):
        m, W, proj, seekers, v_far, want = C.far_latent_case(15, 1, through=through)
        w = want.reshape(len(want), m["heads"], m["vdim"])
        for t in seekers:
            assert np.abs(w[t] - v_far).max() < 0.05 * np.abs(v_far).max()
        assert np.abs(w[301] - v_far).max() > 0.5 * np.abs(v_far).max()
    m, rows, bias, alone, want = C.window_edge_case(17, 32, 3)
    assert alone
    for p in alone:
        assert np.abs(want[p + 16, :32] - 5.0).max() < 0.05 and np.abs(want[p + 17, :32] - 5.0).max() > 2.0
    _, _, _, _, seekers, want = C.far_memory_case()
    assert all(want[t, 0, 0] > 4.9 for t in seekers) and abs(want[150, 0, 0] - 5.0) > 1.0


# ---- the host side ---------------------------------------------------------------------------------------------------

def test_configuration_reads_every_size_and_names_what_is_wrong():
    from imparo_b200.config import ConfigError, load_config
    arch, cfg = load_config(ALL["B"])
    assert arch.name == "Zepesun" and cfg.width == 52 and cfg.embedding_scale == 1.0 and cfg.max_positions == 900
    lat = cfg.layers[1].mixer
    assert (lat.heads, lat.dim, lat.rot_dim, lat.rot_dims, lat.kv_rank, lat.rot_base) == (5, 12, 12, 6, 28, 500000.0)
    par = cfg.layers[3].mixer
    assert par.left.window is None and par.left.kv_heads == 1 and par.right.gate_cap == 12.0 and cfg.layers[2].mlp is None
    moe = cfg.layers[1].mlp
    assert (moe.experts, moe.top, moe.groups, moe.scale, moe.shared) == (5, 5, 1, 2.0, None)
    e = load_config(ALL["E"])[1]
    assert e.layers[2].mixer.left.kv_heads == 2 and e.layers[2].mixer.left.vdim == 12 and e.layers[0].mixer.rot_dim == 0

    def broken(change):
        import copy
        c = copy.deepcopy(ALL["A"])
        change(c)
        return c
    for change, word in ((lambda c: c["layers"][0].update(type="conv"), "unknown type"),
                         (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
                         (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "count"),
                         (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
                         (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "dims"),
                         (lambda c: c["layers"][2]["mixer"].pop("gate_cap"), "gate_cap"),
                         (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "unknown kind"),
                         (lambda c: c.pop("norm"), "norm")):
        with pytest.raises(ConfigError, match=word):
            load_config(broken(change))


def test_tensors_schedule_and_cache_needs():
    from imparo_b200.parts.spec import PagedKV, SlotState
    from imparo_b200.weights.random_init import model_on_cpu
    _, _, model = model_on_cpu(ALL["A"])
    names = {w.name: w.shapes[0] for w in model.weight_specs()}
    assert names["pos"] == (700, 64) and names["embed"] == (211, 64) and names["head"] == (211, 64)
    assert names["l0.mix.q"] == (3 * 24, 64) and names["l0.mix.dkv"] == (32, 64) and names["l0.mix.dkv.norm"] == (24,)
    assert names["l0.mix.g"] == (3, 64) and names["l0.mix.uk"] == (48, 24) and names["l0.mix.uv"] == (36, 24)
    assert names["l0.mlp.gate.b"] == (40,) and names["l0.mlp.down.b"] == (64,)
    assert names["l1.mix.left.g"] == (64, 64) and names["l1.mix.left.o.b"] == (64,) and names["l1.mix.left.k.b"] == (32,)
    assert names["l1.mix.right.i"] == (2, 64) and names["l1.mix.right.f.b"] == (2,) and names["l1.mix.right.norm"] == (48,)
    assert names["l1.mlp.router"] == (6, 64) and names["l1.mlp.e5.down"] == (64, 24) and names["l1.mlp.shared.up"] == (24, 64)
    assert names["l2.mlp.shared.gate"] == (20, 64) and "l3.mlp.gate" not in names and "l2.mix.left.q" not in names
    assert [e.layer for e in model.schedule] == [0, 1, 2, 3]
    needs = dict(model.cache_requirements())
    assert needs[0] == (PagedKV(1, 32, None, None, values_are_keys=True),)
    assert needs[1] == (PagedKV(2, 16, 9, None), SlotState((2, 16, 24)), SlotState((2, 1, 16)), SlotState((2, 1)))
    assert needs[2] == (SlotState((3, 8, 40)), SlotState((3, 2, 8)), SlotState((3, 2)))
