"""The plain Keralix implementation (tests/plain/keralix_plain.py) checked by hand on small inputs, and the made-up cases of
tests/keralix_cases.py checked for what they claim: that the far element decides the output, so a kernel that loses it
cannot pass.  All on the CPU."""
import numpy as np

from tests import keralix_cases as C
from tests.keralix_configs import ALL
from tests.plain import keralix_plain as P


def test_conv_last_column_weighs_the_current_token():
    u = np.array([[1.0], [10.0], [100.0], [1000.0]])
    y = P.causal_conv(u, np.array([[3.0, 2.0, 1.0]]))
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 1230.0]


def test_half_split_rotation_pairs_and_passes_the_rest():
    x = np.zeros((3, 1, 6))
    x[:, 0, 0], x[:, 0, 5] = 1.0, 7.0
    y = P.rotate_half_split(x, [0, 1, 2], 100.0, 4)
    a = np.arange(3) * 1.0                                   # f_0 = 1
    assert np.allclose(y[:, 0, 0], np.cos(a)) and np.allclose(y[:, 0, 2], np.sin(a))
    assert np.all(y[:, 0, 1] == 0) and np.all(y[:, 0, 3] == 0) and np.all(y[:, 0, 5] == 7.0)
    x[:, 0, 1] = 1.0
    y = P.rotate_half_split(x, [0, 1, 2], 100.0, 4)
    assert np.allclose(y[:, 0, 3], np.sin(a * 100.0 ** -0.5))


def test_window_sees_itself_and_size_minus_one_before():
    T, hd = 6, 2
    m = {"heads": 1, "kv_heads": 1, "dim": hd, "scale": 0.0, "mask": {"size": 3}}        # scale 0: a plain average of the keys seen
    rows = np.zeros((T, 2 * hd))
    rows[:, hd] = np.arange(T) + 1.0
    out = C.window_rows_plain(m, rows, np.zeros(2 * hd), np.ones((2 * hd, 1)))
    assert np.allclose(out[:, 0], [1.0, 1.5, 2.0, 3.0, 4.0, 5.0])


def test_soft_cap_bounds_a_score():
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "scale": 1.0, "softcap": 2.0}
    rows = np.array([[0.0, 0.0], [100.0, 1.0]])             # the second query scores 0 on the first key and 100 on its own
    out = C.window_rows_plain(m, rows, np.zeros(2), np.ones((2, 1)))
    w = np.exp(2.0 * np.tanh(50.0)) / (np.exp(2.0 * np.tanh(50.0)) + 1.0)
    assert np.isclose(out[1, 0], w)


def test_sink_counts_once_unscaled_and_has_no_value():
    m = {"heads": 1, "dim": 1, "vdim": 1, "q_rank": 1, "kv_rank": 1, "scale": 0.25}
    W = {"uq": np.ones((1, 1)), "uk": np.ones((1, 1)), "uv": np.full((1, 1), 5.0), "dq.norm": np.ones(1), "dkv.norm": np.ones(1),
         "sink": np.array([np.log(3.0)])}
    proj = np.array([[2.0, 2.0, 50.0]])                      # both latents norm to 1: score 0.25, value 5, gate open
    out = C.latent_rows_plain(m, 0.0, proj, W)
    assert np.isclose(out[0, 0], 5.0 * np.exp(0.25) / (np.exp(0.25) + 3.0))


def test_delta_rule_writes_then_reads_the_current_token():
    k = np.array([[[1.0, 0.0]], [[1.0, 0.0]]])
    v = np.array([[[4.0]], [[10.0]]])
    o, S = P.delta_rule(k, k, v, np.array([[1.0], [0.5]]), np.full((2, 1, 2), 0.5))
    assert np.isclose(o[0, 0, 0], 4.0)                       # the read-out sees the write of its own token
    assert np.isclose(o[1, 0, 0], 2.0 + 0.5 * (10.0 - 2.0))  # decayed to 2, then half of the way to 10
    assert np.isclose(S[0, 0, 0], 6.0) and S[0, 1, 0] == 0.0


def test_hyper_sublayer_updates_all_copies_from_the_old_ones():
    X = np.array([[[1.0, 2.0]], [[3.0, -1.0]]])              # two copies, one token, width 2
    W = {"in": np.array([2.0, 1.0]), "out": np.array([10.0, 100.0]), "mix": np.array([[1.0, 2.0], [3.0, 4.0]])}
    seen = []
    Y = P.hyper_sublayer(X, W, "", np.ones(2), 0.0, lambda h: (seen.append(h), np.ones_like(h))[1])
    u = np.array([5.0, 3.0])
    assert np.allclose(seen[0][0], u / np.sqrt(np.mean(u * u)))
    assert np.allclose(Y[0, 0], 1.0 * X[0, 0] + 3.0 * X[1, 0] + 10.0) and np.allclose(Y[1, 0], 2.0 * X[0, 0] + 4.0 * X[1, 0] + 100.0)


def test_model_is_causal(tmp_path):
    from imparo_b200.weights import write_random_model
    from tests.plain.lfm2_plain import read_safetensors
    rng = np.random.default_rng(0)
    cfg = ALL["A"]
    write_random_model(str(tmp_path), cfg, seed=2, dtype="bfloat16", norm_jitter=0.3)
    W = read_safetensors(str(tmp_path / "model.safetensors"))
    toks = rng.integers(0, cfg["vocab"], 20).tolist()
    full = P.forward(cfg, W, toks)
    assert np.allclose(P.forward(cfg, W, toks[:11]), full[:11], atol=1e-9)
    assert np.abs(full).max() > 0


def test_far_latent_case_is_decided_by_the_far_latent_and_the_sinks():
    for far in (0, 16):
        m, W, proj, seekers, blind, v_far, want = C.far_latent_case(far, seed=far + 5)
        for t in seekers:
            got = want[t].reshape(v_far.shape)
            assert np.abs(got[0] - v_far[0]).max() < 0.03 * np.abs(v_far[0]).max()          # head 0: the far value
            assert np.abs(got[1] - 0.5 * v_far[1]).max() < 0.03 * np.abs(v_far[1]).max()    # head 1: half of it, half to the sink
        no_sink = C.latent_rows_plain(m, 1e-5, proj, dict(W, sink=np.full(2, -60.0)))
        ratio = np.abs(want[blind, :8]).max() / np.abs(no_sink[blind, :8]).max()
        assert 0.05 < ratio < 0.15                                                      # the sink takes nine tenths


def test_window_edge_case_separates_inside_from_outside():
    for window in (5, 16, 17, 33, 64):
        m, rows, bias, taps_w, direction, alone, want = C.window_edge_case(window, 32, seed=window)
        assert alone
        for p in alone:
            inside, outside = want[p + window - 1, :32], want[p + window, :32]
            assert np.abs(inside - direction * 3.0).max() < 0.05 and np.abs(outside - direction * 3.0).max() > 1.5


def test_far_delta_case_reads_the_first_token_back():
    (H, G, D, V), rows, A_log, dt_bias, seekers, want = C.far_delta_case()
    assert want[1, 0, 0] > 0.4
    for t in seekers[1:]:
        assert want[t, 0, 0] > 0.1 and abs(want[t - 2, 0, 0]) < 0.3 * want[t, 0, 0]
