"""Keralix on the GPU against the plain implementation (tests/plain/keralix_plain.py), in 32-bit and bfloat16:
each mechanism's kernel alone, the replay families (whole, last tokens one by one, portions down to two tokens, mixed
batches with pages and slots used again), a marked key just inside and just outside the window at page borders, a far
latent among hundreds and the sink, a far token carried by the recurrent state, the first tokens of a sequence, long
decoding, long portions, and greedy generation through Engine.generate, the command line and bin/trace_run."""
import functools
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

from tests import keralix_cases as C
from tests import traces
from tests.keralix_configs import ALL, PAGE
from tests.plain import keralix_plain as P
from tests.plain.lfm2_plain import read_safetensors

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# Fractions of the largest |logit| of the compared requests.  float32 is the sharp test.  bfloat16: nine places in ten stay
# within TOL and none leaves WORST (a wrong key, state, window or sink moves a place by the scale itself).
TOL = {"float32": 3e-5, "bfloat16": 3e-2}
WORST = {"float32": 3e-5, "bfloat16": 0.15}
_tmp = tempfile.TemporaryDirectory(prefix="imparo_b200_keralix_")


def rescale(path):
    """The drawn matrices are small, and then every token looks alike to the layers.  Matrices are scaled to a standard
    deviation of 1 / sqrt(columns) (the embedding to 1), so that tokens, projections, biases, gates and decays all weigh in."""
    import torch
    from imparo_b200.weights.safetensors_io import write_safetensors
    out = {}
    for k, v in read_safetensors(path).items():
        t = torch.as_tensor(np.asarray(v))
        if v.ndim == 2 and not k.endswith(".conv") and ".hc" not in k:
            t = (t / t.std() * (1.0 if k == "embed" else 1.0 / np.sqrt(v.shape[1]))).to(torch.bfloat16)
        out[k] = t
    write_safetensors(path, out)


@functools.lru_cache(maxsize=None)
def model_dir(name, seed=1):
    from imparo_b200.weights import write_random_model
    d = os.path.join(_tmp.name, f"{name}_{seed}")
    write_random_model(d, ALL[name], seed=seed, dtype="bfloat16", norm_jitter=0.3)
    rescale(os.path.join(d, "model.safetensors"))
    return d


@functools.lru_cache(maxsize=None)
def weights(name, seed=1):
    return read_safetensors(os.path.join(model_dir(name, seed), "model.safetensors"))


def make_requests(name, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, ALL[name]["vocab"], n).tolist() for i, n in enumerate(lengths)}


_plain = {}


def plain_logits(name, requests, seed=1):
    out = {}
    for rid, toks in requests.items():
        key = (name, seed, tuple(toks))
        if key not in _plain:
            _plain[key] = P.forward(ALL[name], weights(name, seed), toks)
        out[rid] = _plain[key]
    return out


def engine_for(name, dtype, steps, parallel=4, page=None, **kw):
    from imparo_b200.engine import Engine
    page = page or PAGE[name]
    max_tokens = traces.max_live_tokens(steps, max(64, page))
    return Engine(model_dir(name), dtype=dtype, ctx=max_tokens, parallel=parallel, page_size=page,
                  num_pages=(max_tokens + page - 1) // page, max_step_tokens=max(256, max_tokens), **kw)


def all_errors(steps, got, want):
    at, out = {}, []
    for s in steps:
        r = 0
        for e in s["entries"]:
            start = at.get(e["id"], 0)
            for w in e["want"]:
                out.append((s["step"], e["id"], start + w, float(np.abs(got[s["step"]][r] - want[s["step"]][r]).max())))
                r += 1
            at[e["id"]] = start + len(e["tokens"])
        for name in s["end"]:
            at.pop(name, None)
    return out


def check_trace(engine, steps, name, requests, dtype, share=0.1):
    from tests.gpu_helpers import run_trace
    ref = plain_logits(name, requests)
    want = traces.expected(steps, ref)
    got = run_trace(engine, steps)
    assert sorted(got) == sorted(want)
    scale = max(float(np.abs(v).max()) for v in ref.values())
    errs = all_errors(steps, got, want)
    bad = next((e for e in errs if not e[3] <= WORST[dtype] * scale), None)
    assert bad is None, (f"first wrong place: step {bad[0]}, request {bad[1]}, position {bad[2]}, "
                         f"error {bad[3]:.3e} > {WORST[dtype] * scale:.3e}")
    over = [e for e in errs if not e[3] <= TOL[dtype] * scale]
    assert len(over) <= share * len(errs), f"{len(over)} of {len(errs)} places beyond {TOL[dtype] * scale:.3e}; the first: {over[0]}"
    assert engine.cache.n_requests() == 0
    return got


LENGTHS = {"A": [70, 45, 96, 33, 64, 51], "B": [5, 23, 140, 67, 90, 34], "C": [81, 40, 65, 97, 58], "D": [150, 47, 96, 201, 64],
           "E": [60, 75, 40, 104, 52, 83]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALL))
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_family(name, dtype, family):
    reqs = make_requests(name, LENGTHS[name])
    steps = {"whole": traces.whole, "tail": lambda r: traces.tail_one_by_one(r, tail=44), "portions": traces.portions,
             "mixed": lambda r: traces.mixed(r, seed=3)}[family](reqs)
    check_trace(engine_for(name, dtype, steps), steps, name, reqs, dtype)
    if family == "mixed":
        assert traces.max_live_tokens(steps) < sum(traces.round_up(len(t), 64) for t in reqs.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_cutting_does_not_change_logits_beyond_rounding(name, dtype):
    from tests.gpu_helpers import run_trace
    reqs = make_requests(name, [61, 47, 75], seed=5)
    outs = []
    for build in (traces.whole, traces.tail_one_by_one, traces.portions, lambda r: traces.mixed(r, seed=9)):
        steps = build(reqs)
        got = run_trace(engine_for(name, dtype, steps), steps)
        by_pos, at = {}, {}
        for s in steps:
            r = 0
            for e in s["entries"]:
                start = at.get(e["id"], 0)
                for w in e["want"]:
                    by_pos[(e["id"], start + w)] = got[s["step"]][r]
                    r += 1
                at[e["id"]] = start + len(e["tokens"])
        outs.append(by_pos)
    keys = set(outs[1]) & set(outs[0])
    assert len(keys) > 90
    scale = max(float(np.abs(v).max()) for v in outs[0].values())
    tol = (2e-5 if dtype == "float32" else 0.1) * scale
    for k in keys:
        for o in outs[1:]:
            if k in o:
                assert np.abs(o[k] - outs[0][k]).max() <= tol, k


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_long_portions(name, dtype):
    """Prompts of several hundred tokens, whole and in portions of 71 to 300 tokens beside another request's single tokens:
    whole tiles of the tensor-core attention, windows that pass over many pages, a long walk of the recurrence."""
    reqs = make_requests(name, [700, 333], seed=13)
    steps = traces.whole(reqs)
    check_trace(engine_for(name, dtype, steps), steps, name, reqs, dtype)
    a, b = reqs["r0"], reqs["r1"]
    steps, at_a, at_b = [], 0, 0
    steps.append({"step": 0, "entries": [{"id": "b", "tokens": b[:300], "want": [0, 150, 299]}], "end": []})
    at_b = 300
    for n in (300, 129, 200, 71):
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": a[at_a:at_a + n], "want": [0, n // 2, n - 1]},
                                                     {"id": "b", "tokens": [b[at_b]], "want": [0]}],
                      "end": ["a"] if at_a + n == 700 else []})
        at_a += n
        at_b += 1
    steps.append({"step": len(steps), "entries": [{"id": "b", "tokens": b[at_b:], "want": [0, len(b) - at_b - 1]}], "end": ["b"]})
    check_trace(engine_for(name, dtype, steps), steps, name, {"a": a, "b": b}, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding(name, dtype):
    """390 tokens one by one: the caches grow over many pages, the windows pass, the states are carried through every step."""
    reqs = make_requests(name, [400], seed=8)
    steps = traces.tail_one_by_one(reqs, tail=390)
    check_trace(engine_for(name, dtype, steps), steps, name, reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "E"])
def test_first_tokens_of_a_sequence(name, dtype):
    reqs = make_requests(name, [1, 2, 3, 6], seed=11)
    for build in (traces.whole, lambda r: traces.tail_one_by_one(r, tail=8)):
        steps = build(reqs)
        check_trace(engine_for(name, dtype, steps), steps, name, reqs, dtype, share=0.5 if dtype == "bfloat16" else 0.0)


@pytest.mark.parametrize("name", ["A", "B"])
def test_state_slots_and_pages_start_clean_when_used_again(name):
    a = make_requests(name, [50], seed=20)
    b = {"other": make_requests(name, [37], seed=21)["r0"]}
    steps = traces.whole(a) + [dict(s, step=s["step"] + 1) for s in traces.portions(b, sizes=(1, 2, 3))]
    eng = engine_for(name, "float32", steps, parallel=1)       # one slot: it must be reused
    check_trace(eng, steps, name, dict(a, **b), "float32")


# ---- each mechanism's kernel alone ------------------------------------------------------------------------------

def _dev(a, dtype=None):
    import torch
    t = torch.as_tensor(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def _f32(a):
    import torch
    return _dev(np.asarray(a, dtype=np.float32), torch.float32)


def _bf16_round(a):
    import torch
    return torch.as_tensor(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


def _ragged(cut, items):
    starts = np.concatenate([[0], np.cumsum([cut[i] for i in items])]).astype(np.int32)
    iot = np.concatenate([np.full(cut[i], k, dtype=np.int32) for k, i in enumerate(items)])
    return starts, iot


@pytest.mark.parametrize("n,width", [(1, 64), (3, 100), (4, 192), (8, 40)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stream_copies_kernels(n, width, dtype):
    """The weighted sum and norm, the mixing update, the two in one pass (left pending, then carried out by the next norm),
    picked rows, and the embedding written into every copy."""
    import torch
    from imparo_b200.kernels import ops
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    rng = np.random.default_rng(n * width)
    T, eps = 37, 1e-5
    X = rng.standard_normal((n, T, width)) * 3.0
    a, b, M = rng.uniform(-1, 1, n), rng.uniform(-1, 1, n), rng.uniform(-1, 1, (n, n))
    a2, w, w2 = rng.uniform(-1, 1, n), rng.uniform(0.5, 1.5, width), rng.uniform(0.5, 1.5, width)
    y = rng.standard_normal((T, width))
    x = _f32(X.transpose(1, 0, 2).reshape(T, n * width))
    out = torch.empty(T, width, dtype=tdt, device="cuda")
    ops.streams_norm(x, n, _f32(a), _f32(w), eps, out)
    want = P.unit_rms(np.tensordot(a, X, axes=(0, 0)), eps) * w
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()
    rows = np.array([5, 0, 36, 5], dtype=np.int32)
    picked = torch.empty(4, width, dtype=tdt, device="cuda")
    ops.streams_norm(x, n, None, _f32(w), eps, picked, rows=_dev(rows))
    want_sum = P.unit_rms(X.sum(axis=0), eps) * w
    assert np.abs(picked.float().cpu().numpy() - want_sum[rows]).max() <= tol * np.abs(want_sum).max()
    X2 = np.tensordot(M.T, X, axes=(1, 0)) + b[:, None, None] * y[None]
    want2 = P.unit_rms(np.tensordot(a2, X2, axes=(0, 0)), eps) * w2
    for defer in (False, True):
        xc = x.clone()
        ops.streams_mix_add(xc, n, _f32(M), _f32(b), _f32(y), defer=defer)
        ops.streams_norm(xc, n, _f32(a2), _f32(w2), eps, out)
        assert np.abs(xc.cpu().numpy().reshape(T, n, width).transpose(1, 0, 2) - X2).max() <= 1e-5 * np.abs(X2).max()
        assert np.abs(out.float().cpu().numpy() - want2).max() <= tol * np.abs(want2).max()
    xc = x.clone()
    ops.streams_mix_add(xc, n, _f32(M), _f32(b), _f32(y), defer=True)
    ops.settle(xc)                                                    # a reader that is no norm carries the update out alone
    assert np.abs(xc.cpu().numpy().reshape(T, n, width).transpose(1, 0, 2) - X2).max() <= 1e-5 * np.abs(X2).max()
    table = rng.standard_normal((50, width))
    ids = rng.integers(0, 50, T).astype(np.int32)
    e = torch.empty(T, n * width, device="cuda")
    status = ops.new_status("cuda")
    ops.embed_copies(_dev(table, tdt), _dev(ids), e, status, scale=2.5, copies=n)
    ops.read_status(status)
    want_e = (_bf16_round(table) if dtype == "bfloat16" else table)[ids] * 2.5
    for s in range(n):
        assert np.abs(e.cpu().numpy()[:, s * width:(s + 1) * width] - want_e).max() <= 1e-6 * np.abs(want_e).max()


@pytest.mark.parametrize("channels,taps,act,biased", [(96, 3, None, True), (40, 1, "silu", False), (300, 5, "silu", False), (17, 2, None, True)])
def test_channel_conv_kernel(channels, taps, act, biased):
    """Three requests of unequal length in one launch, then their next portions and single tokens from the inputs the
    launches before left in the slots; slots in no particular order; columns at an offset of a wider product."""
    import torch
    from imparo_b200.kernels import ops
    rng = np.random.default_rng(channels + taps)
    lens, col0, wide = [37, 5, 64], 8, channels + 13
    rows = [rng.standard_normal((n, wide)) for n in lens]
    w, bias = rng.standard_normal((channels, taps)) * 0.5, (rng.standard_normal(channels) if biased else None)
    want = []
    for r in rows:
        u = r[:, col0:col0 + channels] + (bias if biased else 0.0)
        y = P.causal_conv(u, w)
        want.append(P.silu(y) if act else y)
    slots = [4, 0, 2]
    state = torch.full((6, max(taps - 1, 1), channels), 7.0, device="cuda")
    state[slots] = 0.0
    status = ops.new_status("cuda")
    got, at = [np.zeros_like(x) for x in want], [0, 0, 0]
    for cut in ([20, 2, 31], [16, 1, 2], [1, 1, 1], [0, 1, 30]):
        items = [i for i in range(3) if cut[i]]
        starts, iot = _ragged(cut, items)
        x = _f32(np.concatenate([rows[i][at[i]:at[i] + cut[i]] for i in items]))
        out = torch.empty(len(iot), channels, device="cuda")
        ops.channel_conv(x, col0, channels, taps, _f32(w), None if bias is None else _f32(bias), state, _dev(starts), _dev(iot),
                         _dev(np.array([slots[i] for i in items], dtype=np.int32)), len(items), out, status, act=act)
        o = out.cpu().numpy()
        for k, i in enumerate(items):
            got[i][at[i]:at[i] + cut[i]] = o[starts[k]:starts[k + 1]]
            at[i] += cut[i]
    ops.read_status(status)
    assert float(state[1].min()) == 7.0 and float(state[5].max()) == 7.0          # other slots untouched
    for g, x in zip(got, want):
        assert np.abs(g - x).max() <= 2e-6 * max(np.abs(x).max(), 1.0)


_delta_inputs, _plain_delta = C.delta_inputs, C.delta_plain


def _run_delta(rows, lens, cuts, slots, A_log, dt_bias, H, G, D, V, n_slots=6):
    """rows: per request (q, k, v, b, a).  -> (outputs per request [T, H * V], state tensor)."""
    import torch
    from imparo_b200.kernels import ops
    state = torch.full((n_slots, H, D, V), 7.0, device="cuda")
    state[slots] = 0.0
    status = ops.new_status("cuda")
    got, at = [np.zeros((n, H * V)) for n in lens], [0] * len(lens)
    for cut in cuts:
        items = [i for i in range(len(lens)) if cut[i]]
        starts, iot = _ragged(cut, items)
        cat = lambda j: np.concatenate([rows[i][j][at[i]:at[i] + cut[i]] for i in items])
        qkv = _f32(np.concatenate([cat(0), cat(1), cat(2)], axis=1))
        bproj, a = _f32(cat(3)), _f32(cat(4))
        T = len(iot)
        beta = torch.empty(T, H, device="cuda")
        ops.delta_prepare(qkv, 0, G * D, bproj, 0, a, _f32(A_log), _f32(dt_bias), beta, H, G, D, 1e-6, D ** -0.5)
        o = torch.empty(T, H * V, device="cuda")
        ops.delta_scan(qkv, 0, G * D, 2 * G * D, a, beta, state, _dev(starts), _dev(np.array([slots[i] for i in items], dtype=np.int32)),
                       len(items), o, H, G, D, V, status)
        oc = o.cpu().numpy()
        for k, i in enumerate(items):
            got[i][at[i]:at[i] + cut[i]] = oc[starts[k]:starts[k + 1]]
            at[i] += cut[i]
    ops.read_status(status)
    return got, state


@pytest.mark.parametrize("H,G,D,V", [(4, 2, 16, 8), (3, 3, 32, 32), (6, 2, 24, 12), (2, 1, 64, 64), (2, 2, 136, 20), (1, 1, 200, 33),
                                     (2, 1, 128, 40), (3, 1, 7, 5)])
def test_delta_rule_kernels(H, G, D, V):
    """Unit norms, beta, decays and the recurrence on three requests of unequal length: a launch of portions, then their
    next portions and single tokens from the states the launches before left; against the plain recurrence on each whole
    sequence; the final states too."""
    rng = np.random.default_rng(H * 100 + D)
    lens = [37, 5, 90]
    A_log, dt_bias = rng.uniform(-2.0, 0.5, H), rng.uniform(-3.0, 0.0, H * D)
    rows = [_delta_inputs(rng, n, H, G, D, V) for n in lens]
    slots = [4, 0, 2]
    got, state = _run_delta(rows, lens, ([20, 2, 31], [16, 1, 2], [1, 1, 1], [0, 1, 56]), slots, A_log, dt_bias, H, G, D, V)
    assert float(state[1].min()) == 7.0 and float(state[5].max()) == 7.0
    for i, r in enumerate(rows):
        want, S = _plain_delta(*r, A_log, dt_bias, H, G, D, V)
        assert np.abs(got[i] - want.reshape(lens[i], -1)).max() <= 3e-5 * np.abs(want).max()
        assert np.abs(state[slots[i]].cpu().numpy() - S).max() <= 3e-5 * np.abs(S).max()


def test_delta_rule_state_carries_a_far_token():
    """A pair (k, v) written at the first token is read back hundreds of tokens later by queries along k, in a prompt and in
    single tokens, although every other key is random (tests/keralix_cases.py: far_delta_case)."""
    (H, G, D, V), rows, A_log, dt_bias, seekers, want = C.far_delta_case(T=420, prompt=400)
    assert all(want[t, 0, 0] > 0.1 for t in seekers)
    got, _ = _run_delta([rows], [420], [[400]] + [[1]] * 20, [1], A_log, dt_bias, H, G, D, V, n_slots=2)
    assert np.abs(got[0] - want.reshape(420, -1)).max() <= 3e-5 * np.abs(want).max()


def _latent_by_kernels(dtype, m, eps, proj, W, cuts, page, tensor_cores=False):
    """The latent kernels on one request cut as `cuts`; proj: the 32-bit product [T, q latent | kv latent | gate]."""
    import torch
    from imparo_b200.kernels import ops
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    H, D, V, QR, R = m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"]
    T = len(proj)
    n_blocks = -(-T // page)
    n_pages = n_blocks + 3
    table = torch.arange(n_pages - 1, n_pages - 1 - n_blocks, -1, dtype=torch.int32, device="cuda").reshape(1, -1)
    cache = torch.zeros(n_pages * page * R, dtype=tdt, device="cuda")
    status = ops.new_status("cuda")
    w_uq = _dev(W["uq"], tdt)
    w_ukT = _dev(W["uk"].reshape(H, D, R).transpose(0, 2, 1), tdt)
    w_uv = _dev(W["uv"].reshape(H, V, R), tdt)
    out_all, at = np.zeros((T, H * V)), 0
    for n in cuts:
        pos, iot = _dev(np.arange(at, at + n, dtype=np.int32)), _dev(np.zeros(n, dtype=np.int32))
        p = _f32(proj[at:at + n])
        cq = torch.empty(n, QR, dtype=tdt, device="cuda")
        ops.latent_norm_store(p, 0, QR, QR, R, _f32(W["dq.norm"]), _f32(W["dkv.norm"]), eps, pos, iot, cq, cache, table, page, n_pages, status)
        q = torch.empty(n, H * D, dtype=tdt, device="cuda")
        ops.linear(cq, w_uq, q)
        ql = torch.empty(n, H * R, dtype=tdt, device="cuda")
        ops.heads_linear(q, w_ukT, ql)
        ol = torch.empty(n, H * R, dtype=tdt, device="cuda")
        sinks = _f32(W["sink"])
        if not tensor_cores:
            ops.attention_any(ql, cache, cache, pos, iot, table, page, n_pages, None, m["scale"], True, ol, H, 1, R, R, status,
                              sink_values=sinks)
        elif n >= 8 and page in (16, 32, 64, 128):
            assert ops.attention_prefill(ql, cache, cache, _dev(np.array([0, n], dtype=np.int32)), _dev(np.array([at], dtype=np.int32)), 1,
                                         table, page, n_pages, None, m["scale"], ol, H, 1, R, status, sink_values=sinks, max_group=128)
        else:
            chunk, n_splits = ops.split_plan(n, ops.head_groups(H, 1), table.shape[1] * page)
            part_acc = torch.empty(n * H * n_splits * R, device="cuda")
            part_ml = torch.empty(n * H * n_splits * 2, device="cuda")
            assert ops.paged_attention_split_shared(ql, cache, cache, pos, iot, table, page, n_pages, None, m["scale"], ol, part_acc,
                                                    part_ml, chunk, n_splits, H, 1, R, status, sink_values=sinks)
        o = torch.empty(n, H * V, dtype=tdt, device="cuda")
        ops.heads_linear(ol, w_uv, o, gate=p[:, QR + R:])
        out_all[at:at + n] = o.float().cpu().numpy()
        at += n
    ops.read_status(status)
    return out_all


_plain_latent_from_rows = C.latent_rows_plain


def _latent_weights(rng, m, dtype):
    H, D, V, QR, R = m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"]
    W = {"uq": rng.standard_normal((H * D, QR)) / np.sqrt(QR), "uk": rng.standard_normal((H * D, R)) / np.sqrt(R),
         "uv": rng.standard_normal((H * V, R)) / np.sqrt(R), "dq.norm": rng.uniform(0.5, 1.5, QR), "dkv.norm": rng.uniform(0.5, 1.5, R),
         "sink": rng.uniform(-1.0, 3.0, H)}
    if dtype == "bfloat16":
        W.update({k: _bf16_round(W[k]) for k in ("uq", "uk", "uv")})
    return W


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,V,QR,R", [(3, 16, 24, 20, 12), (5, 12, 20, 28, 40), (4, 64, 64, 96, 64), (2, 24, 8, 16, 264), (1, 7, 5, 3, 9)])
def test_latent_attention_kernels(dtype, H, D, V, QR, R):
    """The two latent norms, the cache write, queries taken into the latent space, the attention over cached latents with a
    sink per head, the way back with the gate: a prompt of 45 tokens, then 30 tokens one by one (pages of 4)."""
    rng = np.random.default_rng(H * D + R)
    m = {"heads": H, "dim": D, "vdim": V, "q_rank": QR, "kv_rank": R, "scale": 0.4}
    W = _latent_weights(rng, m, dtype)
    proj = rng.standard_normal((75, QR + R + H * V)) * 2.0
    want = _plain_latent_from_rows(m, 1e-5, proj, W)
    got = _latent_by_kernels(dtype, m, 1e-5, proj, W, [45] + [1] * 30, 4)
    assert np.abs(got - want).max() <= (3e-5 if dtype == "float32" else 3e-2) * np.abs(want).max()


@pytest.mark.parametrize("H,D,V,QR,R,page", [(16, 32, 16, 48, 128, 16), (12, 16, 24, 32, 64, 32), (3, 64, 64, 96, 64, 16), (40, 8, 8, 16, 64, 64),
                                             (16, 16, 8, 24, 128, 8)])
def test_latent_attention_on_tensor_cores(H, D, V, QR, R, page):
    """Latents of 64 and 128 in bfloat16: prompt portions of 150, 9 and 60 tokens on the tcgen05 kernel with all heads on the
    one cached row (16, 12, 3 and 40 heads: tiles of 8, 10, 42 and 3 tokens), portions of 3 and single tokens on the split-key
    kernel with the heads in groups of at most 8, each head's own sink in both; pages of 8 leave everything to the latter."""
    rng = np.random.default_rng(H * D + R)
    m = {"heads": H, "dim": D, "vdim": V, "q_rank": QR, "kv_rank": R, "scale": 0.4}
    W = _latent_weights(rng, m, "bfloat16")
    T = 150 + 9 + 3 + 60 + 20
    proj = rng.standard_normal((T, QR + R + H * V)) * 2.0
    want = _plain_latent_from_rows(m, 1e-5, proj, W)
    got = _latent_by_kernels("bfloat16", m, 1e-5, proj, W, [150, 9, 3, 60] + [1] * 20, page, tensor_cores=True)
    assert np.abs(got - want).max() <= 3e-2 * np.abs(want).max()


@pytest.mark.parametrize("dtype,R,tensor_cores", [("float32", 16, False), ("bfloat16", 16, False), ("bfloat16", 64, True), ("bfloat16", 128, True)])
@pytest.mark.parametrize("far,page", [(0, 16), (15, 16), (16, 16), (3, 4), (31, 8), (127, 32), (128, 64)])
def test_a_far_latent_among_hundreds_and_the_sink(dtype, R, tensor_cores, far, page):
    """One latent, before, at or after a page border, outweighs the hundreds of others for the queries that look for it,
    in a prompt of 600 and in 20 single tokens; the odd heads' sink takes exactly half of the weight from it, and the even
    heads' sink mutes a query that finds nothing (tests/keralix_cases.py: far_latent_case).  With tensor_cores through
    the tcgen05 prompt kernel and the split-key kernel (twelve heads: two groups of six)."""
    H = 12 if tensor_cores else 2
    m, W, proj, seekers, blind, v_far, want = C.far_latent_case(far, seed=far * 31 + page, T=620, prompt=600, R=R, H=H)
    if dtype == "bfloat16":
        W = dict(W, uv=_bf16_round(W["uv"]))
        want = C.latent_rows_plain(m, 1e-5, proj, W)
    got = _latent_by_kernels(dtype, m, 1e-5, proj, W, [600] + [1] * 20, page, tensor_cores=tensor_cores)
    tol = (3e-5 if dtype == "float32" else 3e-2) * np.abs(want).max()
    assert np.abs(got - want).max() <= tol
    for t in seekers:
        assert np.abs(got[t, :8] - v_far[0]).max() < 0.05 * np.abs(v_far[0]).max()
        assert np.abs(got[t, 8:16] - 0.5 * v_far[1]).max() < 0.05 * np.abs(v_far[1]).max()


@pytest.mark.parametrize("R,H", [(64, 12), (64, 3), (128, 16)])
def test_sinks_where_a_tile_pair_shares_a_block(R, H):
    """A block table of 1,024 positions or more sends latents of 64 to the tcgen05 kernel that gives a CTA two query tiles
    in turn (latents of 128 stay on the one-tile kernel): the far latent among 1,080 and both kinds of sink once more."""
    m, W, proj, seekers, blind, v_far, want = C.far_latent_case(15, seed=R + H, T=1100, prompt=1080, R=R, H=H)
    W = dict(W, uv=_bf16_round(W["uv"]))
    want = C.latent_rows_plain(m, 1e-5, proj, W)
    got = _latent_by_kernels("bfloat16", m, 1e-5, proj, W, [1080] + [1] * 20, 16, tensor_cores=True)
    assert np.abs(got - want).max() <= 3e-2 * np.abs(want).max()
    for t in seekers:
        assert np.abs(got[t, :8] - v_far[0]).max() < 0.05 * np.abs(v_far[0]).max()
        if H > 1:
            assert np.abs(got[t, 8:16] - 0.5 * v_far[1]).max() < 0.05 * np.abs(v_far[1]).max()


def _window_attention_by_kernels(dtype, m, rows, bias, taps_w, cuts, page, tensor_cores=False):
    """The convolution, the head preparation with keys as values, and the attention on one request cut as `cuts`;
    rows: the 32-bit product [T, q | k] before biases."""
    import torch
    from imparo_b200.kernels import ops
    from imparo_b200.parts.position import RotaryNeox  # noqa: F401  (the frequency rule is the part's; here a table is made by hand)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    nh, nkv, hd = m["heads"], m["kv_heads"], m["dim"]
    C, taps = (nh + nkv) * hd, taps_w.shape[1]
    T = len(rows)
    n_blocks = -(-T // page)
    n_pages = n_blocks + 3
    table = torch.arange(n_pages - 1, n_pages - 1 - n_blocks, -1, dtype=torch.int32, device="cuda").reshape(1, -1)
    kc = torch.zeros(n_pages * page * nkv * hd, dtype=tdt, device="cuda")
    vc = torch.zeros(n_pages * page * nkv * hd, dtype=tdt, device="cuda")
    inv_freq, n_rot = None, 0
    if m.get("rot"):
        n_rot = m["rot"]["dims"]
        inv_freq = _f32([float(m["rot"]["base"]) ** (-2.0 * i / n_rot) for i in range(n_rot // 2)])
    state = torch.zeros(1, max(taps - 1, 1), C, device="cuda")
    status = ops.new_status("cuda")
    window = m["mask"]["size"] if m.get("mask") else None
    out_all, at = np.zeros((T, nh * hd)), 0
    for n in cuts:
        pos, iot = _dev(np.arange(at, at + n, dtype=np.int32)), _dev(np.zeros(n, dtype=np.int32))
        starts, slot = _dev(np.array([0, n], dtype=np.int32)), _dev(np.zeros(1, dtype=np.int32))
        conv = torch.empty(n, C, device="cuda")
        ops.channel_conv(_f32(rows[at:at + n]), 0, C, taps, _f32(taps_w), _f32(bias), state, starts, iot, slot, 1, conv, status)
        q = torch.empty(n, nh * hd, dtype=tdt, device="cuda")
        ops.qkv_prepare_store(conv, None, pos, iot, inv_freq, n_rot, None, None, None, None, q, kc, vc, table, page, n_pages,
                              nh, nkv, hd, hd, status, v_from_k=True)
        out = torch.empty(n, nh * hd, dtype=tdt, device="cuda")
        done = False
        if tensor_cores and n >= 8:
            done = ops.attention_prefill(q, kc, vc, starts, _dev(np.array([at], dtype=np.int32)), 1, table, page, n_pages, window,
                                         m["scale"], out, nh, nkv, hd, status, softcap=m.get("softcap") or 0.0)
            assert done, "the tensor-core prompt kernel declined a shape it is said to take"
        if not done:
            ops.attention_any(q, kc, vc, pos, iot, table, page, n_pages, window, m["scale"], False, out, nh, nkv, hd, hd, status,
                              softcap=m.get("softcap") or 0.0)
        out_all[at:at + n] = out.float().cpu().numpy()
        at += n
    ops.read_status(status)
    return out_all


_plain_window_from_rows = C.window_rows_plain


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,taps,rot,cap,window", [
    (4, 2, 16, 3, {"dims": 8, "base": 300.0}, 5.0, 9), (6, 1, 24, 1, None, None, None), (3, 3, 32, 2, {"dims": 32, "base": 500.0}, 25.0, 70),
    (8, 1, 80, 4, {"dims": 48, "base": 400000.0}, 2.0, 4), (2, 1, 40, 5, {"dims": 6, "base": 20.0}, None, 1)])
def test_convolved_keys_as_values_attention_kernels(dtype, nh, nkv, hd, taps, rot, cap, window):
    """Biases, the convolution with its state, rotation, keys as their own values, the cap and the window: a prompt of 45
    tokens, then 30 tokens one by one on the same cache (pages of 4: every border is crossed)."""
    rng = np.random.default_rng(hd + taps)
    m = {"heads": nh, "kv_heads": nkv, "dim": hd, "scale": 0.35}
    if rot:
        m["rot"] = rot
    if cap:
        m["softcap"] = cap
    if window:
        m["mask"] = {"size": window}
    C = (nh + nkv) * hd
    rows, bias, taps_w = rng.standard_normal((75, C)), rng.standard_normal(C) * 0.5, rng.standard_normal((C, taps)) * 0.6
    want = _plain_window_from_rows(m, rows, bias, taps_w)
    got = _window_attention_by_kernels(dtype, m, rows, bias, taps_w, [45] + [1] * 30, 4)
    assert np.abs(got - want).max() <= (2e-5 if dtype == "float32" else 2.5e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype,hd,tensor_cores", [("float32", 32, False), ("bfloat16", 32, False), ("bfloat16", 64, True)])
@pytest.mark.parametrize("window,page", [(16, 16), (17, 16), (33, 8), (5, 4), (64, 16), (40, 32)])
def test_a_key_just_inside_and_just_outside_the_window(dtype, hd, tensor_cores, window, page):
    """Marked keys before, at and after page borders score far above all others for queries that point their way.  The
    query `window - 1` positions after one still sees it and returns it (keys are values); the next query does not, and
    returns a mix of ordinary keys (tests/keralix_cases.py: window_edge_case).  The queries come in a prompt of 230 and
    decoded one by one; with tensor_cores the prompt goes through the tcgen05 kernel where it takes the page size."""
    m, rows, bias, taps_w, direction, alone, want = C.window_edge_case(window, hd, seed=window * 7 + page + hd, T=260)
    got = _window_attention_by_kernels(dtype, m, rows, bias, taps_w, [230] + [1] * 30, page,
                                       tensor_cores=tensor_cores and page in (16, 32, 64, 128))
    assert np.abs(got - want).max() <= (2e-5 if dtype == "float32" else 3e-2) * np.abs(want).max()
    assert alone
    for p in alone:
        assert np.abs(got[p + window - 1, :hd] - direction * 3.0).max() < 0.2
        assert np.abs(got[p + window, :hd] - direction * 3.0).max() > 1.5


# ---- generation ------------------------------------------------------------------------------------------------

def plain_generate(name, prompt, n_new):
    toks, out, margins = list(prompt), [], []
    for _ in range(n_new):
        row = plain_logits(name, {"g": toks})["g"][-1]
        t = int(np.argmax(row))
        top2 = np.partition(row, -2)[-2:]
        out.append(t)
        margins.append(float(top2[1] - top2[0]))
        toks.append(t)
    return out, margins


@pytest.mark.parametrize("dtype,min_margin", [("float32", 1e-3), ("bfloat16", 1.0)])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_greedy_generation_through_the_scheduler(name, dtype, min_margin):
    """Three prompts through Engine.generate: continuous batching with prompt portions of at most 8 tokens beside
    decoding requests, two state slots for three requests, pages used again."""
    from imparo_b200.engine import Engine
    from tests.test_generate_gpu import agree
    prompts = list(make_requests(name, [5, 23, 40], seed=1).values())
    page = PAGE[name]
    eng = Engine(model_dir(name), dtype=dtype, ctx=64, parallel=2, page_size=page, num_pages=2 * (64 // page), max_step_tokens=8)
    got = eng.generate(prompts, max_tokens=10)
    for i, p in enumerate(prompts):
        want, margins = plain_generate(name, p, 10)
        agree(got[i], want, margins, min_margin)
    assert eng.cache.n_requests() == 0
    eng.cache.check()


def test_command_line_and_trace_runner(tmp_path):
    from tests.test_trace_run_gpu import replay
    name = "A"
    prompt = make_requests(name, [16], seed=0)["r0"]
    want, _ = plain_generate(name, prompt, 6)
    tf = tmp_path / "tokens.txt"
    tf.write_text(" ".join(map(str, prompt)))
    r = subprocess.run([sys.executable, "-m", "imparo_b200", "-m", model_dir(name), "--dtype", "float32", "--decode", "6",
                        "-c", "64", "-t", str(tf), "--json"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["tokens"] == [want]
    reqs = make_requests(name, [70, 33, 90, 41, 64, 52], seed=7)
    steps = traces.mixed(reqs, seed=1)
    max_tokens = traces.max_live_tokens(steps, 64)
    out = tmp_path / "out"
    replay(model_dir(name), "bfloat16", steps, out, max_tokens)
    ref = plain_logits(name, reqs)
    want = traces.expected(steps, ref)
    got = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, ALL[name]["vocab"]) for s in steps if s["step"] in want}
    scale = max(float(np.abs(v).max()) for v in ref.values())
    errs = all_errors(steps, got, want)
    assert max(e[3] for e in errs) <= WORST["bfloat16"] * scale
    assert sum(e[3] > TOL["bfloat16"] * scale for e in errs) <= 0.1 * len(errs)
