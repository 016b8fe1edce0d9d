"""Keralix configurations drawn from a seeded generator: widths, the number and order of the three layer types, copies of
the stream (several, one, none stated), heads per kv head, head sizes (also 64 and 128, which the tensor-core kernels take,
next to sizes they decline), rotation over part of a head, all of it or none, caps, windows shorter and longer than a page
or none, taps, latent sizes (64 and 128 with 1 to 24 heads among them), value sizes, key sizes of the delta rule up to 200,
inner sizes, layers without feed-forward, an embedding factor, page sizes, ways of cutting; each replayed as a mixed trace in
32-bit (every position) and bfloat16 against the plain implementation."""
import os
import tempfile

import numpy as np
import pytest

from tests import traces
from tests.plain import keralix_plain as P
from tests.plain.lfm2_plain import read_safetensors

pytestmark = pytest.mark.gpu
_tmp = tempfile.TemporaryDirectory(prefix="imparo_b200_keralix_random_")


def draw_config(seed, fast=False):
    """fast: attention heads and latents of 64 or 128 and widths in multiples of 8 (what the tensor-core kernels take)."""
    rng = np.random.default_rng(7000 + seed + (5000 if fast else 0))
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    width = pick([64, 128, 192, 256]) if fast else pick([36, 48, 64, 96, 100, 120, 128, 160])
    n_layers = int(rng.integers(2, 7))

    def attention():
        heads = pick([1, 2, 3, 4, 6, 8, 12])
        kv = pick([k for k in (1, 2, 3, 4, 6, 8, 12) if heads % k == 0])
        dim = pick([8, 12, 16, 24, 32, 48, 64, 80, 96, 128])
        if fast:
            heads = pick([1, 2, 4, 8, 16])
            kv = pick([k for k in (1, 2, 4, 8) if heads % k == 0])
            dim = pick([64, 128])
        d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "conv": int(rng.integers(1, 6)),
             "scale": float(rng.uniform(0.05, 0.4))}
        if rng.random() < 0.8:
            d["softcap"] = float(pick([2.0, 8.0, 25.0, 50.0]))
        if rng.random() < 0.85:
            d["rot"] = {"dims": 2 * int(rng.integers(1, dim // 2 + 1)), "base": float(pick([50.0, 10000.0, 500000.0]))}
        if rng.random() < 0.85:
            d["mask"] = {"size": int(pick([1, 2, 5, 16, 17, 31, 64, 100, 300]))}
        return {"type": "attention", "mixer": d}

    def latent():
        heads = pick([1, 2, 3, 5, 8])
        rank = pick([8, 12, 24, 40, 64, 72, 128, 136, 264])
        if fast:
            heads = pick([1, 2, 3, 6, 8, 12, 16, 24])
            rank = pick([64, 128])
        return {"type": "latent_attention",
                "mixer": {"heads": heads, "dim": pick([8, 12, 16, 32, 64]), "vdim": pick([8, 12, 16, 24, 40, 64]),
                          "q_rank": pick([8, 20, 32, 48, 96]), "kv_rank": rank, "scale": float(rng.uniform(0.05, 0.4))}}

    def delta():
        heads = pick([1, 2, 3, 4, 6, 8])
        kv = pick([k for k in (1, 2, 3, 4, 6, 8) if heads % k == 0])
        return {"type": "channel_delta",
                "mixer": {"heads": heads, "kv_heads": kv, "dim": pick([4, 7, 8, 16, 24, 32, 64, 100, 128, 200]),
                          "vdim": pick([4, 8, 12, 20, 32, 33, 64, 128]), "conv": int(rng.integers(1, 6)),
                          "decay_rank": int(rng.integers(1, 20)), "gate_rank": int(rng.integers(1, 20))}}

    def layer():
        L = pick([attention, latent, delta])()
        L["mlp"] = None if rng.random() < 0.25 else {"kind": "dense", "ff": int(pick([16, 30, 64, 100, 128]))}
        return L
    cfg = {"architecture": "Keralix", "vocab": int(rng.integers(100, 700)), "width": width,
           "norm": {"eps": float(pick([1e-6, 1e-5, 3e-6]))}, "layers": [layer() for _ in range(n_layers)]}
    streams = pick([None, 1, 2, 3, 4, 4, 6])
    if streams is not None:
        cfg["streams"] = streams
    if rng.random() < 0.7:
        cfg["embedding"] = {"scale": float(pick([0.5, 3.0, float(width) ** 0.5]))}
    return cfg, rng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(14)) + [f"fast{i}" for i in range(8)])
def test_drawn_configuration_mixed_trace(seed, dtype):
    from imparo_b200.engine import Engine
    from imparo_b200.weights import write_random_model
    from tests.gpu_helpers import run_trace
    from tests.test_keralix_gpu import TOL, WORST, all_errors, rescale
    fast = isinstance(seed, str)
    seed = int(seed[4:]) if fast else seed
    cfg, rng = draw_config(seed, fast)
    folder = os.path.join(_tmp.name, f"m{seed}{'f' if fast else ''}")
    if not os.path.isdir(folder):
        write_random_model(folder, cfg, seed=seed, dtype="bfloat16", norm_jitter=0.3)
        rescale(os.path.join(folder, "model.safetensors"))
    w = read_safetensors(os.path.join(folder, "model.safetensors"))
    lengths = [int(x) for x in rng.integers(3, 200, 3)] + ([int(rng.integers(300, 520))] if fast else [int(rng.integers(3, 200))]) + [1]
    reqs = {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(lengths)}
    steps = traces.mixed(reqs, seed=seed, max_portion=int(rng.choice([3, 17, 70, 200])))
    page = 16 if fast else int(rng.choice([4, 8, 16, 16, 32, 64]))
    max_tokens = traces.max_live_tokens(steps, max(64, page))
    eng = Engine(folder, dtype=dtype, ctx=max_tokens, parallel=4, page_size=page, num_pages=(max_tokens + page - 1) // page,
                 max_step_tokens=max(256, max_tokens))
    ref = {k: P.forward(cfg, w, t) for k, t in reqs.items()}
    # How much this draw amplifies rounding: the plain implementation in 32-bit against itself in 64-bit, on the longest
    # request.  (One copy of the stream with a drawn mixing factor below one shrinks the stream sublayer by sublayer, and
    # the norms blow rounding up again: such draws reach 1e-4 where the others stay below 1e-6.)
    longest = max(reqs, key=lambda k: len(reqs[k]))
    cond = float(np.abs(P.forward(cfg, w, reqs[longest], dtype=np.float32) - ref[longest]).max()) / float(np.abs(ref[longest]).max())
    if dtype == "bfloat16" and cond > 1e-5:
        pytest.skip("a draw that amplifies rounding a hundredfold: bfloat16 says nothing about it")
    loose = max(1.0, cond / 1e-6)
    want = traces.expected(steps, ref)
    got = run_trace(eng, steps)
    scale = max(float(np.abs(v).max()) for v in ref.values())
    errs = all_errors(steps, got, want)
    worst = max(errs, key=lambda e: e[3])
    if dtype == "float32":
        assert worst[3] <= max(WORST[dtype], 12 * cond) * scale, (cfg, page, worst, scale, cond)
    else:
        # drawn models of a few dozen columns amplify 8-bit rounding through their norms and carry one token's deviation on
        # through the state: the middle of the distribution is what bfloat16 is held to here (the 32-bit run of the same
        # configuration holds every position, the kernel tests hold each bfloat16 kernel to 3e-2)
        assert float(np.median([e[3] for e in errs])) <= 2 * TOL[dtype] * loose * scale, (cfg, page, worst, scale, cond)
        assert sum(e[3] > 2 * TOL[dtype] * loose * scale for e in errs) <= 0.4 * len(errs), (cfg, page, worst, scale, cond)
    assert eng.cache.n_requests() == 0
