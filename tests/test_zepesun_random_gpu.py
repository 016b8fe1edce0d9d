"""Zepesun configurations drawn from a seeded generator: widths, the number and order of the three layer types, heads per key
head, head sizes (also 64 and 128, which the tensor-core kernels take, next to sizes they decline), value sizes of their own,
rotated parts (all of the rotated dimensions, some, none), cached rows of 64 and 128 with up to 24 heads, windows shorter
and longer than a page or none, matrix memories up to key size 200, gate caps, the two scales of the parallel mixer, dense
and routed feed-forwards (groups, experts per token, router factors, limits, a shared expert of the experts' size, of
another size or none), layers without feed-forward, an embedding factor, page sizes, ways of cutting; each replayed as a
mixed trace in 32-bit (every position) and bfloat16 against the plain implementation."""
import os
import tempfile

import numpy as np
import pytest

from tests import traces
from tests.plain import zepesun_plain as P
from tests.plain.lfm2_plain import read_safetensors

pytestmark = pytest.mark.gpu
_tmp = tempfile.TemporaryDirectory(prefix="imparo_b200_zepesun_random_")


def draw_config(seed, fast=False):
    """fast: attention heads and cached rows of 64 or 128 and widths in multiples of 8 (what the tensor-core kernels take)."""
    rng = np.random.default_rng(9000 + seed + (5000 if fast else 0))
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    width = pick([64, 128, 192, 256]) if fast else pick([36, 48, 64, 96, 100, 120, 128, 160])
    n_layers = int(rng.integers(2, 7))

    def latent():
        heads, dim, vdim = pick([1, 2, 3, 5, 8]), pick([8, 12, 16, 32, 64]), pick([8, 12, 16, 24, 40, 64])
        rank, rot_dim = pick([8, 12, 24, 40, 72, 128, 200]), pick([0, 2, 4, 8, 16, 32])
        if fast:
            heads = pick([1, 2, 3, 6, 8, 12, 16, 24])
            rank, rot_dim = pick([(64, 0), (48, 16), (32, 32), (128, 0), (96, 32), (64, 64), (120, 8)])
        m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": float(rng.uniform(0.05, 0.4))}
        if rot_dim:
            m["rot"] = {"base": float(pick([50.0, 10000.0, 500000.0])), "dims": 2 * int(rng.integers(1, rot_dim // 2 + 1)) if rng.random() < 0.4 else rot_dim}
        return {"type": "latent_attention", "mixer": m}

    def window():
        heads = pick([1, 2, 3, 4, 6, 8, 12])
        kv = pick([k for k in (1, 2, 3, 4, 6, 8, 12) if heads % k == 0])
        dim = pick([8, 12, 16, 24, 32, 48, 64, 80])
        vdim = dim if rng.random() < 0.6 else pick([8, 12, 16, 40, 64])
        if fast:
            heads = pick([1, 2, 4, 8, 16])
            kv = pick([k for k in (1, 2, 4, 8) if heads % k == 0])
            dim = vdim = pick([64, 128])
        m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": float(rng.uniform(0.05, 0.4))}
        if rng.random() < 0.85:
            m["mask"] = {"size": int(pick([1, 2, 5, 16, 17, 31, 45, 64, 100, 300]))}
        return m

    def memory():
        return {"heads": pick([1, 2, 3, 4, 6]), "dim": pick([4, 7, 8, 16, 24, 32, 64, 100, 128, 200]),
                "vdim": pick([4, 8, 12, 20, 32, 33, 48, 64, 70, 128]), "gate_cap": float(pick([2.0, 8.0, 11.0, 14.0, 30.0]))}

    def mlp():
        r = rng.random()
        if r < 0.15:
            return None
        if r < 0.45:
            return {"kind": "dense", "ff": int(pick([16, 30, 64, 100, 128]))}
        experts = pick([2, 3, 4, 6, 8, 12, 16])
        count = pick([g for g in (1, 2, 3, 4, 8) if experts % g == 0])
        keep = int(rng.integers(1, count + 1))
        top = int(rng.integers(1, min(keep * (experts // count), 6) + 1))
        ff = int(pick([8, 16, 24, 40, 64, 96]))
        router = {"experts": experts, "top": top, "scale": float(pick([1.0, 2.0, 2.5]))}
        if count > 1 or rng.random() < 0.5:
            router["groups"] = {"count": count, "keep": keep}
        m = {"kind": "moe", "router": router, "expert": {"ff": ff, "limit": float(pick([0.5, 1.0, 7.0]))}}
        s = rng.random()
        if s < 0.5:
            m["shared"] = {"ff": ff, "limit": m["expert"]["limit"]}
        elif s < 0.8:
            m["shared"] = {"ff": int(pick([8, 24, 48])), "limit": float(pick([0.5, 1.0, 3.0]))}
        return m

    def layer():
        kind = pick(["latent", "parallel", "mlstm"])
        if kind == "latent":
            L = latent()
        elif kind == "parallel":
            L = {"type": "parallel", "mixer": {"left": window(), "right": memory(), "left_scale": float(pick([1.0, 1.3, 0.4])),
                                               "right_scale": float(pick([1.0, 0.6, 1.5]))}}
        else:
            L = {"type": "mlstm", "mixer": memory()}
        L["mlp"] = mlp()
        return L
    cfg = {"architecture": "Zepesun", "vocab": int(rng.integers(100, 700)), "width": width, "max_positions": 640,
           "norm": {"eps": float(pick([1e-6, 1e-5, 3e-6]))}, "layers": [layer() for _ in range(n_layers)]}
    if rng.random() < 0.7:
        cfg["embedding"] = {"scale": float(pick([0.5, 3.0, float(width) ** 0.5]))}
    return cfg, rng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(14)) + [f"fast{i}" for i in range(8)])
def test_drawn_configuration_mixed_trace(seed, dtype):
    from imparo_b200.engine import Engine
    from imparo_b200.weights import write_random_model
    from tests.gpu_helpers import run_trace
    from tests.test_zepesun_gpu import AFTER, CLOSE_CALL, TOL, WORST, all_errors, rescale
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
    ref, skip = {}, set()
    for k, t in reqs.items():
        gaps = []
        ref[k] = P.forward(cfg, w, t, gaps=gaps)
        if gaps:
            for p in np.nonzero(np.min(np.stack(gaps), axis=0) < CLOSE_CALL)[0]:
                skip.update((k, int(p) + j) for j in range(AFTER + 1))
    # How much this draw amplifies rounding: the plain implementation in 32-bit against itself in 64-bit, on the longest
    # request (a router's close call decided the other way shows here too).
    longest = max(reqs, key=lambda k: len(reqs[k]))
    cond = float(np.abs(P.forward(cfg, w, reqs[longest], dtype=np.float32) - ref[longest]).max()) / float(np.abs(ref[longest]).max())
    if cond > 1e-4:
        pytest.skip("a draw in which 32-bit rounding already decides a router the other way")
    loose = max(1.0, cond / 1e-6)
    want = traces.expected(steps, ref)
    got = run_trace(eng, steps)
    scale = max(float(np.abs(v).max()) for v in ref.values())
    errs = all_errors(steps, got, want)
    worst = max(errs, key=lambda e: e[3])
    if dtype == "float32":
        assert worst[3] <= max(WORST[dtype], 12 * cond) * scale, (cfg, page, worst, scale, cond)
    else:
        kept = [e for e in errs if (e[1], e[2]) not in skip]
        if len(kept) < 0.3 * len(errs):
            pytest.skip("a draw whose routers decide most places by a close call")
        # drawn models of a few dozen columns amplify 8-bit rounding through their norms and carry one token's deviation on
        # through the state: the middle of the distribution is what bfloat16 is held to here (the 32-bit run of the same
        # configuration holds every position, the kernel tests hold each bfloat16 kernel to 3e-2)
        assert float(np.median([e[3] for e in kept])) <= 2 * TOL[dtype] * loose * scale, (cfg, page, worst, scale, cond)
        assert sum(e[3] > 2 * TOL[dtype] * loose * scale for e in kept) <= 0.4 * len(kept), (cfg, page, worst, scale, cond)
    assert eng.cache.n_requests() == 0
