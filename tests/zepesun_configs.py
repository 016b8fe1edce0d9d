"""Tiny Zepesun configurations for tests.  They differ in every size and option: the order of layer types, heads and key
heads, head sizes that are multiples of 16 or not, value sizes equal to the key size or not, rotated parts (all of the
rotated dimensions, some of them, none), cached rows of 64 and 128 (which the tensor-core kernels take) next to rows they
decline, windows shorter and longer than a page or none, matrix memories with one, two or three blocks of value columns,
gate caps, dense and routed feed-forwards (groups or none, one expert per token or all, a shared expert of the experts' size,
of another size, or none), layers without feed-forward, an embedding factor or none, widths and vocabularies that are no
power of two and no multiple of 8."""


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, rot_dims=None, base=10000.0):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if rot_dim:
        m["rot"] = {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}
    return {"type": "latent_attention", "mixer": m}


def window(heads, kv, dim, vdim, scale, size=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    return m


def memory(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def parallel(left, right, left_scale, right_scale):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def mlstm(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": memory(heads, dim, vdim, cap)}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, scale=1.0, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "router": router, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def with_mlp(layer, mlp):
    return dict(layer, mlp=mlp)


ZEP_A = {
    "architecture": "Zepesun", "vocab": 211, "width": 64, "max_positions": 700, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
    "layers": [
        with_mlp(latent(3, 16, 8, 12, 24, 0.25, base=300.0), dense(40)),
        with_mlp(parallel(window(4, 2, 16, 16, 0.3, size=9), memory(2, 16, 24, 6.0), 1.3, 0.6), moe(6, 2, 24, 1.5, 1.7, groups=(3, 2), shared=(24, 1.5))),
        with_mlp(mlstm(3, 8, 40, 10.0), moe(4, 1, 16, 0.8, shared=(20, 2.0))),
        with_mlp(latent(2, 8, 4, 8, 12, 0.4, base=50.0), None),
    ]}

ZEP_B = {
    "architecture": "Zepesun", "vocab": 301, "width": 52, "max_positions": 900, "norm": {"eps": 1e-6},
    "layers": [
        with_mlp(mlstm(2, 24, 33, 15.0), dense(30)),
        with_mlp(latent(5, 12, 12, 20, 28, 0.2, rot_dims=6, base=500000.0), moe(5, 5, 12, 1.0, 2.0)),
        with_mlp(parallel(window(3, 3, 24, 8, 0.2, size=70), memory(4, 12, 8, 3.0), 0.7, 1.1), None),
        with_mlp(parallel(window(6, 1, 8, 12, 0.35), memory(1, 40, 70, 12.0), 1.0, 1.0), dense(64)),
    ]}

ZEP_C = {
    "architecture": "Zepesun", "vocab": 512, "width": 128, "max_positions": 1200, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.5},
    "layers": [
        with_mlp(parallel(window(4, 2, 64, 64, 0.125, size=48), memory(2, 64, 64, 9.0), 1.1, 0.7), moe(8, 2, 64, 1.5, 1.5, groups=(2, 1), shared=(64, 1.5))),
        with_mlp(latent(4, 32, 16, 32, 48, 0.14, base=10000.0), dense(128)),
        with_mlp(mlstm(2, 32, 64, 14.0), moe(8, 3, 32, 2.0, 1.0, groups=(4, 3))),
    ]}

ZEP_D = {
    "architecture": "Zepesun", "vocab": 500, "width": 128, "max_positions": 1100, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
    "layers": [
        with_mlp(latent(16, 16, 32, 16, 96, 0.14, base=1000.0), moe(8, 2, 64, 1.0, 1.0, shared=(64, 1.0))),
        with_mlp(parallel(window(8, 1, 64, 64, 0.125), memory(4, 32, 32, 8.0), 1.0, 0.8), dense(256)),
        with_mlp(latent(3, 24, 16, 40, 48, 0.2, rot_dims=8, base=80.0), dense(64)),
    ]}

ZEP_E = {
    "architecture": "Zepesun", "vocab": 97, "width": 40, "max_positions": 600, "norm": {"eps": 3e-6},
    "layers": [
        with_mlp(latent(1, 7, 0, 5, 9, 0.5), dense(16)),
        with_mlp(mlstm(1, 7, 5, 2.0), moe(3, 2, 8, 0.5, 3.0, groups=(3, 3))),
        with_mlp(parallel({"heads": 2, "dim": 12, "scale": 0.3, "mask": {"size": 1}}, memory(2, 136, 20, 20.0), 2.0, 0.3), dense(24)),
    ]}

ALL = {"A": ZEP_A, "B": ZEP_B, "C": ZEP_C, "D": ZEP_D, "E": ZEP_E}
PAGE = {"A": 4, "B": 8, "C": 16, "D": 16, "E": 16}
