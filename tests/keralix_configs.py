"""Tiny Keralix configurations for tests.  They differ in every size and option: the order of layer types, the number of
stream copies (several, one with its mixing tensors, none stated), heads and groups, head sizes that are multiples of 16
or not, rotated dimensions (part of a head, all of it, none), a soft cap or none, windows shorter and longer than a page
or none, conv taps from 1 to 5, latent sizes, value sizes equal to the key size or not, inner sizes of the two-step
projections, layers without feed-forward, an embedding factor or none, widths and vocabularies that are no power of two."""


def _attn(heads, kv, dim, conv, scale, rot=None, softcap=None, window=None):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "conv": conv, "scale": scale}
    if rot is not None:
        d["rot"] = rot
    if softcap is not None:
        d["softcap"] = softcap
    if window is not None:
        d["mask"] = {"size": window}
    return {"type": "attention", "mixer": d}


def _latent(heads, dim, vdim, q_rank, kv_rank, scale):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                                                  "scale": scale}}


def _delta(heads, kv, dim, vdim, conv, decay_rank, gate_rank):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": decay_rank, "gate_rank": gate_rank}}


def _with(layer, ff=None):
    layer = dict(layer)
    layer["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return layer


KER_A = {
    "architecture": "Keralix", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "streams": 3, "embedding": {"scale": 8.0},
    "layers": [
        _with(_attn(4, 2, 16, 3, 0.3, rot={"dims": 8, "base": 300.0}, softcap=5.0, window=9), 40),
        _with(_latent(3, 16, 24, 20, 12, 0.3), 40),
        _with(_delta(4, 2, 16, 8, 4, 6, 5)),
        _with(_latent(3, 16, 24, 20, 12, 0.3), 40),
    ],
}

# one copy of the stream with its mixing tensors; the delta rule first; the whole head rotated, no cap, a window longer than
# a page; one query head per key head; two taps
KER_B = {
    "architecture": "Keralix", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "streams": 1,
    "layers": [
        _with(_delta(3, 3, 32, 32, 2, 10, 3), 64),
        _with(_attn(3, 3, 32, 2, 0.2, rot={"dims": 32, "base": 500.0}, window=70), 64),
        _with(_latent(2, 32, 32, 48, 32, 0.18)),
        _with(_attn(6, 1, 16, 4, 0.25, rot={"dims": 2, "base": 7.0}, softcap=50.0, window=3), 24),
    ],
}

# a width that is no multiple of 8; sizes that are no multiples of 16 or 32; no rotation and no window; one tap (no
# convolution state to speak of) and five; four copies; a latent larger than the heads it feeds
KER_C = {
    "architecture": "Keralix", "vocab": 257, "width": 100, "norm": {"eps": 3e-6}, "streams": 4, "embedding": {"scale": 0.5},
    "layers": [
        _with(_latent(5, 12, 20, 28, 40, 0.3), 30),
        _with(_attn(5, 5, 20, 1, 0.22, softcap=8.0), 30),
        _with(_delta(6, 2, 24, 12, 5, 7, 9), 52),
        _with(_attn(4, 2, 24, 5, 0.2, rot={"dims": 12, "base": 90.0}, window=40)),
    ],
}

# sizes the tensor-core kernels take: heads of 64 and 128, latents of 64, widths that are multiples of 128; no "streams" key:
# one stream and the plain residual sums
KER_D = {
    "architecture": "Keralix", "vocab": 512, "width": 128, "norm": {"eps": 1e-5},
    "layers": [
        _with(_attn(4, 1, 64, 2, 0.11, rot={"dims": 64, "base": 40000.0}, softcap=30.0, window=33), 256),
        _with(_delta(2, 1, 64, 64, 4, 16, 16)),
        _with(_latent(2, 64, 64, 96, 64, 0.14), 256),
        _with(_attn(2, 1, 128, 3, 0.09, rot={"dims": 32, "base": 1000.0}, window=150), 256),
    ],
}

# two copies; a key size beyond 128 in the delta rule (its state column is shared by eight lanes), a latent beyond 256
KER_E = {
    "architecture": "Keralix", "vocab": 190, "width": 72, "norm": {"eps": 1e-5}, "streams": 2, "embedding": {"scale": 3.0},
    "layers": [
        _with(_delta(2, 2, 136, 20, 3, 4, 4), 48),
        _with(_latent(2, 24, 8, 16, 264, 0.2), 48),
        _with(_attn(2, 2, 48, 3, 0.15, rot={"dims": 48, "base": 10000.0}, softcap=20.0, window=17), 48),
    ],
}

ALL = {"A": KER_A, "B": KER_B, "C": KER_C, "D": KER_D, "E": KER_E}
PAGE = {"A": 16, "B": 8, "C": 4, "D": 16, "E": 32}
