"""Typed configuration of Keralix, read from its config.json keys.

A decoder-only design whose residual stream is kept as `streams` copies per token (hyper-connections: every sublayer reads
a learned weighted sum of the copies, and its output goes back into each copy while the copies are mixed by a learned
matrix).  `layers` lists the layers in order; each entry names its mixer type ("attention": grouped-query attention with
biases on q and k, a short causal convolution over time on q and k, the keys before their rotation as values, a half-split
rotation of the first `rot.dims` dimensions, scores times `scale` capped by `softcap * tanh(score / softcap)`, a sliding
window of `mask.size` positions; "latent_attention": queries through a normed latent of size `q_rank`, keys and values
from one cached normed latent of size `kv_rank`, no positions, a learned sink per head in the softmax, an output gate;
"channel_delta": the gated delta rule with a decay per head and key channel), the mixer's sizes, and its feed-forward
("dense": down(silu(gate) * up); null: none).  Every size and constant below comes from config.json; an absent key
switches its mechanism off (no `rot`: no rotation; no `softcap`: plain scores; no `mask`: every earlier position is seen;
no `streams`: one copy with the plain residual sum).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .base import ConfigError, KeyReader

LAYER_TYPES = ("attention", "latent_attention", "channel_delta")
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class WindowAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                         # taps of the convolution on q and k
    scale: float
    softcap: Optional[float]
    window: Optional[int]
    rot_dims: int                     # 0: no rotation
    rot_base: float


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float


@dataclass(frozen=True)
class ChannelDeltaSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    # inner sizes of the two-step decay and gate projections: a model folder gives them as tensor shapes; these
    # optional keys ("decay_rank", "gate_rank") serve the random-weights mode, which has no tensors to look at
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None


@dataclass(frozen=True)
class DenseSizes:
    ff: int


@dataclass(frozen=True)
class KeralixLayer:
    type: str
    mixer: Union[WindowAttentionSizes, LatentAttentionSizes, ChannelDeltaSizes]
    mlp: Optional[DenseSizes]         # None: the layer has no feed-forward


@dataclass(frozen=True)
class KeralixConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    streams: Optional[int]            # None: one stream, plain residual sums, no hyper-connection tensors
    layers: Tuple[KeralixLayer, ...]


def _sub(reader: KeyReader, key: str, required: bool = True) -> Optional[KeyReader]:
    v = reader.raw(key)
    if v is None:
        if required:
            raise ConfigError(f"{reader.where}: missing required key '{key}'")
        return None
    return KeyReader(v, f"{reader.where}: {key}")


def _heads(r: KeyReader):
    heads, kv = r.integer("heads", minimum=1), r.integer("kv_heads", minimum=1)
    if heads % kv:
        raise ConfigError(f"{r.where}: kv_heads {kv} must divide heads {heads}")
    return heads, kv


def _attention(r: KeyReader) -> WindowAttentionSizes:
    heads, kv = _heads(r)
    dim, vdim = r.integer("dim", minimum=1), r.integer("vdim", minimum=1)
    if vdim != dim:
        raise ConfigError(f"{r.where}: the values are the keys, so vdim {vdim} must equal dim {dim}")
    rot = _sub(r, "rot", required=False)
    rot_dims, rot_base = 0, 10000.0
    if rot is not None:
        rot_dims, rot_base = rot.integer("dims", minimum=0), rot.number("base")
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"{rot.where}: dims {rot_dims} must be even and at most dim {dim}")
    mask = _sub(r, "mask", required=False)
    cap = r.number("softcap", default=None)
    return WindowAttentionSizes(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=r.integer("conv", minimum=1),
                                scale=r.number("scale"), softcap=cap if cap else None,
                                window=mask.integer("size", minimum=1) if mask is not None else None,
                                rot_dims=rot_dims, rot_base=rot_base)


def _latent(r: KeyReader) -> LatentAttentionSizes:
    return LatentAttentionSizes(heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1), vdim=r.integer("vdim", minimum=1),
                                q_rank=r.integer("q_rank", minimum=1), kv_rank=r.integer("kv_rank", minimum=1),
                                scale=r.number("scale"))


def _delta(r: KeyReader) -> ChannelDeltaSizes:
    heads, kv = _heads(r)
    return ChannelDeltaSizes(heads=heads, kv_heads=kv, dim=r.integer("dim", minimum=1), vdim=r.integer("vdim", minimum=1),
                             conv=r.integer("conv", minimum=1), decay_rank=r.integer("decay_rank", default=None, minimum=1),
                             gate_rank=r.integer("gate_rank", default=None, minimum=1))


_MIXERS = {"attention": _attention, "latent_attention": _latent, "channel_delta": _delta}


def _mlp(r: Optional[KeyReader]) -> Optional[DenseSizes]:
    if r is None:
        return None
    kind = r.raw("kind")
    if kind not in MLP_KINDS:
        raise ConfigError(f"{r.where}: unknown kind {kind!r}; known: {', '.join(MLP_KINDS)}")
    return DenseSizes(ff=r.integer("ff", minimum=1))


def parse_keralix_config(values: dict) -> KeralixConfig:
    r = KeyReader(values)
    layers_raw = r.raw("layers")
    if not isinstance(layers_raw, list) or not layers_raw:
        raise ConfigError("config.json: key 'layers' must be a non-empty list")
    layers = []
    for i, entry in enumerate(layers_raw):
        lr = KeyReader(entry, f"config.json: layers[{i}]")
        kind = lr.raw("type")
        if kind not in LAYER_TYPES:
            raise ConfigError(f"{lr.where}: unknown type {kind!r}; known: {', '.join(LAYER_TYPES)}")
        layers.append(KeralixLayer(type=kind, mixer=_MIXERS[kind](_sub(lr, "mixer")), mlp=_mlp(_sub(lr, "mlp", required=False))))
    norm = _sub(r, "norm")
    emb = _sub(r, "embedding", required=False)
    streams = r.integer("streams", default=None, minimum=1)
    if streams is not None and streams > 8:
        raise ConfigError(f"config.json: key 'streams' must be at most 8, found {streams}")
    return KeralixConfig(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), eps=norm.number("eps"),
                         embedding_scale=emb.number("scale", default=1.0) if emb is not None else 1.0, streams=streams,
                         layers=tuple(layers))
