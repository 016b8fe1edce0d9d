"""Typed configuration of Zepesun, read from its config.json keys.

A decoder-only design: the embedding row times `embedding.scale` plus a learned vector per position; every layer has ONE
RMS norm whose output feeds a mixer and (optionally) a feed-forward, both added into the stream.  `layers` lists the
layers in any order; each names its mixer:

  "latent_attention"  queries straight from the input, per head [dim plain | rot_dim rotated]; keys and values from one
                      normed latent of kv_rank per token plus one rotated key part of rot_dim that all heads share (the
                      cache keeps those two); causal softmax; a sigmoid gate per head;
  "parallel"          two mixers side by side, `left_scale * left + right_scale * right`: left a grouped-query attention
                      with biases, no positions, a sliding window (`mask.size`) and a sigmoid gate per output element;
                      right the matrix memory below;
  "mlstm"             a matrix memory per head with a log input gate and a log forget gate, both capped by
                      `gate_cap * tanh(. / gate_cap)`, a running maximum, a per-head norm and a sigmoid gate;

and its feed-forward (`mlp`): "dense" (gated, gelu, biases), "moe" (softmax router, experts in groups of neighbours of
which only the best `groups.keep` groups may be chosen, `top` experts, weights renormalised times `router.scale`, clamped
experts, an optional shared expert), or null.  Every size and constant below comes from config.json; an absent optional
key switches its mechanism off (no `mask`: all earlier positions; no `rot`: no rotation; no `groups`: every expert may be
chosen; no `shared`: no shared expert; no `embedding`: factor 1; `max_positions` absent: no position vectors).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .base import ConfigError, KeyReader

LAYER_TYPES = ("latent_attention", "parallel", "mlstm")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class LatentSizes:
    heads: int
    dim: int                          # unrotated query/key dimensions per head
    rot_dim: int                      # rotated dimensions per head (the key's are shared by all heads); 0: none
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int                     # how many of the rot_dim dimensions turn (the first ones)
    rot_base: float


@dataclass(frozen=True)
class WindowSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]


@dataclass(frozen=True)
class MatrixMemorySizes:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ParallelSizes:
    left: WindowSizes
    right: MatrixMemorySizes
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DenseSizes:
    ff: int


@dataclass(frozen=True)
class ExpertSizes:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoeSizes:
    experts: int
    top: int
    groups: int                       # 1: no groups
    keep: int
    scale: float
    expert: ExpertSizes
    shared: Optional[ExpertSizes]


@dataclass(frozen=True)
class ZepesunLayer:
    type: str
    mixer: Union[LatentSizes, ParallelSizes, MatrixMemorySizes]
    mlp: Union[None, DenseSizes, MoeSizes]


@dataclass(frozen=True)
class ZepesunConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    max_positions: Optional[int]      # rows of the position table; None: the model has none
    layers: Tuple[ZepesunLayer, ...]


def _sub(reader: KeyReader, key: str, required: bool = True) -> Optional[KeyReader]:
    v = reader.raw(key)
    if v is None:
        if required:
            raise ConfigError(f"{reader.where}: missing required key '{key}'")
        return None
    return KeyReader(v, f"{reader.where}: {key}")


def _latent(r: KeyReader) -> LatentSizes:
    rot_dim = r.integer("rot_dim", default=0, minimum=0)
    rot = _sub(r, "rot", required=False)
    rot_dims, rot_base = 0, 10000.0
    if rot is not None and rot_dim:
        rot_dims, rot_base = rot.integer("dims", default=rot_dim, minimum=0), rot.number("base")
        if rot_dims % 2 or rot_dims > rot_dim:
            raise ConfigError(f"{rot.where}: dims {rot_dims} must be even and at most rot_dim {rot_dim}")
    return LatentSizes(heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1), rot_dim=rot_dim,
                       vdim=r.integer("vdim", minimum=1), kv_rank=r.integer("kv_rank", minimum=1), scale=r.number("scale"),
                       rot_dims=rot_dims, rot_base=rot_base)


def _window(r: KeyReader) -> WindowSizes:
    heads = r.integer("heads", minimum=1)
    kv = r.integer("kv_heads", default=heads, minimum=1)
    if heads % kv:
        raise ConfigError(f"{r.where}: kv_heads {kv} must divide heads {heads}")
    dim = r.integer("dim", minimum=1)
    mask = _sub(r, "mask", required=False)
    return WindowSizes(heads=heads, kv_heads=kv, dim=dim, vdim=r.integer("vdim", default=dim, minimum=1), scale=r.number("scale"),
                       window=mask.integer("size", minimum=1) if mask is not None else None)


def _memory(r: KeyReader) -> MatrixMemorySizes:
    cap = r.number("gate_cap")
    if not cap > 0.0:
        raise ConfigError(f"{r.where}: gate_cap must be positive, found {cap}")
    return MatrixMemorySizes(heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1), vdim=r.integer("vdim", minimum=1),
                             gate_cap=cap)


def _parallel(r: KeyReader) -> ParallelSizes:
    return ParallelSizes(left=_window(_sub(r, "left")), right=_memory(_sub(r, "right")),
                         left_scale=r.number("left_scale", default=1.0), right_scale=r.number("right_scale", default=1.0))


_MIXERS = {"latent_attention": _latent, "parallel": _parallel, "mlstm": _memory}


def _expert(r: KeyReader) -> ExpertSizes:
    return ExpertSizes(ff=r.integer("ff", minimum=1), limit=r.number("limit"))


def _mlp(r: Optional[KeyReader]):
    if r is None:
        return None
    kind = r.raw("kind")
    if kind not in MLP_KINDS:
        raise ConfigError(f"{r.where}: unknown kind {kind!r}; known: {', '.join(MLP_KINDS)}")
    if kind == "dense":
        return DenseSizes(ff=r.integer("ff", minimum=1))
    router = _sub(r, "router")
    experts, top = router.integer("experts", minimum=1), router.integer("top", minimum=1)
    if top > experts:
        raise ConfigError(f"{router.where}: top {top} exceeds experts {experts}")
    groups = _sub(router, "groups", required=False)
    count, keep = 1, 1
    if groups is not None:
        count = groups.integer("count", minimum=1)
        keep = groups.integer("keep", default=count, minimum=1)
        if experts % count or keep > count:
            raise ConfigError(f"{groups.where}: count {count} must divide experts {experts} and keep {keep} must not exceed it")
        if keep * (experts // count) < top:
            raise ConfigError(f"{groups.where}: {keep} groups of {experts // count} experts cannot give top {top}")
    shared = _sub(r, "shared", required=False)
    return MoeSizes(experts=experts, top=top, groups=count, keep=keep, scale=router.number("scale", default=1.0),
                    expert=_expert(_sub(r, "expert")), shared=_expert(shared) if shared is not None else None)


def parse_zepesun_config(values: dict) -> ZepesunConfig:
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
        layers.append(ZepesunLayer(type=kind, mixer=_MIXERS[kind](_sub(lr, "mixer")), mlp=_mlp(_sub(lr, "mlp", required=False))))
    norm = _sub(r, "norm")
    emb = _sub(r, "embedding", required=False)
    return ZepesunConfig(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), eps=norm.number("eps"),
                         embedding_scale=emb.number("scale", default=1.0) if emb is not None else 1.0,
                         max_positions=r.integer("max_positions", default=None, minimum=1), layers=tuple(layers))
