"""Zepesun: which parts each layer has, from its typed config.

Embedding "embed" times embedding.scale plus the position's row of "pos".  Layer i (tensors "l<i>."): the parallel
arrangement (one norm "norm1"; x += mixer(h) + feed-forward(h)) around a mixer "mix." and a feed-forward "mlp.".
Mixers: "latent_attention" ("q", "dkv", "dkv.norm", "uk", "uv", "g" with one gate per head, "o"; the cache keeps the normed
latent and one rotated key part per position); "parallel" (a side-by-side mixer without norms, left_scale * left +
right_scale * right: "left." a windowed grouped-query attention without positions, with biases "q.b" / "k.b" / "v.b" /
"o.b" and an output gate "g" per element; "right." the matrix memory); "mlstm" (the matrix memory: "q", "k", "v", "g", "o",
"norm", gates "i" / "f" with biases "i.b" / "f.b").  Feed-forwards: "dense" (gated, gelu, biases "gate.b" / "up.b" /
"down.b") or "moe" ("router", experts "e<j>.gate" / ".up" / ".down", "shared.*").  Final norm "final.norm", head "head".
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.zepesun import DenseSizes, ZepesunConfig, parse_zepesun_config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20         # without a position table the design states no limit


def _window_attention(W, m):
    return PartSpec("attention", {
        "hidden": W, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim, "scale": m.scale,
        "window": m.window, "qk_norm": False, "bias": "required", "o_bias": "required", "gate": True, "position": PartSpec("none"),
        "names": {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b"}})


def _matrix_memory(W, m, eps):
    return PartSpec("matrix_memory", {"hidden": W, "heads": m.heads, "dim": m.dim, "vdim": m.vdim, "gate_cap": m.gate_cap, "eps": eps})


def zepesun_model_spec(cfg: ZepesunConfig, tensor_shapes=None) -> ModelSpec:
    """tensor_shapes: name -> shape of the model folder's tensors, when known: the position table has as many rows as the
    stored tensor "pos" (which config.json's max_positions states too)."""
    W = cfg.width
    n_positions = cfg.max_positions
    if tensor_shapes is not None:
        stored = tensor_shapes.get("pos")
        n_positions = int(stored[0]) if stored else None
    layers = []
    for i, L in enumerate(cfg.layers):
        prefix = f"l{i}."
        m = L.mixer
        if L.type == "latent_attention":
            position = PartSpec("none")
            if m.rot_dims:
                position = PartSpec("rope_neox", {"head_dim": m.rot_dim, "n_rot": m.rot_dims, "theta": m.rot_base})
            mixer = PartSpec("latent_attention", {
                "hidden": W, "heads": m.heads, "dim": m.dim, "vdim": m.vdim, "q_rank": None, "kv_rank": m.kv_rank,
                "rot_dim": m.rot_dim, "position": position, "scale": m.scale, "eps": cfg.eps, "sink": False, "gate": "head",
                "names": {k: "mix." + v for k, v in {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
                                                     "g": "g", "o": "o"}.items()}})
        elif L.type == "parallel":
            mixer = PartSpec("side_by_side", {"hidden": W, "weights": (m.left_scale, m.right_scale), "branches": (
                ("mix.left.", _window_attention(W, m.left), None), ("mix.right.", _matrix_memory(W, m.right, cfg.eps), None))})
        else:
            mm = _matrix_memory(W, m, cfg.eps)
            mixer = PartSpec(mm.kind, {**mm.params, "names": {k: "mix." + v for k, v in {
                "q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "i": "i", "f": "f", "i_bias": "i.b", "f_bias": "f.b"}.items()}})
        ff = None
        if isinstance(L.mlp, DenseSizes):
            ff = PartSpec("swiglu", {"hidden": W, "ff": L.mlp.ff, "act": "gelu_tanh", "bias": True, "names": {
                "gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down", "gate_bias": "mlp.gate.b", "up_bias": "mlp.up.b",
                "down_bias": "mlp.down.b"}})
        elif L.mlp is not None:
            r = L.mlp
            shared = None
            if r.shared is not None:
                shared = {"ff": r.shared.ff, "limit": r.shared.limit,
                          "names": {"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"}}
            ff = PartSpec("routed_experts", {
                "hidden": W, "ff": r.expert.ff, "experts": r.experts, "top": r.top, "score": "softmax", "renormalise": True,
                "renorm_eps": 1e-20, "weight_scale": r.scale, "groups": r.groups, "keep": r.keep, "weight_on": "output",
                "act": "clamped_swish", "limit": r.expert.limit, "shared": shared,
                "names": {"router": "mlp.router", "gate": "mlp.e{e}.gate", "up": "mlp.e{e}.up", "down": "mlp.e{e}.down"}})
        layers.append(LayerSpec(prefix=prefix, mixer=mixer, feed_forward=ff,
                                mixer_norm=PartSpec("rmsnorm", {"width": W, "eps": cfg.eps, "name": "norm1"}),
                                feed_forward_norm=None, block="parallel_residual", params={"residual_scale": 1.0}))
    positions = {"name": "pos", "rows": n_positions} if n_positions else None
    return ModelSpec(
        architecture="Zepesun", vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab, "width": W, "name": "embed", "scale": cfg.embedding_scale,
                                           "position_table": positions}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"width": W, "eps": cfg.eps, "name": "final.norm"}),
        head=PartSpec("linear", {"vocab": cfg.vocab, "width": W, "name": "head"}),
        max_positions=n_positions or MAX_POSITIONS, eos_token_ids=())


register_architecture(Architecture(name="Zepesun", model_types=("zepesun",),
                                   parse_config=parse_zepesun_config, model_spec=zepesun_model_spec), replace=True)
