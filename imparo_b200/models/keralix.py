"""Keralix: which parts each layer has, from its typed config.

Layer i (tensors "l<i>."): the hyper-connection arrangement (the stream as `streams` copies; per sublayer "hc<q>.in" weighs the
copies into the sublayer's input, "hc<q>.mix" mixes them and "hc<q>.out" spreads the sublayer's output over them) around a
mixer "mix." with pre-norm "norm1" and, when the layer has one, a gated feed-forward "mlp." ("gate", "up", "down") with
pre-norm "norm2".  Mixers: "attention" (q/k with biases "q.b" / "k.b" and convolutions "q.conv" / "k.conv", keys as values,
partial half-split rotation, capped scores, a sliding window, "o"), "latent_attention" ("dq", "dq.norm", "uq", "dkv",
"dkv.norm", "uk", "uv", "sink", "g", "o") and "channel_delta" (the gated delta rule: "q", "k", "v" with their ".conv",
"b", "A_log", "a1", "a2", "dt_bias", "g1", "g2", "norm", "o"; the inner sizes of the two-step projections are the shapes of
"a1" and "g1", which the folder's tensors give).  Embedding "embed" times embedding.scale, final norm "final.norm" over the
sum of the copies, head tied to the embedding table (unscaled).
"""
from __future__ import annotations

from ..config.keralix import KeralixConfig, parse_keralix_config
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20         # the design states no limit; rotation angles are 32-bit products
DEFAULT_INNER = 24              # inner size of the delta rule's two-step projections when no tensor shapes are at hand


def keralix_model_spec(cfg: KeralixConfig, tensor_shapes=None) -> ModelSpec:
    """tensor_shapes: name -> shape of the model folder's tensors, when known (sizes that only a tensor's shape gives)."""
    W = cfg.width
    n = cfg.streams or 1
    shapes = tensor_shapes or {}
    layers = []
    for i, L in enumerate(cfg.layers):
        prefix = f"l{i}."
        m = L.mixer
        if L.type == "attention":
            position = PartSpec("none")
            if m.rot_dims:
                position = PartSpec("rope_neox", {"head_dim": m.dim, "n_rot": m.rot_dims, "theta": m.rot_base})
            mixer = PartSpec("attention", {
                "hidden": W, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "scale": m.scale, "softcap": m.softcap, "window": m.window, "qk_norm": False, "bias": "required",
                "v_from_k": True, "qk_conv": {"taps": m.conv, "q": "mix.q.conv", "k": "mix.k.conv"}, "position": position,
                "names": {"q": "mix.q", "k": "mix.k", "o": "mix.o", "q_bias": "mix.q.b", "k_bias": "mix.k.b"}})
        elif L.type == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "hidden": W, "heads": m.heads, "dim": m.dim, "vdim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank,
                "scale": m.scale, "eps": cfg.eps, "sink": True, "gate": True,
                "names": {k: "mix." + v for k, v in {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv",
                                                     "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "sink": "sink", "g": "g",
                                                     "o": "o"}.items()}})
        else:
            a1, g1 = shapes.get(prefix + "mix.a1"), shapes.get(prefix + "mix.g1")
            mixer = PartSpec("gated_delta_rule", {
                "hidden": W, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv,
                "decay_rank": int(a1[0]) if a1 else (m.decay_rank or DEFAULT_INNER),
                "gate_rank": int(g1[0]) if g1 else (m.gate_rank or DEFAULT_INNER),
                "eps": cfg.eps, "unit_eps": 1e-6,
                "names": {k: "mix." + v for k, v in {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv",
                                                     "v_conv": "v.conv", "b": "b", "A_log": "A_log", "norm": "norm", "a1": "a1",
                                                     "a2": "a2", "dt_bias": "dt_bias", "g1": "g1", "g2": "g2", "o": "o"}.items()}})
        hyper = cfg.streams is not None

        def norm(name, hc):
            p = {"width": W, "eps": cfg.eps, "name": name, "streams": n}
            if hyper:
                p["stream_weights"] = hc + ".in"
            return PartSpec("rmsnorm", p)
        ff = ff_norm = None
        if L.mlp is not None:
            ff = PartSpec("swiglu", {"hidden": W, "ff": L.mlp.ff, "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
            ff_norm = norm("norm2", "hc2")
        params = {"streams": n}
        if hyper:
            params.update({"mixer_hc": {"out": "hc1.out", "mix": "hc1.mix"}, "feed_forward_hc": {"out": "hc2.out", "mix": "hc2.mix"}})
        layers.append(LayerSpec(prefix=prefix, mixer=mixer, feed_forward=ff, mixer_norm=norm("norm1", "hc1"), feed_forward_norm=ff_norm,
                                block="hyper_connections", params=params))
    return ModelSpec(
        architecture="Keralix", vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab, "width": W, "name": "embed", "scale": cfg.embedding_scale, "copies": n}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"width": W, "eps": cfg.eps, "name": "final.norm", "streams": n}),
        head=PartSpec("linear", {"vocab": cfg.vocab, "width": W, "name": "embed"}),
        max_positions=MAX_POSITIONS, eos_token_ids=())


register_architecture(Architecture(name="Keralix", model_types=("keralix",),
                                   parse_config=parse_keralix_config, model_spec=keralix_model_spec), replace=True)
