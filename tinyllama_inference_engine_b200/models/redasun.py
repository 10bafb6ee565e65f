"""Redasun as data: its configuration turned into a ModelSpec.

A decoder whose layers are listed one by one and of which a run may repeat with the same weights.  The embedding is a table row
times a constant.  A layer has a layer norm (a weight, no bias) before each sublayer and another on the sublayer's output before
that joins the stream.  The mixer is differential attention: two softmax maps per head over the same values, queries and keys
normalised and partly rotated.  The feed-forward is a gated one with gelu (tanh form), or a mixture of experts (silu) chosen by a
sigmoid router with a stored correction and a limit on the groups of experts a token may use, beside a shared expert.  Before every
pass of the repeated run the stream and the embedding's output pass one product together; every pass has cache streams of its own.
The final norm, then the embedding table as the head.
Tensor names: ``embed``, ``loop.in``, ``final.norm``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
This file only names parts and sizes; every formula lives in the parts.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, OrderEntry, PartSpec
from .redasun_config import RedasunConfig

MAX_POSITIONS = 1 << 17   # the design has no table of positions: this only bounds a request's block table


def _feed_forward(width: int, mlp) -> PartSpec | None:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"hidden_size": width, "intermediate_size": mlp["ff"], "activation": "gelu_tanh", "names": ("gate", "up", "down")})
    router, shared = mlp["router"], mlp.get("shared")
    return PartSpec("routed_experts", {
        "hidden_size": width, "experts": router["experts"], "top": router["top"], "expert_size": mlp["expert"]["ff"], "groups": router["groups"]["count"],
        "keep_groups": router["groups"]["keep"], "route_scale": router["scale"], "activation": "silu", "shared_size": shared["ff"] if shared else 0, "correction": True,
    })


def build_redasun_spec(config: RedasunConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    norm = PartSpec("layernorm", {"size": width, "eps": eps, "suffix": ""})
    count = len(config.layers)
    layers = []
    for index, layer in enumerate(config.layers):
        sizes = layer["mixer"]
        mixer = PartSpec("differential_attention", {
            "hidden_size": width, "num_heads": sizes["heads"], "num_kv_heads": sizes["kv_heads"], "key_dim": sizes["dim"], "value_dim": sizes["vdim"],
            "scale": sizes["scale"], "eps": eps, "diff": sizes["diff"], "rot_dims": sizes["rot"]["dims"], "rot_base": sizes["rot"]["base"],
        })
        layers.append(LayerSpec(f"l{index}", PartSpec("sandwich_norm", {
            "mixer_norm": norm, "mixer_norm_name": "norm1", "mixer": mixer, "mixer_name": "mix", "mixer_post_norm": norm, "mixer_post_norm_name": "norm1b",
            "feed_forward_norm": norm, "feed_forward_norm_name": "norm2", "feed_forward": _feed_forward(width, layer["mlp"]), "feed_forward_name": "mlp",
            "feed_forward_post_norm": norm, "feed_forward_post_norm_name": "norm2b",
        })))
    # the order of runs: every run of a layer has a cache stream of its own; a pass of the repeated run starts with the input mix
    loop = config.loop
    runs = [(i, None) for i in range(count)]
    if loop is not None:
        runs = [(i, None) for i in range(loop["start"])]
        for t in range(loop["times"]):
            runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
        runs += [(i, None) for i in range(loop["stop"], count)]
    order, stream = [], 0
    for index, starts_pass in runs:
        if starts_pass is not None:
            layers.append(LayerSpec("loop", PartSpec("stream_input_mix", {"tensor": "loop.in", "size": width, "table": "embed", "vocab_size": config.vocab,
                                                                          "scale": config.embedding_scale, "turn": starts_pass})))
            order.append(OrderEntry(layer=len(layers) - 1, cache=stream))
            stream += 1
        order.append(OrderEntry(layer=index, cache=stream))
        stream += 1
    spec = ModelSpec(
        architecture="Redasun", hidden_size=width, vocab_size=config.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("positioned_embedding", {"vocab_size": config.vocab, "hidden_size": width, "tensor": "embed", "scale": config.embedding_scale}),
        layers=tuple(layers), order=tuple(order),
        final_norm=PartSpec("layernorm", {"size": width, "eps": eps, "suffix": "", "name": "final.norm"}),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "hidden_size": width, "tensor": "embed", "tied_to": None}),
    )
    spec.validate()
    return spec


REDASUN = Architecture(name="Redasun", config_class=RedasunConfig, build_spec=build_redasun_spec)
register_architecture(REDASUN, replace=True)
