"""Kilurax as data: its configuration turned into a ModelSpec.

A decoder whose layers are listed one by one.  The embedding is a table row times a constant plus a row of a second table chosen by
the token and the one before it, under the model's norm.  The norm is an RMS norm over equal groups of a row.  A layer has such a
norm before each sublayer and another on the sublayer's output, which joins the stream times a constant; what a sublayer reads
first passes a short causal convolution over time that is added to its own input.  Three mixers: softmax attention (biased
projections, a partial rotation, grouped heads) added to a state-space layer's output on the same input; a linear-attention layer with one
gate for forgetting and writing; the gated delta rule with one decay per head.  The feed-forward is a mixture of experts chosen by a sigmoid router
whose scores multiply what the experts read, beside a shared expert.  The final norm, then a head of its own.
Tensor names: ``embed``, ``bigram``, ``embed.norm``, ``final.norm``, ``head``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``,
``l<i>.canon1``, ``l<i>.canon2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.  This file only names parts and sizes; every formula lives in the parts.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, OrderEntry, PartSpec
from .kilurax_config import KiluraxConfig

UNIT_EPS = 1e-6           # inside the root of the delta rule's unit norms
MAX_POSITIONS = 1 << 17   # the design has no table of positions: this only bounds a request's block table


def _attention(width: int, sizes: dict) -> PartSpec:
    return PartSpec("mixed_heads_attention", {
        "hidden_size": width, "num_heads": sizes["heads"], "num_kv_heads": sizes["kv_heads"], "key_dim": sizes["dim"], "value_dim": sizes["vdim"],
        "scale": sizes["scale"], "window": 0, "distance_slopes": None, "mix_heads": False, "output_gate": False, "biases": True,
        "rot_dims": sizes["rot"]["dims"], "rot_base": sizes["rot"]["base"], "out_buffer": "mixer_left",   # it runs beside another mixer
    })


def _state_space(width: int, sizes: dict, eps: float) -> PartSpec:
    return PartSpec("state_space_duality", {
        "hidden_size": width, "num_heads": sizes["heads"], "value_dim": sizes["vdim"], "state_dim": sizes["state"], "groups": sizes["groups"], "taps": sizes["conv"],
        "norm_groups": sizes["norm_groups"], "eps": eps,
    })


def _mixer(width: int, kind: str, sizes: dict, eps: float) -> PartSpec:
    if kind == "parallel":
        return PartSpec("parallel_mixers", {"hidden_size": width, "left": _attention(width, sizes["left"]), "right": _state_space(width, sizes["right"], eps),
                                            "left_scale": sizes["left_scale"], "right_scale": sizes["right_scale"]})
    if kind == "hgrn2":
        return PartSpec("hgrn2", {"hidden_size": width, "num_heads": sizes["heads"], "key_dim": sizes["dim"], "value_dim": sizes["vdim"], "eps": eps})
    return PartSpec("gated_delta_rule", {"hidden_size": width, "num_heads": sizes["heads"], "num_kv_heads": sizes["kv_heads"], "key_dim": sizes["dim"],
                                         "value_dim": sizes["vdim"], "taps": sizes["conv"], "eps": eps, "unit_eps": UNIT_EPS})


def _feed_forward(width: int, mlp) -> PartSpec | None:
    if mlp is None:
        return None
    shared = mlp.get("shared")
    return PartSpec("routed_experts", {
        "hidden_size": width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"], "expert_size": mlp["expert"]["ff"], "groups": 1, "keep_groups": 1,
        "route_scale": 1.0, "activation": "silu", "shared_size": shared["ff"] if shared else 0, "correction": False, "normalize": False, "weight_input": True,
    })


def build_kilurax_spec(config: KiluraxConfig) -> ModelSpec:
    width, eps, groups = config.width, config.norm_eps, config.norm_groups
    norm = PartSpec("grouped_rmsnorm", {"size": width, "eps": eps, "groups": groups, "suffix": ""})
    joining = PartSpec("grouped_rmsnorm", {"size": width, "eps": eps, "groups": groups, "suffix": "", "scale": config.residual_mult})   # a branch joins times the constant
    conv = PartSpec("causal_conv_residual", {"size": width, "taps": config.canon_taps}) if config.canon_taps else None
    layers = []
    for index, layer in enumerate(config.layers):
        layers.append(LayerSpec(f"l{index}", PartSpec("sandwich_norm", {
            "mixer_norm": norm, "mixer_norm_name": "norm1", "mixer_filter": conv, "mixer_filter_name": "canon1",
            "mixer": _mixer(width, layer["type"], layer["mixer"], eps), "mixer_name": "mix", "mixer_post_norm": joining, "mixer_post_norm_name": "norm1b",
            "feed_forward_norm": norm, "feed_forward_norm_name": "norm2", "feed_forward_filter": conv, "feed_forward_filter_name": "canon2",
            "feed_forward": _feed_forward(width, layer["mlp"]), "feed_forward_name": "mlp", "feed_forward_post_norm": joining, "feed_forward_post_norm_name": "norm2b",
        })))
    bigram = config.bigram
    spec = ModelSpec(
        architecture="Kilurax", hidden_size=width, vocab_size=config.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("pair_embedding", {
            "vocab_size": config.vocab, "hidden_size": width, "tensor": "embed", "scale": config.embedding_scale,
            "pairs": None if bigram is None else {"tensor": "bigram", "buckets": bigram["buckets"], "mul_prev": bigram["mul_prev"], "mul_cur": bigram["mul_cur"]},
            "norm": {"tensor": "embed.norm", "eps": eps, "groups": groups},
        }),
        layers=tuple(layers), order=tuple(OrderEntry(layer=i, cache=i) for i in range(len(layers))),
        final_norm=PartSpec("grouped_rmsnorm", {"size": width, "eps": eps, "groups": groups, "suffix": "", "name": "final.norm"}),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "hidden_size": width, "tensor": "head", "tied_to": None}),
    )
    spec.validate()
    return spec


KILURAX = Architecture(name="Kilurax", config_class=KiluraxConfig, build_spec=build_kilurax_spec)
register_architecture(KILURAX, replace=True)
