"""Feed-forwards: the gated one, and the plain one of two products with an activation between them."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import ConfigError
from .base import FeedForward, register_part
from .spec import PartSpec, TensorSpec


class GatedMLP(FeedForward):
    """down( act(gate(x)) * up(x) ) with act = SiLU (src/model.cpp:187-203, src/operators.cpp:148-164).

    params: ``hidden_size``, ``intermediate_size``, ``activation`` ("silu"; "gelu_tanh": gelu in its tanh form; or "clamped_sigmoid": with g = min(gate, limit) and
    u = clamp(up, -limit, limit) the product is g * sigmoid(alpha * g) * (u + shift); params ``limit``, ``alpha``, ``shift``),
    optional ``names`` = (gate, up, down) tensor suffixes in full.
    tensors: ``<prefix>.{gate,up}_proj.weight [inter, hidden]``,
    ``<prefix>.down_proj.weight [hidden, inter]``.  gate and up are stacked at load
    time into one ``[2 * inter, hidden]`` product; the activation and the product with
    ``up`` are computed in 32-bit.
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _names(cls, spec: PartSpec, prefix: str) -> tuple[str, str, str]:
        gate, up, down = spec.get("names") or ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
        return f"{prefix}.{gate}", f"{prefix}.{up}", f"{prefix}.{down}"

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, inter = spec["hidden_size"], spec["intermediate_size"]
        gate, up, down = cls._names(spec, prefix)
        if spec.get("names"):
            return [TensorSpec(gate, (inter, hidden), std=hidden ** -0.5), TensorSpec(up, (inter, hidden), std=hidden ** -0.5), TensorSpec(down, (hidden, inter), std=inter ** -0.5)]
        return [TensorSpec(gate, (inter, hidden)), TensorSpec(up, (inter, hidden)), TensorSpec(down, (hidden, inter))]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.activation = spec.get("activation", "silu")
        if self.activation not in ("silu", "gelu_tanh", "clamped_sigmoid"):
            raise ConfigError(f"gated_mlp has no activation {spec.get('activation')!r}")
        if self.activation == "clamped_sigmoid":
            self.limit, self.alpha, self.shift = float(spec["limit"]), float(spec["alpha"]), float(spec["shift"])
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        dtype = runtime.dtype
        gate, up, down = self._names(spec, prefix)
        self.w_gate_up = torch.cat([weights.get(gate, dtype), weights.get(up, dtype)], dim=0).contiguous()
        self.w_down = weights.get(down, dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_down)

    def forward(self, x, ctx, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        act = ws.get("activated", tokens, self.inter, dtype)
        if self.activation == "clamped_sigmoid" and tokens <= ops.fused_rows_limit(dtype, act.device):
            # few rows: the clamps, the gate and the shift are applied in the stacked product's epilogue
            clamp = (self.limit, self.alpha, self.shift)
            if isinstance(x, ops.LazyNorm):
                ops.norm_linear(x, self.w_gate_up, act, gated=True, clamp=clamp)
            else:
                ops.linear_gated(x, self.w_gate_up, act, clamp=clamp)
        elif self.activation == "clamped_sigmoid":
            # the stacked product, then the clamps, the gate and the shift in one row-wise kernel (32-bit inside)
            gate_up = ws.get("gate_up", tokens, 2 * self.inter, dtype)
            if isinstance(x, ops.LazyNorm):
                ops.norm_linear(x, self.w_gate_up, gate_up)
            else:
                ops.linear(x, self.w_gate_up, gate_up)
            ops.clamped_gate_mul(gate_up, act, self.limit, self.alpha, self.shift)
        elif self.activation == "gelu_tanh":
            # few rows: the gate in the stacked product's epilogue; otherwise the product, then the gate in a row-wise kernel (32-bit inside)
            ops.linear_gated(x.tensor() if isinstance(x, ops.LazyNorm) else x, self.w_gate_up, act, activation="gelu_tanh")
        elif tokens <= ops.fused_rows_limit(dtype, act.device):
            # few rows: the gate is applied in the first product's epilogue, the residual add in the second's
            if isinstance(x, ops.LazyNorm):
                ops.norm_linear(x, self.w_gate_up, act, gated=True)
            else:
                ops.linear_gated(x, self.w_gate_up, act)
        elif dtype == torch.bfloat16:
            ops.linear_gated(x.tensor() if isinstance(x, ops.LazyNorm) else x, self.w_gate_up, act)   # picks the fused kernel for its size
        else:
            if isinstance(x, ops.LazyNorm):
                x = x.tensor()
            gate_up = ws.get("gate_up", tokens, 2 * self.inter, dtype)
            ops.linear(x, self.w_gate_up, gate_up)
            ops.silu_mul(gate_up, act)
        if accumulate_into is not None:
            ops.linear_accumulate(act, self.w_down, accumulate_into, prepare)
            return None
        out = ws.get("ff_out", tokens, self.hidden, dtype)
        ops.linear(act, self.w_down, out)
        return out


class DenseMLP(FeedForward):
    """down( act(up(x)) ), no gate and no biases.

    params: ``hidden_size``, ``intermediate_size``, ``activation`` ("relu_squared", "gelu_tanh" or "silu"; ops.ACTIVATIONS),
    optional ``up_name`` / ``down_name`` (the tensors are ``<prefix>.<name>``: "up" and "down" unless given).
    The activation is computed in 32-bit on the first product's (rounded) output.  With few rows the norm in front and the
    activation behind are applied inside the first product and the residual add inside the second, as the gated feed-forward does.
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _names(cls, spec: PartSpec, prefix: str) -> tuple[str, str]:
        return f"{prefix}.{spec.get('up_name', 'up')}", f"{prefix}.{spec.get('down_name', 'down')}"

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, inter = spec["hidden_size"], spec["intermediate_size"]
        up, down = cls._names(spec, prefix)
        return [TensorSpec(up, (inter, hidden), std=hidden ** -0.5), TensorSpec(down, (hidden, inter), std=inter ** -0.5)]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.activation = spec.get("activation", "relu_squared")
        if self.activation not in ops.ACTIVATIONS:
            raise ConfigError(f"dense_mlp has no activation {self.activation!r}; known: {sorted(ops.ACTIVATIONS)}")
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        up, down = self._names(spec, prefix)
        self.w_up = weights.get(up, runtime.dtype).contiguous()
        self.w_down = weights.get(down, runtime.dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_down)

    def forward(self, x, ctx, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        act = ws.get("activated", tokens, self.inter, dtype)
        ops.linear_activated(x, self.w_up, act, self.activation)   # few rows: norm, product and activation are one kernel
        if accumulate_into is not None:
            ops.linear_accumulate(act, self.w_down, accumulate_into, prepare)
            return None
        out = ws.get("ff_out", tokens, self.hidden, dtype)
        ops.linear(act, self.w_down, out)
        return out


class RoutedExperts(FeedForward):
    """A mixture of experts: every token goes through ``top`` of ``experts`` small gated feed-forwards, chosen by a router, and
    (optionally) through a shared one that every token uses.

    Router: z = W_router x and s = sigmoid(z) in 32-bit; an expert's choice score is s plus a stored correction, its weight uses s
    alone.  Experts form ``groups`` equal groups of neighbours; a group's score is the sum of its two largest choice scores, and only
    experts of the ``keep_groups`` best groups can be chosen.  The ``top`` largest choice scores are chosen; their weights are
    s / (sum of the chosen s + 1e-20) * ``route_scale``.  out = sum_k weight_k expert_k(x) + shared(x).
    ``normalize`` False: the weights are the chosen experts' scores as they are (times ``route_scale``).  ``weight_input`` True: the weight
    multiplies what the expert reads and not what it returns, out = sum_k expert_k(weight_k x) + shared(x).

    params: ``hidden_size``, ``experts``, ``top``, ``expert_size`` (an expert's inner width), ``groups``, ``keep_groups``, ``route_scale``,
    ``activation`` ("silu" or "gelu_tanh"), ``shared_size`` (0 or None: no shared expert), ``correction`` (whether the tensor exists),
    ``normalize`` (True), ``weight_input`` (False).
    tensors: ``<prefix>.router`` [experts, hidden], ``<prefix>.correction`` [experts], ``<prefix>.e<i>.{gate,up,down}``,
    ``<prefix>.shared.{gate,up,down}``.  The experts' gate and up rows are stacked per expert at load time, [experts, 2 ff, hidden].
    """

    capturable = True

    @classmethod
    def _shared_spec(cls, spec: PartSpec):
        size = int(spec.get("shared_size") or 0)
        if size <= 0:
            return None
        return PartSpec("gated_mlp", {"hidden_size": spec["hidden_size"], "intermediate_size": size, "activation": spec.get("activation", "silu"), "names": ("gate", "up", "down")})

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, ff = int(spec["hidden_size"]), int(spec["expert_size"])
        specs = []
        for e in range(int(spec["experts"])):
            specs += [TensorSpec(f"{prefix}.e{e}.gate", (ff, hidden), std=hidden ** -0.5), TensorSpec(f"{prefix}.e{e}.up", (ff, hidden), std=hidden ** -0.5),
                      TensorSpec(f"{prefix}.e{e}.down", (hidden, ff), std=ff ** -0.5)]
        specs.append(TensorSpec(f"{prefix}.router", (int(spec["experts"]), hidden), std=hidden ** -0.5))
        if spec.get("correction", True):
            specs.append(TensorSpec(f"{prefix}.correction", (int(spec["experts"]),), std=0.1))
        shared = cls._shared_spec(spec)
        if shared is not None:
            specs += GatedMLP.tensor_specs(shared, f"{prefix}.shared")
        return specs

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.experts, self.top, self.ff = (int(spec[k]) for k in ("hidden_size", "experts", "top", "expert_size"))
        self.groups, self.keep = int(spec.get("groups", 1) or 1), int(spec.get("keep_groups", 1) or 1)
        self.route_scale = float(spec.get("route_scale", 1.0))
        self.activation = spec.get("activation", "silu")
        self.normalize, self.weight_input = bool(spec.get("normalize", True)), bool(spec.get("weight_input", False))
        if self.experts % self.groups or not 0 < self.keep <= self.groups or not 0 < self.top <= self.keep * (self.experts // self.groups):
            raise ConfigError(f"{prefix}: {self.experts} experts in {self.groups} groups of which {self.keep} are kept cannot give {self.top} per token")
        if self.activation not in ops.GATE_KINDS:
            raise ConfigError(f"{prefix}: experts have no activation {self.activation!r}")
        dtype = runtime.dtype
        self.w_gate_up = torch.stack([torch.cat([weights.get(f"{prefix}.e{e}.gate", dtype), weights.get(f"{prefix}.e{e}.up", dtype)], dim=0) for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([weights.get(f"{prefix}.e{e}.down", dtype) for e in range(self.experts)]).contiguous()
        self.router = weights.get(f"{prefix}.router", torch.float32).contiguous()
        self.correction = weights.get(f"{prefix}.correction", torch.float32).contiguous() if spec.get("correction", True) else None
        shared = self._shared_spec(spec)
        self.shared = None if shared is None else GatedMLP(shared, f"{prefix}.shared", weights, runtime)

    def forward(self, x, ctx):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        ids = ws.get("expert_ids", tokens, self.top, torch.int32)
        weights = ws.get("expert_weights", tokens, self.top, torch.float32)
        ops.moe_route(x, self.router, self.correction, ids, weights, self.groups, self.keep, self.route_scale, normalize=self.normalize)
        shared = None if self.shared is None else self.shared.forward(x, ctx)
        out = ws.get("routed_out", tokens, self.hidden, dtype)
        ops.moe_experts(x, self.w_gate_up, self.w_down, ids, weights, shared, out, self.activation, batch=ctx, weight_input=self.weight_input)
        return out


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "routed_experts", RoutedExperts)
register_part("feed_forward", "dense_mlp", DenseMLP)
