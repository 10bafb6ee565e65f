"""RMSNorm, with the residual add fused in front of it; and the layer norm without a bias."""
from __future__ import annotations

import torch

from .. import ops
from .base import Norm, register_part
from .spec import PartSpec, TensorSpec


class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * weight, eps inside the root (src/operators.cpp:22-45).

    params: ``size``, ``eps``, optional ``suffix`` (what follows the prefix in the tensor's name, ".weight" unless given), optional
    ``offset`` (the weight is stored minus this number: 1.0 for a weight stored around zero; added once, in 32-bit, at load time).
    tensors: ``<prefix><suffix> [size]``.
    The statistics, the scale and the residual sum are 32-bit in both precisions;
    the weight is held in 32-bit (exact for a bfloat16 checkpoint).
    """

    capturable = True
    supports_lazy = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        if float(spec.get("offset", 0.0) or 0.0) != 0.0:
            return [TensorSpec(f"{prefix}{spec.get('suffix', '.weight')}", (spec["size"],), init="matrix", std=0.1)]   # stored around zero
        return [TensorSpec(f"{prefix}{spec.get('suffix', '.weight')}", (spec["size"],), init="norm", std=0.1)]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = weights.get(f"{prefix}{spec.get('suffix', '.weight')}", torch.float32).contiguous()
        offset = float(spec.get("offset", 0.0) or 0.0)
        if offset != 0.0:
            self.weight = (self.weight + offset).contiguous()

    def forward(self, residual, delta=None, rows=None, lazy: bool = False):
        """``lazy`` (and nothing to add): hand the norm on to the product that consumes it (ops.LazyNorm)."""
        if lazy and delta is None:
            handle = ops.LazyNorm(residual, self.weight, self.eps, rows, lambda: self.forward(residual, None, rows))
            if rows is None and self.runtime.dtype == torch.bfloat16:
                # where a product that completes the residual may leave this norm's input (ops.linear_accumulate(..., prepare=handle))
                ws = self.runtime.workspace
                handle.buffers = (ws.get("prepared_norm", residual.shape[0], self.size, torch.bfloat16),
                                  ws.get("prepared_squares", residual.shape[0], -(-self.size // 16), torch.float32))
            return handle
        count = residual.shape[0] if rows is None else rows.shape[0]
        out = self.runtime.workspace.get("normed" if rows is None else "normed_rows", count, self.size, self.runtime.dtype)
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows)
        return out


class LayerNorm(Norm):
    """y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * weight: a layer norm with a weight and no bias.

    params: ``size``, ``eps``, optional ``suffix`` (what follows the prefix in the tensor's name, ".weight" unless given).
    tensors: ``<prefix><suffix> [size]``.  Mean, variance, scale and the residual sum are 32-bit in both precisions; the weight is held
    in 32-bit.  ``forward`` adds ``delta`` into the stream first, as the RMS norm does; ``join`` is what a block calls that normalises a
    branch before it joins the stream: ``residual += self(y)``, and in the same kernel the next norm of the stream if one is named.
    """

    capturable = True
    supports_lazy = False
    centred = True
    groups = 1

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(f"{prefix}{spec.get('suffix', '.weight')}", (spec["size"],), init="norm", std=0.1)]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = weights.get(f"{prefix}{spec.get('suffix', '.weight')}", torch.float32).contiguous()

    def forward(self, residual, delta=None, rows=None, lazy: bool = False):
        if delta is not None:
            ops.add_(residual, delta)
        count = residual.shape[0] if rows is None else rows.shape[0]
        out = self.runtime.workspace.get("normed" if rows is None else "normed_rows", count, self.size, self.runtime.dtype)
        ops.branch_norm(residual, None, None, self.weight, out, self.eps, self.centred, rows, groups=self.groups)
        return out

    def join(self, residual, branch, following: "LayerNorm | None" = None):
        """``residual += self(branch)``; with ``following`` (a norm of this kind and eps) also returns ``following(residual)``, one kernel."""
        if following is None:
            ops.branch_norm(residual, branch, self.weight, None, None, self.eps, self.centred, groups=self.groups)
            return None
        out = self.runtime.workspace.get("normed", residual.shape[0], self.size, self.runtime.dtype)
        ops.branch_norm(residual, branch, self.weight, following.weight, out, self.eps, self.centred, groups=self.groups)
        return out


class GroupedRMSNorm(LayerNorm):
    """y = x / sqrt(mean(x^2) + eps) * weight over each of ``groups`` equal consecutive parts of a row, every part with a root mean
    square of its own (one group: the plain RMS norm).

    params: ``size``, ``eps``, ``groups``, optional ``suffix`` and ``scale`` (the weight is multiplied by it once, in 32-bit, at load time:
    a branch that joins the stream times a constant).  ``forward`` and ``join`` are the layer norm's: the norm of a branch, its sum
    into the 32-bit stream and the stream's next norm are one kernel."""

    centred = False

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.groups = int(spec.get("groups", 1) or 1)
        if self.size % self.groups:
            from ..errors import ConfigError

            raise ConfigError(f"{prefix}: a norm over {self.size} columns cannot have {self.groups} equal groups")
        scale = float(spec.get("scale", 1.0))
        if scale != 1.0:
            self.weight = (self.weight * scale).contiguous()


register_part("norm", "grouped_rmsnorm", GroupedRMSNorm)
register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
