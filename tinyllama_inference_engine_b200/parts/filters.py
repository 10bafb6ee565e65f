"""What a layer may put between a norm and the sublayer that reads it."""
from __future__ import annotations

import torch

from .. import ops
from .base import InputFilter, register_part
from .spec import PartSpec, TensorSpec


class CausalConvResidual(InputFilter):
    """y_t = x_t + sum_j w[:, j] x_(t - taps + 1 + j): a short causal convolution over time on every channel, added to its own input;
    zeros before a request's start, no bias.

    params: ``size`` (channels), ``taps``.  tensors: ``<prefix>`` [size, taps], the last column the current token's.  The last
    ``taps - 1`` inputs of a request are its state (32-bit, [taps - 1, size]); the sums are 32-bit.
    """

    capturable = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(prefix, (int(spec["size"]), int(spec["taps"])), std=0.3)]

    @classmethod
    def state_words(cls, spec: PartSpec) -> int:
        return (int(spec["taps"]) - 1) * int(spec["size"])

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.size, self.taps = int(spec["size"]), int(spec["taps"])
        self.weight = weights.get(prefix, torch.float32).contiguous()

    def forward(self, x, ctx, state, offset: int):
        out = self.runtime.workspace.get("filtered", x.shape[0], self.size, x.dtype)
        ops.conv_residual(x, self.weight, state, offset, ctx, out)
        return out


register_part("input_filter", "causal_conv_residual", CausalConvResidual)
