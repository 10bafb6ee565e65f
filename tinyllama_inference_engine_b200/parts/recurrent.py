"""Recurrent mixers: a state of fixed size per request instead of a cache that grows: a gated recurrence per channel, and four mixers
over a matrix of fast weights per head (the gated delta rule with a decay per key channel and with one per head, linear attention whose
forget gate also writes, a state-space layer with a scalar decay per head), which share one recurrence kernel."""
from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, LayerCache, Mixer, register_part
from .spec import PartSpec, TensorSpec


class MinGRU(Mixer):
    """A gated recurrence whose gates read only the current token, so a prompt portion is a scan and not a loop.

    With a = W_z h + b_z and u = W_x h + b_x, per channel: z = sigmoid(a); the candidate is u + 1/2 for u >= 0 and
    sigmoid(u) below; S_t = (1 - z_t) S_{t-1} + z_t cand_t from S = 0; the mixer's output is W_o (S_t * silu(W_g h_t)).

    params: ``hidden_size``, ``width`` (channels of the state).
    tensors: ``<prefix>.z``, ``<prefix>.x``, ``<prefix>.g`` [width, hidden], ``<prefix>.z.b``, ``<prefix>.x.b`` [width],
    ``<prefix>.o`` [hidden, width].  The three input products are stacked into one [3 width, hidden] at load time; biases,
    gates, candidate and state are 32-bit in both precisions, and the state lives in the request's slot of the cache
    manager's state group (zero when the request is admitted).
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, width = spec["hidden_size"], spec["width"]
        std = hidden ** -0.5
        return [
            TensorSpec(f"{prefix}.z", (width, hidden), std=std), TensorSpec(f"{prefix}.z.b", (width,), std=1.0),
            TensorSpec(f"{prefix}.x", (width, hidden), std=std), TensorSpec(f"{prefix}.x.b", (width,), std=0.5),
            TensorSpec(f"{prefix}.g", (width, hidden), std=std), TensorSpec(f"{prefix}.o", (hidden, width), std=width ** -0.5),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return CacheNeed("state", state_shape=(int(spec["width"]),))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden = int(spec["hidden_size"])
        self.width = int(spec["width"])
        dtype = runtime.dtype
        self.w_zxg = torch.cat([weights.get(f"{prefix}.{n}", dtype) for n in ("z", "x", "g")], dim=0).contiguous()
        self.bias_z = weights.get(f"{prefix}.z.b", torch.float32).contiguous()
        self.bias_x = weights.get(f"{prefix}.x.b", torch.float32).contiguous()
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        zxg = ws.get("recurrent_in", tokens, 3 * self.width, dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_zxg, zxg)
        else:
            ops.linear(x, self.w_zxg, zxg)
        gated = ws.get("recurrent_out", tokens, self.width, dtype)
        ops.mingru_scan(zxg, self.bias_z, self.bias_x, cache.state, ctx.seq_starts, ctx.state_slots, gated, ctx.max_q_len)
        if accumulate_into is not None:
            ops.linear_accumulate(gated, self.w_o, accumulate_into, prepare)
            return None
        out = ws.get("mixer_out", tokens, self.hidden, dtype)
        ops.linear(gated, self.w_o, out)
        return out


class ChannelDeltaRule(Mixer):
    """The gated delta rule with one decay per head and key channel: a matrix of fast weights per head that every token first
    lets decay, then corrects towards its value along its key, then reads with its query.

    Per token: q = W_q x, k = W_k x (``kv_heads`` heads of ``dim``; head h reads q/k head h // (heads / kv_heads)), v = W_v x (``heads`` of
    ``vdim``); each passes a short causal convolution over time per channel (``<tensor>.conv`` [channels, taps], the last column the
    current token's, zeros before a request's start) and silu; q and k become unit vectors per head (x / sqrt(sum x^2 + unit_eps)),
    q times dim^-1/2.  beta = sigmoid(W_b x) per head; decay g = exp(-exp(A_log_h) softplus(W_a2 W_a1 x + dt_bias)) per head and key
    channel.  Per head, in this order: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Each head's o is divided by
    its root mean square (``eps``), times ``<prefix>.norm`` [vdim], times sigmoid(W_g2 W_g1 x); then W_o.

    The state (32-bit, zero for a new request) is the heads' matrices and the convolution's last taps - 1 inputs, one flat vector
    in the request's state slot.  Everything after the projections is 32-bit.  The eight input products are one stacked product;
    the two second halves of the low-rank pairs are products of their own.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``key_dim``, ``value_dim``, ``taps``, ``decay_rank``, ``gate_rank``, ``eps``,
    ``unit_eps`` (1e-6).
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _sizes(cls, spec: PartSpec):
        return tuple(int(spec[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "key_dim", "value_dim", "taps", "decay_rank", "gate_rank"))

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, heads, kv, dim, vdim, taps, decay_rank, gate_rank = cls._sizes(spec)
        std = hidden ** -0.5
        return [
            TensorSpec(f"{prefix}.q", (kv * dim, hidden), std=std), TensorSpec(f"{prefix}.q.conv", (kv * dim, taps), std=taps ** -0.5),
            TensorSpec(f"{prefix}.k", (kv * dim, hidden), std=std), TensorSpec(f"{prefix}.k.conv", (kv * dim, taps), std=taps ** -0.5),
            TensorSpec(f"{prefix}.v", (heads * vdim, hidden), std=std), TensorSpec(f"{prefix}.v.conv", (heads * vdim, taps), std=taps ** -0.5),
            TensorSpec(f"{prefix}.b", (heads, hidden), std=std), TensorSpec(f"{prefix}.A_log", (heads,), std=0.5),
            TensorSpec(f"{prefix}.norm", (vdim,), init="norm", std=0.1),
            TensorSpec(f"{prefix}.a1", (decay_rank, hidden), std=std), TensorSpec(f"{prefix}.a2", (heads * dim, decay_rank), std=decay_rank ** -0.5),
            TensorSpec(f"{prefix}.dt_bias", (heads * dim,), std=1.0),
            TensorSpec(f"{prefix}.g1", (gate_rank, hidden), std=std), TensorSpec(f"{prefix}.g2", (heads * vdim, gate_rank), std=gate_rank ** -0.5),
            TensorSpec(f"{prefix}.o", (hidden, heads * vdim), std=(heads * vdim) ** -0.5),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, heads, kv, dim, vdim, taps, _, _ = cls._sizes(spec)
        words, _ = ops.delta_state_words(heads, dim, vdim, 2 * kv * dim + heads * vdim, taps)
        return CacheNeed("state", state_shape=(words,))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.decay_rank, self.gate_rank = self._sizes(spec)
        self.eps, self.unit_eps = float(spec["eps"]), float(spec.get("unit_eps", 1e-6))
        dtype = runtime.dtype
        self.channels = 2 * self.kv_heads * self.dim + self.heads * self.vdim
        _, self.conv_offset = ops.delta_state_words(self.heads, self.dim, self.vdim, self.channels, self.taps)
        self.w_in = torch.cat([weights.get(f"{prefix}.{n}", dtype) for n in ("q", "k", "v", "b", "a1", "g1")], dim=0).contiguous()
        self.beta_offset = self.channels
        self.a1_offset = self.beta_offset + self.heads
        self.g1_offset = self.a1_offset + self.decay_rank
        self.w_a2 = weights.get(f"{prefix}.a2", dtype).contiguous()
        self.w_g2 = weights.get(f"{prefix}.g2", dtype).contiguous()
        self.conv = torch.cat([weights.get(f"{prefix}.{n}.conv", torch.float32) for n in ("q", "k", "v")], dim=0).contiguous()
        self.a_log = weights.get(f"{prefix}.A_log", torch.float32).contiguous()
        self.dt_bias = weights.get(f"{prefix}.dt_bias", torch.float32).contiguous()
        self.out_weight = weights.get(f"{prefix}.norm", torch.float32).contiguous()
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        rows = ws.get("delta_in", tokens, self.w_in.shape[0], dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_in, rows)
        else:
            ops.linear(x, self.w_in, rows)
        decay_in = ws.get("delta_decay_in", tokens, self.heads * self.dim, dtype)
        gate = ws.get("delta_gate", tokens, self.heads * self.vdim, dtype)
        first, second = rows[:, self.a1_offset : self.g1_offset], rows[:, self.g1_offset :]   # the low-rank pairs' first halves, columns of the stacked product
        ops.linear(first, self.w_a2, decay_in)
        ops.linear(second, self.w_g2, gate)
        prep = ws.get("delta_prep", tokens, self.channels + self.heads + self.heads * self.dim, torch.float32)
        ops.delta_prepare(rows, self.beta_offset, decay_in, self.conv, self.a_log, self.dt_bias, cache.state, self.conv_offset, ctx, prep, self.heads,
                          self.kv_heads, self.dim, self.vdim, self.unit_eps, self.dim ** -0.5)
        read = ws.get("delta_read", tokens, self.heads * self.vdim, torch.float32)
        ops.delta_rule(prep, cache.state, ctx, read, self.heads, self.kv_heads, self.dim, self.vdim)
        gated = ws.get("recurrent_out", tokens, self.heads * self.vdim, dtype)
        ops.delta_gate_norm(read, gate, self.out_weight, gated, self.eps, self.heads, self.vdim)
        if accumulate_into is not None:
            ops.linear_accumulate(gated, self.w_o, accumulate_into, prepare)
            return None
        out = ws.get("mixer_out", tokens, self.hidden, dtype)
        ops.linear(gated, self.w_o, out)
        return out


class _MatrixRecurrence(Mixer):
    """What the mixers below share: a matrix of fast weights per head, [dim x vdim] in 32-bit in the request's state, that every token lets
    decay, writes to and reads, S <- diag(g) S + k u^T, o = S^T q, over the rows ``prep`` = [q | k | v | beta | g] that the mixer's own
    preparation leaves in 32-bit (``ops.delta_rule``: u = beta (v - S^T k) for the delta rule, u = beta v otherwise)."""

    capturable = True

    def _recur(self, prep, ctx, cache, heads, kv_heads, dim, vdim, plain):
        read = self.runtime.workspace.get("delta_read", prep.shape[0], heads * vdim, torch.float32)
        ops.delta_rule(prep, cache.state, ctx, read, heads, kv_heads, dim, vdim, plain=plain)
        return read

    def _project(self, gated, accumulate_into, prepare):
        if accumulate_into is not None:
            ops.linear_accumulate(gated, self.w_o, accumulate_into, prepare)
            return None
        out = self.runtime.workspace.get("mixer_out", gated.shape[0], self.hidden, self.runtime.dtype)
        ops.linear(gated, self.w_o, out)
        return out


class GatedDeltaRule(_MatrixRecurrence):
    """The gated delta rule with one decay per head.

    Per token: q = W_q x, k = W_k x (``kv_heads`` heads of ``dim``; head h reads q/k head h // (heads / kv_heads)), v = W_v x (``heads`` of ``vdim``);
    each passes a short causal convolution over time per channel (``<tensor>.conv`` [channels, taps], the last column the current token's,
    zeros before a request's start) and silu; q and k become unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times dim^-1/2.
    beta = sigmoid(W_b x) and g = exp(-exp(A_log_h) softplus(W_a x + dt_bias_h)), one each per head.  Per head, in this order:
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Each head's o is divided by its root mean square (``eps``), times
    ``<prefix>.norm`` [vdim], times silu(W_g x); then W_o.

    The state (32-bit, zero for a new request) is the heads' matrices and the convolution's last taps - 1 inputs.  Everything after the
    projections is 32-bit.  The six input products are one stacked product.
    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``key_dim``, ``value_dim``, ``taps``, ``eps``, ``unit_eps`` (1e-6).
    """

    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _sizes(cls, spec: PartSpec):
        return tuple(int(spec[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "key_dim", "value_dim", "taps"))

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, heads, kv, dim, vdim, taps = cls._sizes(spec)
        std = hidden ** -0.5
        return [
            TensorSpec(f"{prefix}.q", (kv * dim, hidden), std=std), TensorSpec(f"{prefix}.q.conv", (kv * dim, taps), std=taps ** -0.5),
            TensorSpec(f"{prefix}.k", (kv * dim, hidden), std=std), TensorSpec(f"{prefix}.k.conv", (kv * dim, taps), std=taps ** -0.5),
            TensorSpec(f"{prefix}.v", (heads * vdim, hidden), std=std), TensorSpec(f"{prefix}.v.conv", (heads * vdim, taps), std=taps ** -0.5),
            TensorSpec(f"{prefix}.b", (heads, hidden), std=std), TensorSpec(f"{prefix}.A_log", (heads,), std=0.5),
            TensorSpec(f"{prefix}.norm", (vdim,), init="norm", std=0.1), TensorSpec(f"{prefix}.a", (heads, hidden), std=std),
            TensorSpec(f"{prefix}.dt_bias", (heads,), std=1.0), TensorSpec(f"{prefix}.g", (heads * vdim, hidden), std=std),
            TensorSpec(f"{prefix}.o", (hidden, heads * vdim), std=(heads * vdim) ** -0.5),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, heads, kv, dim, vdim, taps = cls._sizes(spec)
        words, _ = ops.delta_state_words(heads, dim, vdim, 2 * kv * dim + heads * vdim, taps)
        return CacheNeed("state", state_shape=(words,))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim, self.taps = self._sizes(spec)
        self.eps, self.unit_eps = float(spec["eps"]), float(spec.get("unit_eps", 1e-6))
        dtype = runtime.dtype
        self.channels = 2 * self.kv_heads * self.dim + self.heads * self.vdim
        _, self.conv_offset = ops.delta_state_words(self.heads, self.dim, self.vdim, self.channels, self.taps)
        stacked = [weights.get(f"{prefix}.{n}", dtype) for n in ("q", "k", "v", "g", "b", "a")]
        self.gate_offset = self.channels
        self.beta_offset = self.gate_offset + self.heads * self.vdim
        self.decay_offset = self.beta_offset + self.heads
        width = self.decay_offset + self.heads
        if width % 8:   # rows of the stacked product start on 16-byte boundaries
            stacked.append(torch.zeros((8 - width % 8, self.hidden), dtype=dtype, device=stacked[0].device))
        self.w_in = torch.cat(stacked, dim=0).contiguous()
        self.conv = torch.cat([weights.get(f"{prefix}.{n}.conv", torch.float32) for n in ("q", "k", "v")], dim=0).contiguous()
        self.a_log = weights.get(f"{prefix}.A_log", torch.float32).contiguous()
        self.dt_bias = weights.get(f"{prefix}.dt_bias", torch.float32).contiguous()
        self.out_weight = weights.get(f"{prefix}.norm", torch.float32).contiguous()
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        rows = ws.get("delta_in", tokens, self.w_in.shape[0], dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_in, rows)
        else:
            ops.linear(x, self.w_in, rows)
        prep = ws.get("delta_prep", tokens, self.channels + self.heads + self.heads * self.dim, torch.float32)
        ops.delta_prepare(rows, self.beta_offset, rows[:, self.decay_offset : self.decay_offset + self.heads], self.conv, self.a_log, self.dt_bias, cache.state,
                          self.conv_offset, ctx, prep, self.heads, self.kv_heads, self.dim, self.vdim, self.unit_eps, self.dim ** -0.5, decay_per_head=True)
        read = self._recur(prep, ctx, cache, self.heads, self.kv_heads, self.dim, self.vdim, plain=False)
        gated = ws.get("recurrent_out", tokens, self.heads * self.vdim, dtype)
        ops.delta_gate_norm(read, rows[:, self.gate_offset : self.beta_offset], self.out_weight, gated, self.eps, self.heads, self.vdim, gate_kind="silu")
        return self._project(gated, accumulate_into, prepare)


class Hgrn2(_MatrixRecurrence):
    """Linear attention with one gate for forgetting and writing: what a channel of the state gives up, it takes from the new value.

    q = silu(W_q x) (``heads`` of ``dim``), v = W_v x (``heads`` of ``vdim``), f = l + (1 - l) sigmoid(W_f x + b_f) per head and channel with the
    stored lower bound l in [0, 1).  Per head S <- diag(f) S + (1 - f) v^T, o = S^T q (no key, no other scale).  Each head's o is divided by
    its root mean square over vdim (``eps``), times ``<prefix>.norm`` [vdim]; heads concatenated; W_o.  State (32-bit, zero for a new request):
    the heads' matrices.  Gates and everything after the projections are 32-bit.  q, f and v are one stacked product.
    params: ``hidden_size``, ``num_heads``, ``key_dim``, ``value_dim``, ``eps``.
    tensors: ``<prefix>.q``, ``<prefix>.f`` [heads dim, hidden], ``<prefix>.f.b``, ``<prefix>.lower`` [heads dim], ``<prefix>.v`` [heads vdim, hidden],
    ``<prefix>.norm`` [vdim], ``<prefix>.o`` [hidden, heads vdim].
    """

    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _sizes(cls, spec: PartSpec):
        return tuple(int(spec[k]) for k in ("hidden_size", "num_heads", "key_dim", "value_dim"))

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, heads, dim, vdim = cls._sizes(spec)
        std = hidden ** -0.5
        return [TensorSpec(f"{prefix}.q", (heads * dim, hidden), std=std), TensorSpec(f"{prefix}.f", (heads * dim, hidden), std=std),
                TensorSpec(f"{prefix}.f.b", (heads * dim,), std=1.0), TensorSpec(f"{prefix}.lower", (heads * dim,), init="uniform", std=0.9),
                TensorSpec(f"{prefix}.v", (heads * vdim, hidden), std=std), TensorSpec(f"{prefix}.norm", (vdim,), init="norm", std=0.1),
                TensorSpec(f"{prefix}.o", (hidden, heads * vdim), std=(heads * vdim) ** -0.5)]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, heads, dim, vdim = cls._sizes(spec)
        return CacheNeed("state", state_shape=(ops.delta_state_words(heads, dim, vdim, 0, 1)[0],))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.heads, self.dim, self.vdim = self._sizes(spec)
        self.eps = float(spec["eps"])
        dtype = runtime.dtype
        stacked = [weights.get(f"{prefix}.{n}", dtype) for n in ("q", "f", "v")]
        width = 2 * self.heads * self.dim + self.heads * self.vdim
        if width % 8:
            stacked.append(torch.zeros((8 - width % 8, self.hidden), dtype=dtype, device=stacked[0].device))
        self.w_in = torch.cat(stacked, dim=0).contiguous()
        self.f_bias = weights.get(f"{prefix}.f.b", torch.float32).contiguous()
        self.lower = weights.get(f"{prefix}.lower", torch.float32).contiguous()
        self.out_weight = weights.get(f"{prefix}.norm", torch.float32).contiguous()
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        rows = ws.get("hgrn2_in", tokens, self.w_in.shape[0], dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_in, rows)
        else:
            ops.linear(x, self.w_in, rows)
        prep = ws.get("hgrn2_prep", tokens, 3 * self.heads * self.dim + self.heads * self.vdim + self.heads, torch.float32)
        ops.hgrn2_prepare(rows, self.f_bias, self.lower, prep, self.heads, self.dim, self.vdim)
        read = self._recur(prep, ctx, cache, self.heads, self.heads, self.dim, self.vdim, plain=True)
        normed = ws.get("recurrent_out", tokens, self.heads * self.vdim, dtype)
        ops.delta_gate_norm(read, None, self.out_weight, normed, self.eps, self.heads, self.vdim, gate_kind=None)
        return self._project(normed, accumulate_into, prepare)


class StateSpaceDuality(_MatrixRecurrence):
    """A state-space layer with a scalar decay per head (the form that is also linear attention).

    W_in x = [z: inner | x: inner | B: G N | C: G N | dt: heads] with inner = heads * vdim; x, B and C pass a causal convolution per channel
    (``<prefix>.conv`` [inner + 2 G N, taps] with the bias ``<prefix>.conv.b``, the last column the current token's, zeros before a request's start)
    and silu; dt = softplus(dt + dt_bias) as it comes out, with no bounds put on it.  Per head h (group h // (heads / G)): S <- exp(-exp(A_log_h) dt) S + dt B x^T with S [N x vdim],
    y = S^T C + D_h x.  y (heads concatenated) times silu(z), then an RMS norm over each of ``norm_groups`` equal parts (``eps``), times
    ``<prefix>.norm`` [inner]; W_o.  State (32-bit, zero for a new request): the heads' matrices and the convolution's last taps - 1 inputs.
    Step sizes, decays, the recurrence, the gate and the norm are 32-bit.
    params: ``hidden_size``, ``num_heads``, ``value_dim``, ``state_dim`` (N), ``groups`` (G), ``taps``, ``norm_groups``, ``eps``.
    """

    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _sizes(cls, spec: PartSpec):
        return tuple(int(spec[k]) for k in ("hidden_size", "num_heads", "value_dim", "state_dim", "groups", "taps"))

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, heads, vdim, n, groups, taps = cls._sizes(spec)
        inner, channels = heads * vdim, heads * vdim + 2 * groups * n
        return [TensorSpec(f"{prefix}.in", (inner + channels + heads, hidden), std=hidden ** -0.5), TensorSpec(f"{prefix}.conv", (channels, taps), std=taps ** -0.5),
                TensorSpec(f"{prefix}.conv.b", (channels,), std=0.2), TensorSpec(f"{prefix}.dt_bias", (heads,), std=1.0), TensorSpec(f"{prefix}.A_log", (heads,), std=0.5),
                TensorSpec(f"{prefix}.D", (heads,), std=1.0), TensorSpec(f"{prefix}.norm", (inner,), init="norm", std=0.1),
                TensorSpec(f"{prefix}.o", (hidden, inner), std=inner ** -0.5)]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, heads, vdim, n, groups, taps = cls._sizes(spec)
        return CacheNeed("state", state_shape=(ops.delta_state_words(heads, n, vdim, heads * vdim + 2 * groups * n, taps)[0],))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.heads, self.vdim, self.n, self.groups, self.taps = self._sizes(spec)
        self.eps, self.norm_groups = float(spec["eps"]), int(spec.get("norm_groups", 1) or 1)
        self.out_scale = float(spec.get("out_scale", 1.0))
        dtype = runtime.dtype
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n
        _, self.conv_offset = ops.delta_state_words(self.heads, self.n, self.vdim, self.channels, self.taps)
        self.w_in = weights.get(f"{prefix}.in", dtype).contiguous()
        self.conv = weights.get(f"{prefix}.conv", torch.float32).contiguous()
        self.conv_bias = weights.get(f"{prefix}.conv.b", torch.float32).contiguous()
        self.a_log = weights.get(f"{prefix}.A_log", torch.float32).contiguous()
        self.dt_bias = weights.get(f"{prefix}.dt_bias", torch.float32).contiguous()
        self.skip = weights.get(f"{prefix}.D", torch.float32).contiguous()
        self.out_weight = weights.get(f"{prefix}.norm", torch.float32).contiguous()
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        rows = ws.get("ssd_in", tokens, self.w_in.shape[0], dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_in, rows)
        else:
            ops.linear(x, self.w_in, rows)
        gn = self.groups * self.n
        prep = ws.get("ssd_prep", tokens, 2 * gn + self.inner + self.heads + self.heads * self.n, torch.float32)
        ops.ssd_prepare(rows, self.conv, self.conv_bias, self.a_log, self.dt_bias, cache.state, self.conv_offset, ctx, prep, self.heads, self.groups, self.n, self.vdim)
        read = self._recur(prep, ctx, cache, self.heads, self.groups, self.n, self.vdim, plain=True)
        gated = ws.get("recurrent_out", tokens, self.inner, dtype)
        ops.ssd_finish(read, prep, 2 * gn, rows, self.skip, self.out_weight, gated, self.eps, self.heads, self.vdim, self.norm_groups)
        return self._project(gated, accumulate_into, prepare)


register_part("mixer", "gated_delta_rule", GatedDeltaRule)
register_part("mixer", "hgrn2", Hgrn2)
register_part("mixer", "state_space_duality", StateSpaceDuality)
register_part("mixer", "mingru", MinGRU)
register_part("mixer", "channel_delta_rule", ChannelDeltaRule)
