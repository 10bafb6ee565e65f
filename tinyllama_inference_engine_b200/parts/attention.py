"""Attention over the paged cache: grouped-query attention with a position encoding; attention whose heads are biased by
distance, mixed before the softmax and gated after it; attention with normalised queries and keys under a window that keeps
the first tokens; and latent attention, which caches one small vector per token for all heads."""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .base import CacheNeed, LayerCache, Mixer, build_part, register_part
from .spec import PartSpec, TensorSpec


class Attention(Mixer):
    """q, k, v projections, position encoding, cache write, attention, output projection.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``position`` (a PartSpec), optional ``window`` (0 = every earlier token) and
    ``scale`` (default head_dim ** -0.5).
    tensors: ``<prefix>.{q,k,v}_proj.weight [heads * head_dim, hidden]``,
    ``<prefix>.o_proj.weight [hidden, num_heads * head_dim]``; no biases
    (src/model_config.cpp:81-95).

    The reference issues three projections (src/cuda/model.cu:412-421); here their
    weights are stacked once at load time and one product yields ``[q | k | v]``.
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, d = spec["hidden_size"], spec["head_dim"]
        q, kv = spec["num_heads"] * d, spec["num_kv_heads"] * d
        return [
            TensorSpec(f"{prefix}.q_proj.weight", (q, hidden)),
            TensorSpec(f"{prefix}.k_proj.weight", (kv, hidden)),
            TensorSpec(f"{prefix}.v_proj.weight", (kv, hidden)),
            TensorSpec(f"{prefix}.o_proj.weight", (hidden, q)),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return CacheNeed("pages", kv_heads=spec["num_kv_heads"], head_dim=spec["head_dim"], window=int(spec.get("window", 0) or 0))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden = int(spec["hidden_size"])
        self.q_heads = int(spec["num_heads"])
        self.kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.window = int(spec.get("window", 0) or 0)
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        dtype = runtime.dtype
        self.w_qkv = torch.cat([weights.get(f"{prefix}.{n}_proj.weight", dtype) for n in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = weights.get(f"{prefix}.o_proj.weight", dtype).contiguous()
        self.position = build_part("position", spec["position"], prefix, weights, runtime)
        self.qkv_width = (self.q_heads + 2 * self.kv_heads) * self.head_dim

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        qkv = ws.get("qkv", tokens, self.qkv_width, dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_qkv, qkv)
        else:
            ops.linear(x, self.w_qkv, qkv)
        table = self.position.rotary_table()
        if table is None:
            self.position.apply(qkv, ctx, self.q_heads, self.kv_heads, self.head_dim)
            inv_freq, rotary_dim = None, 0
        else:
            inv_freq, rotary_dim = table
        mixed = ws.get("attention", tokens, self.q_heads * self.head_dim, dtype)
        ops.attention_step(qkv, ctx.positions, ctx.token_seq, cache.block_table, inv_freq, rotary_dim, cache.pages, mixed,
                           self.q_heads, self.kv_heads, self.head_dim, cache.page_size, self.window, self.scale,
                           write_cache=cache.writes, batch=ctx)
        if accumulate_into is not None:
            ops.linear_accumulate(mixed, self.w_o, accumulate_into, prepare)
            return None
        out = ws.get("mixer_out", tokens, self.hidden, dtype)
        ops.linear(mixed, self.w_o, out)
        return out


class MixedHeadsAttention(Mixer):
    """Grouped heads without a rotation: positions enter through a distance bias, the heads' scores are mixed by a learned matrix
    before the softmax, and the concatenated heads pass an output gate before the output projection.

    Score of query head g at position i for key j: (q_g . k_j) * scale - slope_g (i - j); head h sees sum_g M[h, g] score_g;
    key j is visible while 0 <= i - j (and i - j < window, if there is a window); an ordinary softmax over the visible keys;
    out = W_o (concat_h(softmax_h . v) * sigmoid(W_gate x)).

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads`` (query head h reads key/value head h // (heads / kv heads)),
    ``key_dim`` (queries and keys), ``value_dim``, ``scale``, ``window`` (0: every earlier token), ``distance_slopes``
    (one slope per head, or None for no bias), ``mix_heads`` (tensor ``<prefix>.talk`` [heads, heads], row h mixing into head h),
    ``output_gate`` (tensor ``<prefix>.g`` [heads * value_dim, hidden]); optional ``biases`` (q, k, v and the output projection have one each, the
    tensor's name with ``.b`` added, added in 32-bit) and ``rot_dims`` / ``rot_base`` (of every q and k head the first ``rot_dims`` columns turn, column i
    with column i + rot_dims / 2, by position * rot_base^(-2i / rot_dims); keys are cached turned); optional ``out_buffer`` (the workspace buffer
    the output is written to, "mixer_out" unless given: a mixer that runs beside another one needs a buffer of its own).
    tensors: ``<prefix>.q`` [heads * key_dim, hidden], ``<prefix>.k`` [kv * key_dim, hidden], ``<prefix>.v`` [kv * value_dim, hidden],
    ``<prefix>.o`` [hidden, heads * value_dim].  q, k, v and the gate are one stacked product.  Keys and values are
    two planes of a page (of different widths if ``key_dim != value_dim``); scores, mix, softmax and the gate are 32-bit.
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _sizes(cls, spec: PartSpec) -> tuple[int, int, int, int, int]:
        return int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["key_dim"]), int(spec["value_dim"])

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, heads, kv, key_dim, value_dim = cls._sizes(spec)
        std = hidden ** -0.5
        specs = [TensorSpec(f"{prefix}.q", (heads * key_dim, hidden), std=std), TensorSpec(f"{prefix}.k", (kv * key_dim, hidden), std=std),
                 TensorSpec(f"{prefix}.v", (kv * value_dim, hidden), std=std)]
        if spec.get("mix_heads"):
            specs.append(TensorSpec(f"{prefix}.talk", (heads, heads), std=heads ** -0.5))
        if spec.get("output_gate"):
            specs.append(TensorSpec(f"{prefix}.g", (heads * value_dim, hidden), std=std))
        specs.append(TensorSpec(f"{prefix}.o", (hidden, heads * value_dim), std=(heads * value_dim) ** -0.5))
        if spec.get("biases"):
            specs += [TensorSpec(f"{prefix}.q.b", (heads * key_dim,), std=0.5), TensorSpec(f"{prefix}.k.b", (kv * key_dim,), std=0.5),
                      TensorSpec(f"{prefix}.v.b", (kv * value_dim,), std=0.5), TensorSpec(f"{prefix}.o.b", (hidden,), std=0.5)]
        return specs

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, _, kv, key_dim, value_dim = cls._sizes(spec)
        return CacheNeed("pages", window=int(spec.get("window", 0) or 0), planes=((kv, key_dim), (kv, value_dim)))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.heads, self.kv_heads, self.key_dim, self.value_dim = self._sizes(spec)
        self.window = int(spec.get("window", 0) or 0)
        self.scale = float(spec["scale"]) if spec.get("scale") is not None else self.key_dim ** -0.5
        dtype = runtime.dtype
        stacked = [weights.get(f"{prefix}.{n}", dtype) for n in ("q", "k", "v")]
        self.k_offset = self.heads * self.key_dim
        self.v_offset = self.k_offset + self.kv_heads * self.key_dim
        self.gate_offset = -1
        if spec.get("output_gate"):
            self.gate_offset = self.v_offset + self.kv_heads * self.value_dim
            stacked.append(weights.get(f"{prefix}.g", dtype))
        self.w_in = torch.cat(stacked, dim=0).contiguous()
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()
        slopes = spec.get("distance_slopes")
        self.slopes = None if slopes is None else torch.tensor([float(v) for v in slopes], dtype=torch.float32, device=runtime.device)
        self.mix = weights.get(f"{prefix}.talk", torch.float32).contiguous() if spec.get("mix_heads") else None
        self.folded_slopes = ops.fast.folded_slopes(self.slopes, self.mix) if self.slopes is not None and self.slopes.is_cuda else None
        self.biases = self.out_bias = None
        if spec.get("biases"):
            self.biases = tuple(weights.get(f"{prefix}.{n}.b", torch.float32).contiguous() for n in ("q", "k", "v"))
            self.out_bias = weights.get(f"{prefix}.o.b", torch.float32).contiguous()
        self.rot_dims = int(spec.get("rot_dims", 0) or 0)
        self.inv_freq = None
        if self.rot_dims:
            # frequencies in 64-bit, rounded once: the angle is float(position) * frequency in 32-bit inside the kernel
            exponent = -2.0 * np.arange(self.rot_dims // 2, dtype=np.float64) / float(self.rot_dims)
            self.inv_freq = torch.from_numpy(np.power(float(spec["rot_base"]), exponent).astype(np.float32)).to(runtime.device)
        if self.biases is not None or self.rot_dims:
            # the kernels of few rows take neither: such a layer is handed finished tensors and returns its output
            self.accepts_lazy_norm = self.fuses_residual_add = self.prepares_next_norm = False

    def adds_to_residual(self, rows: int) -> bool:
        return self.out_bias is None and ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        rows = ws.get("qkv_gate", tokens, self.w_in.shape[0], dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_in, rows)
        else:
            ops.linear(x, self.w_in, rows)
        if self.biases is not None or self.rot_dims:
            ops.rotary_store_planes(rows, self.k_offset, self.v_offset, self.biases, self.inv_freq, self.rot_dims, ctx.positions, ctx.token_seq, cache, self.heads,
                                    self.kv_heads, self.key_dim, self.value_dim)
        elif cache.writes:
            ops.store_kv_planes(rows, self.k_offset, self.v_offset, ctx.positions, ctx.token_seq, cache, self.kv_heads, self.key_dim, self.value_dim)
        mixed = ws.get("attention", tokens, self.heads * self.value_dim, dtype)
        ops.mixed_heads_attention(rows, self.gate_offset, ctx.positions, ctx.token_seq, cache, self.slopes, self.mix, mixed, self.heads, self.kv_heads,
                                  self.key_dim, self.value_dim, self.window, self.scale, batch=ctx, folded_slopes=self.folded_slopes)
        if accumulate_into is not None:
            ops.linear_accumulate(mixed, self.w_o, accumulate_into, prepare)
            return None
        out = ws.get(self.spec.get("out_buffer", "mixer_out"), tokens, self.hidden, dtype)
        ops.linear(mixed, self.w_o, out)
        if self.out_bias is not None:
            ops.add_bias(out, self.out_bias)
        return out


class NormedKeyAttention(Mixer):
    """Grouped heads without positions: queries and keys are divided by their root mean square per head before the product.

    score = (q^ . k^) * scale with x^ = x / sqrt(mean(x^2) + eps); query position i sees key j if j <= i and (i - j < window or
    j < keep_first) (``window`` 0: every earlier key); an ordinary softmax; head h's output is multiplied by sigmoid((W_g x)_h), one
    number per head, if ``head_gate``; out = W_o concat(heads).  With ``values`` = "keys" the values are the keys as projected,
    before the norm, and there is no value projection (then value_dim = key_dim); with "projection" there is ``<prefix>.v``.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``key_dim``, ``value_dim``, ``scale``, ``eps``, ``window``, ``keep_first``,
    ``values``, ``head_gate``.  tensors: ``<prefix>.q`` [heads * key_dim, hidden], ``<prefix>.k`` [kv * key_dim, hidden], ``<prefix>.v``
    [kv * value_dim, hidden] (if projected), ``<prefix>.g`` [heads, hidden] (if gated), ``<prefix>.o`` [hidden, heads * value_dim].
    The cache holds two planes per token: the normalised keys and the values; a window group keeps the pages of the first
    ``keep_first`` tokens.  Norms, scores, softmax and the gate are 32-bit.
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _sizes(cls, spec: PartSpec) -> tuple[int, int, int, int, int]:
        return int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["key_dim"]), int(spec["value_dim"])

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, heads, kv, key_dim, value_dim = cls._sizes(spec)
        std = hidden ** -0.5
        specs = [TensorSpec(f"{prefix}.q", (heads * key_dim, hidden), std=std), TensorSpec(f"{prefix}.k", (kv * key_dim, hidden), std=std)]
        if spec.get("values", "projection") != "keys":
            specs.append(TensorSpec(f"{prefix}.v", (kv * value_dim, hidden), std=std))
        if spec.get("head_gate"):
            specs.append(TensorSpec(f"{prefix}.g", (heads, hidden), std=std))
        return specs + [TensorSpec(f"{prefix}.o", (hidden, heads * value_dim), std=(heads * value_dim) ** -0.5)]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, _, kv, key_dim, value_dim = cls._sizes(spec)
        window = int(spec.get("window", 0) or 0)
        return CacheNeed("pages", window=window, planes=((kv, key_dim), (kv, value_dim)), keep_first=int(spec.get("keep_first", 0) or 0) if window > 0 else 0)

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.heads, self.kv_heads, self.key_dim, self.value_dim = self._sizes(spec)
        self.window = int(spec.get("window", 0) or 0)
        self.keep_first = int(spec.get("keep_first", 0) or 0)
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.values_are_keys = spec.get("values", "projection") == "keys"
        if self.values_are_keys and self.value_dim != self.key_dim:
            from ..errors import ConfigError

            raise ConfigError(f"{prefix}: values that are the keys have the keys' width ({self.key_dim}), not {self.value_dim}")
        dtype = runtime.dtype
        stacked = [weights.get(f"{prefix}.q", dtype), weights.get(f"{prefix}.k", dtype)]
        self.k_offset = self.heads * self.key_dim
        width = self.k_offset + self.kv_heads * self.key_dim
        self.v_offset = self.k_offset
        if not self.values_are_keys:
            self.v_offset = width
            stacked.append(weights.get(f"{prefix}.v", dtype))
            width += self.kv_heads * self.value_dim
        self.gate_offset = -1
        if spec.get("head_gate"):
            self.gate_offset = width
            stacked.append(weights.get(f"{prefix}.g", dtype))
            width += self.heads
        if width % 8:   # rows of the stacked product start on 16-byte boundaries (what the tensor-core attention kernels read them by)
            stacked.append(torch.zeros((8 - width % 8, self.hidden), dtype=dtype, device=stacked[0].device))
        self.w_in = torch.cat(stacked, dim=0).contiguous()
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        rows = ws.get("qk_gate", tokens, self.w_in.shape[0], dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_in, rows)
        else:
            ops.linear(x, self.w_in, rows)
        ops.normed_store(rows, self.k_offset, self.v_offset, ctx.positions, ctx.token_seq, cache, self.heads, self.kv_heads, self.key_dim, self.value_dim, self.eps)
        mixed = ws.get("attention", tokens, self.heads * self.value_dim, dtype)
        ops.mixed_heads_attention(rows, self.gate_offset, ctx.positions, ctx.token_seq, cache, None, None, mixed, self.heads, self.kv_heads, self.key_dim,
                                  self.value_dim, self.window, self.scale, batch=ctx, keep_first=self.keep_first, gate_per_head=True)
        if accumulate_into is not None:
            ops.linear_accumulate(mixed, self.w_o, accumulate_into, prepare)
            return None
        out = ws.get("mixer_out", tokens, self.hidden, dtype)
        ops.linear(mixed, self.w_o, out)
        return out


class LatentAttention(Mixer):
    """Attention whose keys and values are expanded from one latent vector per token, with a rotated key part shared by all heads
    and, optionally, a sink in the softmax.

    Per token: q = W_q x, head by head [plain | rot]; W_dkv x = [rank | rot]; the latent c is the first ``rank`` columns under an RMS norm
    with a weight, the last ``rot`` columns are one key part for every head, rotated by position like the queries' rot parts (pairs
    (2i, 2i + 1) of the first ``rot_dims`` columns by angle position * base^(-2i / rot_dims)).  Head h has keys [W_uk,h c | shared part]
    and values W_uv,h c; causal; softmax whose denominator also holds exp(sink_h) if ``sink``; out = W_o concat(heads).

    Only [c | rotated part] is cached (one plane, one head, rank + rot wide).  The products with W_uk and W_uv are moved across the
    attention: q~_h = W_uk,h^T q_plain,h, so that the score is [q~_h | q_rot,h] . [c_j | rot_j] and head h's weighted sum of latents,
    sum_j p_j c_j, is multiplied by W_uv,h afterwards.  All heads then read the same cached rows: attention with one key/value
    head whose values are the first ``rank`` columns of its keys.

    params: ``hidden_size``, ``num_heads``, ``plain_dim``, ``rot_dim``, ``value_dim``, ``rank``, ``scale``, ``eps``, ``rot_dims``, ``rot_base``,
    ``sink``.  tensors: ``<prefix>.q`` [heads * (plain + rot), hidden], ``<prefix>.dkv`` [rank + rot, hidden], ``<prefix>.dkv.norm`` [rank],
    ``<prefix>.uk`` [heads * plain, rank], ``<prefix>.uv`` [heads * value_dim, rank], ``<prefix>.sink`` [heads], ``<prefix>.o`` [hidden, heads * value_dim].
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, heads, plain, rot, vdim, rank = (int(spec[k]) for k in ("hidden_size", "num_heads", "plain_dim", "rot_dim", "value_dim", "rank"))
        std = hidden ** -0.5
        specs = [TensorSpec(f"{prefix}.q", (heads * (plain + rot), hidden), std=std), TensorSpec(f"{prefix}.dkv", (rank + rot, hidden), std=std),
                 TensorSpec(f"{prefix}.dkv.norm", (rank,), init="norm", std=0.1), TensorSpec(f"{prefix}.uk", (heads * plain, rank), std=rank ** -0.5),
                 TensorSpec(f"{prefix}.uv", (heads * vdim, rank), std=rank ** -0.5)]
        if spec.get("sink"):
            specs.append(TensorSpec(f"{prefix}.sink", (heads,), std=1.0))
        return specs + [TensorSpec(f"{prefix}.o", (hidden, heads * vdim), std=(heads * vdim) ** -0.5)]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return CacheNeed("pages", planes=((1, int(spec["rank"]) + int(spec["rot_dim"])),))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.heads, self.plain, self.rot, self.vdim, self.rank = (int(spec[k]) for k in ("hidden_size", "num_heads", "plain_dim", "rot_dim", "value_dim", "rank"))
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.rot_dims = int(spec["rot_dims"])
        dtype = runtime.dtype
        self.w_in = torch.cat([weights.get(f"{prefix}.q", dtype), weights.get(f"{prefix}.dkv", dtype)], dim=0).contiguous()
        self.latent_offset = self.heads * (self.plain + self.rot)
        self.latent_weight = weights.get(f"{prefix}.dkv.norm", torch.float32).contiguous()
        # W_uk per head, transposed: [heads, rank, plain], the operand of q~ = W_uk^T q; W_uv per head [heads, vdim, rank]
        self.w_uk_t = weights.get(f"{prefix}.uk", dtype).view(self.heads, self.plain, self.rank).transpose(1, 2).contiguous()
        self.w_uv = weights.get(f"{prefix}.uv", dtype).view(self.heads, self.vdim, self.rank).contiguous()
        self.sinks = weights.get(f"{prefix}.sink", torch.float32).contiguous() if spec.get("sink") else None
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()
        # frequencies in 64-bit, rounded once: the angle is float(position) * frequency in 32-bit inside the kernel
        exponent = -2.0 * np.arange(self.rot_dims // 2, dtype=np.float64) / float(self.rot_dims)
        self.inv_freq = torch.from_numpy(np.power(float(spec["rot_base"]), exponent).astype(np.float32)).to(runtime.device)

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        rows = ws.get("latent_in", tokens, self.w_in.shape[0], dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_in, rows)
        else:
            ops.linear(x, self.w_in, rows)
        width = self.rank + self.rot
        flat_queries = ws.get("latent_queries", tokens, self.heads * width, dtype)
        ops.latent_store(rows, self.latent_offset, self.latent_weight, self.eps, self.inv_freq, self.rot_dims, ctx.positions, ctx.token_seq, cache, flat_queries,
                         self.heads, self.plain, self.rot, self.rank)
        queries = flat_queries.view(tokens, self.heads, width)
        per_head = rows[:, : self.latent_offset].view(tokens, self.heads, self.plain + self.rot)
        ops.head_linear(per_head[:, :, : self.plain], self.w_uk_t, queries[:, :, : self.rank])
        summed = ws.get("latent_sums", tokens, self.heads * self.rank, dtype)
        ops.mixed_heads_attention(flat_queries, -1, ctx.positions, ctx.token_seq, cache, None, None, summed, self.heads, 1, width,
                                  self.rank, 0, self.scale, batch=ctx, sinks=self.sinks, values_in_keys=True)
        mixed = ws.get("attention", tokens, self.heads * self.vdim, dtype)
        ops.head_linear(summed.view(tokens, self.heads, self.rank), self.w_uv, mixed.view(tokens, self.heads, self.vdim))
        if accumulate_into is not None:
            ops.linear_accumulate(mixed, self.w_o, accumulate_into, prepare)
            return None
        out = ws.get("mixer_out", tokens, self.hidden, dtype)
        ops.linear(mixed, self.w_o, out)
        return out


class DifferentialAttention(Mixer):
    """Attention whose every head takes the difference of two softmax maps over the same values.

    q has ``num_heads`` x 2 vectors of ``key_dim`` and k has ``num_kv_heads`` x 2, head by head as [map 1 | map 2]; v has ``num_kv_heads``
    vectors of ``value_dim``.  Every q and k vector passes an RMS norm with a weight ([key_dim], one for q and one for k, shared by all
    heads and maps) and then a rotation of its first ``rot_dims`` columns (column i with column i + rot_dims / 2, by position *
    rot_base^(-2 i / rot_dims)).  Per head: a_m = softmax(scale q_m . k_m) v (causal) for m = 1, 2, o = a_1 - lambda a_2 with
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + ``diff`` (one number for the layer, from four stored vectors), then
    o / sqrt(mean(o^2) + eps) * (1 - ``diff``); W_o on the concatenated heads.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``key_dim``, ``value_dim``, ``scale``, ``eps``, ``diff``, ``rot_dims``, ``rot_base``.
    tensors: ``<prefix>.q`` [2 heads key_dim, hidden], ``<prefix>.k`` [2 kv key_dim, hidden], ``<prefix>.v`` [kv value_dim, hidden], ``<prefix>.q.norm``,
    ``<prefix>.k.norm`` [key_dim], ``<prefix>.{lq1,lk1,lq2,lk2}`` [key_dim], ``<prefix>.o`` [hidden, heads value_dim].  q, k and v are one stacked
    product.  The cache holds a key plane of 2 kv vectors per token (normalised and rotated) and a value plane of kv vectors.
    Norms, angles, scores, softmax, the difference and its norm are 32-bit.
    """

    capturable = True

    @classmethod
    def _sizes(cls, spec: PartSpec) -> tuple[int, int, int, int, int]:
        return int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["key_dim"]), int(spec["value_dim"])

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, heads, kv, dim, vdim = cls._sizes(spec)
        std = hidden ** -0.5
        specs = [TensorSpec(f"{prefix}.q", (2 * heads * dim, hidden), std=std), TensorSpec(f"{prefix}.k", (2 * kv * dim, hidden), std=std),
                 TensorSpec(f"{prefix}.v", (kv * vdim, hidden), std=std), TensorSpec(f"{prefix}.q.norm", (dim,), init="norm", std=0.1),
                 TensorSpec(f"{prefix}.k.norm", (dim,), init="norm", std=0.1)]
        specs += [TensorSpec(f"{prefix}.{name}", (dim,), std=0.1) for name in ("lq1", "lk1", "lq2", "lk2")]
        return specs + [TensorSpec(f"{prefix}.o", (hidden, heads * vdim), std=(heads * vdim) ** -0.5)]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, _, kv, dim, vdim = cls._sizes(spec)
        return CacheNeed("pages", planes=((2 * kv, dim), (kv, vdim)))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim = self._sizes(spec)
        self.scale, self.eps, self.diff = float(spec["scale"]), float(spec["eps"]), float(spec["diff"])
        self.rot_dims = int(spec.get("rot_dims", 0) or 0)
        dtype = runtime.dtype
        stacked = [weights.get(f"{prefix}.{n}", dtype) for n in ("q", "k", "v")]
        self.k_offset = 2 * self.heads * self.dim
        self.v_offset = self.k_offset + 2 * self.kv_heads * self.dim
        width = self.v_offset + self.kv_heads * self.vdim
        if width % 8:   # rows of the stacked product start on 16-byte boundaries
            stacked.append(torch.zeros((8 - width % 8, self.hidden), dtype=dtype, device=stacked[0].device))
        self.w_in = torch.cat(stacked, dim=0).contiguous()
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()
        self.q_weight = weights.get(f"{prefix}.q.norm", torch.float32).contiguous()
        self.k_weight = weights.get(f"{prefix}.k.norm", torch.float32).contiguous()
        # lambda: one number for the layer, worked out once in 32-bit
        l = {name: weights.get(f"{prefix}.{name}", torch.float32) for name in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = float(torch.exp((l["lq1"] * l["lk1"]).sum()) - torch.exp((l["lq2"] * l["lk2"]).sum())) + self.diff
        # frequencies in 64-bit, rounded once: the angle is float(position) * frequency in 32-bit inside the kernel
        exponent = -2.0 * np.arange(self.rot_dims // 2, dtype=np.float64) / float(max(self.rot_dims, 1))
        self.inv_freq = torch.from_numpy(np.power(float(spec.get("rot_base", 10000.0)), exponent).astype(np.float32)).to(runtime.device)

    def forward(self, x, ctx, cache: LayerCache):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        rows = ws.get("diff_qkv", tokens, self.w_in.shape[0], dtype)
        ops.linear(x, self.w_in, rows)
        ops.diff_store(rows, self.k_offset, self.v_offset, self.q_weight, self.k_weight, self.eps, self.inv_freq, self.rot_dims, ctx.positions, ctx.token_seq, cache,
                       self.heads, self.kv_heads, self.dim, self.vdim)
        mixed = ws.get("attention", tokens, self.heads * self.vdim, dtype)
        ops.diff_attention(rows, ctx.positions, ctx.token_seq, cache, mixed, self.heads, self.kv_heads, self.dim, self.vdim, self.scale, self.lam, self.eps,
                           1.0 - self.diff, batch=ctx)
        out = ws.get("mixer_out", tokens, self.hidden, dtype)
        ops.linear(mixed, self.w_o, out)
        return out


register_part("mixer", "attention", Attention)
register_part("mixer", "differential_attention", DifferentialAttention)
register_part("mixer", "mixed_heads_attention", MixedHeadsAttention)
register_part("mixer", "normed_key_attention", NormedKeyAttention)
register_part("mixer", "latent_attention", LatentAttention)
