"""Host wrappers of the engine's CUDA kernels.

Every function here launches a hand-written sm_100a kernel on the current CUDA
stream.  There is no CPU fallback and no library model code behind them: tensors
must live on a CUDA device, and a missing compiler or a failed build raises
``KernelError``.  Matrix products of the bfloat16 path may go to the vendor library
(as the reference's do, src/cuda/kernels.cu:342-368) until the engine's own
tensor-core kernel covers the shape; the 32-bit path always uses the engine's own
32-bit product.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..errors import KernelError
from .build import build_library, load_library

CORE_SOURCES = ["elementwise.cu", "rowwise.cu", "norm_branch.cu", "rope_cache.cu", "attention_generic.cu", "gemm_fp32.cu", "sampling.cu"]
RECURRENT_SOURCES = ["recurrent.cu"]              # compiled when a model with a recurrent mixer is first stepped
MIXED_ATTENTION_SOURCES = ["attention_mixed.cu"]   # likewise for attention with a distance bias, mixed heads or an output gate
DELTA_RULE_SOURCES = ["delta_rule.cu"]             # likewise for the gated delta rule
DIFF_ATTENTION_SOURCES = ["attention_diff.cu"]     # likewise for differential attention
MOE_SOURCES = ["moe.cu", "moe_grouped.cu", "moe_grouped_tc.cu"]   # likewise for a feed-forward of routed experts
SEQUENCE_SOURCES = ["sequence_filters.cu"]         # likewise for an embedding that reads the token before, a convolution in front of a sublayer
_F32, _BF16 = 0, 1
launch_count = 0  # kernels of this engine launched by this process (a claim the bench reports)


def core():
    lib = load_library("tlie_core", CORE_SOURCES)
    if not getattr(lib, "_tlie_typed", False):
        lib.tlie_uniform_from.restype = c_float
        lib.tlie_uniform_from.argtypes = [c_longlong, c_longlong]
        lib._tlie_typed = True
    return lib


def build_all() -> list:
    """Compile every kernel set (used by the build check); returns the library paths."""
    return [build_library("tlie_core", CORE_SOURCES), build_library("tlie_recurrent", RECURRENT_SOURCES),
            build_library("tlie_attention_mixed", MIXED_ATTENTION_SOURCES), build_library(f"tlie_delta_rule_l{DELTA_LANES}", DELTA_RULE_SOURCES, {"TLIE_DELTA_LANES": DELTA_LANES}),
            build_library("tlie_attention_diff", DIFF_ATTENTION_SOURCES), build_library("tlie_moe", MOE_SOURCES),
            build_library("tlie_sequence", SEQUENCE_SOURCES)] + fast.build_all()


def _code(tensor: torch.Tensor) -> int:
    if tensor.dtype == torch.float32:
        return _F32
    if tensor.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {tensor.dtype}", code="invalid_dtype")


def _ptr(tensor: torch.Tensor | None) -> c_void_p:
    if tensor is None:
        return c_void_p(0)
    if not tensor.is_cuda:
        raise KernelError("this engine has no CPU path: a kernel was given a tensor that is not on a CUDA device")
    if not tensor.is_contiguous():
        raise KernelError("kernels take contiguous tensors")
    return c_void_p(tensor.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> c_void_p:
    """The handle of torch's current stream on the current device.

    Every kernel launch asks for it; ``torch.cuda.current_stream()`` builds a Stream object each time (several microseconds, a
    fifth of the host time of a short prompt step), the two calls used here only read the handle."""
    if _raw_stream is not None and _device_index is not None:
        return c_void_p(_raw_stream(_device_index()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(status: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if status != 0:
        raise KernelError(f"{what} failed to launch: CUDA error {status}")


def _i32(tensor: torch.Tensor | None, what: str) -> c_void_p:
    if tensor is not None and tensor.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {tensor.dtype}", code="invalid_dtype")
    return _ptr(tensor)


# --- the device's error word -------------------------------------------------------------
# Kernels that can notice a fault without a host in the loop record it in one int32 per device: bit 0, a bounded wait
# inside a tensor-core kernel gave up (its results are garbage); bit 1, a token id outside the vocabulary reached the
# embedding (row 0 was read instead).  The engine reads the word wherever it synchronises with the device anyway.
_error_flags: dict[torch.device, torch.Tensor] = {}
DEVICE_ERRORS = {1: "a bounded wait inside a tensor-core kernel gave up; the step's results are not valid",
                 2: "a token id outside the vocabulary reached the embedding kernel (non-finite logits upstream?)",
                 4: "a position beyond the table of learned position vectors reached the embedding kernel"}


def error_flag(device: torch.device) -> torch.Tensor:
    """The device's error word (int32 [1]); kernels set bits in it, ``raise_for_error_word`` names and clears them."""
    device = torch.device(device)
    if device not in _error_flags:
        _error_flags[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[device]


def raise_for_error_word(word: int, device: torch.device) -> None:
    """Raise KernelError if ``word`` (a host copy of the device's error word) has a bit set, clearing the word on the device."""
    if word:
        error_flag(device).zero_()
        reasons = [text for bit, text in DEVICE_ERRORS.items() if word & bit] or [f"unknown error bits {word:#x}"]
        raise KernelError("the device reported: " + "; ".join(reasons))


def check_device_errors(device: torch.device) -> None:
    """Read the device's error word (this synchronises) and raise if a kernel reported a fault."""
    device = torch.device(device)
    if device in _error_flags:
        raise_for_error_word(int(_error_flags[device].item()), device)


# --- rows --------------------------------------------------------------------------------
def embedding(table: torch.Tensor, ids: torch.Tensor, residual: torch.Tensor) -> None:
    """residual[t] = float(table[ids[t]]); an id outside the table reads row 0 and sets bit 1 of the device's error word."""
    rows, hidden = residual.shape
    if table.shape[1] != hidden:
        raise KernelError("embedding: the table's width is not the residual's", code="invalid_shape")
    _check(core().tlie_embedding(_code(table), _ptr(table), _i32(ids, "ids"), _ptr(residual), c_int(rows), c_int(hidden), c_int(table.shape[0]),
                                 _ptr(error_flag(residual.device)), _stream()), "embedding")


def embedding_positions(table, place_table, ids, positions, norm_weight, eps: float, residual, scale: float = 1.0) -> None:
    """residual[t] = norm(float(table[ids[t]]) * scale + float(place_table[positions[t]])), all in 32-bit, in one kernel.

    ``place_table`` (learned vectors by position) and ``norm_weight`` (an RMS norm with ``eps`` inside the root) may each be None.
    A position beyond the table reads its last row and sets bit 2 of the device's error word."""
    rows, hidden = residual.shape
    if table.shape[1] != hidden or (place_table is not None and (place_table.shape[1] != hidden or place_table.dtype != table.dtype)):
        raise KernelError("embedding_positions: the tables' widths and dtypes must be the residual's width and each other's", code="invalid_shape")
    if residual.dtype != torch.float32 or (norm_weight is not None and (norm_weight.dtype != torch.float32 or norm_weight.numel() != hidden)):
        raise KernelError("embedding_positions: the residual stream and the norm weight are 32-bit", code="invalid_dtype")
    _check(core().tlie_embedding_positions(_code(table), _ptr(table), _ptr(place_table), _i32(ids, "ids"), _i32(positions, "positions"), _ptr(norm_weight),
                                           c_float(eps), c_float(scale), _ptr(residual), c_int(rows), c_int(hidden), c_int(table.shape[0]),
                                           c_int(0 if place_table is None else place_table.shape[0]), _ptr(error_flag(residual.device)), _stream()),
           "embedding_positions")


ACTIVATIONS = {"relu_squared": 0, "gelu_tanh": 1, "silu": 2}


def activation(kind: str, x, out) -> None:
    """out = act(x) element by element, 32-bit inside (``out`` may be ``x``): the square of relu, gelu in its tanh form
    0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))), or silu."""
    if kind not in ACTIVATIONS:
        raise KernelError(f"no activation {kind!r}; known: {sorted(ACTIVATIONS)}", code="invalid_argument")
    if out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("activation: the output must have the input's shape and dtype", code="invalid_shape")
    _check(core().tlie_activation(_code(x), c_int(ACTIVATIONS[kind]), _ptr(x), _ptr(out), c_longlong(x.numel()), _stream()), "activation")


def add_rmsnorm(residual, delta, weight, eps: float, out, rows=None) -> None:
    """Optional ``residual += delta`` in 32-bit, then ``out = rmsnorm(residual) * weight``.

    With ``rows`` (int32) only those rows are normalised (and ``delta`` must be None).
    """
    if residual.dtype != torch.float32 or weight.dtype != torch.float32:
        raise KernelError("the residual stream and norm weights are 32-bit", code="invalid_dtype")
    if rows is not None and delta is not None:
        raise KernelError("add_rmsnorm cannot add a delta while gathering rows")
    out_rows, hidden = out.shape
    if weight.numel() != hidden or residual.shape[1] != hidden:
        raise KernelError("add_rmsnorm: widths differ", code="invalid_shape")
    if delta is not None and (delta.shape != residual.shape or delta.dtype != out.dtype):
        raise KernelError("add_rmsnorm: delta must match the residual's shape and the output's dtype", code="invalid_shape")
    _check(
        core().tlie_add_rmsnorm(_code(out), _ptr(residual), _ptr(delta), _i32(rows, "rows"), _ptr(weight), c_float(eps), _ptr(out), c_int(out_rows), c_int(hidden), _stream()),
        "add_rmsnorm",
    )


def add_(residual, delta) -> None:
    _check(core().tlie_add(_code(delta), _ptr(residual), _ptr(delta), c_longlong(residual.numel()), _stream()), "add")


def silu_mul(gate_up, out) -> None:
    rows, inter = out.shape
    if gate_up.shape != (rows, 2 * inter) or gate_up.dtype != out.dtype:
        raise KernelError("silu_mul: gate_up must be [rows, 2 * inter] of the output's dtype", code="invalid_shape")
    _check(core().tlie_silu_mul(_code(out), _ptr(gate_up), _ptr(out), c_int(rows), c_int(inter), _stream()), "silu_mul")


GATE_KINDS = {"silu": 0, "gelu_tanh": 1}


def gate_mul(gate_up, out, kind: str = "silu") -> None:
    """out = act(gate) * up for the two halves of ``gate_up``'s rows, 32-bit inside; ``kind``: "silu" or "gelu_tanh"."""
    rows, inter = out.shape
    if gate_up.shape != (rows, 2 * inter) or gate_up.dtype != out.dtype or kind not in GATE_KINDS:
        raise KernelError("gate_mul: gate_up must be [rows, 2 * inter] of the output's dtype, kind one of " + ", ".join(GATE_KINDS), code="invalid_shape")
    _check(core().tlie_gate_mul(_code(out), _ptr(gate_up), _ptr(out), c_int(rows), c_int(inter), c_int(GATE_KINDS[kind]), _stream()), "gate_mul")


def branch_norm(residual, y, post_weight, next_weight, out, eps: float, centred: bool = True, rows=None, groups: int = 1) -> None:
    """One kernel around a residual branch: ``residual += norm(y) * post_weight`` (if ``y`` is given), then
    ``out = norm(residual[rows]) * next_weight`` (if ``out`` is given; ``rows`` None: every row in order, and only then may ``y`` be given).
    ``centred``: the layer norm without a bias, (x - mean) / sqrt(mean((x - mean)^2) + eps); else x / sqrt(mean(x^2) + eps).
    ``groups``: the statistics are taken over each of that many equal consecutive parts of a row.
    The stream, the statistics and the weights are 32-bit; ``y`` and ``out`` share a dtype."""
    width = residual.shape[1]
    if groups < 1 or width % groups:
        raise KernelError(f"branch_norm: a row of {width} cannot be cut into {groups} equal parts", code="invalid_shape")
    count = residual.shape[0] if rows is None else rows.shape[0]
    if residual.dtype != torch.float32 or (y is not None and (y.shape != residual.shape or rows is not None)) or (out is not None and out.shape != (count, width)):
        raise KernelError("branch_norm: a 32-bit stream [T, width], y of its shape, out [rows, width]", code="invalid_shape")
    for weight in (post_weight, next_weight):
        if weight is not None and (weight.dtype != torch.float32 or weight.numel() != width):
            raise KernelError("branch_norm: norm weights are 32-bit [width]", code="invalid_shape")
    if y is not None and out is not None and y.dtype != out.dtype:
        raise KernelError("branch_norm: y and out share a dtype", code="invalid_dtype")
    if y is None and out is None:
        return
    _check(core().tlie_branch_norm(_code(y if y is not None else out), _ptr(residual), _ptr(y), _ptr(post_weight if y is not None else None),
                                   _ptr(next_weight if out is not None else None), _ptr(out), _i32(rows, "rows"), c_float(eps), c_int(1 if centred else 0),
                                   c_int(count), c_int(width), c_int(groups), _stream()), "branch_norm")


def stream_with_embedding(residual, table, ids, scale: float, out) -> None:
    """out[t] = [residual[t] | table[ids[t]] * scale], rounded to ``out``'s dtype (the table's): the stream beside the embedding's output."""
    rows, width = residual.shape
    if residual.dtype != torch.float32 or table.shape[1] != width or out.shape != (rows, 2 * width) or out.dtype != table.dtype:
        raise KernelError("stream_with_embedding: a 32-bit stream [T, width], a table [vocab, width], out [T, 2 width] of the table's dtype", code="invalid_shape")
    _check(core().tlie_stream_with_embedding(_code(out), _ptr(residual), _ptr(table), _i32(ids, "ids"), c_float(scale), _ptr(out), c_int(rows), c_int(width),
                                             c_int(table.shape[0]), _ptr(error_flag(residual.device)), _stream()), "stream_with_embedding")


def add_row_vector(residual, delta, vector) -> None:
    """residual[t] += delta[t] (if given) + vector, in 32-bit: a learned vector joins every row of the stream."""
    rows, hidden = residual.shape
    if residual.dtype != torch.float32 or vector.dtype != torch.float32 or vector.numel() != hidden or (delta is not None and delta.shape != residual.shape):
        raise KernelError("add_row_vector: a 32-bit residual [rows, hidden], a 32-bit vector [hidden], a delta of the residual's shape", code="invalid_shape")
    _check(core().tlie_add_row_vector(_code(delta) if delta is not None else _F32, _ptr(residual), _ptr(delta), _ptr(vector), c_int(rows), c_int(hidden), _stream()),
           "add_row_vector")


def complete_and_round(residual, delta, out) -> None:
    """residual += delta (if given), then out = the residual in ``out``'s dtype: the finished stream as a product's operand."""
    if residual.dtype != torch.float32 or out.shape != residual.shape or (delta is not None and (delta.shape != residual.shape or delta.dtype != out.dtype)):
        raise KernelError("complete_and_round: the residual is 32-bit; delta and out have its shape and one dtype", code="invalid_shape")
    _check(core().tlie_complete_and_round(_code(out), _ptr(residual), _ptr(delta), _ptr(out), c_longlong(residual.numel()), _stream()), "complete_and_round")


def clamped_gate_mul(gate_up, out, limit: float, alpha: float, shift: float) -> None:
    """out = g sigmoid(alpha g) (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit), for gate_up = [gate | up]."""
    rows, inter = out.shape
    if gate_up.shape != (rows, 2 * inter) or gate_up.dtype != out.dtype:
        raise KernelError("clamped_gate_mul: gate_up must be [rows, 2 * inter] of the output's dtype", code="invalid_shape")
    _check(core().tlie_clamped_gate_mul(_code(out), _ptr(gate_up), _ptr(out), c_int(rows), c_int(inter), c_float(limit), c_float(alpha), c_float(shift), _stream()),
           "clamped_gate_mul")


def scale_rows(x, factor: float) -> None:
    """x *= factor in place (32-bit)."""
    if x.dtype != torch.float32:
        raise KernelError("scale_rows takes a 32-bit tensor", code="invalid_dtype")
    _check(core().tlie_scale_rows(_ptr(x), c_float(factor), c_longlong(x.numel()), _stream()), "scale_rows")


def gather_gated(z, table, ids, out, offset: int) -> None:
    """out[t, d] = gelu_tanh(z[t, d]) * table[ids[t], offset + d]: a slice of a second token table, gated."""
    rows, dim = out.shape
    if z.shape != out.shape or z.dtype != out.dtype or table.dtype != out.dtype or table.dim() != 2:
        raise KernelError("gather_gated: z, out [rows, dim] and the table are of one dtype", code="invalid_shape")
    _check(core().tlie_gather_gated(_code(out), _ptr(z), _ptr(table), _i32(ids, "ids"), _ptr(out), c_int(rows), c_int(dim), c_int(table.shape[1]), c_int(offset),
                                    c_int(table.shape[0]), _stream()), "gather_gated")


def unit_norm_add(residual, y, weight, eps: float) -> None:
    """residual[t] += y[t] / sqrt(mean(y[t]^2) + eps) * weight, statistics and sum in 32-bit."""
    rows, hidden = residual.shape
    if residual.dtype != torch.float32 or weight.dtype != torch.float32 or weight.numel() != hidden or y.shape != residual.shape:
        raise KernelError("unit_norm_add: a 32-bit residual and weight, y of the residual's shape", code="invalid_shape")
    _check(core().tlie_unit_norm_add(_code(y), _ptr(residual), _ptr(y), _ptr(weight), c_float(eps), c_int(rows), c_int(hidden), _stream()), "unit_norm_add")


# --- matrix products --------------------------------------------------------------------
HEAD_LINEAR_LIBRARY_ROWS = 64    # from this many bfloat16 rows on the per-head product is one batched library product


def head_linear(x, weight, out) -> None:
    """out[t, h, :] = weight[h] . x[t, h, :] for every head: x [T, H, K] and out [T, H, N] may be views with strides of their own
    (last axis contiguous), weight [H, N, K] contiguous.  32-bit sums, ascending k (a row's bits depend on the row alone) in the
    engine's own kernel; bfloat16 steps of many rows go to the library's batched product, as the other products of their size do."""
    rows, heads, k_in = x.shape
    n_out = weight.shape[1]
    if weight.shape != (heads, n_out, k_in) or out.shape != (rows, heads, n_out) or x.stride(2) != 1 or out.stride(2) != 1 or not weight.is_contiguous():
        raise KernelError("head_linear: x [T, H, K], weight [H, N, K], out [T, H, N] with contiguous last axes", code="invalid_shape")
    if x.dtype != weight.dtype or out.dtype != x.dtype:
        raise KernelError("head_linear: one dtype for x, weight and out", code="invalid_dtype")
    if not x.is_cuda:
        raise KernelError("this engine has no CPU path: a kernel was given a tensor that is not on a CUDA device")
    if x.dtype == torch.bfloat16 and rows >= HEAD_LINEAR_LIBRARY_ROWS:
        torch.bmm(x.transpose(0, 1), weight.transpose(1, 2), out=out.transpose(0, 1))
        return
    _check(core().tlie_head_linear(_code(x), c_void_p(x.data_ptr()), c_longlong(x.stride(0)), c_longlong(x.stride(1)), _ptr(weight), c_void_p(out.data_ptr()),
                                   c_longlong(out.stride(0)), c_longlong(out.stride(1)), c_int(rows), c_int(heads), c_int(n_out), c_int(k_in), _stream()), "head_linear")


def linear(x, weight, out) -> None:
    """out[M, N] = x[M, K] . weight[N, K]^T in the tensors' dtype (32-bit accumulation); ``x`` may be a run of columns of wider rows."""
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"linear: shapes {tuple(x.shape)} x {tuple(weight.shape)}^T -> {tuple(out.shape)} do not fit", code="invalid_shape")
    if x.dtype == torch.float32:
        if weight.dtype != torch.float32 or out.dtype != torch.float32:
            raise KernelError("linear: the 32-bit path takes 32-bit weights and outputs", code="invalid_dtype")
        if not x.is_cuda or x.stride(1) != 1:
            raise KernelError("linear: x must be on a CUDA device with contiguous rows")
        _check(core().tlie_gemm_nt_f32(c_void_p(x.data_ptr()), _ptr(weight), _ptr(out), c_int(M), c_int(N), c_int(K), c_longlong(x.stride(0)), _stream()), "gemm_nt_f32")
        return
    fast.linear_bf16(x, weight, out)


def fused_rows_limit(dtype: torch.dtype, device: torch.device) -> int:
    """Up to how many rows a step may use the fused decode kernels (0: never, as in the 32-bit path)."""
    if dtype != torch.bfloat16 or device.type != "cuda":
        return 0
    return fast.FUSED_MAX_ROWS


# A product that completes the residual leaves the next norm's input for the product after it, from this many rows on
# (measured per decode step of the 1.1B shapes: 2 % slower with 1 or 2 rows, 2 to 3 % faster with 4 to 8).
use_prepared_norms = True
PREPARED_NORM_MIN_ROWS = 3


class LazyNorm:
    """A normalised activation that is not computed yet: rmsnorm(residual[rows]) * weight.

    A product that can apply the norm while it loads its operand takes this in the place of a tensor
    (``norm_linear``); anything else calls ``tensor()``.  ``prepared``: set by the product that completed the residual
    (``linear_accumulate(..., prepare=this)``) to (bfloat16(residual * weight), sums of squares per 16 columns), which
    ``norm_linear`` then reads instead of working them out again in every thread block.
    """

    def __init__(self, residual, weight, eps: float, rows, materialize):
        self.residual, self.weight, self.eps, self.rows = residual, weight, eps, rows
        self._materialize = materialize
        self.shape = (residual.shape[0] if rows is None else rows.shape[0], residual.shape[1])
        self.prepared = None
        self.buffers = None    # where ``prepared`` is to be written (buffers of fixed address), or None for fresh ones

    def tensor(self):
        return self._materialize()


def norm_linear(x: "LazyNorm", weight, out, gated: bool = False, clamp=None) -> None:
    """out = rmsnorm(residual) * norm_weight . weight^T in one kernel (``gated``: silu(gate) * up of the two halves; with ``clamp`` =
    (limit, alpha, shift) the clamped gate of ``clamped_gate_mul`` instead)."""
    epilogue = "gated" if gated else "store"
    if fast.gemv_fits(out.shape[0], weight.shape[1], norm=True, gated=gated):
        if x.prepared is not None:
            fast.gemv_fused(x.prepared[0], weight, out, prepared=(x.prepared[1], x.eps), epilogue=epilogue, clamp=clamp)
        else:
            fast.gemv_fused(x.residual, weight, out, norm=(x.weight, x.eps, x.rows), epilogue=epilogue, clamp=clamp)
    elif clamp is not None:
        gate_up = torch.empty((out.shape[0], weight.shape[0]), dtype=out.dtype, device=out.device)
        linear(x.tensor(), weight, gate_up)
        clamped_gate_mul(gate_up, out, *clamp)
    elif fast.use_skinny and x.prepared is not None and fast.skinny_fits(out.shape[0], weight, x.prepared[0]) and out.is_contiguous():
        # the rows' scale is applied to the product's result: the operand is bfloat16(residual * norm weight) as it was left
        fast.gemm_skinny(x.prepared[0], weight, out, epilogue=epilogue, prepared=(x.prepared[1], x.eps))
    elif gated:
        linear_gated(x.tensor(), weight, out)
    else:
        linear(x.tensor(), weight, out)


def linear_activated(x, weight, out, kind: str) -> None:
    """out = act(x . weight^T), the activation applied to the product as it is stored (rounded to the output's dtype first, as when
    the product is stored and ``activation`` run over it).  ``x``: a tensor or a ``LazyNorm``.  One kernel for up to 16 bfloat16 rows
    (norm in front, activation behind); a product and an elementwise kernel otherwise."""
    lazy = isinstance(x, LazyNorm)
    if out.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and fast.gemv_fits(out.shape[0], weight.shape[1], norm=lazy, N=None if lazy else weight.shape[0]):
        if lazy and x.prepared is not None:
            fast.gemv_fused(x.prepared[0], weight, out, prepared=(x.prepared[1], x.eps), activation=kind)
            return
        if lazy:
            fast.gemv_fused(x.residual, weight, out, norm=(x.weight, x.eps, x.rows), activation=kind)
            return
        if x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.stride(0) % 8 == 0:
            fast.gemv_fused(x, weight, out, activation=kind)
            return
    if lazy:
        norm_linear(x, weight, out)
    else:
        linear(x, weight, out)
    activation(kind, out, out)


def can_accumulate(rows: int, weight) -> bool:
    """Whether ``linear_accumulate`` is one kernel for a step of this many rows beyond the fused row limit."""
    return fast.can_accumulate(rows, weight)


def linear_accumulate(x, weight, residual, prepare: "LazyNorm | None" = None) -> None:
    """residual += x . weight^T, the sum in 32-bit, in one kernel (bfloat16 x; up to 16 rows in the register-fed weight-streaming
    kernel, up to 127 in the tensor-core one, for prompt portions in the tensor-core product's epilogue).

    ``prepare``: the lazy norm of this residual (all rows) that the next product will consume; the kernel then leaves that
    norm's input beside the residual (``prepare.prepared``), written by the threads that hold the finished sums."""
    rows = x.shape[0]
    preparing = (prepare is not None and prepare.rows is None and prepare.residual is residual and use_prepared_norms
                 and residual.shape[0] >= PREPARED_NORM_MIN_ROWS)
    if fast.gemv_fits(rows, weight.shape[1], norm=False, N=weight.shape[0]):
        if preparing:
            buffers = fast.prepared_norm_buffers(residual.shape[0], residual.shape[1], residual.device) if prepare.buffers is None else prepare.buffers
            fast.gemv_fused(x, weight, residual, epilogue="accumulate", prepare=(prepare.weight, buffers[0], buffers[1]))
            prepare.prepared = buffers
        else:
            fast.gemv_fused(x, weight, residual, epilogue="accumulate")
    elif fast.use_skinny and fast.skinny_fits(rows, weight, x) and residual.is_contiguous():
        buffers = None
        if preparing:
            buffers = fast.prepared_norm_buffers(residual.shape[0], residual.shape[1], residual.device) if prepare.buffers is None else prepare.buffers
            runs = fast.skinny_square_runs(rows, weight.shape[0], weight.shape[1])   # this kernel's partial sums per row: one per CTA that finishes a run of columns
            if runs > buffers[1].shape[1]:
                buffers = None   # a narrow matrix cut many ways: more partial sums than the buffer has room for
        if buffers is not None:
            squares = buffers[1][:, :runs]
            fast.gemm_skinny(x, weight, residual, epilogue="accumulate", prepare=(prepare.weight, buffers[0], squares))
            prepare.prepared = (buffers[0], squares)
        else:
            fast.gemm_skinny(x, weight, residual, epilogue="accumulate")
    elif x.dtype == torch.bfloat16 and fast.can_accumulate(rows, weight) and x.is_contiguous() and residual.is_contiguous():
        fast.gemm_tcgen05_accumulate(x, weight, residual)
    else:
        delta = torch.empty((rows, weight.shape[0]), dtype=x.dtype, device=x.device)
        linear(x, weight, delta)
        add_(residual, delta)


def linear_gated(x, weight, out, clamp=None, activation: str = "silu") -> None:
    """out = act(x . gate^T) * (x . up^T) for weight = [gate rows | up rows], in one kernel where one takes the shape (``clamp``: see
    ``norm_linear``; ``activation``: "silu", or "gelu_tanh", which the small-step kernel has in its epilogue and larger steps run
    as a kernel behind the product)."""
    if activation != "silu":
        if activation not in GATE_KINDS or clamp is not None:
            raise KernelError(f"linear_gated: no gate {activation!r} (with a clamp: silu only)", code="invalid_argument")
        if x.dtype == torch.bfloat16 and fast.gemv_fits(x.shape[0], weight.shape[1], norm=False, gated=True) and x.stride(1) == 1 and x.stride(0) % 8 == 0:
            fast.gemv_fused(x, weight, out, epilogue="gated", gate=activation)
            return
        gate_up = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        linear(x, weight, gate_up)
        gate_mul(gate_up, out, activation)
        return
    if x.dtype == torch.bfloat16 and fast.gemv_fits(x.shape[0], weight.shape[1], norm=False, gated=True):
        fast.gemv_fused(x, weight, out, epilogue="gated", clamp=clamp)
    elif clamp is not None:
        gate_up = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        linear(x, weight, gate_up)
        clamped_gate_mul(gate_up, out, *clamp)
    elif fast.use_tcgen05 and fast.gated_takes(x.shape[0], weight.shape[0], weight.shape[1]) and weight.shape[1] % 8 == 0 and x.is_contiguous():
        fast.gemm_tcgen05_gated(x, weight, out)
    elif fast.use_skinny and fast.skinny_fits(x.shape[0], weight, x) and out.is_contiguous() and out.dtype == torch.bfloat16:
        fast.gemm_skinny(x, weight, out, epilogue="gated")
    else:
        gate_up = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        linear(x, weight, gate_up)
        silu_mul(gate_up, out)


# --- position encoding and cache write ---------------------------------------------------
def rope_store(qkv, positions, token_seq, block_table, inv_freq, rotary_dim: int, pages, q_heads: int, kv_heads: int, head_dim: int, page_size: int, write_cache: bool = True) -> None:
    """Rotate q (in place) and k, and store k, v of every token into its request's pages."""
    tokens = qkv.shape[0]
    if qkv.shape[1] != (q_heads + 2 * kv_heads) * head_dim:
        raise KernelError("rope_store: qkv width does not fit the head counts", code="invalid_shape")
    if write_cache and pages.dtype != qkv.dtype:
        raise KernelError("rope_store: pages and qkv differ in dtype", code="invalid_dtype")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("rope_store: inv_freq must hold rotary_dim / 2 32-bit frequencies", code="invalid_shape")
    _check(
        core().tlie_rope_store(
            _code(qkv), _ptr(qkv), _i32(positions, "positions"), _i32(token_seq, "token_seq"), _i32(block_table, "block_table"),
            c_int(block_table.shape[1]), _ptr(inv_freq), c_int(rotary_dim if inv_freq is not None else 0), _ptr(pages if write_cache else None),
            c_int(tokens), c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(page_size), c_int(1 if write_cache else 0), _stream(),
        ),
        "rope_store",
    )


# --- attention -----------------------------------------------------------------------------
def paged_attention(qkv, pages, positions, token_seq, block_table, out, q_heads: int, kv_heads: int, head_dim: int, page_size: int, window: int = 0, scale: float | None = None, batch=None) -> None:
    """Attention of every query row over its request's cached keys up to its own position.

    ``qkv`` rows start with the (already rotated) q heads; ``batch`` may carry the
    step's shape so that a faster kernel can be chosen for bfloat16.
    """
    tokens = qkv.shape[0]
    if head_dim % 16 != 0 or head_dim > 256:
        raise KernelError(f"attention kernels take head sizes that are multiples of 16 up to 256, got {head_dim}", code="invalid_shape")
    if q_heads % kv_heads != 0:
        raise KernelError("attention: query heads must be a multiple of key/value heads", code="invalid_shape")
    if scale is None:
        scale = head_dim ** -0.5
    if qkv.dtype == torch.bfloat16:
        if fast.paged_attention_bf16(qkv, pages, positions, token_seq, block_table, out, q_heads, kv_heads, head_dim, page_size, window, scale, batch):
            return
    _check(
        core().tlie_paged_attention_generic(
            _code(qkv), _ptr(qkv), c_int(qkv.shape[1]), _ptr(pages), _i32(positions, "positions"), _i32(token_seq, "token_seq"),
            _i32(block_table, "block_table"), c_int(block_table.shape[1]), _ptr(out), c_int(tokens), c_int(q_heads), c_int(kv_heads),
            c_int(head_dim), c_int(page_size), c_int(window), c_float(scale), _stream(),
        ),
        "paged_attention_generic",
    )


def attention_step(qkv, positions, token_seq, block_table, inv_freq, rotary_dim: int, pages, out, q_heads: int, kv_heads: int,
                   head_dim: int, page_size: int, window: int = 0, scale: float | None = None, write_cache: bool = True, batch=None) -> None:
    """Rotate q and k, store k and v in the pages, and attend: ``rope_store`` then ``paged_attention``, in one kernel where one exists."""
    if qkv.dtype == torch.bfloat16:
        if fast.can_fuse_rope_into_decode(batch, qkv, head_dim, q_heads, kv_heads, inv_freq, rotary_dim):
            splits = fast.decode_splits(batch.num_seqs, kv_heads, batch.max_seq_len)
            fast.decode_attention(qkv, pages, positions, block_table, out, q_heads, kv_heads, head_dim, page_size, window,
                                  head_dim ** -0.5 if scale is None else scale, splits, fuse_rope=True, inv_freq=inv_freq, write_cache=write_cache)
            return
    rope_store(qkv, positions, token_seq, block_table, inv_freq, rotary_dim, pages, q_heads, kv_heads, head_dim, page_size, write_cache)
    paged_attention(qkv, pages, positions, token_seq, block_table, out, q_heads, kv_heads, head_dim, page_size, window, scale, batch)


# --- recurrences ---------------------------------------------------------------------------
GATED_RECURRENCE_MAX_RUNS = 64


def recurrent():
    return load_library("tlie_recurrent", RECURRENT_SOURCES)


def mingru_scan(zxg, bias_z, bias_x, state, seq_starts, state_slots, out, max_rows: int) -> None:
    """The minGRU recurrence over every entry's rows, from and into the entries' state slots.

    ``zxg`` [T, 3 W]: the stacked product (gate, candidate and output-gate pre-activations); per channel
    z = sigmoid(a + bias_z), u = x + bias_x, cand = u + 1/2 if u >= 0 else sigmoid(u), S = (1 - z) S + z cand,
    out = S * silu(g).  ``state`` [slots, W] is 32-bit and is read at ``state_slots[entry]`` and left at the entry's last row.
    ``max_rows``: the longest entry of the step (decides into how many runs the kernel cuts an entry)."""
    tokens, width = out.shape
    entries = state_slots.shape[0]
    if zxg.shape != (tokens, 3 * width) or zxg.dtype != out.dtype:
        raise KernelError("mingru_scan: the stacked product must be [rows, 3 * width] of the output's dtype", code="invalid_shape")
    if state.dtype != torch.float32 or state.shape[1] != width or bias_z.dtype != torch.float32 or bias_x.dtype != torch.float32 or bias_z.numel() != width or bias_x.numel() != width:
        raise KernelError("mingru_scan: state [slots, width] and the two biases [width] are 32-bit", code="invalid_dtype")
    if seq_starts.shape[0] != entries + 1:
        raise KernelError("mingru_scan: seq_starts holds one more word than there are entries", code="invalid_shape")
    runs = 1 if max_rows <= 1 else min(GATED_RECURRENCE_MAX_RUNS, max(2, -(-max_rows // 16)))
    _check(recurrent().tlie_mingru_scan(_code(zxg), _ptr(zxg), _ptr(bias_z), _ptr(bias_x), _ptr(state), _i32(seq_starts, "seq_starts"),
                                        _i32(state_slots, "state_slots"), _ptr(out), c_int(entries), c_int(width), c_int(runs), _stream()), "mingru_scan")


import os as _os

# lanes that share a column of the delta rule's state (8 or 16): the matrix is stored [4 ceil(dim / (4 lanes))][vdim][lanes] per head
DELTA_LANES = int(_os.environ.get("TLIE_DELTA_LANES", "8"))


def delta_rule_library():
    return load_library(f"tlie_delta_rule_l{DELTA_LANES}", DELTA_RULE_SOURCES, {"TLIE_DELTA_LANES": DELTA_LANES})


def delta_state_words(heads: int, dim: int, vdim: int, channels: int, taps: int) -> tuple[int, int]:
    """(words of a request's delta-rule state, where the convolution's inputs start in it): the heads' matrices, then taps - 1 rows of inputs."""
    matrices = heads * 4 * (-(-dim // (4 * DELTA_LANES))) * DELTA_LANES * vdim
    return matrices + (taps - 1) * channels, matrices


def _single_rows(ctx) -> int:
    """1 if every entry of the step brings exactly one row (a kernel that keeps a request's last inputs then renews them itself, without a second launch)."""
    return 1 if getattr(ctx, "max_q_len", 0) == 1 else 0


def _state_rows(state, what: str):
    """(pointer, words between two requests' slots) of a per-request state [slots, words] in 32-bit; it may be a run of columns of wider rows."""
    if state is None or state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or not state.is_cuda:
        raise KernelError(f"{what}: the per-request state is 32-bit [slots, words] on a CUDA device", code="invalid_shape")
    return c_void_p(state.data_ptr()), c_longlong(state.stride(0))


def delta_prepare(rows, beta_offset: int, decay_in, taps, a_log, dt_bias, state, conv_offset: int, ctx, prep, heads: int, kv_heads: int, dim: int, vdim: int,
                  unit_eps: float, q_scale: float, decay_per_head: bool = False) -> None:
    """What the delta rule's recurrence reads, per token, in 32-bit: ``prep[t] = [q | k | v | beta | decay]``.

    ``rows`` [T, >= channels + heads] starts with the products for q, k (``kv_heads * dim`` each) and v (``heads * vdim``) and holds the
    beta pre-activations from ``beta_offset``.  q, k, v pass a causal convolution over time per channel (``taps`` [channels, n], last
    column the current token's; the inputs before an entry's first row are read from the request's state at ``conv_offset``) and silu;
    q and k become unit vectors per head (``unit_eps`` inside the root), q times ``q_scale``; beta = sigmoid; decay =
    exp(-exp(a_log[h]) softplus(decay_in + dt_bias)) per head and key channel.  Afterwards the state's convolution inputs are moved on.
    ``decay_per_head``: ``decay_in`` [T, heads] (it may be a run of columns of ``rows``) and ``dt_bias`` [heads] give one decay per head, for all its key channels."""
    tokens = rows.shape[0]
    decays = heads if decay_per_head else heads * dim
    channels = 2 * kv_heads * dim + heads * vdim
    width = channels + heads + heads * dim
    if prep.shape != (tokens, width) or prep.dtype != torch.float32 or state.dtype != torch.float32 or state.dim() != 2:
        raise KernelError("delta_prepare: prep is 32-bit [rows, 2 G dim + H vdim + H + H dim], the state 32-bit [slots, words]", code="invalid_shape")
    if decay_in.shape != (tokens, decays) or decay_in.dtype != rows.dtype or decay_in.stride(1) != 1 or tuple(taps.shape)[0] != channels or taps.dtype != torch.float32:
        raise KernelError("delta_prepare: decay_in [rows, H dim] (or [rows, H]) of the rows' dtype, taps 32-bit [channels, n]", code="invalid_shape")
    if a_log.dtype != torch.float32 or dt_bias.dtype != torch.float32 or a_log.numel() != heads or dt_bias.numel() != decays or rows.stride(1) != 1:
        raise KernelError("delta_prepare: a_log [H] and dt_bias [H dim] (or [H]) are 32-bit", code="invalid_shape")
    state_ptr, state_stride = _state_rows(state, "delta_prepare")
    _check(delta_rule_library().tlie_delta_prepare(_code(rows), c_void_p(rows.data_ptr()), c_int(rows.stride(0)), c_int(beta_offset), c_void_p(decay_in.data_ptr()),
                                                   c_longlong(decay_in.stride(0)), c_int(1 if decay_per_head else 0), _ptr(taps), _ptr(a_log),
                                                   _ptr(dt_bias), state_ptr, state_stride, c_longlong(conv_offset), _i32(ctx.token_seq, "token_seq"),
                                                   _i32(ctx.seq_starts, "seq_starts"), _i32(ctx.state_slots, "state_slots"), _ptr(prep), c_int(tokens), c_int(ctx.num_seqs),
                                                   c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_int(taps.shape[1]), c_float(unit_eps), c_float(q_scale),
                                                   c_int(_single_rows(ctx)), _stream()),
           "delta_prepare")


def delta_rule(prep, state, ctx, out, heads: int, kv_heads: int, dim: int, vdim: int, plain: bool = False) -> None:
    """The gated delta rule over every entry's rows in order, from and into the entries' state slots: per head
    S <- diag(decay) S; u = beta (v - S^T k); S <- S + k u^T; out = S^T q.  ``out`` is 32-bit [T, heads * vdim].
    ``plain``: u = beta v, the recurrence of linear attention with a decay (nothing is taken back before the write).
    ``prep`` rows are [q: kv_heads dim | k: kv_heads dim | v: heads vdim | beta: heads | decay: heads dim]."""
    tokens = prep.shape[0]
    if out.shape != (tokens, heads * vdim) or out.dtype != torch.float32 or prep.dtype != torch.float32 or prep.shape[1] != 2 * kv_heads * dim + heads * (vdim + 1 + dim):
        raise KernelError("delta_rule: prep [rows, 2 G dim + H vdim + H + H dim] and out [rows, H vdim] are 32-bit", code="invalid_shape")
    state_ptr, state_stride = _state_rows(state, "delta_rule")
    _check(delta_rule_library().tlie_delta_rule(_ptr(prep), state_ptr, state_stride, _i32(ctx.seq_starts, "seq_starts"), _i32(ctx.state_slots, "state_slots"),
                                                _ptr(out), c_int(ctx.num_seqs), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_int(1 if plain else 0), _stream()),
           "delta_rule")


HEAD_GATES = {"sigmoid": 0, "silu": 1, None: 2}


def delta_gate_norm(o, gate, weight, out, eps: float, heads: int, vdim: int, gate_kind: str | None = "sigmoid") -> None:
    """out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * weight * act(gate[t, h]) per head (``weight`` [vdim] shared by the heads);
    ``gate_kind``: "sigmoid", "silu", or None for no gate (``gate`` is then not read)."""
    tokens = o.shape[0]
    if gate_kind not in HEAD_GATES:
        raise KernelError(f"delta_gate_norm: no gate {gate_kind!r}", code="invalid_argument")
    if o.dtype != torch.float32 or weight.dtype != torch.float32 or weight.numel() != vdim or out.shape != (tokens, heads * vdim):
        raise KernelError("delta_gate_norm: o 32-bit [rows, H vdim], weight 32-bit [vdim], out of o's shape", code="invalid_shape")
    if gate_kind is not None and (gate.shape != out.shape or gate.dtype != out.dtype or gate.stride(1) != 1 or not gate.is_cuda):
        raise KernelError("delta_gate_norm: gate and out are of one dtype and shape (the gate may be a run of columns of wider rows)", code="invalid_shape")
    gate_ptr, gate_stride = (c_void_p(0), 0) if gate_kind is None else (c_void_p(gate.data_ptr()), gate.stride(0))
    _check(delta_rule_library().tlie_delta_gate_norm(_code(out), _ptr(o), gate_ptr, c_longlong(gate_stride), _ptr(weight), _ptr(out), c_float(eps), c_int(tokens),
                                                     c_int(heads), c_int(vdim), c_int(HEAD_GATES[gate_kind]), _stream()), "delta_gate_norm")


def hgrn2_prepare(rows, f_bias, lower, prep, heads: int, dim: int, vdim: int) -> None:
    """What the plain recurrence reads for a mixer whose forget gate also writes: ``rows`` = [q: H dim | f: H dim | v: H vdim] (products);
    ``prep[t]`` = [silu(q) | 1 - f | v | 1 | f] with f = lower + (1 - lower) sigmoid(f + f_bias), all 32-bit (``f_bias`` may be None)."""
    tokens = rows.shape[0]
    if rows.shape[1] < 2 * heads * dim + heads * vdim or rows.stride(1) != 1 or prep.dtype != torch.float32 or prep.shape != (tokens, 3 * heads * dim + heads * vdim + heads):
        raise KernelError("hgrn2_prepare: rows [T, >= 2 H dim + H vdim], prep 32-bit [T, 3 H dim + H vdim + H]", code="invalid_shape")
    if lower.dtype != torch.float32 or lower.numel() != heads * dim or (f_bias is not None and (f_bias.dtype != torch.float32 or f_bias.numel() != heads * dim)):
        raise KernelError("hgrn2_prepare: the lower bound and the bias are 32-bit [H dim]", code="invalid_shape")
    _check(delta_rule_library().tlie_hgrn2_prepare(_code(rows), c_void_p(rows.data_ptr()), c_int(rows.stride(0)), _ptr(f_bias), _ptr(lower), _ptr(prep), c_int(tokens),
                                                   c_int(heads), c_int(dim), c_int(vdim), _stream()), "hgrn2_prepare")


def ssd_prepare(rows, taps, conv_bias, a_log, dt_bias, state, conv_offset: int, ctx, prep, heads: int, groups: int, n: int, vdim: int) -> None:
    """What the plain recurrence reads for a state-space layer: ``rows`` = [z: inner | x: inner | B: G n | C: G n | dt: H] (products, inner = H vdim).
    x, B, C pass a causal convolution per channel (``taps`` 32-bit [inner + 2 G n, taps], ``conv_bias`` or None; the inputs before an entry's first row
    are read from the request's state at ``conv_offset``, which is moved on afterwards) and silu; dt = softplus(dt + dt_bias);
    ``prep[t]`` = [C | B | x | dt | exp(-exp(a_log[h]) dt) for the n channels of head h], all 32-bit."""
    tokens = rows.shape[0]
    inner, channels = heads * vdim, heads * vdim + 2 * groups * n
    if rows.shape[1] != inner + channels + heads or rows.stride(1) != 1 or prep.dtype != torch.float32 or prep.shape != (tokens, 2 * groups * n + inner + heads + heads * n):
        raise KernelError("ssd_prepare: rows [T, 2 inner + 2 G n + H], prep 32-bit [T, 2 G n + inner + H + H n]", code="invalid_shape")
    if taps.dtype != torch.float32 or taps.shape[0] != channels or a_log.dtype != torch.float32 or a_log.numel() != heads or dt_bias.dtype != torch.float32 or dt_bias.numel() != heads:
        raise KernelError("ssd_prepare: taps 32-bit [channels, n]; a_log and dt_bias 32-bit [H]", code="invalid_shape")
    state_ptr, state_stride = _state_rows(state, "ssd_prepare")
    _check(delta_rule_library().tlie_ssd_prepare(_code(rows), c_void_p(rows.data_ptr()), c_int(rows.stride(0)), _ptr(taps), _ptr(conv_bias), _ptr(a_log), _ptr(dt_bias), state_ptr,
                                                 state_stride, c_longlong(conv_offset), _i32(ctx.token_seq, "token_seq"), _i32(ctx.seq_starts, "seq_starts"),
                                                 _i32(ctx.state_slots, "state_slots"), _ptr(prep), c_int(tokens), c_int(ctx.num_seqs), c_int(heads), c_int(groups), c_int(n),
                                                 c_int(vdim), c_int(taps.shape[1]), c_int(_single_rows(ctx)), _stream()), "ssd_prepare")


def ssd_finish(read, prep, x_offset: int, rows, skip, weight, out, eps: float, heads: int, vdim: int, norm_groups: int) -> None:
    """out = norm((read + skip[h] x) silu(z)) * weight: ``read`` 32-bit [T, H vdim] is the recurrence's output, x the value columns of ``prep`` (from
    ``x_offset``), z the first H vdim columns of ``rows``; the RMS norm runs over each of ``norm_groups`` equal parts of a row (``eps`` inside the root)."""
    tokens, inner = read.shape[0], heads * vdim
    if read.dtype != torch.float32 or read.shape != (tokens, inner) or prep.dtype != torch.float32 or out.shape != (tokens, inner) or out.dtype != rows.dtype or rows.stride(1) != 1:
        raise KernelError("ssd_finish: read and prep are 32-bit, out [T, H vdim] of the rows' dtype", code="invalid_shape")
    if skip.dtype != torch.float32 or skip.numel() != heads or weight.dtype != torch.float32 or weight.numel() != inner or inner % norm_groups:
        raise KernelError("ssd_finish: skip 32-bit [H], weight 32-bit [H vdim], norm_groups a divisor of H vdim", code="invalid_shape")
    _check(delta_rule_library().tlie_ssd_finish(_code(out), _ptr(read), _ptr(prep), c_int(prep.shape[1]), c_int(x_offset), c_void_p(rows.data_ptr()), c_int(rows.stride(0)),
                                                _ptr(skip), _ptr(weight), _ptr(out), c_float(eps), c_int(tokens), c_int(heads), c_int(vdim), c_int(norm_groups), _stream()),
           "ssd_finish")


# --- what looks back along a request ---------------------------------------------------------------
def sequence_library():
    return load_library("tlie_sequence", SEQUENCE_SOURCES)


def pair_embedding(table, pairs, ctx, state, state_offset: int, weight, eps: float, scale: float, residual, buckets: int, mul_prev: int, mul_cur: int, groups: int) -> None:
    """residual[t] = norm(table[id_t] * scale + pairs[(id_{t-1} mul_prev + id_t mul_cur) mod buckets]) in 32-bit: a second table's row chosen by the token
    and the one before it (row ``buckets`` for a request's first token).  The token before a step's first row of a request is the word
    ``state_offset`` of the request's state (the id's bits), renewed after the step.  ``pairs`` None: no second table; ``weight`` None: no norm;
    the norm is an RMS norm over each of ``groups`` equal parts of a row."""
    rows, width = residual.shape
    if residual.dtype != torch.float32 or table.shape[1] != width or (pairs is not None and (pairs.shape != (buckets + 1, width) or pairs.dtype != table.dtype)):
        raise KernelError("pair_embedding: a 32-bit residual [T, width], a table [vocab, width], pairs [buckets + 1, width] of the table's dtype", code="invalid_shape")
    if weight is not None and (weight.dtype != torch.float32 or weight.numel() != width):
        raise KernelError("pair_embedding: the norm weight is 32-bit [width]", code="invalid_shape")
    state_ptr, state_stride = (c_void_p(0), c_longlong(0)) if pairs is None else _state_rows(state, "pair_embedding")
    _check(sequence_library().tlie_pair_embedding(_code(table), _ptr(table), _ptr(pairs), _i32(ctx.token_ids, "ids"), _i32(ctx.positions, "positions"),
                                                  _i32(ctx.token_seq, "token_seq"), _i32(ctx.seq_starts, "seq_starts"), _i32(ctx.state_slots, "state_slots"), state_ptr,
                                                  state_stride, c_longlong(state_offset), _ptr(weight), c_float(eps), c_float(scale), _ptr(residual), c_int(rows),
                                                  c_int(ctx.num_seqs), c_int(width), c_int(table.shape[0]), c_int(buckets), c_longlong(mul_prev), c_longlong(mul_cur),
                                                  c_int(groups), c_int(_single_rows(ctx)), _ptr(error_flag(residual.device)), _stream()), "pair_embedding")


def conv_residual(x, taps, state, state_offset: int, ctx, out) -> None:
    """out[t, c] = x[t, c] + sum_j taps[c, j] x[t - n + 1 + j, c] along every request (zeros before its start), 32-bit inside.  The n - 1 inputs
    before a step's first row of a request are read from the request's state at ``state_offset`` ([n - 1, channels]), which is moved on afterwards."""
    rows, channels = x.shape
    if out.shape != x.shape or out.dtype != x.dtype or out.data_ptr() == x.data_ptr() or taps.dtype != torch.float32 or taps.shape[0] != channels:
        raise KernelError("conv_residual: out has x's shape and dtype and is another buffer; taps are 32-bit [channels, n]", code="invalid_shape")
    state_ptr, state_stride = (c_void_p(0), c_longlong(0)) if taps.shape[1] == 1 else _state_rows(state, "conv_residual")
    _check(sequence_library().tlie_conv_residual(_code(x), _ptr(x), _ptr(taps), state_ptr, state_stride, c_longlong(state_offset), _i32(ctx.token_seq, "token_seq"),
                                                 _i32(ctx.seq_starts, "seq_starts"), _i32(ctx.state_slots, "state_slots"), _ptr(out), c_int(rows), c_int(ctx.num_seqs),
                                                 c_int(channels), c_int(taps.shape[1]), c_int(_single_rows(ctx)), _stream()), "conv_residual")


def add_bias(x, bias) -> None:
    """x[t, c] += bias[c] in place (``bias`` 32-bit [width]), 32-bit inside."""
    if bias.dtype != torch.float32 or x.dim() != 2 or bias.numel() != x.shape[1]:
        raise KernelError("add_bias: x [rows, width], bias 32-bit [width]", code="invalid_shape")
    _check(sequence_library().tlie_add_bias(_code(x), _ptr(x), _ptr(bias), c_int(x.shape[0]), c_int(x.shape[1]), _stream()), "add_bias")


def scaled_sum(x, y, a: float, b: float, out) -> None:
    """out = a x + b y, 32-bit inside (``out`` may be ``x`` or ``y``)."""
    if x.shape != y.shape or out.shape != x.shape or x.dtype != y.dtype or out.dtype != x.dtype:
        raise KernelError("scaled_sum: x, y and out share a shape and a dtype", code="invalid_shape")
    _check(sequence_library().tlie_scaled_sum(_code(x), _ptr(x), _ptr(y), c_float(a), c_float(b), _ptr(out), c_longlong(x.numel()), _stream()), "scaled_sum")


# --- attention with mixed heads --------------------------------------------------------------
def mixed_attention():
    return load_library("tlie_attention_mixed", MIXED_ATTENTION_SOURCES)


def _plane_pointers(cache, heads: int, key_dim: int, value_dim: int):
    """Where the key plane and the value plane of a layer's pages start, and each one's page stride in elements."""
    if cache.pages is not None:   # equal planes: [pages, 2, heads, page_size, width]
        pages = cache.pages
        if pages.dim() != 5 or pages.shape[1] != 2 or tuple(pages.shape[2:]) != (heads, cache.page_size, key_dim) or key_dim != value_dim or not pages.is_contiguous():
            raise KernelError("attention pages must be contiguous [pages, 2, kv heads, page size, width]", code="invalid_shape")
        plane = heads * cache.page_size * key_dim
        return pages, _ptr(pages), 2 * plane, c_void_p(pages.data_ptr() + plane * pages.element_size()), 2 * plane
    k_pages, v_pages = cache.plane_pages
    if tuple(k_pages.shape[1:]) != (heads, cache.page_size, key_dim) or tuple(v_pages.shape[1:]) != (heads, cache.page_size, value_dim) or k_pages.dtype != v_pages.dtype:
        raise KernelError("attention planes must be [pages, kv heads, page size, key width] and [.., value width]", code="invalid_shape")
    return k_pages, _ptr(k_pages), heads * cache.page_size * key_dim, _ptr(v_pages), heads * cache.page_size * value_dim


def normed_store(rows, k_offset: int, v_offset: int, positions, token_seq, cache, heads: int, kv_heads: int, key_dim: int, value_dim: int, eps: float,
                 q_weight=None, k_weight=None) -> None:
    """Divide every query head (in place) and key head of ``rows`` by its root mean square (``eps`` inside the root; times a 32-bit
    weight [key_dim] if given); write the normalised keys into the key plane of the tokens' pages and the ``kv_heads * value_dim``
    columns from ``v_offset`` into the value plane as they are (``v_offset == k_offset``: the values are the keys before the norm)."""
    pages, k_ptr, k_stride, v_ptr, v_stride = _plane_pointers(cache, kv_heads, key_dim, value_dim)
    if pages.dtype != rows.dtype:
        raise KernelError("normed_store: pages and rows differ in dtype", code="invalid_dtype")
    table = cache.block_table
    _check(mixed_attention().tlie_normed_store(_code(rows), _ptr(rows), c_int(rows.shape[1]), c_int(k_offset), c_int(v_offset), _ptr(q_weight), _ptr(k_weight), c_float(eps),
                                               _i32(positions, "positions"), _i32(token_seq, "token_seq"), _i32(table, "block_table"), c_int(table.shape[1]), k_ptr,
                                               c_longlong(k_stride), v_ptr, c_longlong(v_stride), c_int(rows.shape[0]), c_int(heads), c_int(kv_heads), c_int(key_dim),
                                               c_int(value_dim), c_int(cache.page_size), c_int(1 if cache.writes else 0), _stream()), "normed_store")


def _latent_plane(cache, width: int):
    pages = cache.pages
    if pages is None or pages.dim() != 5 or tuple(pages.shape[1:]) != (1, 1, cache.page_size, width) or not pages.is_contiguous():
        raise KernelError("latent attention pages must be contiguous [pages, 1, 1, page size, rank + rot]", code="invalid_shape")
    return pages


def latent_store(rows, latent_offset: int, weight, eps: float, inv_freq, rot_dims: int, positions, token_seq, cache, queries, heads: int, plain: int, rot: int, rank: int) -> None:
    """Latent attention's cache write and rotation: ``rows[:, latent_offset:]`` = [rank | rot] becomes [rms-normed latent (32-bit ``weight``) |
    rotated shared key part] in the token's cache row; the ``rot`` columns behind the ``plain`` ones of every query head are rotated into
    ``queries`` [T, heads * (rank + rot)], behind each head's first ``rank`` columns (which are left alone).
    Pairs (2i, 2i + 1) of the first ``rot_dims`` columns turn by position * inv_freq[i]."""
    pages = _latent_plane(cache, rank + rot)
    if queries.shape != (rows.shape[0], heads * (rank + rot)) or queries.dtype != rows.dtype:
        raise KernelError("latent_store: queries must be [rows, heads * (rank + rot)] of the rows' dtype", code="invalid_shape")
    if pages.dtype != rows.dtype or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2 or weight.dtype != torch.float32 or weight.numel() != rank:
        raise KernelError("latent_store: pages of the rows' dtype; inv_freq [rot_dims / 2] and weight [rank] 32-bit", code="invalid_shape")
    table = cache.block_table
    _check(mixed_attention().tlie_latent_store(_code(rows), _ptr(rows), c_int(rows.shape[1]), c_int(latent_offset), _ptr(weight), c_float(eps), _ptr(inv_freq), c_int(rot_dims),
                                               _i32(positions, "positions"), _i32(token_seq, "token_seq"), _i32(table, "block_table"), c_int(table.shape[1]), _ptr(pages),
                                               c_longlong(cache.page_size * (rank + rot)), c_int(rows.shape[0]), c_int(heads), c_int(plain), c_int(rot), c_int(rank),
                                               c_int(cache.page_size), c_int(1 if cache.writes else 0), _ptr(queries), _stream()), "latent_store")


def store_kv_planes(rows, k_offset: int, v_offset: int, positions, token_seq, cache, kv_heads: int, key_dim: int, value_dim: int) -> None:
    """Copy every token's keys (``kv_heads * key_dim`` columns of ``rows`` from ``k_offset``) and values (from ``v_offset``) into the
    pages its request holds for its position.  ``cache``: the layer's ``LayerCache`` (one tensor of two equal planes, or a tensor per plane)."""
    pages, k_ptr, k_stride, v_ptr, v_stride = _plane_pointers(cache, kv_heads, key_dim, value_dim)
    if pages.dtype != rows.dtype:
        raise KernelError("store_kv_planes: pages and rows differ in dtype", code="invalid_dtype")
    table = cache.block_table
    _check(mixed_attention().tlie_store_kv_planes(_code(rows), _ptr(rows), c_int(rows.shape[1]), c_int(k_offset), c_int(v_offset), _i32(positions, "positions"),
                                                  _i32(token_seq, "token_seq"), _i32(table, "block_table"), c_int(table.shape[1]), k_ptr, c_longlong(k_stride),
                                                  v_ptr, c_longlong(v_stride), c_int(rows.shape[0]), c_int(kv_heads), c_int(key_dim), c_int(value_dim),
                                                  c_int(cache.page_size), _stream()), "store_kv_planes")


def rotary_store_planes(rows, k_offset: int, v_offset: int, biases, inv_freq, rot_dims: int, positions, token_seq, cache, heads: int, kv_heads: int, key_dim: int,
                        value_dim: int) -> None:
    """Biases, a partial rotation and the cache write in one kernel: every q, k and v vector of ``rows`` gets its bias (``biases`` = (q, k, v), 32-bit
    or None each); of every q and k head the first ``rot_dims`` columns turn, column i with column i + rot_dims / 2, by position * inv_freq[i];
    q is left in place, k goes into the key plane and v into the value plane of the token's page."""
    pages, k_ptr, k_stride, v_ptr, v_stride = _plane_pointers(cache, kv_heads, key_dim, value_dim)
    if pages.dtype != rows.dtype or rot_dims % 2 or rot_dims > key_dim or (rot_dims > 0 and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2)):
        raise KernelError("rotary_store_planes: pages of the rows' dtype; inv_freq 32-bit [rot_dims / 2], rot_dims even and at most key_dim", code="invalid_shape")
    q_bias, k_bias, v_bias = biases if biases is not None else (None, None, None)
    for bias, count in ((q_bias, heads * key_dim), (k_bias, kv_heads * key_dim), (v_bias, kv_heads * value_dim)):
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != count):
            raise KernelError("rotary_store_planes: biases are 32-bit, one number per column", code="invalid_shape")
    table = cache.block_table
    _check(mixed_attention().tlie_rotary_store_planes(_code(rows), _ptr(rows), c_int(rows.shape[1]), c_int(k_offset), c_int(v_offset), _ptr(q_bias), _ptr(k_bias), _ptr(v_bias),
                                                      _ptr(inv_freq if rot_dims > 0 else None), c_int(rot_dims), _i32(positions, "positions"), _i32(token_seq, "token_seq"),
                                                      _i32(table, "block_table"), c_int(table.shape[1]), k_ptr, c_longlong(k_stride), v_ptr, c_longlong(v_stride),
                                                      c_int(rows.shape[0]), c_int(heads), c_int(kv_heads), c_int(key_dim), c_int(value_dim), c_int(cache.page_size),
                                                      c_int(1 if cache.writes else 0), _stream()), "rotary_store_planes")


def mixed_heads_attention(rows, gate_offset: int, positions, token_seq, cache, slopes, mix, out, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                          window: int, scale: float, batch=None, folded_slopes=None, keep_first: int = 0, gate_per_head: bool = False, sinks=None,
                          values_in_keys: bool = False) -> None:
    """Attention over the paged keys with a distance bias, the heads' scores mixed before the softmax, and an output gate.

    ``rows`` [T, >= heads * key_dim]: each row starts with its query heads; ``gate_offset`` (>= 0) names the column where
    ``heads * value_dim`` gate pre-activations start (the output is multiplied by their sigmoid), -1 for none.  Score of query
    head g at position i for key j: (q . k) * scale - slopes[g] * (i - j) (``slopes`` 32-bit [heads] or None); head h then sees
    sum_g mix[h, g] score_g (``mix`` 32-bit [heads, heads] or None); keys with 0 <= i - j (< window if window > 0) are visible.
    ``batch``: the step's context, from which a faster kernel is chosen where one fits; ``folded_slopes``: ``fast.folded_slopes(slopes, mix)``
    if the caller keeps it (it is worked out here otherwise).  ``keep_first``: with a window, the keys at positions below it stay visible.
    ``gate_per_head``: the gate is ``heads`` columns, one per head.  ``sinks`` (32-bit [heads]): exp(sink_h) joins the softmax's denominator.
    ``values_in_keys``: the cache has one plane of one key/value head whose rows are the keys and whose first ``value_dim`` columns are the values."""
    tokens = rows.shape[0]
    if heads % kv_heads != 0 or out.shape != (tokens, heads * value_dim) or out.dtype != rows.dtype:
        raise KernelError("mixed_heads_attention: out must be [rows, heads * value_dim] of the rows' dtype, heads a multiple of kv heads", code="invalid_shape")
    for name, tensor, count in (("slopes", slopes, heads), ("mix", mix, heads * heads)):
        if tensor is not None and (tensor.dtype != torch.float32 or tensor.numel() != count):
            raise KernelError(f"mixed_heads_attention: {name} must be 32-bit with {count} elements", code="invalid_shape")
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != heads):
        raise KernelError("mixed_heads_attention: sinks must be 32-bit with one element per head", code="invalid_shape")
    v_row_stride = value_dim
    if values_in_keys:
        if kv_heads != 1 or value_dim > key_dim:
            raise KernelError("mixed_heads_attention: values inside the keys need one key/value head and value_dim <= key_dim", code="invalid_shape")
        pages = _latent_plane(cache, key_dim)
        k_ptr = v_ptr = _ptr(pages)
        k_stride = v_stride = cache.page_size * key_dim
        v_row_stride = key_dim
    else:
        pages, k_ptr, k_stride, v_ptr, v_stride = _plane_pointers(cache, kv_heads, key_dim, value_dim)
    if pages.dtype != rows.dtype:
        raise KernelError("mixed_heads_attention: pages and rows differ in dtype", code="invalid_dtype")
    table = cache.block_table
    if (values_in_keys and window == 0 and gate_offset < 0 and slopes is None and mix is None and rows.shape[1] == heads * key_dim
            and fast.latent_prefill_takes(batch, rows, key_dim, value_dim)):
        fast.latent_prefill(rows, batch, table, k_ptr, k_stride, sinks, out, heads, key_dim, value_dim, cache.page_size, scale)
        return
    plain_options = sinks is None and not values_in_keys   # what the tensor-core kernels with two planes know
    if plain_options and rows.dtype == torch.bfloat16 and fast.mixed_prefill_takes(batch, rows, cache.page_size, kv_heads if mix is not None else 1, key_dim, value_dim, gate_offset,
                                                                                   gate_per_head):
        folded = folded_slopes if folded_slopes is not None else fast.folded_slopes(slopes, mix)
        fast.mixed_prefill(rows, gate_offset, batch, table, (k_ptr, k_stride, v_ptr, v_stride), folded, mix, out, heads, kv_heads, key_dim, value_dim,
                           cache.page_size, window, scale, keep_first if window > 0 else 0, gate_per_head)
        return
    # few rows over long contexts (decode steps): every row's keys are dealt to several CTAs
    splits, partial = 1, None
    if batch is not None and tokens * 2 <= fast.sm_count():
        reach = min(window + keep_first, batch.max_seq_len) if window > 0 else batch.max_seq_len
        splits = max(1, min(2 * fast.sm_count() // tokens, -(-reach // 32), 64))   # down to one tile of 32 keys per CTA
        if plain_options and fast.mixed_decode_takes(rows, heads, kv_heads, key_dim, value_dim, gate_offset, mix is not None, gate_per_head):
            fast.mixed_decode(rows, gate_offset, positions, token_seq, table, (k_ptr, k_stride, v_ptr, v_stride), slopes, mix, out, heads, kv_heads, key_dim,
                              value_dim, cache.page_size, window, scale, splits, keep_first if window > 0 else 0, gate_per_head)
            return
        if splits > 1:
            partial = fast.mixed_scratch(rows.device, tokens * splits * (heads * value_dim + 2 * heads), torch.float32)
    _check(mixed_attention().tlie_mixed_heads_attention(_code(rows), _ptr(rows), c_int(rows.shape[1]), c_int(gate_offset), k_ptr, c_longlong(k_stride), v_ptr,
                                                        c_longlong(v_stride), _i32(positions, "positions"), _i32(token_seq, "token_seq"), _i32(table, "block_table"),
                                                        c_int(table.shape[1]), _ptr(slopes), _ptr(mix), _ptr(out), c_int(tokens), c_int(heads), c_int(kv_heads),
                                                        c_int(key_dim), c_int(value_dim), c_int(cache.page_size), c_int(window), c_float(scale), c_int(splits), _ptr(partial),
                                                        c_int(keep_first if window > 0 else 0), c_int(1 if gate_per_head else 0), _ptr(sinks), c_int(v_row_stride), _stream()),
           "mixed_heads_attention")


# --- differential attention --------------------------------------------------------------------
def diff_attention_library():
    return load_library("tlie_attention_diff", DIFF_ATTENTION_SOURCES)


def _diff_planes(cache, kv_heads: int, dim: int, vdim: int):
    """The key plane (two vectors per key/value head: one per map) and the value plane of a layer's pages."""
    if len(cache.plane_pages) != 2:
        raise KernelError("differential attention keeps a key plane [pages, 2 kv heads, page size, dim] and a value plane [pages, kv heads, page size, vdim]", code="invalid_shape")
    k_pages, v_pages = cache.plane_pages
    if tuple(k_pages.shape[1:]) != (2 * kv_heads, cache.page_size, dim) or tuple(v_pages.shape[1:]) != (kv_heads, cache.page_size, vdim) or k_pages.dtype != v_pages.dtype:
        raise KernelError("differential attention keeps a key plane [pages, 2 kv heads, page size, dim] and a value plane [pages, kv heads, page size, vdim]", code="invalid_shape")
    return k_pages, v_pages, 2 * kv_heads * cache.page_size * dim, kv_heads * cache.page_size * vdim


def diff_store(rows, k_offset: int, v_offset: int, q_weight, k_weight, eps: float, inv_freq, rot_dims: int, positions, token_seq, cache, heads: int, kv_heads: int,
               dim: int, vdim: int) -> None:
    """Differential attention's norm, rotation and cache write.  ``rows`` [T, >= 2 heads dim + 2 kv dim + kv vdim]: queries head by head as
    [map 1 | map 2], keys from ``k_offset`` laid out the same way, values from ``v_offset``.  Every query and key vector is divided by its root
    mean square (``eps`` inside the root) and multiplied by a 32-bit weight [dim]; then its first ``rot_dims`` columns turn, column i with
    column i + rot_dims / 2, by position * inv_freq[i].  Queries are left in place; keys and values go into the token's pages."""
    k_pages, v_pages, k_stride, v_stride = _diff_planes(cache, kv_heads, dim, vdim)
    if k_pages.dtype != rows.dtype or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2 or rot_dims % 2 or rot_dims > dim:
        raise KernelError("diff_store: pages of the rows' dtype; inv_freq 32-bit [rot_dims / 2], rot_dims even and at most dim", code="invalid_shape")
    for weight in (q_weight, k_weight):
        if weight.dtype != torch.float32 or weight.numel() != dim:
            raise KernelError("diff_store: the query and key norms' weights are 32-bit [dim]", code="invalid_shape")
    table = cache.block_table
    _check(diff_attention_library().tlie_diff_store(_code(rows), _ptr(rows), c_int(rows.shape[1]), c_int(k_offset), c_int(v_offset), _ptr(q_weight), _ptr(k_weight),
                                                    c_float(eps), _ptr(inv_freq), c_int(rot_dims), _i32(positions, "positions"), _i32(token_seq, "token_seq"),
                                                    _i32(table, "block_table"), c_int(table.shape[1]), _ptr(k_pages), c_longlong(k_stride), _ptr(v_pages),
                                                    c_longlong(v_stride), c_int(rows.shape[0]), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim),
                                                    c_int(cache.page_size), c_int(1 if cache.writes else 0), _stream()), "diff_store")


def diff_attention(rows, positions, token_seq, cache, out, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, lam: float, eps: float, out_scale: float,
                   batch=None) -> None:
    """Causal differential attention over the paged keys.  Head h has two maps, softmax(scale q_m . k_m) v for m = 1, 2 over the same
    values (query vectors 2 h and 2 h + 1 of ``rows``, key vectors 2 g and 2 g + 1 of key/value head g = h // (heads / kv_heads));
    out_h = o / sqrt(mean(o^2) + eps) * out_scale with o = map 1 - lam * map 2.  ``batch``: the step's context, from which the kernel and
    the number of runs a row's keys are cut into are chosen."""
    tokens = rows.shape[0]
    if heads % kv_heads != 0 or out.shape != (tokens, heads * vdim) or out.dtype != rows.dtype:
        raise KernelError("diff_attention: out must be [rows, heads * vdim] of the rows' dtype, heads a multiple of kv heads", code="invalid_shape")
    k_pages, v_pages, k_stride, v_stride = _diff_planes(cache, kv_heads, dim, vdim)
    if k_pages.dtype != rows.dtype:
        raise KernelError("diff_attention: pages and rows differ in dtype", code="invalid_dtype")
    table = cache.block_table
    if rows.dtype == torch.bfloat16 and fast.diff_prefill_takes(batch, rows, cache.page_size, dim, vdim):
        fast.diff_prefill(rows, batch, table, (k_pages, k_stride, v_pages, v_stride), out, heads, kv_heads, dim, vdim, cache.page_size, scale, lam, eps, out_scale)
        return
    if batch is not None and fast.diff_decode_takes(rows, cache.page_size, dim, vdim):
        fast.diff_decode(rows, positions, token_seq, table, (k_pages, k_stride, v_pages, v_stride), out, heads, kv_heads, dim, vdim, cache.page_size, scale, lam, eps,
                         out_scale, batch.max_seq_len)
        return
    runs = 1
    if batch is not None and tokens * kv_heads * 2 <= fast.sm_count():
        runs = max(1, min(2 * fast.sm_count() // (tokens * kv_heads), -(-batch.max_seq_len // 32), 64))   # down to one tile of 32 keys per CTA
    parts = fast.mixed_scratch(rows.device, tokens * runs * 2 * heads * (vdim + 2), torch.float32)
    _check(diff_attention_library().tlie_diff_attention(_code(rows), _ptr(rows), c_int(rows.shape[1]), _ptr(k_pages), c_longlong(k_stride), _ptr(v_pages),
                                                        c_longlong(v_stride), _i32(positions, "positions"), _i32(token_seq, "token_seq"), _i32(table, "block_table"),
                                                        c_int(table.shape[1]), _ptr(parts), _ptr(out), c_int(tokens), c_int(heads), c_int(kv_heads), c_int(dim),
                                                        c_int(vdim), c_int(cache.page_size), c_float(scale), c_float(lam), c_float(eps), c_float(out_scale),
                                                        c_int(runs), _stream()), "diff_attention")


# --- routed experts ------------------------------------------------------------------------------
def moe_library():
    return load_library("tlie_moe", MOE_SOURCES)


def moe_route(x, router, correction, ids, weights, groups: int, keep: int, route_scale: float, normalize: bool = True) -> None:
    """Per token of ``x`` [T, width]: s = sigmoid(router x) (``router`` 32-bit [experts, width], sums in 32-bit), choice = s + ``correction``
    (32-bit [experts] or None).  Experts form ``groups`` equal groups of neighbours; a group's score is the sum of its two largest choice
    scores and only experts of the ``keep`` best groups can be chosen.  ``ids`` int32 [T, top] receives the experts of the ``top`` largest
    choice scores (the lower index on ties), ``weights`` 32-bit [T, top] their s / (sum of the chosen s + 1e-20) * ``route_scale``
    (``normalize`` False: s * ``route_scale``, the scores as they are)."""
    tokens, width = x.shape
    experts, top = router.shape[0], ids.shape[1]
    if router.dtype != torch.float32 or router.shape[1] != width or ids.dtype != torch.int32 or ids.shape != (tokens, top) or weights.dtype != torch.float32 or weights.shape != (tokens, top):
        raise KernelError("moe_route: a 32-bit router [experts, width], int32 ids and 32-bit weights [T, top]", code="invalid_shape")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != experts):
        raise KernelError("moe_route: the correction is 32-bit [experts]", code="invalid_shape")
    _check(moe_library().tlie_moe_route(_code(x), _ptr(x), _ptr(router), _ptr(correction), _ptr(ids), _ptr(weights), c_int(tokens), c_int(width), c_int(experts),
                                        c_int(groups), c_int(keep), c_int(top), c_float(route_scale), c_int(1 if normalize else 0), _stream()), "moe_route")


def moe_experts(x, gate_up, down, ids, weights, shared, out, activation: str = "silu", batch=None, weight_input: bool = False) -> None:
    """out[t] = sum_k weights[t, k] * W_down[e] (act(W_gate[e] x[t]) * (W_up[e] x[t])) for e = ids[t, k], plus ``shared[t]`` if given.
    ``gate_up`` [experts, 2 ff, width] (an expert's gate rows, then its up rows), ``down`` [experts, width, ff].  Steps of few rows and the
    32-bit path read each chosen expert's rows directly; bfloat16 prompt portions sort the (token, expert) pairs by expert and run
    the experts' products on the tensor cores.  ``weight_input``: the weight multiplies what the expert reads instead of what it returns,
    out[t] = sum_k expert_e(weights[t, k] x[t]) (the two differ: the experts are not linear)."""
    tokens, width = x.shape
    experts, two_ff, _ = gate_up.shape
    ff, top = two_ff // 2, ids.shape[1]
    if gate_up.shape != (experts, 2 * ff, width) or down.shape != (experts, width, ff) or out.shape != (tokens, width) or gate_up.dtype != x.dtype or down.dtype != x.dtype or out.dtype != x.dtype:
        raise KernelError("moe_experts: gate_up [experts, 2 ff, width], down [experts, width, ff], out [T, width], one dtype", code="invalid_shape")
    if shared is not None and (shared.shape != out.shape or shared.dtype != out.dtype):
        raise KernelError("moe_experts: the shared branch has the output's shape and dtype", code="invalid_shape")
    if activation not in GATE_KINDS:
        raise KernelError(f"moe_experts: no activation {activation!r}", code="invalid_argument")
    if x.dtype == torch.bfloat16 and fast.moe_grouped_takes(tokens, top, width, ff, experts):
        fast.moe_grouped(x, gate_up, down, ids, weights, shared, out, GATE_KINDS[activation], weight_input)
        return
    act = fast.mixed_scratch(x.device, tokens * top * ff, x.dtype)
    _check(moe_library().tlie_moe_experts(_code(x), _ptr(x), _ptr(gate_up), _ptr(down), _ptr(ids), _ptr(weights), _ptr(shared), _ptr(act), _ptr(out), c_int(tokens),
                                          c_int(width), c_int(ff), c_int(top), c_int(GATE_KINDS[activation]), c_int(1 if weight_input else 0), _stream()), "moe_experts")


# --- sampling ------------------------------------------------------------------------------
def argmax(logits, out) -> None:
    """out[r] = index of the largest logit of row r, the lowest index on ties."""
    if logits.dtype != torch.float32:
        raise KernelError("sampling takes 32-bit logits", code="invalid_dtype")
    _check(core().tlie_argmax(_ptr(logits), c_int(logits.shape[0]), c_int(logits.shape[1]), _i32(out, "out"), _stream()), "argmax")


def sample(logits, temperature, top_p, seeds, counters, out) -> None:
    """Temperature / top-p sampling per row; rows with temperature <= 0 are greedy."""
    if logits.dtype != torch.float32 or temperature.dtype != torch.float32 or top_p.dtype != torch.float32:
        raise KernelError("sampling takes 32-bit logits, temperatures and top_p", code="invalid_dtype")
    if seeds.dtype != torch.int64 or counters.dtype != torch.int64:
        raise KernelError("sampling takes int64 seeds and counters", code="invalid_dtype")
    _check(
        core().tlie_sample(_ptr(logits), c_int(logits.shape[0]), c_int(logits.shape[1]), _ptr(temperature), _ptr(top_p), _ptr(seeds), _ptr(counters), _i32(out, "out"), _stream()),
        "sample",
    )


def decode_advance(token_ids, sampled, positions, seq_lens, first_positions, counters, mailbox=None, steps_done=None) -> None:
    """token_ids = sampled; positions, seq_lens, first_positions and counters move on by one.

    ``mailbox``: a pinned host int32 tensor of ``count + 2`` words that the kernel writes over the bus (the tokens, the device error
    word, then the number of the step from the device counter ``steps_done``), so that the host can poll for the step's result."""
    count = token_ids.shape[0]
    box, flag, done = c_void_p(0), c_void_p(0), c_void_p(0)
    if mailbox is not None:
        if mailbox.dtype != torch.int32 or not mailbox.is_pinned() or mailbox.numel() < count + 2 or steps_done is None or steps_done.dtype != torch.int32:
            raise KernelError("decode_advance: the mailbox is pinned host int32 of count + 2 words, with a device int32 step counter", code="invalid_shape")
        box, flag, done = c_void_p(mailbox.data_ptr()), _ptr(error_flag(token_ids.device)), _ptr(steps_done)
    _check(
        core().tlie_decode_advance(_i32(token_ids, "token_ids"), _i32(sampled, "sampled"), _i32(positions, "positions"), _i32(seq_lens, "seq_lens"),
                                   _i32(first_positions, "first_positions"), _ptr(counters), c_int(count), box, flag, done, _stream()),
        "decode_advance",
    )


def uniform_from(seed: int, counter: int) -> float:
    """The uniform number in [0, 1) that draw ``counter`` of a request with ``seed`` uses."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + (counter + 1) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / 16777216.0


from . import fast  # noqa: E402  (the bfloat16 kernels; at the end because it refers back to this module)
