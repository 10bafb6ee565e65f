// Small per-token work that looks back along a request: an embedding that also reads the token before, and a short causal
// convolution in front of a sublayer.  What lies before a step's first row of a request comes from the request's state.
//
//   pair_embedding       x[t] = table[id_t] * scale + pairs[(id_{t-1} * mul_prev + id_t * mul_cur) mod buckets]   (row ``buckets`` for a
//                        request's first token), then an RMS norm over each of ``groups`` equal parts of the row, times a weight;
//                        sums, statistics and the result (the residual stream) are 32-bit.  The token before a step's first row is
//                        one word of the request's state, which ``last_token`` renews after the step.
//   conv_residual        out[t, c] = x[t, c] + sum_j taps[c, j] x[t - n + 1 + j, c]  (zeros before a request's start; the last n - 1
//                        inputs of a request are its state, moved on by ``conv_inputs_keep``).  32-bit inside.
//   scaled_sum           out = a * x + b * y, 32-bit inside: two branches that read the same input join.
//   add_bias             x[t, c] += bias[c], 32-bit inside.
#include <cstdint>
#include "common.cuh"

namespace tlie {

constexpr int kFilterMaxTaps = 16;
constexpr int kFilterMaxGroups = 256;

template <typename T>
__global__ void __launch_bounds__(256) pair_embedding_kernel(const T* __restrict__ table, const T* __restrict__ pairs, const int* __restrict__ ids,
                                                             const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ seq_starts,
                                                             const int* __restrict__ state_slots, const float* __restrict__ state, long long state_stride,
                                                             long long state_offset, const float* __restrict__ weight, float eps, float scale, float* __restrict__ residual,
                                                             int width, int vocab, int buckets, long long mul_prev, long long mul_cur, int groups,
                                                             int* __restrict__ error_flag, float* __restrict__ renew) {
  extern __shared__ float row_s[];
  __shared__ float scratch[32];
  __shared__ float invs[kFilterMaxGroups];
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && error_flag != nullptr) atomicOr(error_flag, 2);
    id = 0;
  }
  const T* pair_row = nullptr;
  if (pairs != nullptr) {
    long long index = buckets;   // a request's first token
    if (positions[t] > 0) {
      const int entry = token_seq[t];
      int before = t > seq_starts[entry] ? ids[t - 1] : __float_as_int(state[(size_t)state_slots[entry] * state_stride + state_offset]);
      if (before < 0 || before >= vocab) before = 0;
      index = ((long long)before * mul_prev + (long long)id * mul_cur) % buckets;
    }
    pair_row = pairs + (size_t)index * width;
  }
  const T* token_row = table + (size_t)id * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) row_s[i] = to_float(token_row[i]) * scale + (pair_row != nullptr ? to_float(pair_row[i]) : 0.0f);
  __syncthreads();
  // a step of single rows: this CTA is the only one that touches its request's word, and every thread has read it by now
  if (renew != nullptr && threadIdx.x == 0) renew[(size_t)state_slots[token_seq[t]] * state_stride + state_offset] = __int_as_float(ids[t]);
  float* out = residual + (size_t)t * width;
  if (weight == nullptr) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[i] = row_s[i];
    return;
  }
  const int part = width / groups;
  for (int g = 0; g < groups; ++g) {
    float squares = 0.0f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) squares += row_s[g * part + i] * row_s[g * part + i];
    const float inv = 1.0f / sqrtf(block_sum(squares, scratch) / (float)part + eps);
    if (threadIdx.x == 0) invs[g] = inv;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < width; i += blockDim.x) out[i] = row_s[i] * invs[i / part] * weight[i];
}

// after the step: every entry's last token becomes the "token before" of its request
__global__ void last_token_kernel(const int* __restrict__ ids, const int* __restrict__ seq_starts, const int* __restrict__ state_slots, float* __restrict__ state,
                                  long long state_stride, long long state_offset, int entries) {
  const int entry = blockIdx.x * blockDim.x + threadIdx.x;
  if (entry >= entries) return;
  const int end = seq_starts[entry + 1];
  if (end > seq_starts[entry]) state[(size_t)state_slots[entry] * state_stride + state_offset] = __int_as_float(ids[end - 1]);
}

template <typename T>
__global__ void __launch_bounds__(256) conv_residual_kernel(const T* __restrict__ x, const float* __restrict__ taps_w, const float* __restrict__ state, long long state_stride,
                                                            long long state_offset, const int* __restrict__ token_seq, const int* __restrict__ seq_starts,
                                                            const int* __restrict__ state_slots, T* __restrict__ out, int channels, int taps, int keep) {
  const int t = blockIdx.x;
  const int entry = token_seq[t];
  const int first = seq_starts[entry];
  const int r = t - first;
  float* kept = const_cast<float*>(state) + (size_t)state_slots[entry] * state_stride + state_offset;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    const float now = to_float(x[(size_t)t * channels + c]);
    float sum = taps_w[c * taps + taps - 1] * now;
    for (int j = 0; j < taps - 1; ++j) {
      const int back = r - (taps - 1) + j;
      const float past = back >= 0 ? to_float(x[(size_t)(first + back) * channels + c]) : kept[(size_t)(taps - 1 + back) * channels + c];
      sum += taps_w[c * taps + j] * past;
      if (keep && j > 0) kept[(size_t)(j - 1) * channels + c] = past;   // a step of single rows: this thread alone reads and renews its channel's inputs
    }
    if (keep && taps > 1) kept[(size_t)(taps - 2) * channels + c] = now;
    out[(size_t)t * channels + c] = from_float<T>(now + sum);
  }
}

// The same for rows whose channels are a multiple of 8 and whose rows start on 16-byte boundaries: a thread takes eight neighbouring channels,
// 16 bytes (bfloat16) or two loads of 16 (32-bit) per row it reads.  Each channel's sum runs in the same order as in the kernel above.
__device__ __forceinline__ void filter_load8(const float* src, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void filter_load8(const __nv_bfloat16* src, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(pairs[i]);
    v[2 * i] = f.x, v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void filter_store8(float* dst, const float (&v)[8]) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void filter_store8(__nv_bfloat16* dst, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) pairs[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(dst) = raw;
}

template <typename T>
__global__ void __launch_bounds__(256) conv_residual_wide_kernel(const T* __restrict__ x, const float* __restrict__ taps_w, const float* __restrict__ state, long long state_stride,
                                                                 long long state_offset, const int* __restrict__ token_seq, const int* __restrict__ seq_starts,
                                                                 const int* __restrict__ state_slots, T* __restrict__ out, int channels, int taps, int rows, int keep) {
  const int per_row = channels / 8;
  const int index = blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= rows * per_row) return;
  const int t = index / per_row, c0 = (index - t * per_row) * 8;
  const int entry = token_seq[t];
  const int first = seq_starts[entry];
  const int r = t - first;
  float* kept = const_cast<float*>(state) + (size_t)state_slots[entry] * state_stride + state_offset;
  float now[8], sum[8], past[8];
  filter_load8(x + (size_t)t * channels + c0, now);
#pragma unroll
  for (int i = 0; i < 8; ++i) sum[i] = taps_w[(c0 + i) * taps + taps - 1] * now[i];
  for (int j = 0; j < taps - 1; ++j) {
    const int back = r - (taps - 1) + j;
    if (back >= 0) {
      filter_load8(x + (size_t)(first + back) * channels + c0, past);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) past[i] = kept[(size_t)(taps - 1 + back) * channels + c0 + i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sum[i] += taps_w[(c0 + i) * taps + j] * past[i];
    if (keep && j > 0) {   // a step of single rows: this thread alone reads and renews its channels' inputs
#pragma unroll
      for (int i = 0; i < 8; ++i) kept[(size_t)(j - 1) * channels + c0 + i] = past[i];
    }
  }
  if (keep && taps > 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) kept[(size_t)(taps - 2) * channels + c0 + i] = now[i];
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) now[i] += sum[i];
  filter_store8(out + (size_t)t * channels + c0, now);
}

// the last taps - 1 inputs of every entry, kept for the request's next step (older ones move up where the entry brought fewer)
template <typename T>
__global__ void conv_inputs_keep_kernel(const T* __restrict__ x, float* __restrict__ state, long long state_stride, long long state_offset,
                                        const int* __restrict__ seq_starts, const int* __restrict__ state_slots, int channels, int taps) {
  const int entry = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int first = seq_starts[entry], count = seq_starts[entry + 1] - first;
  float* kept = state + (size_t)state_slots[entry] * state_stride + state_offset;
  float keep[kFilterMaxTaps];
  for (int i = 0; i < taps - 1; ++i) {
    const int back = count - (taps - 1) + i;
    keep[i] = back >= 0 ? to_float(x[(size_t)(first + back) * channels + c]) : kept[(size_t)(taps - 1 + back) * channels + c];
  }
  for (int i = 0; i < taps - 1; ++i) kept[(size_t)i * channels + c] = keep[i];
}

template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ x, const T* __restrict__ y, float a, float b, T* __restrict__ out, size_t count) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = from_float<T>(a * to_float(x[i]) + b * to_float(y[i]));
}

template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, int width, size_t count) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) x[i] = from_float<T>(to_float(x[i]) + bias[i % width]);
}

}  // namespace tlie

using namespace tlie;

// ``pairs`` null: no second table.  ``weight`` null: no norm.  ``single_rows`` 1: every entry of the step brings exactly one row.  The state word at ``state_offset`` of a request's slot holds the bits of
// the request's last token id (a new request's is never read: its first position is 0).
TLIE_EXPORT int tlie_pair_embedding(int dtype, const void* table, const void* pairs, const int* ids, const int* positions, const int* token_seq, const int* seq_starts,
                                    const int* state_slots, float* state, long long state_stride, long long state_offset, const float* weight, float eps, float scale,
                                    float* residual, int rows, int entries, int width, int vocab, int buckets, long long mul_prev, long long mul_cur, int groups,
                                    int single_rows, int* error_flag, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (groups < 1 || groups > kFilterMaxGroups || width % groups != 0 || (pairs != nullptr && (buckets < 1 || state == nullptr)) || (size_t)width * sizeof(float) > 48 * 1024)
    return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)width * sizeof(float);
  float* renew = (single_rows && pairs != nullptr && rows == entries) ? state : nullptr;   // every entry brings one row: no second launch
  if (dtype == TLIE_F32)
    pair_embedding_kernel<float><<<rows, 256, smem, stream>>>((const float*)table, (const float*)pairs, ids, positions, token_seq, seq_starts, state_slots, state, state_stride,
                                                              state_offset, weight, eps, scale, residual, width, vocab, buckets, mul_prev, mul_cur, groups, error_flag, renew);
  else
    pair_embedding_kernel<__nv_bfloat16><<<rows, 256, smem, stream>>>((const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs, ids, positions, token_seq, seq_starts,
                                                                      state_slots, state, state_stride, state_offset, weight, eps, scale, residual, width, vocab, buckets,
                                                                      mul_prev, mul_cur, groups, error_flag, renew);
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess || pairs == nullptr || renew != nullptr) return (int)status;
  last_token_kernel<<<(entries + 127) / 128, 128, 0, stream>>>(ids, seq_starts, state_slots, state, state_stride, state_offset, entries);
  return (int)cudaGetLastError();
}

// ``single_rows`` 1: every entry of the step brings exactly one row; the kernel then renews the kept inputs itself and there is no second launch.
TLIE_EXPORT int tlie_conv_residual(int dtype, const void* x, const float* taps_w, float* state, long long state_stride, long long state_offset, const int* token_seq,
                                   const int* seq_starts, const int* state_slots, void* out, int rows, int entries, int channels, int taps, int single_rows,
                                   cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int keep = (single_rows && rows == entries && taps > 1) ? 1 : 0;
  if (taps < 1 || taps > kFilterMaxTaps || (taps > 1 && state == nullptr)) return (int)cudaErrorInvalidValue;
  const bool wide = channels % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;   // which kernel runs depends on the sizes alone
  const int wide_blocks = (int)(((long long)rows * (channels / 8) + 255) / 256);
  if (dtype == TLIE_F32) {
    if (wide)
      conv_residual_wide_kernel<float><<<wide_blocks, 256, 0, stream>>>((const float*)x, taps_w, state, state_stride, state_offset, token_seq, seq_starts, state_slots,
                                                                        (float*)out, channels, taps, rows, keep);
    else
      conv_residual_kernel<float><<<rows, 256, 0, stream>>>((const float*)x, taps_w, state, state_stride, state_offset, token_seq, seq_starts, state_slots, (float*)out,
                                                            channels, taps, keep);
  } else {
    if (wide)
      conv_residual_wide_kernel<__nv_bfloat16><<<wide_blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, taps_w, state, state_stride, state_offset, token_seq, seq_starts,
                                                                                state_slots, (__nv_bfloat16*)out, channels, taps, rows, keep);
    else
      conv_residual_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>((const __nv_bfloat16*)x, taps_w, state, state_stride, state_offset, token_seq, seq_starts, state_slots,
                                                                    (__nv_bfloat16*)out, channels, taps, keep);
  }
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess || taps == 1 || keep) return (int)status;
  const dim3 grid((channels + 127) / 128, entries);
  if (dtype == TLIE_F32)
    conv_inputs_keep_kernel<float><<<grid, 128, 0, stream>>>((const float*)x, state, state_stride, state_offset, seq_starts, state_slots, channels, taps);
  else
    conv_inputs_keep_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)x, state, state_stride, state_offset, seq_starts, state_slots, channels, taps);
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_scaled_sum(int dtype, const void* x, const void* y, float a, float b, void* out, long long count, cudaStream_t stream) {
  if (count <= 0) return 0;
  const int blocks = (int)((count + 255) / 256);
  if (dtype == TLIE_F32)
    scaled_sum_kernel<float><<<blocks, 256, 0, stream>>>((const float*)x, (const float*)y, a, b, (float*)out, (size_t)count);
  else
    scaled_sum_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)y, a, b, (__nv_bfloat16*)out, (size_t)count);
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_add_bias(int dtype, void* x, const float* bias, int rows, int width, cudaStream_t stream) {
  const size_t count = (size_t)rows * width;
  if (count == 0) return 0;
  const int blocks = (int)((count + 255) / 256);
  if (dtype == TLIE_F32)
    add_bias_kernel<float><<<blocks, 256, 0, stream>>>((float*)x, bias, width, count);
  else
    add_bias_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)x, bias, width, count);
  return (int)cudaGetLastError();
}
