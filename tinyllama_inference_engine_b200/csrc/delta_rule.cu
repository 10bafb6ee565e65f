// The gated delta rule with one decay per head and key channel, over the rows of a step, with the state a request carries.
//
// Per head, with a state S [dim x vdim] (32-bit, zero for a new request) and per token q, k (unit vectors, q scaled), v,
// beta in (0, 1) and a decay g in (0, 1) per key channel:
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the read-out sees the token's own write)
// Every column of S is independent of the others (S[:, j] sees v_j and u_j only), so a column is owned by a group of 8
// lanes that split the key channels; a token costs a group three partial dot products (k . S_j, q . S_j, q . k, reduced
// together by shuffles) and one pass of updates.  o is worked out as q . (g S)_j + (q . k) u_j.
//
// Kernels:
//   delta_prepare    per (token, head): the short causal convolution of q, k, v over time (the taps before an entry's first row come
//                    from the request's convolution state) with silu, unit norms of q and k per head, q's scale,
//                    beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)): all 32-bit, into one row of ``prep``
//   delta_conv_state per entry: the last taps - 1 inputs of the convolution, kept for the next step
//   delta_rule       the recurrence: one CTA per (entry, head, 16 columns), rows in order, the operands of the next twelve rows
//                    on their way (asynchronous copies into a ring of 16) while a block of four is worked on between two barriers
//   delta_gate_norm  per (token, head): o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate)
//
// The same recurrence without the correction (``plain``: u = beta v) serves other linear-attention mixers: with decay f, key 1 - f and
// beta 1 it is S <- diag(f) S + (1 - f) v^T (hgrn2_prepare); with one decay per head, key B, value x, beta dt and query C it is the
// state-space model S <- a S + dt B x^T, y = S^T C (ssd_prepare, and ssd_finish for the skip term, the gate and the grouped norm).
// ``decay_per_head``: one decay per head (g = exp(-exp(A_log_h) softplus(a_h + dt_bias_h))), written to all the head's key channels.
//
// State of a request (32-bit words): for every head the matrix in the order the recurrence reads it,
// [4 ceil(dim / 32)][vdim][8] (lane l of a column's 8 holds key channels 32 (i / 4) + 4 l + i % 4 at [i][j][l]: four neighbours per
// 16-byte read of the staged operands), then the convolution's inputs [taps - 1][channels].  (TLIE_DELTA_LANES=16 at compile time,
// and the same number on the host, gives a column 16 lanes and 8 columns to a CTA: twice the warps; measured slower.)
#include "common.cuh"

namespace tlie {

#ifndef TLIE_DELTA_LANES
#define TLIE_DELTA_LANES 8
#endif
constexpr int kDeltaLanes = TLIE_DELTA_LANES;        // lanes that share a column of the state (8 or 16; the host lays the state out for the same number)
constexpr int kDeltaColumns = 128 / kDeltaLanes;     // columns per CTA
constexpr int kDeltaThreads = kDeltaLanes * kDeltaColumns;
constexpr int kDeltaMaxTaps = 16;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// prep row: [q: G dim | k: G dim | v: H vdim | beta: H | decay: H dim]
// One CTA per (token, head): blockIdx.y < 2 G is a q head (then a k head): convolution, silu, unit norm (q also scaled); the others are
// the value heads: convolution and silu, and beside them the head's beta and its dim decays.  Few rows (decoded tokens) then still
// fill the SMs, and a thread's loads (the taps of one channel) do not wait for one another.
template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(const T* __restrict__ rows, int row_stride, int beta_offset, const T* __restrict__ a, long long a_stride,
                                                            int decay_per_head, const float* __restrict__ taps_w,
                                                            const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ state,
                                                            long long state_stride, long long conv_offset, const int* __restrict__ token_seq,
                                                            const int* __restrict__ seq_starts, const int* __restrict__ state_slots, float* __restrict__ prep,
                                                            int heads, int kv_heads, int dim, int vdim, int taps, float unit_eps, float q_scale, int keep) {
  __shared__ float conv_s[256];   // the convolved and activated channels of a q or k head (dim <= 256)
  __shared__ float scratch[32];
  const int t = blockIdx.x, part = blockIdx.y;
  const int entry = token_seq[t];
  const int first = seq_starts[entry];
  const int r = t - first;
  const int qk = kv_heads * dim;
  const int channels = 2 * qk + heads * vdim;
  float* conv_state = const_cast<float*>(state) + (size_t)state_slots[entry] * state_stride + conv_offset;
  const int width = channels + heads + heads * dim;
  float* out = prep + (size_t)t * width;
  const bool unit = part < 2 * kv_heads;
  const int c0 = unit ? part * dim : 2 * qk + (part - 2 * kv_heads) * vdim;
  const int count = unit ? dim : vdim;
  float squares = 0.0f;
  for (int d = threadIdx.x; d < count; d += blockDim.x) {
    const int c = c0 + d;
    float sum = 0.0f;
    for (int j = 0; j < taps; ++j) {
      const int back = r - (taps - 1) + j;   // row of the entry this tap reads; negative: before this step
      const float x = back >= 0 ? to_float(rows[(size_t)(first + back) * row_stride + c]) : conv_state[(size_t)(taps - 1 + back) * channels + c];
      sum += taps_w[c * taps + j] * x;
      if (keep && j > 0) conv_state[(size_t)(j - 1) * channels + c] = x;   // a step of single rows: this thread alone reads and renews its channel's inputs
    }
    const float y = sum * sigmoid_f(sum);
    if (unit) {
      conv_s[d] = y;
      squares += y * y;
    } else {
      out[c] = y;
    }
  }
  if (unit) {
    const float inv = (1.0f / sqrtf(block_sum(squares, scratch) + unit_eps)) * (part < kv_heads ? q_scale : 1.0f);
    for (int d = threadIdx.x; d < count; d += blockDim.x) out[c0 + d] = conv_s[d] * inv;   // a thread reads back what it wrote itself
    return;
  }
  const int h = part - 2 * kv_heads;
  if (threadIdx.x == 0) out[channels + h] = sigmoid_f(to_float(rows[(size_t)t * row_stride + beta_offset + h]));
  const float rate = expf(a_log[h]);
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    const int i = h * dim + d;
    const int from = decay_per_head ? h : i;
    out[channels + heads + i] = expf(-rate * softplus_f(to_float(a[(size_t)t * a_stride + from]) + dt_bias[from]));
  }
}

template <typename T>
__global__ void delta_conv_state_kernel(const T* __restrict__ rows, int row_stride, float* __restrict__ state, long long state_stride, long long conv_offset,
                                        const int* __restrict__ seq_starts, const int* __restrict__ state_slots, int channels, int taps) {
  const int entry = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int first = seq_starts[entry], count = seq_starts[entry + 1] - first;
  float* conv_state = state + (size_t)state_slots[entry] * state_stride + conv_offset;
  float keep[kDeltaMaxTaps];
  for (int i = 0; i < taps - 1; ++i) {
    const int back = count - (taps - 1) + i;
    keep[i] = back >= 0 ? to_float(rows[(size_t)(first + back) * row_stride + c]) : conv_state[(size_t)(taps - 1 + back) * channels + c];
  }
  for (int i = 0; i < taps - 1; ++i) conv_state[(size_t)i * channels + c] = keep[i];
}

constexpr int kDeltaStages = 16;   // rows whose operands are in flight or staged ahead of the one being worked on
constexpr int kDeltaBlock = 4;     // rows between two barriers: their copies are one group, and the compiler may overlap their work

__device__ __forceinline__ void delta_copy_word(float* dst, const float* src) {
  const unsigned to = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(to), "l"(src));
}
__device__ __forceinline__ void delta_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void delta_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// R: key channels a lane has registers for (a multiple of 4, dim <= 8 R); the state holds 4 ceil(dim / 32) of them per lane.
// A row's operands ([q | k | g] of the head, the CTA's 16 values, beta) are copied asynchronously into a ring of kDeltaStages
// buffers, several rows ahead, so that a row's turn never waits for memory; padding words are zeroed once and never copied.
// PLAIN: u = beta v needs nothing of the state, so the chain from one row to the next is S <- g S + k u alone and the read-out's sums and
// shuffles (o = S^T q of the new state) hang off it; with the correction u waits for k . S_j, reduced over the column's lanes, in every row.
template <int R, bool PLAIN>
__global__ void __launch_bounds__(kDeltaThreads) delta_rule_kernel(const float* __restrict__ prep, float* __restrict__ state, long long state_stride,
                                                                  const int* __restrict__ seq_starts, const int* __restrict__ state_slots, float* __restrict__ out,
                                                                  int heads, int kv_heads, int dim, int vdim) {
  extern __shared__ __align__(16) float stage_s[];   // kDeltaStages buffers of [q: 8 R | k: 8 R | g: 8 R | v: 16 | beta | 3 unused]
  constexpr int kPadded = kDeltaLanes * R;
  constexpr int kRow = 3 * kPadded + kDeltaColumns + 4;
  constexpr int kLoads = (kRow + kDeltaThreads - 1) / kDeltaThreads;
  const int column_blocks = (vdim + kDeltaColumns - 1) / kDeltaColumns;
  const int head = blockIdx.x / column_blocks, block = blockIdx.x - head * column_blocks;
  const int entry = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & (kDeltaLanes - 1), column = block * kDeltaColumns + tid / kDeltaLanes;
  const bool live = column < vdim;
  const int first = seq_starts[entry], count = seq_starts[entry + 1] - first;
  const int kv = head / (heads / kv_heads);
  const int qk = kv_heads * dim;
  const int width = 2 * qk + heads * vdim + heads + heads * dim;
  const int held = 4 * ((dim + 4 * kDeltaLanes - 1) / (4 * kDeltaLanes));   // key channels per lane that are stored
  const size_t matrix = (size_t)held * vdim * kDeltaLanes;
  float* mine = state + (size_t)state_slots[entry] * state_stride + (size_t)head * matrix;

  // where each word of a staged row comes from in a prep row (-1: padding, stays zero)
  int source[kLoads];
#pragma unroll
  for (int i = 0; i < kLoads; ++i) {
    const int w = tid + i * kDeltaThreads;
    int at = -1;
    if (w < kPadded) at = w < dim ? kv * dim + w : -1;
    else if (w < 2 * kPadded) at = w - kPadded < dim ? qk + kv * dim + (w - kPadded) : -1;
    else if (w < 3 * kPadded) at = w - 2 * kPadded < dim ? 2 * qk + heads * vdim + heads + head * dim + (w - 2 * kPadded) : -1;
    else if (w < 3 * kPadded + kDeltaColumns) at = block * kDeltaColumns + (w - 3 * kPadded) < vdim ? 2 * qk + head * vdim + block * kDeltaColumns + (w - 3 * kPadded) : -1;
    else if (w == 3 * kPadded + kDeltaColumns) at = 2 * qk + heads * vdim + head;
    source[i] = at;
  }
  for (int i = tid; i < kDeltaStages * kRow; i += kDeltaThreads) stage_s[i] = 0.0f;
  __syncthreads();
  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) S[i] = (live && i < held) ? mine[((size_t)i * vdim + column) * kDeltaLanes + lane] : 0.0f;

  auto issue = [&](int block_of_rows) {   // one group per block of rows, empty past the end, so that the count of groups in flight is the same at every step
#pragma unroll
    for (int n = 0; n < kDeltaBlock; ++n) {
      const int row = block_of_rows * kDeltaBlock + n;
      if (row < count) {
        const float* from = prep + (size_t)(first + row) * width;
        float* to = stage_s + (row % kDeltaStages) * kRow;
#pragma unroll
        for (int i = 0; i < kLoads; ++i)
          if (source[i] >= 0) delta_copy_word(to + tid + i * kDeltaThreads, from + source[i]);
      }
    }
    delta_commit();
  };
  constexpr int kBlocksAhead = kDeltaStages / kDeltaBlock - 1;
#pragma unroll
  for (int ahead = 0; ahead < kBlocksAhead; ++ahead) issue(ahead);
  const int blocks = (count + kDeltaBlock - 1) / kDeltaBlock;
  for (int block_of_rows = 0; block_of_rows < blocks; ++block_of_rows) {
    delta_wait<kBlocksAhead - 1>();   // this thread's copies of this block's rows have landed ...
    __syncthreads();                  // ... and so have everyone's; and everyone is done with the block before, whose buffers are written next
    issue(block_of_rows + kBlocksAhead);
    if constexpr (PLAIN) {
      // the block's four rows: the state's chain first, every row leaving its share of the read-out; then the four sums across the column's
      // lanes side by side, so that a round of shuffles is waited for once per block and not once per row
      float reads[kDeltaBlock];
#pragma unroll
      for (int n = 0; n < kDeltaBlock; ++n) {
        const int row = block_of_rows * kDeltaBlock + n;
        reads[n] = 0.0f;
        if (row < count) {
          const float* cur = stage_s + (row % kDeltaStages) * kRow;
          const float u = cur[3 * kPadded + kDeltaColumns] * cur[3 * kPadded + (tid / kDeltaLanes)];   // beta v
          float read2[2] = {0.0f, 0.0f};
#pragma unroll
          for (int j = 0; j < R / 4; ++j) {
            const float4 q4 = *reinterpret_cast<const float4*>(cur + j * 4 * kDeltaLanes + lane * 4);
            const float4 k4 = *reinterpret_cast<const float4*>(cur + kPadded + j * 4 * kDeltaLanes + lane * 4);
            const float4 g4 = *reinterpret_cast<const float4*>(cur + 2 * kPadded + j * 4 * kDeltaLanes + lane * 4);
            const float q[4] = {q4.x, q4.y, q4.z, q4.w}, k[4] = {k4.x, k4.y, k4.z, k4.w}, g[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int i = 4 * j + c;
              S[i] = S[i] * g[c] + k[c] * u;
              read2[c & 1] += q[c] * S[i];
            }
          }
          reads[n] = read2[0] + read2[1];
        }
      }
#pragma unroll
      for (int offset = kDeltaLanes / 2; offset > 0; offset >>= 1)
#pragma unroll
        for (int n = 0; n < kDeltaBlock; ++n) reads[n] += __shfl_xor_sync(0xffffffffu, reads[n], offset);
#pragma unroll
      for (int n = 0; n < kDeltaBlock; ++n) {
        const int row = block_of_rows * kDeltaBlock + n;
        if (row < count && live && lane == 0) out[(size_t)(first + row) * heads * vdim + head * vdim + column] = reads[n];
      }
    } else {
#pragma unroll
    for (int n = 0; n < kDeltaBlock; ++n) {
      const int row = block_of_rows * kDeltaBlock + n;
      if (row >= count) break;
      const float* cur = stage_s + (row % kDeltaStages) * kRow;
      // k . (g S)_j, q . (g S)_j, q . k (this lane's share), each in two chains of sums
      float reach2[2] = {0.0f, 0.0f}, read2[2] = {0.0f, 0.0f}, both2[2] = {0.0f, 0.0f};
      float kk[R];
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const float4 q4 = *reinterpret_cast<const float4*>(cur + j * 4 * kDeltaLanes + lane * 4);
        const float4 k4 = *reinterpret_cast<const float4*>(cur + kPadded + j * 4 * kDeltaLanes + lane * 4);
        const float4 g4 = *reinterpret_cast<const float4*>(cur + 2 * kPadded + j * 4 * kDeltaLanes + lane * 4);
        const float q[4] = {q4.x, q4.y, q4.z, q4.w}, k[4] = {k4.x, k4.y, k4.z, k4.w}, g[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int i = 4 * j + c;
          S[i] *= g[c];
          reach2[c & 1] += k[c] * S[i];
          read2[c & 1] += q[c] * S[i];
          both2[c & 1] += q[c] * k[c];
          kk[i] = k[c];
        }
      }
      float reach = reach2[0] + reach2[1], read = read2[0] + read2[1], both = both2[0] + both2[1];
#pragma unroll
      for (int offset = kDeltaLanes / 2; offset > 0; offset >>= 1) {
        reach += __shfl_xor_sync(0xffffffffu, reach, offset);
        read += __shfl_xor_sync(0xffffffffu, read, offset);
        both += __shfl_xor_sync(0xffffffffu, both, offset);
      }
      const float v = cur[3 * kPadded + (tid / kDeltaLanes)], beta = cur[3 * kPadded + kDeltaColumns];
      const float u = beta * (v - reach);
#pragma unroll
      for (int i = 0; i < R; ++i) S[i] += kk[i] * u;
      if (live && lane == 0) out[(size_t)(first + row) * heads * vdim + head * vdim + column] = read + both * u;
    }
    }
  }
  delta_wait<0>();
  if (live && count > 0) {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (i < held) mine[((size_t)i * vdim + column) * kDeltaLanes + lane] = S[i];
  }
}

// a warp per (token, head)
template <typename T>
__global__ void delta_gate_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long gate_stride, const float* __restrict__ weight, T* __restrict__ out,
                                       float eps, int heads, int vdim, size_t pairs, int gate_kind) {
  const size_t pair = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  const int lane = threadIdx.x & 31;
  const float* row = o + pair * vdim;
  float squares = 0.0f;
  for (int d = lane; d < vdim; d += 32) squares += row[d] * row[d];
  const float inv = rsqrtf(warp_sum(squares) / (float)vdim + eps);
  for (int d = lane; d < vdim; d += 32) {
    float factor = 1.0f;   // gate_kind 0: sigmoid(gate); 1: silu(gate); 2: no gate
    if (gate_kind != 2) {
      const float z = to_float(gate[(pair / heads) * gate_stride + (pair % heads) * vdim + d]);   // the gate may be a run of columns of wider rows
      factor = gate_kind == 1 ? z * sigmoid_f(z) : sigmoid_f(z);
    }
    out[pair * vdim + d] = from_float<T>(row[d] * inv * weight[d] * factor);
  }
}

// prep rows of the same layout for a recurrence whose forget gate also writes: rows = [q: H dim | f: H dim | v: H vdim] (products),
// q = silu(q); f = lower + (1 - lower) sigmoid(f + f_bias) is the decay, 1 - f the key; beta = 1.  A thread per number, so that a step of few rows still fills SMs.
template <typename T>
__global__ void __launch_bounds__(256) hgrn2_prepare_kernel(const T* __restrict__ rows, int row_stride, const float* __restrict__ f_bias, const float* __restrict__ lower,
                                                            float* __restrict__ prep, int heads, int dim, int vdim) {
  const int t = blockIdx.x;
  const T* row = rows + (size_t)t * row_stride;
  const int qk = heads * dim, values = heads * vdim;
  float* out = prep + (size_t)t * (3 * qk + values + heads);
  const int w = blockIdx.y * blockDim.x + threadIdx.x;   // one piece of work a thread: a (q, f) channel, a value or a head's beta
  if (w < qk) {
    const float q = to_float(row[w]);
    const float low = lower[w];
    const float f = low + (1.0f - low) * sigmoid_f(to_float(row[qk + w]) + (f_bias != nullptr ? f_bias[w] : 0.0f));
    out[w] = q * sigmoid_f(q);
    out[qk + w] = 1.0f - f;
    out[2 * qk + values + heads + w] = f;
  } else if (w < qk + values) {
    out[2 * qk + (w - qk)] = to_float(row[2 * qk + (w - qk)]);
  } else if (w < qk + values + heads) {
    out[2 * qk + values + (w - qk - values)] = 1.0f;
  }
}

// prep rows of the same layout for a state-space layer: rows = [z: inner | x: inner | B: G N | C: G N | dt: H] (products, inner = H vdim).
// x, B and C pass a causal convolution over time per channel (taps [channels, n] with a bias, the last column the current token's;
// inputs before an entry's first row come from the request's state at ``conv_offset``) and silu; dt = softplus(dt + dt_bias); the
// query is C, the key B, the value x, beta = dt and the decay exp(-exp(A_log_h) dt) for all N channels of head h.  A thread per number.
template <typename T>
__global__ void __launch_bounds__(256) ssd_prepare_kernel(const T* __restrict__ rows, int row_stride, const float* __restrict__ taps_w, const float* __restrict__ conv_bias,
                                                          const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ state,
                                                          long long state_stride, long long conv_offset, const int* __restrict__ token_seq,
                                                          const int* __restrict__ seq_starts, const int* __restrict__ state_slots, float* __restrict__ prep, int heads,
                                                          int groups, int n, int vdim, int taps, int keep) {
  const int t = blockIdx.x;
  const int entry = token_seq[t];
  const int first = seq_starts[entry];
  const int r = t - first;
  const int inner = heads * vdim, gn = groups * n;
  const int channels = inner + 2 * gn;
  float* conv_state = const_cast<float*>(state) + (size_t)state_slots[entry] * state_stride + conv_offset;
  float* out = prep + (size_t)t * (2 * gn + inner + heads + heads * n);
  const int w = blockIdx.y * blockDim.x + threadIdx.x;   // one piece of work a thread: a channel of the convolution, or one key channel's decay of a head
  // the step sizes and decays of the heads whose channels this CTA writes: once per head, not once per channel
  __shared__ float dt_s[258], decay_s[258];
  const int lo = max((int)(blockIdx.y * blockDim.x), channels), hi = min((int)((blockIdx.y + 1) * blockDim.x), channels + heads * n);
  const int h0 = lo < hi ? (lo - channels) / n : 0;
  if (lo < hi) {
    const int h1 = (hi - 1 - channels) / n;
    for (int j = threadIdx.x; j <= h1 - h0; j += blockDim.x) {
      const float dt = softplus_f(to_float(rows[(size_t)t * row_stride + 2 * inner + 2 * gn + h0 + j]) + dt_bias[h0 + j]);
      dt_s[j] = dt;
      decay_s[j] = expf(-expf(a_log[h0 + j]) * dt);
    }
  }
  __syncthreads();
  if (w < channels) {
    const int c = w;
    float sum = conv_bias != nullptr ? conv_bias[c] : 0.0f;
    for (int j = 0; j < taps; ++j) {
      const int back = r - (taps - 1) + j;
      const float x = back >= 0 ? to_float(rows[(size_t)(first + back) * row_stride + inner + c]) : conv_state[(size_t)(taps - 1 + back) * channels + c];
      sum += taps_w[c * taps + j] * x;
      if (keep && j > 0) conv_state[(size_t)(j - 1) * channels + c] = x;   // a step of single rows: this thread alone reads and renews its channel's inputs
    }
    const float y = sum * sigmoid_f(sum);
    // x -> the values; B -> the keys; C -> the queries
    const int at = c < inner ? 2 * gn + c : (c < inner + gn ? gn + (c - inner) : c - inner - gn);
    out[at] = y;
  } else if (w < channels + heads * n) {
    const int h = (w - channels) / n, i = (w - channels) - h * n;
    if (i == 0) out[2 * gn + inner + h] = dt_s[h - h0];
    out[2 * gn + inner + heads + h * n + i] = decay_s[h - h0];
  }
}

// y = (o + D_h x) silu(z), then an RMS norm over each of ``norm_groups`` equal parts of the inner width, times a weight: the state-space
// layer's read-out made ready for the output product.  x is read from the prep rows (their value columns).  One CTA per token.
template <typename T>
__global__ void __launch_bounds__(256) ssd_finish_kernel(const float* __restrict__ o, const float* __restrict__ prep, int prep_stride, int x_offset, const T* __restrict__ rows,
                                                         int row_stride, const float* __restrict__ skip, const float* __restrict__ weight, T* __restrict__ out, float eps,
                                                         int heads, int vdim, int norm_groups) {
  extern __shared__ float gated_s[];
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int inner = heads * vdim, part = inner / norm_groups;
  for (int i = threadIdx.x; i < inner; i += blockDim.x) {
    const float z = to_float(rows[(size_t)t * row_stride + i]);
    gated_s[i] = (o[(size_t)t * inner + i] + skip[i / vdim] * prep[(size_t)t * prep_stride + x_offset + i]) * (z * sigmoid_f(z));
  }
  __syncthreads();
  for (int g = 0; g < norm_groups; ++g) {
    float squares = 0.0f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) squares += gated_s[g * part + i] * gated_s[g * part + i];
    const float inv = 1.0f / sqrtf(block_sum(squares, scratch) / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += blockDim.x) out[(size_t)t * inner + g * part + i] = from_float<T>(gated_s[g * part + i] * inv * weight[g * part + i]);
  }
}

template <int R, bool PLAIN>
static int launch_delta_rule(const float* prep, float* state, long long state_stride, const int* seq_starts, const int* state_slots, float* out, int entries,
                             int heads, int kv_heads, int dim, int vdim, cudaStream_t stream) {
  const int column_blocks = (vdim + kDeltaColumns - 1) / kDeltaColumns;
  const size_t smem = kDeltaStages * (size_t)(3 * kDeltaLanes * R + kDeltaColumns + 4) * sizeof(float);
  if (smem > 48 * 1024) {   // the widest heads' ring of staged rows is beyond what a kernel may ask for without saying so
    cudaError_t e = cudaFuncSetAttribute(delta_rule_kernel<R, PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  delta_rule_kernel<R, PLAIN><<<dim3(heads * column_blocks, entries), kDeltaThreads, smem, stream>>>(prep, state, state_stride, seq_starts, state_slots, out, heads,
                                                                                                  kv_heads, dim, vdim);
  return (int)cudaGetLastError();
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_delta_prepare(int dtype, const void* rows, int row_stride, int beta_offset, const void* a, long long a_stride, int decay_per_head,
                                   const float* taps_w, const float* a_log,
                                   const float* dt_bias, float* state, long long state_stride, long long conv_offset, const int* token_seq, const int* seq_starts,
                                   const int* state_slots, float* prep, int tokens, int entries, int heads, int kv_heads, int dim, int vdim, int taps, float unit_eps,
                                   float q_scale, int single_rows, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (taps < 1 || taps > kDeltaMaxTaps || kv_heads < 1 || heads % kv_heads != 0 || 2 * kv_heads + heads > 65535) return (int)cudaErrorInvalidValue;
  const int channels = 2 * kv_heads * dim + heads * vdim;
  if (dim > 256) return (int)cudaErrorInvalidValue;
  const dim3 parts(tokens, 2 * kv_heads + heads);
  const int keep = (single_rows && tokens == entries && taps > 1) ? 1 : 0;   // every entry brings one row: the kernel renews the kept inputs itself
  if (dtype == TLIE_F32)
    delta_prepare_kernel<float><<<parts, 128, 0, stream>>>((const float*)rows, row_stride, beta_offset, (const float*)a, a_stride, decay_per_head, taps_w, a_log, dt_bias, state, state_stride,
                                                           conv_offset, token_seq, seq_starts, state_slots, prep, heads, kv_heads, dim, vdim, taps, unit_eps, q_scale, keep);
  else
    delta_prepare_kernel<__nv_bfloat16><<<parts, 128, 0, stream>>>((const __nv_bfloat16*)rows, row_stride, beta_offset, (const __nv_bfloat16*)a, a_stride, decay_per_head, taps_w, a_log, dt_bias,
                                                                   state, state_stride, conv_offset, token_seq, seq_starts, state_slots, prep, heads, kv_heads, dim,
                                                                   vdim, taps, unit_eps, q_scale, keep);
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess || taps == 1 || keep) return (int)status;
  const dim3 grid((channels + 127) / 128, entries);
  if (dtype == TLIE_F32)
    delta_conv_state_kernel<float><<<grid, 128, 0, stream>>>((const float*)rows, row_stride, state, state_stride, conv_offset, seq_starts, state_slots, channels, taps);
  else
    delta_conv_state_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)rows, row_stride, state, state_stride, conv_offset, seq_starts, state_slots,
                                                                     channels, taps);
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_delta_rule(const float* prep, float* state, long long state_stride, const int* seq_starts, const int* state_slots, float* out, int entries,
                                int heads, int kv_heads, int dim, int vdim, int plain, cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (dim < 1 || dim > 256 || kv_heads < 1 || heads % kv_heads != 0) return (int)cudaErrorInvalidValue;
  const int r = 4 * ((dim + 4 * kDeltaLanes - 1) / (4 * kDeltaLanes));
#define TLIE_DELTA(R) \
  if (r <= R)   \
    return plain ? launch_delta_rule<R, true>(prep, state, state_stride, seq_starts, state_slots, out, entries, heads, kv_heads, dim, vdim, stream) \
                 : launch_delta_rule<R, false>(prep, state, state_stride, seq_starts, state_slots, out, entries, heads, kv_heads, dim, vdim, stream)
  TLIE_DELTA(4);
  TLIE_DELTA(8);
  TLIE_DELTA(12);
  TLIE_DELTA(16);
  TLIE_DELTA(24);
  TLIE_DELTA(32);
#undef TLIE_DELTA
  return (int)cudaErrorInvalidValue;
}

TLIE_EXPORT int tlie_delta_gate_norm(int dtype, const float* o, const void* gate, long long gate_stride, const float* weight, void* out, float eps, int tokens, int heads,
                                     int vdim, int gate_kind, cudaStream_t stream) {
  const size_t pairs = (size_t)tokens * heads;
  if (pairs == 0) return 0;
  if (gate_kind < 0 || gate_kind > 2 || (gate_kind != 2 && gate == nullptr)) return (int)cudaErrorInvalidValue;
  const int blocks = (int)((pairs + 3) / 4);
  if (dtype == TLIE_F32)
    delta_gate_norm_kernel<float><<<blocks, 128, 0, stream>>>(o, (const float*)gate, gate_stride, weight, (float*)out, eps, heads, vdim, pairs, gate_kind);
  else
    delta_gate_norm_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(o, (const __nv_bfloat16*)gate, gate_stride, weight, (__nv_bfloat16*)out, eps, heads, vdim, pairs, gate_kind);
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_hgrn2_prepare(int dtype, const void* rows, int row_stride, const float* f_bias, const float* lower, float* prep, int tokens, int heads, int dim,
                                   int vdim, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const dim3 grid(tokens, (heads * dim + heads * vdim + heads + 255) / 256);
  if (dtype == TLIE_F32)
    hgrn2_prepare_kernel<float><<<grid, 256, 0, stream>>>((const float*)rows, row_stride, f_bias, lower, prep, heads, dim, vdim);
  else
    hgrn2_prepare_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)rows, row_stride, f_bias, lower, prep, heads, dim, vdim);
  return (int)cudaGetLastError();
}

// The convolution's inputs (columns [inner, inner + channels) of ``rows``) are moved on in the request's state afterwards.
TLIE_EXPORT int tlie_ssd_prepare(int dtype, const void* rows, int row_stride, const float* taps_w, const float* conv_bias, const float* a_log, const float* dt_bias,
                                 float* state, long long state_stride, long long conv_offset, const int* token_seq, const int* seq_starts, const int* state_slots,
                                 float* prep, int tokens, int entries, int heads, int groups, int n, int vdim, int taps, int single_rows, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (taps < 1 || taps > kDeltaMaxTaps || groups < 1 || heads % groups != 0) return (int)cudaErrorInvalidValue;
  const int inner = heads * vdim, channels = inner + 2 * groups * n;
  const int keep = (single_rows && tokens == entries && taps > 1) ? 1 : 0;
  const dim3 work(tokens, (channels + heads * n + 255) / 256);
  if (dtype == TLIE_F32)
    ssd_prepare_kernel<float><<<work, 256, 0, stream>>>((const float*)rows, row_stride, taps_w, conv_bias, a_log, dt_bias, state, state_stride, conv_offset, token_seq,
                                                          seq_starts, state_slots, prep, heads, groups, n, vdim, taps, keep);
  else
    ssd_prepare_kernel<__nv_bfloat16><<<work, 256, 0, stream>>>((const __nv_bfloat16*)rows, row_stride, taps_w, conv_bias, a_log, dt_bias, state, state_stride,
                                                                  conv_offset, token_seq, seq_starts, state_slots, prep, heads, groups, n, vdim, taps, keep);
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess || taps == 1 || keep) return (int)status;
  const dim3 grid((channels + 127) / 128, entries);
  if (dtype == TLIE_F32)
    delta_conv_state_kernel<float><<<grid, 128, 0, stream>>>((const float*)rows + inner, row_stride, state, state_stride, conv_offset, seq_starts, state_slots, channels, taps);
  else
    delta_conv_state_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)rows + inner, row_stride, state, state_stride, conv_offset, seq_starts,
                                                                     state_slots, channels, taps);
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_ssd_finish(int dtype, const float* o, const float* prep, int prep_stride, int x_offset, const void* rows, int row_stride, const float* skip,
                                const float* weight, void* out, float eps, int tokens, int heads, int vdim, int norm_groups, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int inner = heads * vdim;
  if (norm_groups < 1 || inner % norm_groups != 0 || (size_t)inner * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)inner * sizeof(float);
  if (dtype == TLIE_F32)
    ssd_finish_kernel<float><<<tokens, 256, smem, stream>>>(o, prep, prep_stride, x_offset, (const float*)rows, row_stride, skip, weight, (float*)out, eps, heads, vdim,
                                                            norm_groups);
  else
    ssd_finish_kernel<__nv_bfloat16><<<tokens, 256, smem, stream>>>(o, prep, prep_stride, x_offset, (const __nv_bfloat16*)rows, row_stride, skip, weight,
                                                                    (__nv_bfloat16*)out, eps, heads, vdim, norm_groups);
  return (int)cudaGetLastError();
}
