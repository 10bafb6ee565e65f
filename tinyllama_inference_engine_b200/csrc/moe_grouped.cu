// Routed experts for prompt portions on the tensor cores, bfloat16 (the mathematics of moe.cu).
//
// The step's (token, chosen expert) pairs ("slots": token * top + k) are sorted by expert, so that every expert's rows lie
// together; then every expert is two products over its own rows, cut into tiles of 64 rows:
//
//   moe_sort     one CTA: counts per expert, their running sum, the slots in expert order, and the list of row tiles
//                (expert, first row, rows); nothing is read back on the host, the grids are sized for the most tiles there can be.
//   moe_grouped  <GATED>  act[p] = act(W_gate[e] x[token(p)]) * (W_up[e] x[token(p)])       for the sorted rows p of expert e
//                <DOWN>   y[slot(p)] = weight[slot(p)] * W_down[e] act[p]                    32-bit, by slot
//                ``weight_input``: the weight multiplies what the expert reads instead (its two first products are linear in it, so
//                act(w g) * (w u) in the gated epilogue, 32-bit, and no weight behind W_down)
//                64 x 64 tiles (the gated one: 64 gate and the 64 up columns beside them), k in blocks of 32 through two cp.async
//                stages, mma.sync m16n8k16 with 32-bit accumulators, a warp per 16 rows.
//   moe_combine  out[t] = sum_k y[t * top + k] + shared[t]: the chosen experts in the order they were chosen, so that a row's
//                sum does not depend on what else is in the step.
#include "common.cuh"
#include "mma_utils.cuh"

namespace tlie {

constexpr int kGM = 64, kGN = 64, kGK = 32;
constexpr int kGRow = kGK + 8;   // padded shared-memory rows (elements)
constexpr int kGThreads = 128;

__device__ __forceinline__ float grouped_act(float z, int kind) {
  if (kind == 1) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z / (1.0f + expf(-z));
}

// meta: [0] number of tiles, then (expert, first sorted row, rows) per tile
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ ids, int slots, int experts, int* __restrict__ sorted_slots, int* __restrict__ meta) {
  extern __shared__ int sort_smem[];   // counts [experts], cursor [experts]
  int* counts = sort_smem;
  int* cursor = counts + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int s = threadIdx.x; s < slots; s += blockDim.x) atomicAdd(&counts[ids[s]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      cursor[e] = at;
      for (int r = 0; r < counts[e]; r += kGM) {
        meta[1 + 3 * tiles] = e;
        meta[2 + 3 * tiles] = at + r;
        meta[3 + 3 * tiles] = min(kGM, counts[e] - r);
        ++tiles;
      }
      at += counts[e];
    }
    meta[0] = tiles;
  }
  __syncthreads();
  for (int s = threadIdx.x; s < slots; s += blockDim.x) sorted_slots[atomicAdd(&cursor[ids[s]], 1)] = s;
}

// GATED: a [tokens][K] gathered by slot / top, w [experts][2 N][K], out bfloat16 [slots][N] by sorted row.
// DOWN:  a [slots][K] by sorted row, w [experts][N][K], out 32-bit [slots][N] by slot, times the slot's weight.
template <bool GATED>
__global__ void __launch_bounds__(kGThreads) moe_grouped_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w, const int* __restrict__ sorted_slots,
                                                                const int* __restrict__ meta, const float* __restrict__ weights, void* __restrict__ out, int N, int K,
                                                                int top, int kind, int weight_input) {
  constexpr int kB = GATED ? 2 : 1;
  __shared__ __align__(16) __nv_bfloat16 a_s[2][kGM][kGRow];
  __shared__ __align__(16) __nv_bfloat16 b_s[2][kB][kGN][kGRow];
  __shared__ int row_slot[kGM];
  const int tile = blockIdx.x;
  if (tile >= meta[0]) return;
  const int expert = meta[1 + 3 * tile], row0 = meta[2 + 3 * tile], rows = meta[3 + 3 * tile];
  const int n0 = blockIdx.y * kGN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < kGM) row_slot[threadIdx.x] = threadIdx.x < rows ? sorted_slots[row0 + threadIdx.x] : 0;
  __syncthreads();
  const __nv_bfloat16* w_e = w + (size_t)expert * (GATED ? 2 : 1) * N * K;
  auto issue = [&](int kb) {
    const int k0 = kb * kGK;
    if (k0 < K) {
      const int stage = kb & 1;
      for (int idx = threadIdx.x; idx < kGM * (kGK / 8); idx += kGThreads) {
        const int row = idx / (kGK / 8), chunk = idx % (kGK / 8);
        const bool valid = row < rows && k0 + chunk * 8 < K;
        const size_t source = GATED ? (size_t)(row_slot[row] / top) : (size_t)(row0 + row);
        cp_async_16(&a_s[stage][row][chunk * 8], valid ? a + source * K + k0 + chunk * 8 : a, valid);
      }
      for (int idx = threadIdx.x; idx < kB * kGN * (kGK / 8); idx += kGThreads) {
        const int chunk = idx % (kGK / 8), row = (idx / (kGK / 8)) % kGN, half = idx / (kGK / 8 * kGN);
        const bool valid = n0 + row < N && k0 + chunk * 8 < K;
        cp_async_16(&b_s[stage][half][row][chunk * 8], valid ? w_e + ((size_t)half * N + n0 + row) * K + k0 + chunk * 8 : w_e, valid);
      }
    }
    cp_async_commit();
  };
  float acc[kB][kGN / 8][4];
#pragma unroll
  for (int h = 0; h < kB; ++h)
#pragma unroll
    for (int j = 0; j < kGN / 8; ++j) acc[h][j][0] = acc[h][j][1] = acc[h][j][2] = acc[h][j][3] = 0.0f;
  const int k_blocks = (K + kGK - 1) / kGK;
  issue(0);
  for (int kb = 0; kb < k_blocks; ++kb) {
    issue(kb + 1);
    cp_async_wait<1>();
    __syncthreads();
    const int stage = kb & 1;
#pragma unroll
    for (int ks = 0; ks < kGK / 16; ++ks) {
      unsigned qa[4];
      ldmatrix_x4(qa, &a_s[stage][warp * 16 + (lane & 15)][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int h = 0; h < kB; ++h)
#pragma unroll
        for (int jp = 0; jp < kGN / 16; ++jp) {
          unsigned b[4];
          ldmatrix_x4(b, &b_s[stage][h][(jp * 2 + (lane >> 4)) * 8 + (lane & 7)][ks * 16 + ((lane >> 3) & 1) * 8]);
          mma_bf16(acc[h][jp * 2], qa, b[0], b[1]);
          mma_bf16(acc[h][jp * 2 + 1], qa, b[2], b[3]);
        }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + 8 * r;
    if (row >= rows) continue;
    if (GATED) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)(row0 + row) * N;
      const float scale = weight_input ? weights[row_slot[row]] : 1.0f;
#pragma unroll
      for (int j = 0; j < kGN / 8; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + j * 8 + 2 * t + c;
          if (n < N) dst[n] = __float2bfloat16_rn(grouped_act(scale * acc[0][j][r * 2 + c], kind) * (scale * acc[kB - 1][j][r * 2 + c]));
        }
    } else {
      const int slot = row_slot[row];
      const float weight = weight_input ? 1.0f : weights[slot];
      float* dst = reinterpret_cast<float*>(out) + (size_t)slot * N;
#pragma unroll
      for (int j = 0; j < kGN / 8; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + j * 8 + 2 * t + c;
          if (n < N) dst[n] = weight * acc[0][j][r * 2 + c];
        }
    }
  }
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const __nv_bfloat16* __restrict__ shared, __nv_bfloat16* __restrict__ out, int width, int top, size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width;
    const int n = (int)(i - t * width);
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) sum += y[(t * top + k) * width + n];
    if (shared != nullptr) sum += __bfloat162float(shared[i]);
    out[i] = __float2bfloat16_rn(sum);
  }
}

}  // namespace tlie

using namespace tlie;

// Scratch: sorted_slots int32 [tokens * top], meta int32 [1 + 3 * (tokens * top / 64 + experts)], act bfloat16 [tokens * top, ff],
// y 32-bit [tokens * top, width].  ``shared`` bfloat16 [tokens, width] or null.
TLIE_EXPORT int tlie_moe_grouped(const void* x, const void* gate_up, const void* down, const int* ids, const float* weights, const void* shared, int* sorted_slots,
                                 int* meta, void* act, float* y, void* out, int tokens, int width, int ff, int experts, int top, int kind, int weight_input,
                                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const long long slots = (long long)tokens * top;
  if (width % 8 != 0 || ff % 8 != 0 || experts <= 0 || experts > 4096 || slots > (1LL << 30) || kind < 0 || kind > 1) return (int)cudaErrorInvalidValue;
  const int max_tiles = (int)(slots / kGM) + experts;
  moe_sort_kernel<<<1, 1024, 2 * experts * sizeof(int), stream>>>(ids, (int)slots, experts, sorted_slots, meta);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  moe_grouped_kernel<true><<<dim3(max_tiles, (ff + kGN - 1) / kGN), kGThreads, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate_up, sorted_slots, meta,
                                                                                            weights, act, ff, width, top, kind, weight_input);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  moe_grouped_kernel<false><<<dim3(max_tiles, (width + kGN - 1) / kGN), kGThreads, 0, stream>>>((const __nv_bfloat16*)act, (const __nv_bfloat16*)down, sorted_slots, meta,
                                                                                                weights, y, width, ff, top, kind, weight_input);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const size_t total = (size_t)tokens * width;
  const size_t blocks = (total + 255) / 256;
  const size_t most = (size_t)device_sm_count() * 16;
  moe_combine_kernel<<<(int)(blocks < most ? blocks : most), 256, 0, stream>>>(y, (const __nv_bfloat16*)shared, (__nv_bfloat16*)out, width, top, total);
  return (int)cudaGetLastError();
}
