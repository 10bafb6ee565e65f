// Routed experts for long prompt portions on the 5th-generation tensor cores, bfloat16 (the mathematics of moe.cu).
//
// The step's (token, chosen expert) pairs ("slots": token * top + k) are laid out by expert, every expert's rows starting at a
// multiple of 128, so that a 128-row tile belongs to ONE expert and the two products of all experts are two launches of a
// persistent TMA / tcgen05 kernel whose B operand starts at the tile's expert:
//
//   moe_layout     one CTA: counts per expert, their padded running sum, every slot's row, every row's token (-1: padding),
//                  and the expert of every 128-row tile.  Nothing is read back on the host: grids and scratch are sized for the
//                  most tiles there can be (slots / 128 + experts) and the kernels read the tile count on the device.
//   moe_gather     xs[row] = x[token(row)] (zeros for padding rows), so that TMA fetches an expert's rows as one box.  Where the weight
//                  multiplies what an expert reads (``weight_input``), the row is gathered times its weight and the sum below takes no weights.
//   moe_tc <GATED> act[row] = act(W_gate[e] xs[row]) * (W_up[e] xs[row])      tile 128 x (128 gate + 128 up columns)
//          <DOWN>  y[row]   = W_down[e] act[row]                               32-bit, tile 128 x 256
//   moe_tc_combine out[t] = sum_k weight[t, k] y[row(t, k)] + shared[t]: the chosen experts in the order they were chosen, so
//                  that a token's sum does not depend on what else is in the step.
// Roles (warp 0 TMA producer, warp 1 MMA issuer, warps 2..5 epilogue), the ring of stages, the two alternating accumulators in
// tensor memory and the bounded waits are those of gemm_tcgen05.cu.  Tiles are walked with the row tile fastest: the CTAs that
// run together then work on few column blocks of every expert, whose weights come from memory once and from L2 for the
// expert's other row tiles, while the gathered rows stay in L2 from one column block to the next.
#include "tcgen05_utils.cuh"

namespace tlie {

constexpr int kTcBN = 256;
constexpr int kTcStageBytes = (kBM + kTcBN) * kBK * 2;
constexpr int kTcStages = 4;
constexpr int kTcStoreBuffers = 2;
constexpr int kTcBoxBytes = kAddBoxBytes;   // the larger of the two kinds of staging boxes (32-bit)
constexpr int kTcStoreBytes = kStoreWarps * kTcStoreBuffers * kTcBoxBytes;
constexpr int kTcSmemBytes = kTcStages * kTcStageBytes + kTcStoreBytes + 1024 + 256;
constexpr int kTcTmemCols = 512;            // two accumulators of 256 columns
static_assert(kTcSmemBytes <= 227 * 1024, "shared memory of one CTA");

template <int ACT>
__device__ __forceinline__ float tc_act(float z) {
  if (ACT == 1) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z / (1.0f + expf(-z));
}

// meta: [0] number of 128-row tiles, [1 + i] the expert of tile i.  row_of_slot [slots]; token_of_row [max_rows] holds the row's slot (token * top + k).
__global__ void __launch_bounds__(1024) moe_layout_kernel(const int* __restrict__ ids, int slots, int experts, int top, int max_rows, int* __restrict__ row_of_slot,
                                                          int* __restrict__ token_of_row, int* __restrict__ meta) {
  extern __shared__ int layout_smem[];   // counts [experts], cursor [experts]
  int* counts = layout_smem;
  int* cursor = counts + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  for (int r = threadIdx.x; r < max_rows; r += blockDim.x) token_of_row[r] = -1;
  __syncthreads();
  for (int s = threadIdx.x; s < slots; s += blockDim.x) atomicAdd(&counts[ids[s]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      cursor[e] = at;
      for (int r = 0; r < counts[e]; r += kBM) meta[1 + tiles++] = e;
      at = tiles * kBM;
    }
    meta[0] = tiles;
  }
  __syncthreads();
  for (int s = threadIdx.x; s < slots; s += blockDim.x) {
    const int row = atomicAdd(&cursor[ids[s]], 1);
    row_of_slot[s] = row;
    token_of_row[row] = s;
  }
}

// a warp per row, 16 bytes a lane at a time
__global__ void __launch_bounds__(256) moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ token_of_row, const int* __restrict__ meta,
                                                         const float* __restrict__ input_weights, __nv_bfloat16* __restrict__ xs, int width, int top) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= meta[0] * kBM) return;
  const int slot = token_of_row[row];
  const int token = slot < 0 ? -1 : slot / top;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(token < 0 ? 0 : token) * width);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)row * width);
  if (input_weights == nullptr || token < 0) {
    for (int i = lane; i < width / 8; i += 32) dst[i] = token < 0 ? make_uint4(0, 0, 0, 0) : src[i];
    return;
  }
  const float w = input_weights[slot];   // the expert reads its token times the token's weight
  for (int i = lane; i < width / 8; i += 32) {
    uint4 raw = src[i];
    __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(pairs[j]);
      pairs[j] = __floats2bfloat162_rn(f.x * w, f.y * w);
    }
    dst[i] = raw;
  }
}

// One warp's 32 rows of a gated tile: act(gate) * up of 32 columns at a time as bfloat16 into a staging box, written by a bulk
// tensor store (columns past N are clipped by the tensor map).
template <int ACT>
__device__ __forceinline__ void tc_store_gated(uint32_t tmem_acc, int row0, int n0, int N, const CUtensorMap* map_out, uint8_t* staging, int lane, int& boxes) {
  const int swizzle = (lane >> 1) & 3;   // 64-byte swizzle: 16-byte chunk j of row r lies at chunk j ^ ((r / 2) % 4)
#pragma unroll 1
  for (int c = 0; c < (kTcBN / 2) / kStoreCols && n0 + c * kStoreCols < N; ++c) {
    uint32_t gate[32], up[32], packed[kStoreCols / 2];
    tmem_load_32(tmem_acc + c * kStoreCols, gate);
    tmem_load_32(tmem_acc + kTcBN / 2 + c * kStoreCols, up);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < kStoreCols / 2; ++i)
      packed[i] = pack_bf16(tc_act<ACT>(__uint_as_float(gate[2 * i])) * __uint_as_float(up[2 * i]), tc_act<ACT>(__uint_as_float(gate[2 * i + 1])) * __uint_as_float(up[2 * i + 1]));
    uint8_t* box = staging + (boxes % kTcStoreBuffers) * kTcBoxBytes;
    ++boxes;
    if (lane == 0) bulk_wait_read<kTcStoreBuffers - 1>();   // the store that last read this box is done with it
    __syncwarp();
    uint8_t* my_row = box + lane * (kStoreCols * 2);
#pragma unroll
    for (int j = 0; j < kStoreCols / 8; ++j)
      *reinterpret_cast<uint4*>(my_row + ((j ^ swizzle) << 4)) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map_out, box, n0 + c * kStoreCols, row0);
      asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    }
  }
}

// One warp's 32 rows of a 32-bit tile, 32 columns (128 bytes a row, 128-byte swizzle) per bulk tensor store.
__device__ __forceinline__ void tc_store_f32(uint32_t tmem_acc, int row0, int n0, int N, const CUtensorMap* map_out, uint8_t* staging, int lane, int& boxes) {
  const int swizzle = lane & 7;
#pragma unroll 1
  for (int c = 0; c < kTcBN / kStoreCols && n0 + c * kStoreCols < N; ++c) {
    uint32_t r[32];
    tmem_load_32(tmem_acc + c * kStoreCols, r);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
    uint8_t* box = staging + (boxes % kTcStoreBuffers) * kTcBoxBytes;
    ++boxes;
    if (lane == 0) bulk_wait_read<kTcStoreBuffers - 1>();
    __syncwarp();
    uint8_t* my_row = box + lane * (kStoreCols * 4);
#pragma unroll
    for (int j = 0; j < kStoreCols / 4; ++j) *reinterpret_cast<uint4*>(my_row + ((j ^ swizzle) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map_out, box, n0 + c * kStoreCols, row0);
      asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    }
  }
}

// GATED: a = gathered rows [rows, K = width], b = gate_up [experts * 2 N, K] with N = ff, out = act bfloat16 [rows, N].
// DOWN:  a = act [rows, K = ff], b = down [experts * N, K] with N = width, out = y 32-bit [rows, N].
// Rows of B past an expert's own (the last column block of an N that is no multiple of the tile) belong to the next expert or are
// filled with zeros; their columns are never stored.
template <bool GATED, int ACT>
__global__ void __launch_bounds__(kGemmThreads)
    moe_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_out,
                  const int* __restrict__ meta, int N, int K, int* __restrict__ error_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzled tiles need 1024-byte alignment
  uint8_t* staging = tiles + kTcStages * kTcStageBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + kTcStoreBytes);
  uint64_t* empty = full + kTcStages;
  uint64_t* accum_full = empty + kTcStages;    // [2]: the MMAs of a tile are done
  uint64_t* accum_empty = accum_full + 2;      // [2]: the epilogue has read the accumulator
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kTileN = GATED ? kTcBN / 2 : kTcBN;   // output columns of a tile
  const int n_blocks = (N + kTileN - 1) / kTileN;
  const int k_blocks = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&accum_full[a], 1);
      mbar_init(&accum_empty[a], 4);   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_holder)), "r"(kTcTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;
  grid_launch_dependents();
  grid_dependency_wait();   // the layout, the gathered rows and (DOWN) the activations are the kernels' before this one
  const int m_tiles = meta[0];
  const int num_tiles = m_tiles * n_blocks;

  if (warp == 0) {
    if (lane == 0) {   // TMA producer
      RingPosition<kTcStages> ring;
      const uint32_t tiles_addr = smem_u32(tiles), full_addr = smem_u32(full), empty_addr = smem_u32(empty);
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m_tile = tile % m_tiles, n0 = (tile / m_tiles) * kTileN;
        const int b_row = meta[1 + m_tile] * (GATED ? 2 * N : N) + n0;
        for (int kb = 0; kb < k_blocks; ++kb, ring.advance()) {
          ok = mbar_wait(empty_addr + 8 * ring.stage, ring.phase ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t a_tile = tiles_addr + ring.stage * kTcStageBytes, b_tile = a_tile + kBM * kBK * 2;
          const uint32_t bar = full_addr + 8 * ring.stage;
          mbar_expect_tx(bar, kTcStageBytes);
          tma_load_2d(a_tile, &map_a, kb * kBK, m_tile * kBM, bar);
          if (GATED) {
            tma_load_2d(b_tile, &map_b, kb * kBK, b_row, bar);                                   // gate rows
            tma_load_2d(b_tile + (kTcBN / 2) * kBK * 2, &map_b, kb * kBK, b_row + N, bar);      // up rows
          } else {
            tma_load_2d(b_tile, &map_b, kb * kBK, b_row, bar);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {   // MMA issuer
      constexpr uint32_t idesc = umma_instr_desc(kBM, kTcBN);
      RingPosition<kTcStages> ring;
      const uint32_t tiles_low = umma_desc_low(smem_u32(tiles)), full_addr = smem_u32(full), empty_addr = smem_u32(empty);
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        ok = mbar_wait(&accum_empty[acc], ((local >> 1) & 1) ^ 1, abort_flag);   // the epilogue has drained this accumulator
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_acc = tmem_base + acc * kTcBN;
        for (int kb = 0; kb < k_blocks; ++kb, ring.advance()) {
          ok = mbar_wait(full_addr + 8 * ring.stage, ring.phase, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t a_low = tiles_low + ring.stage * (kTcStageBytes >> 4), b_low = a_low + ((kBM * kBK * 2) >> 4);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)   // 16 k = 32 bytes further inside the 128-byte swizzle span
            umma_bf16(tmem_acc, a_low + k * ((kUmmaK * 2) >> 4), b_low + k * ((kUmmaK * 2) >> 4), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty_addr + 8 * ring.stage);   // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(&accum_full[acc]);
      }
    }
  }
  if (warp >= 2) {   // epilogue: warp w reads tensor-memory lanes 32 * (w % 4) ... + 31
    const int sub = warp & 3;
    uint8_t* my_staging = staging + sub * kTcStoreBuffers * kTcBoxBytes;
    int local = 0, boxes = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const int m0 = (tile % m_tiles) * kBM, n0 = (tile / m_tiles) * kTileN;
      if (!mbar_wait(&accum_full[acc], (local >> 1) & 1, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t tmem_acc = tmem_base + acc * kTcBN + ((uint32_t)(sub * 32) << 16);
      if (GATED)
        tc_store_gated<ACT>(tmem_acc, m0 + sub * 32, n0, N, &map_out, my_staging, lane, boxes);
      else
        tc_store_f32(tmem_acc, m0 + sub * 32, n0, N, &map_out, my_staging, lane, boxes);
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&accum_empty[acc])) : "memory");
    }
    if (lane == 0) bulk_wait_all();   // this warp's staging boxes have been read and written out
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  }
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(error_flag, 1);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // copies in flight may still be landing in this CTA's shared memory
  }
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTcTmemCols));
  }
}

// four columns a thread
__global__ void __launch_bounds__(256) moe_tc_combine_kernel(const float* __restrict__ y, const int* __restrict__ row_of_slot, const float* __restrict__ weights,
                                                             const __nv_bfloat16* __restrict__ shared, __nv_bfloat16* __restrict__ out, int width, int top, size_t quads) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / (width / 4);
    const int n = (int)(i - t * (width / 4)) * 4;
    float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int k = 0; k < top; ++k) {
      const float w = weights != nullptr ? weights[t * top + k] : 1.0f;
      const float4 v = *reinterpret_cast<const float4*>(y + (size_t)row_of_slot[t * top + k] * width + n);
      sum.x = fmaf(w, v.x, sum.x);
      sum.y = fmaf(w, v.y, sum.y);
      sum.z = fmaf(w, v.z, sum.z);
      sum.w = fmaf(w, v.w, sum.w);
    }
    if (shared != nullptr) {
      const uint2 s = *reinterpret_cast<const uint2*>(shared + t * width + n);
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&s.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&s.y);
      sum.x += __low2float(lo);
      sum.y += __high2float(lo);
      sum.z += __low2float(hi);
      sum.w += __high2float(hi);
    }
    uint2 packed;
    packed.x = pack_bf16(sum.x, sum.y);
    packed.y = pack_bf16(sum.z, sum.w);
    *reinterpret_cast<uint2*>(out + t * width + n) = packed;
  }
}

template <bool GATED, int ACT>
static int launch_moe_tc(const void* a, const void* b, void* out, const int* meta, int max_rows, int b_rows, int N, int K, int* error_flag, cudaStream_t stream) {
  CUtensorMap map_a, map_b, map_out;
  if (!make_map(&map_a, a, max_rows, K, kBM) || !make_map(&map_b, b, b_rows, K, GATED ? kTcBN / 2 : kTcBN)) return (int)cudaErrorInvalidValue;
  if (!(GATED ? make_store_map(&map_out, out, max_rows, N) : make_add_map(&map_out, out, max_rows, N))) return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_tc_kernel<GATED, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  constexpr int kTileN = GATED ? kTcBN / 2 : kTcBN;
  const long long most = (long long)(max_rows / kBM) * ((N + kTileN - 1) / kTileN);
  const int sm_count = device_sm_count();
  return (int)launch_pdl(moe_tc_kernel<GATED, ACT>, dim3((unsigned)(most < sm_count ? most : sm_count)), dim3(kGemmThreads), kTcSmemBytes, stream, map_a, map_b, map_out,
                         meta, N, K, error_flag);
}

}  // namespace tlie

using namespace tlie;

// Scratch, with max_rows = (tokens * top / 128 + experts) * 128: row_of_slot int32 [tokens * top], token_of_row int32 [max_rows],
// meta int32 [1 + max_rows / 128], xs bfloat16 [max_rows, width], act bfloat16 [max_rows, ff], y 32-bit [max_rows, width].
// ``shared`` bfloat16 [tokens, width] or null.  All of 16-byte aligned bases; width and ff multiples of 8.
TLIE_EXPORT int tlie_moe_grouped_tc(const void* x, const void* gate_up, const void* down, const int* ids, const float* weights, const void* shared, int* row_of_slot,
                                    int* token_of_row, int* meta, void* xs, void* act, float* y, void* out, int tokens, int width, int ff, int experts, int top,
                                    int kind, int weight_input, int* error_flag, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const long long slots = (long long)tokens * top;
  if (width % 8 != 0 || ff % 8 != 0 || experts <= 0 || experts > 4096 || slots > (1LL << 30) || kind < 0 || kind > 1 || error_flag == nullptr) return (int)cudaErrorInvalidValue;
  if ((long long)experts * 2 * ff > 2147483647LL || (long long)experts * width > 2147483647LL) return (int)cudaErrorInvalidValue;
  const int max_rows = ((int)(slots / kBM) + experts) * kBM;
  moe_layout_kernel<<<1, 1024, 2 * experts * sizeof(int), stream>>>(ids, (int)slots, experts, top, max_rows, row_of_slot, token_of_row, meta);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  moe_gather_kernel<<<max_rows / 8, 256, 0, stream>>>((const __nv_bfloat16*)x, token_of_row, meta, weight_input ? weights : nullptr, (__nv_bfloat16*)xs, width, top);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  int rc = kind == 1 ? launch_moe_tc<true, 1>(xs, gate_up, act, meta, max_rows, experts * 2 * ff, ff, width, error_flag, stream)
                     : launch_moe_tc<true, 0>(xs, gate_up, act, meta, max_rows, experts * 2 * ff, ff, width, error_flag, stream);
  if (rc != 0) return rc;
  rc = launch_moe_tc<false, 0>(act, down, y, meta, max_rows, experts * width, width, ff, error_flag, stream);
  if (rc != 0) return rc;
  const size_t quads = (size_t)tokens * (width / 4);
  const size_t blocks = (quads + 255) / 256;
  const size_t most = (size_t)device_sm_count() * 16;
  moe_tc_combine_kernel<<<(int)(blocks < most ? blocks : most), 256, 0, stream>>>(y, row_of_slot, weight_input ? nullptr : weights, (const __nv_bfloat16*)shared, (__nv_bfloat16*)out, width, top, quads);
  return (int)cudaGetLastError();
}
