// Differential attention for prompt portions on the tensor cores, bfloat16 (the mathematics of attention_diff.cu).
//
// One CTA per (tile of rows of one request, head), one warp per 16 rows.  A head's two maps read key vectors 2 g and 2 g + 1 of
// its key/value head g and the same values, so a tile of 64 keys is fetched once for both: two key tiles and one value tile per
// stage, through a ring of two stages (cp.async).  Per map: Q_m . K_m^T and P_m . V on mma.sync m16n8k16 with 32-bit
// accumulators; the mask, the running maximum and sum are 32-bit.  Both maps' outputs stay in registers to the end, where
// o = a1 - lambda a2, its root mean square over the head's values and the scale are applied before the one store: nothing of the
// two maps is rounded before the difference.
//
// Compile-time: KEY_DIM, VALUE_DIM (multiples of 16).
#include "common.cuh"
#include "mma_utils.cuh"

#ifndef KEY_DIM
#define KEY_DIM 64
#endif
#ifndef VALUE_DIM
#define VALUE_DIM 64
#endif

namespace tlie {

constexpr int kD = KEY_DIM, kVD = VALUE_DIM;
constexpr int kKeys = 64;
constexpr int kKRow = kD + 8, kVRow = kVD + 8, kQRow = 2 * kD + 8;   // padded shared-memory rows (elements)
constexpr int kStages = 2;
constexpr size_t kSmemLimit = 227 * 1024;
constexpr size_t kStageElements = (size_t)2 * kKeys * kKRow + (size_t)kKeys * kVRow;
constexpr size_t smem_for(int rows) { return ((size_t)rows * kQRow + kStages * kStageElements) * sizeof(__nv_bfloat16); }
// rows per CTA: 128 where the two maps' accumulators leave registers for 256 threads' worth of them, else 64
constexpr int kRows = (kVD <= 64 && smem_for(128) <= kSmemLimit) ? 128 : (smem_for(64) <= kSmemLimit ? 64 : (smem_for(32) <= kSmemLimit ? 32 : (smem_for(16) <= kSmemLimit ? 16 : 0)));
constexpr int kWarps = kRows > 0 ? kRows / 16 : 1;
constexpr int kThreads = kWarps * 32;
constexpr float kLog2e = 1.4426950408889634f;

// one plane's rows of a tile for one head: [64][ROW] in shared memory; a page holds a multiple of 16 keys
template <int WIDTH, int ROW>
__device__ __forceinline__ void load_plane(__nv_bfloat16* smem, const __nv_bfloat16* pages, long long page_stride, const int* table, int key0, int n_keys, int head,
                                           int page_size) {
  constexpr int kChunks = WIDTH / 8;
  for (int idx = threadIdx.x; idx < kKeys * kChunks; idx += kThreads) {
    const int chunk = idx % kChunks, row = idx / kChunks;
    const int key = key0 + row;
    const bool valid = key < n_keys;
    const long long page = valid ? table[key / page_size] : 0;
    const __nv_bfloat16* src = pages + page * page_stride + ((size_t)head * page_size + key % page_size) * WIDTH + chunk * 8;
    cp_async_16(smem + (size_t)row * ROW + chunk * 8, valid ? src : pages, valid);
  }
}

constexpr int kMinBlocks = (kRows > 0 && 2 * smem_for(kRows > 0 ? kRows : 16) <= kSmemLimit && kVD <= 32) ? 2 : 1;

__global__ void __launch_bounds__(kThreads, kMinBlocks)
    diff_prefill_kernel(const __nv_bfloat16* __restrict__ rows, int row_stride, const __nv_bfloat16* __restrict__ k_pages, long long k_page_stride,
                        const __nv_bfloat16* __restrict__ v_pages, long long v_page_stride, const int* __restrict__ seq_starts,
                        const int* __restrict__ first_positions, const int* __restrict__ block_table, int table_stride, __nv_bfloat16* __restrict__ out, int heads,
                        int kv_heads, int page_size, float scale, float lambda, float eps, float out_scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [kRows][kQRow]: [map 1 | map 2] of this head
  __nv_bfloat16* ring = q_smem + (size_t)kRows * kQRow;                 // [kStages]{K map 1 [64][kKRow], K map 2, V [64][kVRow]}
  const int seq = blockIdx.y, head = blockIdx.z;
  const int seq_start = seq_starts[seq];
  const int q_len = seq_starts[seq + 1] - seq_start;
  const int row_in_seq = (gridDim.x - 1 - blockIdx.x) * kRows;   // later tiles see more keys: they start first
  if (row_in_seq >= q_len) return;
  const int row0 = seq_start + row_in_seq;
  const int kvh = head / (heads / kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rows_here = min(kRows, q_len - row_in_seq);
  const int pos0 = first_positions[seq] + row_in_seq;
  const int n_keys = pos0 + rows_here;
  const int* table = block_table + (size_t)seq * table_stride;

  constexpr int kQChunks = 2 * kD / 8;
  for (int idx = threadIdx.x; idx < kRows * kQChunks; idx += kThreads) {
    const int row = idx / kQChunks, chunk = idx - row * kQChunks;
    const bool valid = row < rows_here;
    const __nv_bfloat16* src = rows + (size_t)(row0 + (valid ? row : 0)) * row_stride + (size_t)head * 2 * kD + chunk * 8;
    cp_async_16(q_smem + (size_t)row * kQRow + chunk * 8, src, valid);
  }
  const int tiles = (n_keys + kKeys - 1) / kKeys;
  auto issue = [&](int tile) {
    if (tile < tiles) {
      __nv_bfloat16* stage = ring + (size_t)(tile % kStages) * kStageElements;
      load_plane<kD, kKRow>(stage, k_pages, k_page_stride, table, tile * kKeys, n_keys, kvh * 2, page_size);
      load_plane<kD, kKRow>(stage + (size_t)kKeys * kKRow, k_pages, k_page_stride, table, tile * kKeys, n_keys, kvh * 2 + 1, page_size);
      load_plane<kVD, kVRow>(stage + (size_t)2 * kKeys * kKRow, v_pages, v_page_stride, table, tile * kKeys, n_keys, kvh, page_size);
    }
    cp_async_commit();   // a group per tile, empty past the end
  };
  issue(0);   // in one group with the queries

  const int my_row[2] = {warp * 16 + g, warp * 16 + g + 8};
  int my_pos[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) my_pos[r] = pos0 + min(my_row[r], rows_here - 1);   // rows past the end behave like the last row; never stored
  float o[2][kVD / 8][4];
  float row_max[2][2], row_sum[2][2];
#pragma unroll
  for (int m = 0; m < 2; ++m) {
#pragma unroll
    for (int i = 0; i < kVD / 8; ++i) o[m][i][0] = o[m][i][1] = o[m][i][2] = o[m][i][3] = 0.0f;
    row_max[m][0] = row_max[m][1] = -INFINITY;
    row_sum[m][0] = row_sum[m][1] = 0.0f;
  }
  const float scale2 = scale * kLog2e;
  const int warp_last_pos = pos0 + min(warp * 16 + 15, rows_here - 1);

  for (int tile = 0; tile < tiles; ++tile) {
    issue(tile + 1);
    cp_async_wait<1>();   // everything but the tile issued ahead has landed
    __syncthreads();
    const __nv_bfloat16* stage = ring + (size_t)(tile % kStages) * kStageElements;
    const __nv_bfloat16* v_smem = stage + (size_t)2 * kKeys * kKRow;
    const int key0 = tile * kKeys;
    if (key0 <= warp_last_pos) {   // some row of this warp sees some key of this tile
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const __nv_bfloat16* k_smem = stage + (size_t)m * kKeys * kKRow;
        float s_frag[kKeys / 8][4];
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) s_frag[j][0] = s_frag[j][1] = s_frag[j][2] = s_frag[j][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) {
          unsigned qa[4];
          ldmatrix_x4(qa, q_smem + (size_t)(warp * 16 + (lane & 15)) * kQRow + m * kD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int jp = 0; jp < kKeys / 16; ++jp) {
            unsigned b[4];
            const int row = (jp * 2 + (lane >> 4)) * 8 + (lane & 7);
            const int col = ks * 16 + ((lane >> 3) & 1) * 8;
            ldmatrix_x4(b, k_smem + (size_t)row * kKRow + col);
            mma_bf16(s_frag[jp * 2], qa, b[0], b[1]);
            mma_bf16(s_frag[jp * 2 + 1], qa, b[2], b[3]);
          }
        }
        // scores in units of log2; keys after a row's position are masked
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = key0 + j * 8 + 2 * t + (e & 1);
            const int r = e >> 1;
            const float v = key <= my_pos[r] ? s_frag[j][e] * scale2 : -INFINITY;
            s_frag[j][e] = v;
            tile_max[r] = fmaxf(tile_max[r], v);
          }
        }
        float rescale[2], base[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
          tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
          const float new_max = fmaxf(row_max[m][r], tile_max[r]);
          base[r] = (new_max == -INFINITY) ? 0.0f : new_max;
          rescale[r] = exp2f(row_max[m][r] - base[r]);
          row_max[m][r] = new_max;
          row_sum[m][r] *= rescale[r];
        }
        unsigned pa[kKeys / 16][4];
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) {
          const float p0 = exp2_approx(s_frag[j][0] - base[0]);
          const float p1 = exp2_approx(s_frag[j][1] - base[0]);
          const float p2 = exp2_approx(s_frag[j][2] - base[1]);
          const float p3 = exp2_approx(s_frag[j][3] - base[1]);
          row_sum[m][0] += p0 + p1;
          row_sum[m][1] += p2 + p3;
          pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
          pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int i = 0; i < kVD / 8; ++i) {
          o[m][i][0] *= rescale[0];
          o[m][i][1] *= rescale[0];
          o[m][i][2] *= rescale[1];
          o[m][i][3] *= rescale[1];
        }
#pragma unroll
        for (int kk = 0; kk < kKeys / 16; ++kk) {
#pragma unroll
          for (int np = 0; np < kVD / 16; ++np) {
            unsigned b[4];
            const int row = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
            const int col = np * 16 + (lane >> 4) * 8;
            ldmatrix_x4_trans(b, v_smem + (size_t)row * kVRow + col);
            mma_bf16(o[m][np * 2], pa[kk], b[0], b[1]);
            mma_bf16(o[m][np * 2 + 1], pa[kk], b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();   // everyone is done with this stage before the ring comes round to it
  }
  cp_async_wait<0>();
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      row_sum[m][r] += __shfl_xor_sync(0xffffffffu, row_sum[m][r], 1);
      row_sum[m][r] += __shfl_xor_sync(0xffffffffu, row_sum[m][r], 2);
    }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const float inv1 = 1.0f / row_sum[0][r], inv2 = lambda / row_sum[1][r];
    float squares = 0.0f;
#pragma unroll
    for (int i = 0; i < kVD / 8; ++i) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const float d = o[0][i][r * 2 + c] * inv1 - o[1][i][r * 2 + c] * inv2;
        o[0][i][r * 2 + c] = d;
        squares += d * d;
      }
    }
    squares += __shfl_xor_sync(0xffffffffu, squares, 1);
    squares += __shfl_xor_sync(0xffffffffu, squares, 2);
    if (my_row[r] >= rows_here) continue;
    const float norm = out_scale / sqrtf(squares / (float)kVD + eps);
    __nv_bfloat16* dst = out + ((size_t)(row0 + my_row[r]) * heads + head) * kVD + 2 * t;
#pragma unroll
    for (int i = 0; i < kVD / 8; ++i)
      *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[0][i][r * 2] * norm, o[0][i][r * 2 + 1] * norm);
  }
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_diff_prefill_tile_rows() { return kRows; }

// ``rows`` [tokens, row_stride]: the queries, normalised and rotated, head by head as [map 1 | map 2].  ``longest``: the most rows any entry of the step has.
TLIE_EXPORT int tlie_diff_prefill(const void* rows, int row_stride, const void* k_pages, long long k_page_stride, const void* v_pages, long long v_page_stride,
                                  const int* seq_starts, const int* first_positions, const int* block_table, int table_stride, void* out, int tokens, int entries,
                                  int longest, int heads, int kv_heads, int page_size, float scale, float lambda, float eps, float out_scale, cudaStream_t stream) {
  if (tokens <= 0 || entries <= 0) return 0;
  if (kRows == 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || page_size % 16 != 0 || heads > 65535 || entries > 65535 || row_stride % 8 != 0)
    return (int)cudaErrorInvalidValue;
  constexpr size_t smem = smem_for(kRows > 0 ? kRows : 16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(diff_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tile_rows = kRows > 0 ? kRows : 16;
  const dim3 grid((longest + tile_rows - 1) / tile_rows, entries, heads);
  diff_prefill_kernel<<<grid, kThreads, smem, stream>>>((const __nv_bfloat16*)rows, row_stride, (const __nv_bfloat16*)k_pages, k_page_stride,
                                                        (const __nv_bfloat16*)v_pages, v_page_stride, seq_starts, first_positions, block_table, table_stride,
                                                        (__nv_bfloat16*)out, heads, kv_heads, page_size, scale, lambda, eps, out_scale);
  return (int)cudaGetLastError();
}
