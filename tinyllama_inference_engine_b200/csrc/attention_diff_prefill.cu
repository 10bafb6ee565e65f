// Differential attention for prompt portions on the tensor cores, bfloat16 (the mathematics of attention_diff.cu).
//
// One CTA per (tile of rows of one request, head); TWO warps per 16 rows, one for each of the head's two maps.  The maps read key
// vectors 2 g and 2 g + 1 of the head's key/value head g and the same values, so a tile of 64 keys is fetched once for both: two key
// tiles and one value tile per stage, through a ring of two stages (cp.async).  A warp computes Q_m . K_m^T and P_m . V of its map on
// mma.sync m16n8k16 with 32-bit accumulators; the mask, the running maximum and sum are 32-bit.  (One warp for both maps was built
// first: its 2 x 16 x VALUE_DIM accumulators took 255 registers at a value width of 128, eight warps an SM were all that fitted,
// and they issued an instruction in 37% of the cycles with the tensor pipe busy in 17%.)  At the end the second map's warp hands
// lambda a2 over in shared memory as 32-bit numbers and the first map's warp forms o = a1 - lambda a2, takes its root mean square
// over the head's values and stores once: nothing of the two maps is rounded before the difference.
// Tiles that lie wholly before a warp's first row skip the mask; the accumulators are rescaled only when a maximum moved.
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
constexpr int kXRow = kVD + 8;                                       // a row of the second map's hand-over (32-bit words)
constexpr int kStages = 2;
constexpr size_t kSmemLimit = 227 * 1024;
constexpr size_t kStageElements = (size_t)2 * kKeys * kKRow + (size_t)kKeys * kVRow;
constexpr size_t max_of(size_t a, size_t b) { return a > b ? a : b; }
// the hand-over reuses the ring once the last tile is done
constexpr size_t smem_for(int rows) { return (size_t)rows * kQRow * sizeof(__nv_bfloat16) + max_of(kStages * kStageElements * sizeof(__nv_bfloat16), (size_t)rows * kXRow * sizeof(float)); }
// rows per CTA.  Sixteen warps an SM are the aim: 128 rows for narrow values; else two CTAs of 64 rows where two fit, one of 128 rows
// where only that fits and the accumulators (VALUE_DIM / 2 registers a thread) leave room for 512 threads; else what fits.
constexpr int kRows = (kVD <= 64 && smem_for(128) <= kSmemLimit) ? 128
                    : (kVD <= 128 && 2 * smem_for(64) > kSmemLimit && smem_for(128) <= kSmemLimit) ? 128
                    : (smem_for(64) <= kSmemLimit ? 64 : (smem_for(32) <= kSmemLimit ? 32 : (smem_for(16) <= kSmemLimit ? 16 : 0)));
constexpr int kWarps = kRows > 0 ? 2 * (kRows / 16) : 2;
constexpr int kThreads = kWarps * 32;
constexpr float kLog2e = 1.4426950408889634f;

// a key's page and place in it: pages of a power of two keys (``page_shift`` >= 0) need no division
__device__ __forceinline__ void place_of(int key, int page_size, int page_shift, int& page_index, int& slot) {
  if (page_shift >= 0) {
    page_index = key >> page_shift;
    slot = key & (page_size - 1);
  } else {
    page_index = key / page_size;
    slot = key - page_index * page_size;
  }
}

// one plane's rows of a tile for one head: [64][ROW] in shared memory; a page holds a multiple of 16 keys
template <int WIDTH, int ROW, int THREADS>
__device__ __forceinline__ void load_plane(__nv_bfloat16* smem, const __nv_bfloat16* pages, long long page_stride, const int* table, int key0, int n_keys, int head,
                                           int page_size, int page_shift, int thread) {
  constexpr int kChunks = WIDTH / 8;
#pragma unroll
  for (int idx0 = 0; idx0 < kKeys * kChunks; idx0 += THREADS) {
    const int idx = idx0 + thread;
    if ((kKeys * kChunks) % THREADS != 0 && idx >= kKeys * kChunks) break;
    const int chunk = idx % kChunks, row = idx / kChunks;
    const int key = key0 + row;
    const bool valid = key < n_keys;
    int page_index, slot;
    place_of(valid ? key : 0, page_size, page_shift, page_index, slot);
    const long long page = valid ? table[page_index] : 0;
    const __nv_bfloat16* src = pages + page * page_stride + ((size_t)head * page_size + slot) * WIDTH + chunk * 8;
    cp_async_16(smem + (size_t)row * ROW + chunk * 8, valid ? src : pages, valid);
  }
}

constexpr int kMinBlocks = (kRows > 0 && kThreads <= 256 && 2 * smem_for(kRows > 0 ? kRows : 16) <= kSmemLimit && kVD <= 128) ? 2 : 1;

__global__ void __launch_bounds__(kThreads, kMinBlocks)
    diff_prefill_kernel(const __nv_bfloat16* __restrict__ rows, int row_stride, const __nv_bfloat16* __restrict__ k_pages, long long k_page_stride,
                        const __nv_bfloat16* __restrict__ v_pages, long long v_page_stride, const int* __restrict__ seq_starts,
                        const int* __restrict__ first_positions, const int* __restrict__ block_table, int table_stride, __nv_bfloat16* __restrict__ out, int heads,
                        int kv_heads, int page_size, int page_shift, float scale, float lambda, float eps, float out_scale) {
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
  const int row_warp = warp >> 1, m = warp & 1;   // the warp's 16 rows and its map
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
      load_plane<kD, kKRow, kThreads>(stage, k_pages, k_page_stride, table, tile * kKeys, n_keys, kvh * 2, page_size, page_shift, threadIdx.x);
      load_plane<kD, kKRow, kThreads>(stage + (size_t)kKeys * kKRow, k_pages, k_page_stride, table, tile * kKeys, n_keys, kvh * 2 + 1, page_size, page_shift, threadIdx.x);
      load_plane<kVD, kVRow, kThreads>(stage + (size_t)2 * kKeys * kKRow, v_pages, v_page_stride, table, tile * kKeys, n_keys, kvh, page_size, page_shift, threadIdx.x);
    }
    cp_async_commit();   // a group per tile, empty past the end
  };
  issue(0);   // in one group with the queries

  const int my_row[2] = {row_warp * 16 + g, row_warp * 16 + g + 8};
  int my_pos[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) my_pos[r] = pos0 + min(my_row[r], rows_here - 1);   // rows past the end behave like the last row; never stored
  float o[kVD / 8][4];
#pragma unroll
  for (int i = 0; i < kVD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
  const float scale2 = scale * kLog2e;
  const int warp_first_pos = pos0 + min(row_warp * 16, rows_here - 1);
  const int warp_last_pos = pos0 + min(row_warp * 16 + 15, rows_here - 1);

  for (int tile = 0; tile < tiles; ++tile) {
    issue(tile + 1);
    cp_async_wait<1>();   // everything but the tile issued ahead has landed
    __syncthreads();
    const __nv_bfloat16* stage = ring + (size_t)(tile % kStages) * kStageElements;
    const __nv_bfloat16* v_smem = stage + (size_t)2 * kKeys * kKRow;
    const __nv_bfloat16* k_smem = stage + (size_t)m * kKeys * kKRow;
    const int key0 = tile * kKeys;
    if (key0 <= warp_last_pos) {   // some row of this warp sees some key of this tile
      float s_frag[kKeys / 8][4];
#pragma unroll
      for (int j = 0; j < kKeys / 8; ++j) s_frag[j][0] = s_frag[j][1] = s_frag[j][2] = s_frag[j][3] = 0.0f;
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) {
        unsigned qa[4];
        ldmatrix_x4(qa, q_smem + (size_t)(row_warp * 16 + (lane & 15)) * kQRow + m * kD + ks * 16 + (lane >> 4) * 8);
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
      // scores in units of log2; keys after a row's position are masked (only tiles that reach past the warp's first row have any)
      float tile_max[2] = {-INFINITY, -INFINITY};
      if (key0 + kKeys - 1 > warp_first_pos) {
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
      } else {
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float v = s_frag[j][e] * scale2;
            s_frag[j][e] = v;
            tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
          }
        }
      }
      float rescale[2], base[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        const float new_max = fmaxf(row_max[r], tile_max[r]);
        base[r] = (new_max == -INFINITY) ? 0.0f : new_max;
        rescale[r] = exp2f(row_max[r] - base[r]);
        row_max[r] = new_max;
        row_sum[r] *= rescale[r];
      }
      unsigned pa[kKeys / 16][4];
#pragma unroll
      for (int j = 0; j < kKeys / 8; ++j) {
        const float p0 = exp2_approx(s_frag[j][0] - base[0]);
        const float p1 = exp2_approx(s_frag[j][1] - base[0]);
        const float p2 = exp2_approx(s_frag[j][2] - base[1]);
        const float p3 = exp2_approx(s_frag[j][3] - base[1]);
        row_sum[0] += p0 + p1;
        row_sum[1] += p2 + p3;
        pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
        pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
      if (__any_sync(0xffffffffu, rescale[0] != 1.0f || rescale[1] != 1.0f)) {   // a maximum moved somewhere in the warp's rows
#pragma unroll
        for (int i = 0; i < kVD / 8; ++i) {
          o[i][0] *= rescale[0];
          o[i][1] *= rescale[0];
          o[i][2] *= rescale[1];
          o[i][3] *= rescale[1];
        }
      }
#pragma unroll
      for (int kk = 0; kk < kKeys / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < kVD / 16; ++np) {
          unsigned b[4];
          const int row = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
          const int col = np * 16 + (lane >> 4) * 8;
          ldmatrix_x4_trans(b, v_smem + (size_t)row * kVRow + col);
          mma_bf16(o[np * 2], pa[kk], b[0], b[1]);
          mma_bf16(o[np * 2 + 1], pa[kk], b[2], b[3]);
        }
      }
    }
    __syncthreads();   // everyone is done with this stage before the ring comes round to it
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
  }
  // the ring is free (the loop ended on a barrier, nothing is in flight): the second map's lambda a2 crosses it as 32-bit numbers
  float* hand_over = reinterpret_cast<float*>(ring);
  if (m == 1) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float inv2 = lambda / row_sum[r];
      float* dst = hand_over + (size_t)my_row[r] * kXRow + 2 * t;
#pragma unroll
      for (int i = 0; i < kVD / 8; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][r * 2] * inv2, o[i][r * 2 + 1] * inv2);
    }
  }
  __syncthreads();
  if (m == 1) return;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const float inv1 = 1.0f / row_sum[r];
    const float* other = hand_over + (size_t)my_row[r] * kXRow + 2 * t;
    float squares = 0.0f;
#pragma unroll
    for (int i = 0; i < kVD / 8; ++i) {
      const float2 a2 = *reinterpret_cast<const float2*>(other + i * 8);
      const float d0 = o[i][r * 2] * inv1 - a2.x, d1 = o[i][r * 2 + 1] * inv1 - a2.y;
      o[i][r * 2] = d0;
      o[i][r * 2 + 1] = d1;
      squares += d0 * d0 + d1 * d1;
    }
    squares += __shfl_xor_sync(0xffffffffu, squares, 1);
    squares += __shfl_xor_sync(0xffffffffu, squares, 2);
    if (my_row[r] >= rows_here) continue;
    const float norm = out_scale / sqrtf(squares / (float)kVD + eps);
    __nv_bfloat16* dst = out + ((size_t)(row0 + my_row[r]) * heads + head) * kVD + 2 * t;
#pragma unroll
    for (int i = 0; i < kVD / 8; ++i)
      *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][r * 2] * norm, o[i][r * 2 + 1] * norm);
  }
}

// --- steps of few rows per entry (decoded tokens, short portions) ----------------------------------------------------------------
// The rows of the products are the HEADS of one token's key/value group (up to 16 a chunk), all at the token's position.  A CTA of
// four warps takes tiles of 64 keys (tile p, p + parts, ...; usually one) through the same ring as above; warp w works on map w & 1
// and on one half of the value columns (both halves compute the map's scores, which are cheap beside waiting for the tile), and
// writes its running maximum, sum and weighted values as one part per (head, map).  The parts are joined, subtracted and
// normalised by diff_merge (attention_diff.cu), as the general kernel's are.
constexpr int kDecThreads = 128;
constexpr int kPairs = kVD / 16;                 // pairs of 8-column blocks of the values
constexpr int kHalfPairs = (kPairs + 1) / 2;     // a warp's share
constexpr size_t dec_smem_for(int stages) { return ((size_t)16 * kQRow + (size_t)stages * kStageElements) * sizeof(__nv_bfloat16); }
constexpr int kDecStages = dec_smem_for(2) <= kSmemLimit ? 2 : (dec_smem_for(1) <= kSmemLimit ? 1 : 0);

// grid (tokens, kv heads * chunks of 16 heads, CTAs along the keys); parts: [token][part][2 H][kVD + 2] = (max in powers of two, sum, weighted values)
__global__ void __launch_bounds__(kDecThreads)
    diff_decode_kernel(const __nv_bfloat16* __restrict__ rows, int row_stride, const __nv_bfloat16* __restrict__ k_pages, long long k_page_stride,
                       const __nv_bfloat16* __restrict__ v_pages, long long v_page_stride, const int* __restrict__ positions, const int* __restrict__ token_seq,
                       const int* __restrict__ block_table, int table_stride, float* __restrict__ parts, int heads, int kv_heads, int page_size, int page_shift,
                       float scale) {
  constexpr int kRing = kDecStages > 0 ? kDecStages : 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [16 heads][kQRow]: [map 1 | map 2]
  __nv_bfloat16* ring = q_smem + (size_t)16 * kQRow;
  const int token = blockIdx.x;
  const int group = heads / kv_heads, chunks = (group + 15) / 16;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y - kvh * chunks;
  const int head0 = kvh * group + chunk * 16;
  const int heads_here = min(16, group - chunk * 16);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = warp & 1, half = warp >> 1;
  const int g = lane >> 2, t = lane & 3;
  const int total_parts = gridDim.z, part = blockIdx.z;
  const int pos = positions[token];
  const int n_keys = pos + 1;
  const int* table = block_table + (size_t)token_seq[token] * table_stride;
  const int tiles = (n_keys + kKeys - 1) / kKeys;

  constexpr int kQChunks = 2 * kD / 8;
  for (int idx = threadIdx.x; idx < 16 * kQChunks; idx += kDecThreads) {
    const int row = idx / kQChunks, chunk_q = idx - row * kQChunks;
    const bool valid = row < heads_here;
    const __nv_bfloat16* src = rows + (size_t)token * row_stride + (size_t)(head0 + (valid ? row : 0)) * 2 * kD + chunk_q * 8;
    cp_async_16(q_smem + (size_t)row * kQRow + chunk_q * 8, src, valid);
  }
  auto issue = [&](int tile) {
    if (tile < tiles) {
      __nv_bfloat16* stage = ring + (size_t)((tile / total_parts) % kRing) * kStageElements;
      load_plane<kD, kKRow, kDecThreads>(stage, k_pages, k_page_stride, table, tile * kKeys, n_keys, kvh * 2, page_size, page_shift, threadIdx.x);
      load_plane<kD, kKRow, kDecThreads>(stage + (size_t)kKeys * kKRow, k_pages, k_page_stride, table, tile * kKeys, n_keys, kvh * 2 + 1, page_size, page_shift, threadIdx.x);
      load_plane<kVD, kVRow, kDecThreads>(stage + (size_t)2 * kKeys * kKRow, v_pages, v_page_stride, table, tile * kKeys, n_keys, kvh, page_size, page_shift, threadIdx.x);
    }
    cp_async_commit();   // a group per tile, empty past the end
  };
  issue(part);   // in one group with the queries

  float o[2 * kHalfPairs][4];
#pragma unroll
  for (int i = 0; i < 2 * kHalfPairs; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
  const float scale2 = scale * kLog2e;
  for (int tile = part; tile < tiles; tile += total_parts) {
    if (kRing > 1) {
      issue(tile + total_parts);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* stage = ring + (size_t)((tile / total_parts) % kRing) * kStageElements;
    const __nv_bfloat16* k_smem = stage + (size_t)m * kKeys * kKRow;
    const __nv_bfloat16* v_smem = stage + (size_t)2 * kKeys * kKRow;
    const int key0 = tile * kKeys;
    float s_frag[kKeys / 8][4];
#pragma unroll
    for (int j = 0; j < kKeys / 8; ++j) s_frag[j][0] = s_frag[j][1] = s_frag[j][2] = s_frag[j][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
      unsigned qa[4];
      ldmatrix_x4(qa, q_smem + (size_t)(lane & 15) * kQRow + m * kD + ks * 16 + (lane >> 4) * 8);
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
    float tile_max_r[2] = {-INFINITY, -INFINITY};   // every row is at the token's position: one mask, but a maximum per row
#pragma unroll
    for (int j = 0; j < kKeys / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + j * 8 + 2 * t + (e & 1);
        const float v = key <= pos ? s_frag[j][e] * scale2 : -INFINITY;
        s_frag[j][e] = v;
        tile_max_r[e >> 1] = fmaxf(tile_max_r[e >> 1], v);
      }
    }
    float rescale[2], base[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max_r[r] = fmaxf(tile_max_r[r], __shfl_xor_sync(0xffffffffu, tile_max_r[r], 1));
      tile_max_r[r] = fmaxf(tile_max_r[r], __shfl_xor_sync(0xffffffffu, tile_max_r[r], 2));
      const float new_max = fmaxf(row_max[r], tile_max_r[r]);   // key0 <= pos: the tile's first key is visible, so new_max is finite
      base[r] = new_max;
      rescale[r] = exp2f(row_max[r] - base[r]);
      row_max[r] = new_max;
      row_sum[r] *= rescale[r];
    }
    unsigned pa[kKeys / 16][4];
#pragma unroll
    for (int j = 0; j < kKeys / 8; ++j) {
      const float p0 = exp2_approx(s_frag[j][0] - base[0]);
      const float p1 = exp2_approx(s_frag[j][1] - base[0]);
      const float p2 = exp2_approx(s_frag[j][2] - base[1]);
      const float p3 = exp2_approx(s_frag[j][3] - base[1]);
      row_sum[0] += p0 + p1;
      row_sum[1] += p2 + p3;
      pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
      pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int i = 0; i < 2 * kHalfPairs; ++i) {
      o[i][0] *= rescale[0];
      o[i][1] *= rescale[0];
      o[i][2] *= rescale[1];
      o[i][3] *= rescale[1];
    }
#pragma unroll
    for (int kk = 0; kk < kKeys / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < kHalfPairs; ++np) {
        const int pair = half * kHalfPairs + np;
        if (pair < kPairs) {
          unsigned b[4];
          const int row = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
          const int col = pair * 16 + (lane >> 4) * 8;
          ldmatrix_x4_trans(b, v_smem + (size_t)row * kVRow + col);
          mma_bf16(o[np * 2], pa[kk], b[0], b[1]);
          mma_bf16(o[np * 2 + 1], pa[kk], b[2], b[3]);
        }
      }
    }
    __syncthreads();   // everyone is done with this stage before it is filled again
    if (kRing == 1) issue(tile + total_parts);
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    const int row = g + 8 * r;
    if (row >= heads_here) continue;
    float* dst = parts + (((size_t)token * total_parts + part) * 2 * heads + (size_t)(head0 + row) * 2 + m) * (kVD + 2);
    if (t == 0 && half == 0) {
      dst[0] = row_max[r];   // a part without a tile: -infinity and a sum of 0, which the merge passes over
      dst[1] = row_sum[r];
    }
#pragma unroll
    for (int np = 0; np < kHalfPairs; ++np) {
      const int pair = half * kHalfPairs + np;
      if (pair < kPairs) {
        *reinterpret_cast<float2*>(dst + 2 + pair * 16 + 2 * t) = make_float2(o[np * 2][r * 2], o[np * 2][r * 2 + 1]);
        *reinterpret_cast<float2*>(dst + 2 + pair * 16 + 8 + 2 * t) = make_float2(o[np * 2 + 1][r * 2], o[np * 2 + 1][r * 2 + 1]);
      }
    }
  }
}

}  // namespace tlie

using namespace tlie;

static int page_shift_of(int page_size) {
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  return (1 << shift) == page_size ? shift : -1;
}

// 1 if this kernel set has the kernel for steps of few rows (a tile of keys and values fits shared memory), else 0
TLIE_EXPORT int tlie_diff_decode_warps() { return kDecStages > 0 ? 1 : 0; }

// ``parts``: 32-bit scratch [tokens, ctas, 2 heads, VALUE_DIM + 2], which diff_merge (the general kernel set) joins.
TLIE_EXPORT int tlie_diff_decode(const void* rows, int row_stride, const void* k_pages, long long k_page_stride, const void* v_pages, long long v_page_stride,
                                 const int* positions, const int* token_seq, const int* block_table, int table_stride, float* parts, int tokens, int heads,
                                 int kv_heads, int page_size, float scale, int ctas, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (kDecStages == 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || page_size % 16 != 0 || row_stride % 8 != 0 || ctas < 1 || ctas > 65535) return (int)cudaErrorInvalidValue;
  const int chunks = (heads / kv_heads + 15) / 16;
  if ((long long)kv_heads * chunks > 65535) return (int)cudaErrorInvalidValue;
  constexpr size_t smem = dec_smem_for(kDecStages > 0 ? kDecStages : 1);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(diff_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  diff_decode_kernel<<<dim3(tokens, kv_heads * chunks, ctas), kDecThreads, smem, stream>>>(
      (const __nv_bfloat16*)rows, row_stride, (const __nv_bfloat16*)k_pages, k_page_stride, (const __nv_bfloat16*)v_pages, v_page_stride, positions, token_seq,
      block_table, table_stride, parts, heads, kv_heads, page_size, page_shift_of(page_size), scale);
  return (int)cudaGetLastError();
}

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
                                                        (__nv_bfloat16*)out, heads, kv_heads, page_size, page_shift_of(page_size), scale, lambda, eps, out_scale);
  return (int)cudaGetLastError();
}
