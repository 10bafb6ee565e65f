// Differential attention over the paged cache: every head has two softmax maps over the same values, and its output is the
// first map's minus lambda times the second's, divided by its root mean square and scaled.  The general kernels (any sizes,
// both storage types, 32-bit arithmetic), for prompt portions and decoded tokens alike.
//
// A row of the step holds, head by head, the queries [map 1 | map 2] (2 H vectors of ``dim``), then the keys laid out the same
// way (2 G vectors) and the values (G vectors of ``vdim``).  Query head h reads key/value head h / (H / G).
//
//   diff_store      per vector of q and k: RMS norm over dim with a weight, then the first ``rot_dims`` columns turn (column i with
//                   column i + rot_dims / 2, by position * inv_freq[i], 32-bit angles); q in place, k and v into the token's pages.
//   diff_attention  per (token, key/value head, run of key tiles): the running maximum, sum and weighted values of every
//                   (head, map) of the group, written as parts.
//   diff_merge      per (token, head): the parts of both maps joined, a1 - lambda a2, its root mean square taken out, times
//                   ``out_scale``.
//
// Pages: keys [page][2 G][slot][dim], values [page][G][slot][vdim], each with a page stride of its own.  Key tiles of 32 start
// at position 0, so a row's sums run in an order that depends on its position and on the number of runs alone.
#include "common.cuh"

namespace tlie {

constexpr int kDiffKeys = 32;          // keys per tile: a lane each
constexpr int kDiffMaxPerLane = 8;     // widths up to 256
constexpr float kDiffLog2e = 1.4426950408889634f;

template <typename T>
__global__ void __launch_bounds__(128) diff_store_kernel(T* __restrict__ rows, int row_stride, int k_offset, int v_offset, const float* __restrict__ q_weight,
                                                         const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq, int rot_dims,
                                                         const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ block_table,
                                                         int table_stride, T* __restrict__ k_pages, long long k_page_stride, T* __restrict__ v_pages,
                                                         long long v_page_stride, int q_vectors, int k_vectors, int v_heads, int dim, int vdim, int page_size,
                                                         int write_cache) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int page = write_cache ? block_table[(size_t)token_seq[t] * table_stride + pos / page_size] : -1;
  const int slot = pos % page_size;
  T* row = rows + (size_t)t * row_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (page >= 0)
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < v_heads * vdim; i += blockDim.x * gridDim.y) {
      const int head = i / vdim, d = i - head * vdim;
      v_pages[(size_t)page * v_page_stride + ((size_t)head * page_size + slot) * vdim + d] = row[v_offset + i];
    }
  const int half = rot_dims / 2;
  const float where = (float)pos;
  for (int n = blockIdx.y * warps + warp; n < q_vectors + k_vectors; n += warps * gridDim.y) {
    const bool is_key = n >= q_vectors;
    T* vector = is_key ? row + k_offset + (size_t)(n - q_vectors) * dim : row + (size_t)n * dim;
    const float* weight = is_key ? k_weight : q_weight;
    float mine[kDiffMaxPerLane], partner[kDiffMaxPerLane];
    float squares = 0.0f;
#pragma unroll
    for (int i = 0; i < kDiffMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      mine[i] = partner[i] = 0.0f;
      if (d < dim) {
        mine[i] = to_float(vector[d]);
        squares += mine[i] * mine[i];
        if (d < rot_dims) {
          const int other = d < half ? d + half : d - half;
          partner[i] = to_float(vector[other]) * weight[other];
        }
      }
    }
    const float inv = 1.0f / sqrtf(warp_sum(squares) / (float)dim + eps);
    __syncwarp();   // every lane has read its partner before anything of the vector is written
#pragma unroll
    for (int i = 0; i < kDiffMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d >= dim) continue;
      float v = (mine[i] * inv) * weight[d];
      if (d < rot_dims) {
        float sine, cosine;
        sincosf(where * inv_freq[d < half ? d : d - half], &sine, &cosine);
        const float p = partner[i] * inv;
        v = d < half ? v * cosine - p * sine : v * cosine + p * sine;
      }
      if (!is_key)
        vector[d] = from_float<T>(v);
      else if (page >= 0)
        k_pages[(size_t)page * k_page_stride + ((size_t)(n - q_vectors) * page_size + slot) * dim + d] = from_float<T>(v);
    }
  }
}

// One tile's rows of one head's plane into shared memory as 32-bit numbers: [32][stride]; keys past ``end`` are zero.
template <typename T>
__device__ __forceinline__ void stage_tile(float* dst, int stride, const T* pages, long long page_stride, const int* table, int head, int key0, int end, int width,
                                           int page_size) {
  for (int i = threadIdx.x; i < kDiffKeys * width; i += blockDim.x) {
    const int j = i / width, d = i - j * width;
    const int key = key0 + j;
    float v = 0.0f;
    if (key < end) {
      const long long page = table[key / page_size];
      v = to_float(pages[page * page_stride + ((size_t)head * page_size + key % page_size) * width + d]);
    }
    dst[j * stride + d] = v;
  }
}

// grid (tokens, G * chunks, runs); a warp per (head of the chunk, map).  parts: [token][run][2 H][vdim + 2] = (max, sum, weighted values).
template <typename T>
__global__ void __launch_bounds__(512) diff_attention_kernel(const T* __restrict__ rows, int row_stride, const T* __restrict__ k_pages, long long k_page_stride,
                                                             const T* __restrict__ v_pages, long long v_page_stride, const int* __restrict__ positions,
                                                             const int* __restrict__ token_seq, const int* __restrict__ block_table, int table_stride,
                                                             float* __restrict__ parts, int heads, int kv_heads, int dim, int vdim, int page_size, float scale,
                                                             int chunk_heads) {
  extern __shared__ float diff_smem[];
  const int t = blockIdx.x, runs = gridDim.z, run = blockIdx.z;
  const int group = heads / kv_heads;
  const int chunks = (group + chunk_heads - 1) / chunk_heads;
  const int kv = blockIdx.y / chunks, chunk = blockIdx.y - kv * chunks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_stride = dim | 1;   // an odd number of words between rows: a lane per key reads without bank conflicts
  float* q_s = diff_smem;                                   // [2 chunk_heads][dim]
  float* k_s = q_s + 2 * chunk_heads * dim;                 // [2][32][k_stride]
  float* v_s = k_s + 2 * kDiffKeys * k_stride;              // [32][vdim]
  const int pos = positions[t];
  const int* table = block_table + (size_t)token_seq[t] * table_stride;
  const int tiles = pos / kDiffKeys + 1;
  const int per_run = (tiles + runs - 1) / runs;
  const int first_tile = run * per_run, end_tile = min(tiles, first_tile + per_run);
  const int head_in_chunk = warp >> 1, map = warp & 1;
  const int head = kv * group + chunk * chunk_heads + head_in_chunk;
  const bool live = chunk * chunk_heads + head_in_chunk < group;
  for (int i = threadIdx.x; i < 2 * chunk_heads * dim; i += blockDim.x) {
    const int vector = i / dim, d = i - vector * dim;
    const int h = kv * group + chunk * chunk_heads + (vector >> 1);
    q_s[i] = (chunk * chunk_heads + (vector >> 1) < group) ? to_float(rows[(size_t)t * row_stride + ((size_t)h * 2 + (vector & 1)) * dim + d]) : 0.0f;
  }
  float acc[kDiffMaxPerLane];
#pragma unroll
  for (int i = 0; i < kDiffMaxPerLane; ++i) acc[i] = 0.0f;
  float row_max = -INFINITY, row_sum = 0.0f;
  const float scale2 = scale * kDiffLog2e;
  for (int tile = first_tile; tile < end_tile; ++tile) {
    const int key0 = tile * kDiffKeys;
    __syncthreads();   // the tile before is read; q_s is written
    stage_tile(k_s, k_stride, k_pages, k_page_stride, table, kv * 2, key0, pos + 1, dim, page_size);
    stage_tile(k_s + kDiffKeys * k_stride, k_stride, k_pages, k_page_stride, table, kv * 2 + 1, key0, pos + 1, dim, page_size);
    stage_tile(v_s, vdim, v_pages, v_page_stride, table, kv, key0, pos + 1, vdim, page_size);
    __syncthreads();
    if (!live) continue;
    const float* q = q_s + warp * dim;
    const float* k = k_s + (map * kDiffKeys + lane) * k_stride;
    float dot = 0.0f;
    for (int d = 0; d < dim; ++d) dot = fmaf(q[d], k[d], dot);
    const float s = key0 + lane <= pos ? dot * scale2 : -INFINITY;
    const float new_max = fmaxf(row_max, warp_max(s));   // key0 <= pos: some key of the tile is visible
    const float rescale = exp2f(row_max - new_max);
    const float p = exp2f(s - new_max);
    row_sum = row_sum * rescale + warp_sum(p);
    row_max = new_max;
#pragma unroll
    for (int i = 0; i < kDiffMaxPerLane; ++i) acc[i] *= rescale;
    for (int j = 0; j < kDiffKeys; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
      for (int i = 0; i < kDiffMaxPerLane; ++i)
        if (lane + 32 * i < vdim) acc[i] = fmaf(pj, v_s[j * vdim + lane + 32 * i], acc[i]);
    }
  }
  if (!live) return;
  float* part = parts + (((size_t)t * runs + run) * 2 * heads + (size_t)head * 2 + map) * (vdim + 2);
  if (lane == 0) {
    part[0] = row_max;
    part[1] = row_sum;
  }
#pragma unroll
  for (int i = 0; i < kDiffMaxPerLane; ++i)
    if (lane + 32 * i < vdim) part[2 + lane + 32 * i] = acc[i];
}

// grid (tokens, heads), 128 threads: a thread per value column (widths up to 256: two columns each).  Dynamic shared memory: 4 runs
// floats.  The runs' maxima and sums are fetched side by side first and turned into one weight per (map, run), so that the loop over
// the runs' weighted values is a row of independent loads: with a branch and an exponential between two loads, every run of a decoded
// token's many cost a round trip to L2 of its own.  A run that saw no key has the sum 0, weight 0 and zeros for values.
template <typename T>
__global__ void __launch_bounds__(128) diff_merge_kernel(const float* __restrict__ parts, T* __restrict__ out, int runs, int heads, int vdim, float lambda, float eps,
                                                         float out_scale) {
  extern __shared__ float merge_smem[];   // [2][runs] maxima, then [2][runs] weights (sums first)
  __shared__ float scratch[32];
  float* top_s = merge_smem;
  float* w_s = merge_smem + 2 * runs;
  const int t = blockIdx.x, head = blockIdx.y;
  const size_t step = (size_t)2 * heads * (vdim + 2);
  const float* base = parts + ((size_t)t * runs * 2 * heads + (size_t)head * 2) * (vdim + 2);
  for (int i = threadIdx.x; i < 2 * runs; i += blockDim.x) {
    const int map = i / runs, r = i - map * runs;
    const float* pair = base + r * step + (size_t)map * (vdim + 2);
    top_s[i] = pair[0];
    w_s[i] = pair[1];
  }
  __syncthreads();
  float inv[2];
#pragma unroll
  for (int map = 0; map < 2; ++map) {
    float top = -INFINITY;
    for (int r = 0; r < runs; ++r) top = fmaxf(top, top_s[map * runs + r]);
    float total = 0.0f;
    for (int r = 0; r < runs; ++r) {
      const float sum = w_s[map * runs + r];
      total += sum == 0.0f ? 0.0f : sum * exp2f(top_s[map * runs + r] - top);
    }
    inv[map] = 1.0f / total;
    __syncthreads();
    for (int i = threadIdx.x; i < runs; i += blockDim.x) {
      const float sum = w_s[map * runs + i];
      w_s[map * runs + i] = sum == 0.0f ? 0.0f : exp2f(top_s[map * runs + i] - top);
    }
  }
  __syncthreads();
  float o[2] = {0.0f, 0.0f};
#pragma unroll
  for (int map = 0; map < 2; ++map) {
    const float* first = base + (size_t)map * (vdim + 2) + 2;
    float a[2] = {0.0f, 0.0f};
#pragma unroll 8
    for (int r = 0; r < runs; ++r) {
      const float w = w_s[map * runs + r];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if ((int)threadIdx.x + 128 * i < vdim) a[i] = fmaf(first[r * step + threadIdx.x + 128 * i], w, a[i]);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) o[i] = map == 0 ? a[i] * inv[0] : o[i] - lambda * (a[i] * inv[1]);
  }
  float squares = 0.0f;
#pragma unroll
  for (int i = 0; i < 2; ++i)
    if ((int)threadIdx.x + 128 * i < vdim) squares += o[i] * o[i];
  const float norm = out_scale / sqrtf(block_sum(squares, scratch) / (float)vdim + eps);
#pragma unroll
  for (int i = 0; i < 2; ++i)
    if ((int)threadIdx.x + 128 * i < vdim) out[((size_t)t * heads + head) * vdim + threadIdx.x + 128 * i] = from_float<T>(o[i] * norm);
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_diff_store(int dtype, void* rows, int row_stride, int k_offset, int v_offset, const float* q_weight, const float* k_weight, float eps,
                                const float* inv_freq, int rot_dims, const int* positions, const int* token_seq, const int* block_table, int table_stride,
                                void* k_pages, long long k_page_stride, void* v_pages, long long v_page_stride, int tokens, int heads, int kv_heads, int dim,
                                int vdim, int page_size, int write_cache, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dim > 32 * kDiffMaxPerLane || rot_dims < 0 || rot_dims > dim || rot_dims % 2 != 0) return (int)cudaErrorInvalidValue;
  // a warp per vector where the step is small (every vector is a read, a reduction and a write that wait for one another: a token's
  // vectors one after the other in four warps took 22 us for 8 tokens); a step of many tokens keeps more vectors per warp (more CTAs than that were measured: slower)
  const int vectors = 2 * heads + 2 * kv_heads;
  int per_token = (vectors + 3) / 4;
  while (per_token > 1 && (long long)tokens * per_token > 8192) per_token = (per_token + 1) / 2;
  if (per_token > 65535) per_token = 65535;
  const dim3 store_grid(tokens, per_token);
  if (dtype == TLIE_F32)
    diff_store_kernel<float><<<store_grid, 128, 0, stream>>>((float*)rows, row_stride, k_offset, v_offset, q_weight, k_weight, eps, inv_freq, rot_dims, positions, token_seq,
                                                         block_table, table_stride, (float*)k_pages, k_page_stride, (float*)v_pages, v_page_stride, 2 * heads,
                                                         2 * kv_heads, kv_heads, dim, vdim, page_size, write_cache);
  else
    diff_store_kernel<__nv_bfloat16><<<store_grid, 128, 0, stream>>>((__nv_bfloat16*)rows, row_stride, k_offset, v_offset, q_weight, k_weight, eps, inv_freq, rot_dims,
                                                                 positions, token_seq, block_table, table_stride, (__nv_bfloat16*)k_pages, k_page_stride,
                                                                 (__nv_bfloat16*)v_pages, v_page_stride, 2 * heads, 2 * kv_heads, kv_heads, dim, vdim, page_size,
                                                                 write_cache);
  return (int)cudaGetLastError();
}

// ``parts``: 32-bit scratch [tokens, runs, 2 heads, vdim + 2].  ``out`` [tokens, heads * vdim] of ``dtype``.
TLIE_EXPORT int tlie_diff_attention(int dtype, const void* rows, int row_stride, const void* k_pages, long long k_page_stride, const void* v_pages,
                                    long long v_page_stride, const int* positions, const int* token_seq, const int* block_table, int table_stride, float* parts,
                                    void* out, int tokens, int heads, int kv_heads, int dim, int vdim, int page_size, float scale, float lambda, float eps,
                                    float out_scale, int runs, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || dim > 32 * kDiffMaxPerLane || vdim > 32 * kDiffMaxPerLane || runs < 1 || runs > 2048)
    return (int)cudaErrorInvalidValue;
  const int group = heads / kv_heads;
  const int chunk_heads = group < 8 ? group : 8;
  const int chunks = (group + chunk_heads - 1) / chunk_heads;
  if ((long long)kv_heads * chunks > 65535) return (int)cudaErrorInvalidValue;
  const size_t smem = ((size_t)2 * chunk_heads * dim + (size_t)2 * kDiffKeys * (dim | 1) + (size_t)kDiffKeys * vdim) * sizeof(float);
  const dim3 grid(tokens, kv_heads * chunks, runs);
  const int threads = 64 * chunk_heads;
  cudaError_t e;
  if (dtype == TLIE_F32) {
    e = cudaFuncSetAttribute(diff_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    diff_attention_kernel<float><<<grid, threads, smem, stream>>>((const float*)rows, row_stride, (const float*)k_pages, k_page_stride, (const float*)v_pages,
                                                                  v_page_stride, positions, token_seq, block_table, table_stride, parts, heads, kv_heads, dim, vdim,
                                                                  page_size, scale, chunk_heads);
  } else {
    e = cudaFuncSetAttribute(diff_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    diff_attention_kernel<__nv_bfloat16><<<grid, threads, smem, stream>>>((const __nv_bfloat16*)rows, row_stride, (const __nv_bfloat16*)k_pages, k_page_stride,
                                                                          (const __nv_bfloat16*)v_pages, v_page_stride, positions, token_seq, block_table,
                                                                          table_stride, parts, heads, kv_heads, dim, vdim, page_size, scale, chunk_heads);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const dim3 merge_grid(tokens, heads);
  if (dtype == TLIE_F32)
    diff_merge_kernel<float><<<merge_grid, 128, (size_t)4 * runs * sizeof(float), stream>>>(parts, (float*)out, runs, heads, vdim, lambda, eps, out_scale);
  else
    diff_merge_kernel<__nv_bfloat16><<<merge_grid, 128, (size_t)4 * runs * sizeof(float), stream>>>(parts, (__nv_bfloat16*)out, runs, heads, vdim, lambda, eps, out_scale);
  return (int)cudaGetLastError();
}

// The parts of another kernel's runs (csrc/attention_diff_prefill.cu's steps of few rows), joined as above.
TLIE_EXPORT int tlie_diff_merge(int dtype, const float* parts, void* out, int tokens, int heads, int vdim, int runs, float lambda, float eps, float out_scale,
                                cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || heads > 65535 || vdim > 32 * kDiffMaxPerLane || runs < 1 || runs > 2048) return (int)cudaErrorInvalidValue;
  const dim3 merge_grid(tokens, heads);
  if (dtype == TLIE_F32)
    diff_merge_kernel<float><<<merge_grid, 128, (size_t)4 * runs * sizeof(float), stream>>>(parts, (float*)out, runs, heads, vdim, lambda, eps, out_scale);
  else
    diff_merge_kernel<__nv_bfloat16><<<merge_grid, 128, (size_t)4 * runs * sizeof(float), stream>>>(parts, (__nv_bfloat16*)out, runs, heads, vdim, lambda, eps, out_scale);
  return (int)cudaGetLastError();
}
