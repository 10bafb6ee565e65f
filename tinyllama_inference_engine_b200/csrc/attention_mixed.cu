// Paged attention whose heads talk to one another before the softmax, with a distance bias and an output gate: the general
// kernel (any sizes, both storage types, 32-bit arithmetic), for prompt portions and decoded tokens alike.
//
// For query token t at position i of its request, key position j, query head g (key/value head g / (H / G)):
//   raw_g(i, j)   = (q_g . k_j) * scale - slope_g * (i - j)              (slopes optional)
//   mixed_h(i, j) = sum_g M[h, g] raw_g(i, j)                             (M optional: H x H, row h mixes into head h)
//   visible: 0 <= i - j, and i - j < window if window > 0; with keep_first > 0 the keys j < keep_first stay visible behind the window
//   out_h = softmax_j(mixed_h) . v_j                                      (values of value_dim, keys of key_dim)
//   out   = concat_h(out_h) * sigmoid(gate)                               (gate optional: H * value_dim columns of the same row, or H: one per head)
// ``sinks`` (optional, one per head): the softmax's denominator also holds exp(sink_h), a weight that belongs to no key.
// ``v_row_stride``: elements between two slots of the value plane (value_dim unless the values are a part of wider rows, as when
// they are the leading columns of the keys themselves).
// The mix needs every head's score of a (query, key) pair in one place, so a CTA owns one query token with all its heads: per
// tile of 32 keys the warps take the heads' raw scores (a lane per key), then the mixed rows with their running maximum and sum
// (a warp per head), then every thread adds the tile into its share of the H * value_dim outputs.  Tiles start at the first
// visible key, so the order of a row's sums depends on the row's position alone: rows are bit-identical however the step was
// cut or batched.
//
// Pages: keys [page][kv head][slot][key_dim] and values [page][kv head][slot][value_dim], each with a page stride of its own
// (two planes of one tensor when the sizes agree, two tensors when they do not).
#include "common.cuh"

namespace tlie {

constexpr int kMixKeys = 32;        // keys per tile: a lane each
constexpr int kMixThreads = 256;

// k and v of the step's tokens into their pages.
template <typename T>
__global__ void store_kv_planes_kernel(const T* __restrict__ rows, int row_stride, int k_offset, int v_offset, const int* __restrict__ positions,
                                       const int* __restrict__ token_seq, const int* __restrict__ block_table, int table_stride,
                                       T* __restrict__ k_pages, long long k_page_stride, T* __restrict__ v_pages, long long v_page_stride,
                                       int kv_heads, int key_dim, int value_dim, int page_size) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int page = block_table[(size_t)token_seq[t] * table_stride + pos / page_size];
  if (page < 0) return;   // a position its request holds no page for is never read either
  const int slot = pos % page_size;
  const T* row = rows + (size_t)t * row_stride;
  for (int i = threadIdx.x; i < kv_heads * key_dim; i += blockDim.x) {
    const int head = i / key_dim, d = i - head * key_dim;
    k_pages[(size_t)page * k_page_stride + ((size_t)head * page_size + slot) * key_dim + d] = row[k_offset + i];
  }
  for (int i = threadIdx.x; i < kv_heads * value_dim; i += blockDim.x) {
    const int head = i / value_dim, d = i - head * value_dim;
    v_pages[(size_t)page * v_page_stride + ((size_t)head * page_size + slot) * value_dim + d] = row[v_offset + i];
  }
}

// Biases, a partial rotation and the cache write for attention whose keys and values are planes of different widths.  A row of
// ``rows`` holds the products [q: heads x key_dim | ... k at k_offset: kv_heads x key_dim | ... v at v_offset: kv_heads x value_dim].
// Each vector gets its bias (32-bit, null: none); of every q and k head the first ``rot_dims`` columns turn, column i with column
// i + rot_dims / 2, by position * inv_freq[i] (angle, sine and cosine in 32-bit); q is left in place, k and v go into the token's page.
template <typename T>
__global__ void __launch_bounds__(256) rotary_store_planes_kernel(T* __restrict__ rows, int row_stride, int k_offset, int v_offset, const float* __restrict__ q_bias,
                                                                  const float* __restrict__ k_bias, const float* __restrict__ v_bias, const float* __restrict__ inv_freq,
                                                                  int rot_dims, const int* __restrict__ positions, const int* __restrict__ token_seq,
                                                                  const int* __restrict__ block_table, int table_stride, T* __restrict__ k_pages, long long k_page_stride,
                                                                  T* __restrict__ v_pages, long long v_page_stride, int heads, int kv_heads, int key_dim, int value_dim,
                                                                  int page_size, int write_cache) {
  extern __shared__ float turn_s[];   // the token's cosines [rot_dims / 2], then its sines: worked out once, used by every head
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int page = write_cache ? block_table[(size_t)token_seq[t] * table_stride + pos / page_size] : -1;
  const int slot = pos % page_size;
  T* row = rows + (size_t)t * row_stride;
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &turn_s[half + i], &turn_s[i]);
  // values first: they need no angle
  if (page >= 0)
    for (int i = threadIdx.x; i < kv_heads * value_dim; i += blockDim.x) {
      const int head = i / value_dim, d = i - head * value_dim;
      float a = to_float(row[v_offset + i]);
      if (v_bias != nullptr) a += v_bias[i];
      v_pages[(size_t)page * v_page_stride + ((size_t)head * page_size + slot) * value_dim + d] = from_float<T>(a);
    }
  __syncthreads();
  const int units = key_dim - half;   // per head: ``half`` pairs, then the columns that do not turn
  for (int i = threadIdx.x; i < (heads + kv_heads) * units; i += blockDim.x) {
    const int h = i / units, u = i - h * units;
    const bool is_key = h >= heads;
    const int head = is_key ? h - heads : h;
    T* vec = row + (is_key ? k_offset : 0) + (size_t)head * key_dim;
    const float* bias = is_key ? k_bias : q_bias;
    T* dst = (is_key && page >= 0) ? k_pages + (size_t)page * k_page_stride + ((size_t)head * page_size + slot) * key_dim : nullptr;
    if (u < half) {
      float a = to_float(vec[u]), b = to_float(vec[u + half]);
      if (bias != nullptr) a += bias[head * key_dim + u], b += bias[head * key_dim + u + half];
      const float cosine = turn_s[u], sine = turn_s[half + u];
      const T first = from_float<T>(a * cosine - b * sine), second = from_float<T>(b * cosine + a * sine);
      if (!is_key) vec[u] = first, vec[u + half] = second;
      if (dst != nullptr) dst[u] = first, dst[u + half] = second;
    } else {
      const int d = u + half;
      float a = to_float(vec[d]);
      if (bias != nullptr) a += bias[head * key_dim + d];
      const T value = from_float<T>(a);
      if (!is_key) vec[d] = value;
      if (dst != nullptr) dst[d] = value;
    }
  }
}

// Queries and keys divided by their root mean square per head (optionally times a weight), then the cache write: the normalised
// keys into the key plane and ``kv_heads * value_dim`` columns from ``v_offset`` into the value plane as they are (with
// ``v_offset == k_offset`` the values are the keys before the norm).  q is normalised in place.  A warp per head.
template <typename T>
__global__ void __launch_bounds__(128) normed_store_kernel(T* __restrict__ rows, int row_stride, int k_offset, int v_offset, const float* __restrict__ q_weight,
                                                           const float* __restrict__ k_weight, float eps, const int* __restrict__ positions,
                                                           const int* __restrict__ token_seq, const int* __restrict__ block_table, int table_stride,
                                                           T* __restrict__ k_pages, long long k_page_stride, T* __restrict__ v_pages, long long v_page_stride,
                                                           int heads, int kv_heads, int key_dim, int value_dim, int page_size, int write_cache) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int page = write_cache ? block_table[(size_t)token_seq[t] * table_stride + pos / page_size] : -1;
  const int slot = pos % page_size;
  T* row = rows + (size_t)t * row_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (page >= 0)   // values first: they may be the keys, which are still as the product left them
    for (int i = threadIdx.x; i < kv_heads * value_dim; i += blockDim.x) {
      const int head = i / value_dim, d = i - head * value_dim;
      v_pages[(size_t)page * v_page_stride + ((size_t)head * page_size + slot) * value_dim + d] = row[v_offset + i];
    }
  for (int h = warp; h < heads + kv_heads; h += warps) {
    const bool is_key = h >= heads;
    T* head_row = is_key ? row + k_offset + (h - heads) * key_dim : row + h * key_dim;
    const float* weight = is_key ? k_weight : q_weight;
    float squares = 0.0f;
    for (int d = lane; d < key_dim; d += 32) {
      const float v = to_float(head_row[d]);
      squares += v * v;
    }
    const float inv = rsqrtf(warp_sum(squares) / (float)key_dim + eps);
    for (int d = lane; d < key_dim; d += 32) {
      const T v = from_float<T>(to_float(head_row[d]) * inv * (weight ? weight[d] : 1.0f));
      if (!is_key)
        head_row[d] = v;
      else if (page >= 0)
        k_pages[(size_t)page * k_page_stride + ((size_t)(h - heads) * page_size + slot) * key_dim + d] = v;
    }
  }
}

// Latent attention's cache write and rotation.  A row holds ``heads`` queries of [plain | rot] and, from ``latent_offset``, the
// down projection [rank | rot].  The first ``rank`` columns are normalised (RMS, weight) into the latent; the last ``rot`` are a key
// part that all heads share and that is rotated: pairs (2i, 2i + 1) of its first ``rot_dims`` columns turn by position * inv_freq[i]
// (32-bit angles).  [latent | rotated part] goes into the token's cache row; the queries' rotated parts go into ``queries``
// [T, heads, rank + rot] behind the ``rank`` columns that the product with the keys' expansion fills.
template <typename T>
__global__ void __launch_bounds__(128) latent_store_kernel(const T* __restrict__ rows, int row_stride, int latent_offset, const float* __restrict__ weight, float eps,
                                                           const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions,
                                                           const int* __restrict__ token_seq, const int* __restrict__ block_table, int table_stride,
                                                           T* __restrict__ pages, long long page_stride, int heads, int plain, int rot, int rank, int page_size,
                                                           int write_cache, T* __restrict__ queries) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int page = write_cache ? block_table[(size_t)token_seq[t] * table_stride + pos / page_size] : -1;
  const T* row = rows + (size_t)t * row_stride;
  T* cached = page >= 0 ? pages + (size_t)page * page_stride + (size_t)(pos % page_size) * (rank + rot) : nullptr;
  float squares = 0.0f;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    const float v = to_float(row[latent_offset + d]);
    squares += v * v;
  }
  const float inv = rsqrtf(block_sum(squares, scratch) / (float)rank + eps);
  if (cached)
    for (int d = threadIdx.x; d < rank; d += blockDim.x) cached[d] = from_float<T>(to_float(row[latent_offset + d]) * inv * weight[d]);
  // the rot parts: the shared key part is vector ``heads`` and goes into the cache row, the queries' parts are vectors 0 .. heads - 1
  // and go behind the ``rank`` columns of their head in ``queries``; a thread per pair of columns
  const int pairs = rot / 2;
  T* query_row = queries + (size_t)t * heads * (rank + rot);
  for (int i = threadIdx.x; i < (heads + 1) * pairs; i += blockDim.x) {
    const int vector = i / pairs, pair = i - vector * pairs;
    const T* at = vector < heads ? row + vector * (plain + rot) + plain : row + latent_offset + rank;
    T* to = vector < heads ? query_row + vector * (rank + rot) + rank : (cached ? cached + rank : nullptr);
    if (!to) continue;
    if (2 * pair + 1 < rot_dims) {
      float sine, cosine;
      sincosf((float)pos * inv_freq[pair], &sine, &cosine);
      const float a = to_float(at[2 * pair]), b = to_float(at[2 * pair + 1]);
      to[2 * pair] = from_float<T>(a * cosine - b * sine);
      to[2 * pair + 1] = from_float<T>(b * cosine + a * sine);
    } else {   // columns that do not rotate
      to[2 * pair] = at[2 * pair];
      to[2 * pair + 1] = at[2 * pair + 1];
    }
  }
}

__device__ __forceinline__ float dot_row(const float* __restrict__ q, const float* __restrict__ k, int n) {
  float dot = 0.0f;
  if ((n & 3) == 0) {
    for (int d = 0; d < n; d += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(k + d);
      dot += q[d] * kv.x;
      dot += q[d + 1] * kv.y;
      dot += q[d + 2] * kv.z;
      dot += q[d + 3] * kv.w;
    }
  } else {
    for (int d = 0; d < n; ++d) dot += q[d] * k[d];
  }
  return dot;
}

__device__ __forceinline__ float dot_row(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int n) {
  float dot = 0.0f;
  if ((n & 7) == 0) {
    for (int d = 0; d < n; d += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        dot += q[d + 2 * i] * __bfloat162float(pairs[i].x);
        dot += q[d + 2 * i + 1] * __bfloat162float(pairs[i].y);
      }
    }
  } else {
    for (int d = 0; d < n; ++d) dot += q[d] * __bfloat162float(k[d]);
  }
  return dot;
}

// A tile's rows of one plane (``heads`` x ``count`` rows of ``width``) from their pages into shared memory, rows ``stride`` apart.
// 16 bytes per load where the width allows it: all of a thread's loads are in flight together.
template <typename T>
__device__ __forceinline__ void stage_plane(T* __restrict__ dst, int stride, const T* __restrict__ pages, const long long* __restrict__ row_at,
                                            int head_stride, int heads, int count, int width, bool aligned) {
  constexpr int kVec = 16 / sizeof(T);
  constexpr int kBatch = 8;   // loads a thread has in flight before it stores them: a load followed by its own store would wait for the one before
  if (width % kVec == 0 && aligned) {
    const int chunks = width / kVec;
    const int total = heads * kMixKeys * chunks;
    for (int i0 = threadIdx.x; i0 < total; i0 += kBatch * kMixThreads) {
      uint4 raw[kBatch];
      int at[kBatch];
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const int i = i0 + b * kMixThreads;
        const int chunk = i % chunks, j = (i / chunks) % kMixKeys, c = i / (chunks * kMixKeys);
        at[b] = (i < total && j < count) ? (c * kMixKeys + j) * stride + chunk * kVec : -1;
        if (at[b] >= 0) raw[b] = *reinterpret_cast<const uint4*>(pages + row_at[j] + (size_t)c * head_stride + chunk * kVec);
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        if (at[b] < 0) continue;
        unsigned* out = reinterpret_cast<unsigned*>(dst + at[b]);   // rows are 4-byte aligned, not 16
        out[0] = raw[b].x;
        out[1] = raw[b].y;
        out[2] = raw[b].z;
        out[3] = raw[b].w;
      }
    }
  } else {
    const int total = heads * kMixKeys * width;
    for (int i0 = threadIdx.x; i0 < total; i0 += kBatch * kMixThreads) {
      T raw[kBatch];
      int at[kBatch];
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const int i = i0 + b * kMixThreads;
        const int d = i % width, j = (i / width) % kMixKeys, c = i / (width * kMixKeys);
        at[b] = (i < total && j < count) ? (c * kMixKeys + j) * stride + d : -1;
        if (at[b] >= 0) raw[b] = pages[row_at[j] + (size_t)c * head_stride + d];
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b)
        if (at[b] >= 0) dst[at[b]] = raw[b];
    }
  }
}

__device__ __forceinline__ float dot_staged(const float* __restrict__ q, const float* __restrict__ k, int n) {
  float dot = 0.0f;
  for (int d = 0; d < n; ++d) dot += q[d] * k[d];
  return dot;
}

__device__ __forceinline__ float dot_staged(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int n) {
  float dot = 0.0f;
  if ((n & 1) == 0) {
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(k);
    for (int d = 0; d < n / 2; ++d) {
      const float2 kv = __bfloat1622float2(pairs[d]);
      dot += q[2 * d] * kv.x;
      dot += q[2 * d + 1] * kv.y;
    }
  } else {
    for (int d = 0; d < n; ++d) dot += q[d] * __bfloat162float(k[d]);
  }
  return dot;
}

// Shared-memory row stride of a staged key tile: lanes read different rows at the same column, so rows are an odd number of
// 4-byte words apart where the width allows it.
template <typename T>
__host__ __device__ constexpr int staged_key_stride(int key_dim) {
  return sizeof(T) == 4 ? key_dim + 1 : ((key_dim & 1) ? key_dim + 1 : (((key_dim / 2) & 1) ? key_dim : key_dim + 2));
}

template <typename T, int ACC>
__global__ void __launch_bounds__(kMixThreads) mixed_heads_attention_kernel(
    const T* __restrict__ rows, int row_stride, int gate_offset, const T* __restrict__ k_pages, long long k_page_stride,
    const T* __restrict__ v_pages, long long v_page_stride, const int* __restrict__ positions, const int* __restrict__ token_seq,
    const int* __restrict__ block_table, int table_stride, const float* __restrict__ slopes, const float* __restrict__ mix, T* __restrict__ out,
    int heads, int kv_heads, int key_dim, int value_dim, int page_size, int window, float scale, float* __restrict__ partial, int staged,
    int keep_first, int gate_per_head, const float* __restrict__ sinks, int v_row_stride) {
  extern __shared__ __align__(16) unsigned char smem_bytes[];
  long long* k_at = reinterpret_cast<long long*>(smem_bytes);   // [32] where a key's row starts in its plane (head 0)
  long long* v_at = k_at + kMixKeys;
  float* q_s = reinterpret_cast<float*>(v_at + kMixKeys);   // [heads][key_dim]
  float* mix_s = q_s + heads * key_dim;          // [heads][heads]
  float* raw_s = mix_s + (mix ? heads * heads : 0);   // [heads][32]
  float* p_s = raw_s + heads * kMixKeys;         // [heads][32]
  float* max_s = p_s + heads * kMixKeys;         // [heads] running maximum
  float* sum_s = max_s + heads;                  // [heads] running sum
  float* rescale_s = sum_s + heads;              // [heads] what this tile shrinks the sums so far by
  // ``staged``: the tile's keys and values of every key/value head pass through shared memory (wide loads, all in flight at once,
  // every row read from memory once however many heads share it); sizes too large for that read their rows from global memory.
  const int k_stride = staged_key_stride<T>(key_dim);
  T* k_t = reinterpret_cast<T*>(smem_bytes + (((size_t)((rescale_s + heads) - reinterpret_cast<float*>(smem_bytes)) * sizeof(float)) + 15) / 16 * 16);
  T* v_t = k_t + (size_t)kv_heads * kMixKeys * k_stride;   // [kv heads][32][value_dim]; k_t is [kv heads][32][k_stride]

  const int t = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int warps = kMixThreads / 32;
  const int pos = positions[t];
  const int* table = block_table + (size_t)token_seq[t] * table_stride;
  const T* row = rows + (size_t)t * row_stride;
  const int group = heads / kv_heads;
  const int outputs = heads * value_dim;

  for (int i = tid; i < heads * key_dim; i += kMixThreads) q_s[i] = to_float(row[i]);
  if (mix)
    for (int i = tid; i < heads * heads; i += kMixThreads) mix_s[i] = mix[i];
  for (int i = tid; i < heads; i += kMixThreads) {
    max_s[i] = -INFINITY;
    sum_s[i] = 0.0f;
  }

  float acc[ACC];
  int head_of[ACC], value_at[ACC], staged_at[ACC];   // the output's head, and where its element lies in a token's value plane entry / in the staged tile
#pragma unroll
  for (int i = 0; i < ACC; ++i) {
    const int o = tid + i * kMixThreads;
    acc[i] = 0.0f;
    head_of[i] = o < outputs ? o / value_dim : 0;
    value_at[i] = (head_of[i] / group) * page_size * v_row_stride + (o - head_of[i] * value_dim);
    staged_at[i] = (head_of[i] / group) * kMixKeys * value_dim + (o - head_of[i] * value_dim);
  }

  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  // With gridDim.y > 1 the row's key tiles are dealt to that many CTAs in runs; each leaves its unnormalised sums, maxima and
  // totals in ``partial`` and merge_mixed_kernel puts them together.
  // The visible keys are numbered 0, 1, ...: first the ``kept`` keys that stay visible behind the window, then the window's.
  const int kept = min(keep_first, lo);
  const int visible = kept + (pos - lo + 1);
  const int splits = gridDim.y;
  const int tiles = (visible + kMixKeys - 1) / kMixKeys;
  const int tiles_each = (tiles + splits - 1) / splits;
  const int first_key = blockIdx.y * tiles_each * kMixKeys;
  const int last_key = min(visible - 1, first_key + tiles_each * kMixKeys - 1);
  const bool v_aligned = (v_row_stride * (int)sizeof(T)) % 16 == 0 && (v_page_stride * (long long)sizeof(T)) % 16 == 0;
  for (int base = first_key; base <= last_key; base += kMixKeys) {
    const int count = min(kMixKeys, last_key - base + 1);
    __syncthreads();   // the tile before is done with k_at / v_at (and, the first time, q_s and the running sums are in place)
    if (tid < count) {
      const int key = base + tid < kept ? base + tid : lo + (base + tid - kept);
      const long long page = table[key / page_size];
      const int slot = key % page_size;
      k_at[tid] = page * k_page_stride + (long long)slot * key_dim;
      v_at[tid] = page * v_page_stride + (long long)slot * v_row_stride;
    }
    __syncthreads();
    if (staged) {
      stage_plane(k_t, k_stride, k_pages, k_at, page_size * key_dim, kv_heads, count, key_dim, true);
      stage_plane(v_t, value_dim, v_pages, v_at, page_size * v_row_stride, kv_heads, count, value_dim, v_aligned);
      __syncthreads();
    }
    // raw scores: a warp per head, a lane per key
    for (int g = warp; g < heads; g += warps) {
      float raw = 0.0f;
      if (lane < count) {
        if (staged)
          raw = dot_staged(q_s + g * key_dim, k_t + (size_t)((g / group) * kMixKeys + lane) * k_stride, key_dim) * scale;
        else
          raw = dot_row(q_s + g * key_dim, k_pages + k_at[lane] + (size_t)(g / group) * page_size * key_dim, key_dim) * scale;
        if (slopes) raw -= slopes[g] * (float)(pos - (base + lane < kept ? base + lane : lo + (base + lane - kept)));
      }
      raw_s[g * kMixKeys + lane] = raw;
    }
    __syncthreads();
    // the heads' scores mixed, and the softmax's running maximum and sum: a warp per head
    for (int h = warp; h < heads; h += warps) {
      float score;
      if (mix) {
        // four sums side by side: one chain of dependent adds would wait for every load in turn
        float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float* weights = mix_s + h * heads;
        int g = 0;
#pragma unroll 2
        for (; g + 4 <= heads; g += 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) part[i] += weights[g + i] * raw_s[(g + i) * kMixKeys + lane];
        }
        for (; g < heads; ++g) part[0] += weights[g] * raw_s[g * kMixKeys + lane];
        score = (part[0] + part[1]) + (part[2] + part[3]);
      } else {
        score = raw_s[h * kMixKeys + lane];
      }
      if (lane >= count) score = -INFINITY;
      const float before = max_s[h];
      const float now = fmaxf(before, warp_max(score));
      const float shrink = expf(before - now);   // exp(-inf) = 0 on the first tile
      const float p = lane < count ? expf(score - now) : 0.0f;
      const float total = warp_sum(p);
      p_s[h * kMixKeys + lane] = p;
      __syncwarp();
      if (lane == 0) {
        max_s[h] = now;
        sum_s[h] = sum_s[h] * shrink + total;
        rescale_s[h] = shrink;
      }
    }
    __syncthreads();
    // weights times values: every thread its share of the outputs
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] *= rescale_s[head_of[i]];
    if (staged && outputs == ACC * kMixThreads) {   // every accumulator is in use: no guards
#pragma unroll 2
      for (int j = 0; j < count; ++j) {
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[i] += p_s[head_of[i] * kMixKeys + j] * to_float(v_t[staged_at[i] + j * value_dim]);
      }
    } else if (staged) {
      for (int j = 0; j < count; ++j) {
#pragma unroll
        for (int i = 0; i < ACC; ++i)
          if (tid + i * kMixThreads < outputs) acc[i] += p_s[head_of[i] * kMixKeys + j] * to_float(v_t[staged_at[i] + j * value_dim]);
      }
    } else {
      for (int j = 0; j < count; ++j) {
        const T* v_row = v_pages + v_at[j];
#pragma unroll
        for (int i = 0; i < ACC; ++i)
          if (tid + i * kMixThreads < outputs) acc[i] += p_s[head_of[i] * kMixKeys + j] * to_float(v_row[value_at[i]]);
      }
    }
  }
  __syncthreads();
  if (splits > 1) {
    float* mine = partial + ((size_t)t * splits + blockIdx.y) * (outputs + 2 * heads);
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
      const int o = tid + i * kMixThreads;
      if (o < outputs) mine[o] = acc[i];
    }
    for (int i = tid; i < heads; i += kMixThreads) {
      mine[outputs + i] = max_s[i];
      mine[outputs + heads + i] = sum_s[i];
    }
    return;
  }
  for (int h = tid; h < heads; h += kMixThreads) {   // what an accumulator of head h is multiplied by: 1 / the softmax's denominator
    if (sinks) {
      const float top = fmaxf(max_s[h], sinks[h]);
      const float shrink = expf(max_s[h] - top);
      rescale_s[h] = shrink / (sum_s[h] * shrink + expf(sinks[h] - top));
    } else {
      rescale_s[h] = 1.0f / sum_s[h];
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < ACC; ++i) {
    const int o = tid + i * kMixThreads;
    if (o < outputs) {
      float v = acc[i] * rescale_s[head_of[i]];
      if (gate_offset >= 0) {
        const float g = to_float(row[gate_offset + (gate_per_head ? head_of[i] : o)]);
        v *= 1.0f / (1.0f + expf(-g));
      }
      out[(size_t)t * outputs + o] = from_float<T>(v);
    }
  }
}

// The parts of a row put together: out = sum_s acc_s e^(max_s - max) / sum_s total_s e^(max_s - max), then the gate.  A CTA per
// (row, head), a thread per output element: its loads over the parts do not depend on one another.
template <typename T>
__global__ void merge_mixed_kernel(const float* __restrict__ partial, const T* __restrict__ rows, int row_stride, int gate_offset, T* __restrict__ out,
                                   int heads, int value_dim, int splits, int gate_per_head, const float* __restrict__ sinks) {
  __shared__ float weight_s[64];   // at most 64 parts: each part's e^(max - highest), then divided by the sum of the parts' totals
  __shared__ float scratch[2];
  const int t = blockIdx.x, h = blockIdx.y;
  const int outputs = heads * value_dim;
  const size_t part_size = (size_t)outputs + 2 * heads;
  const float* mine = partial + (size_t)t * splits * part_size;
  if (threadIdx.x < 32) {   // one warp: a lane per part (two at most), all loads in one round trip
    const int lane = threadIdx.x;
    float top[2], sum[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int s = lane + 32 * i;
      top[i] = s < splits ? mine[s * part_size + outputs + h] : -INFINITY;
      sum[i] = s < splits ? mine[s * part_size + outputs + heads + h] : 0.0f;
    }
    const float highest = sinks ? fmaxf(warp_max(fmaxf(top[0], top[1])), sinks[h]) : warp_max(fmaxf(top[0], top[1]));
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float weight = expf(top[i] - highest);   // a part that saw no key has maximum -inf: weight 0
      if (lane + 32 * i < splits) weight_s[lane + 32 * i] = weight;
      total += sum[i] * weight;
    }
    total = warp_sum(total);
    if (sinks) total += expf(sinks[h] - highest);
    if (lane == 0) scratch[0] = 1.0f / total;
  }
  __syncthreads();
  const float inv = scratch[0];
  for (int d = threadIdx.x; d < value_dim; d += blockDim.x) {
    const int o = h * value_dim + d;
    float value[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int s = 0;
    for (; s + 4 <= splits; s += 4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) value[i] += mine[(s + i) * part_size + o] * weight_s[s + i];
    }
    for (; s < splits; ++s) value[0] += mine[s * part_size + o] * weight_s[s];
    float v = ((value[0] + value[1]) + (value[2] + value[3])) * inv;
    if (gate_offset >= 0) {
      const float g = to_float(rows[(size_t)t * row_stride + gate_offset + (gate_per_head ? h : o)]);
      v *= 1.0f / (1.0f + expf(-g));
    }
    out[(size_t)t * outputs + o] = from_float<T>(v);
  }
}

template <typename T, int ACC>
static int launch_mixed(const void* rows, int row_stride, int gate_offset, const void* k_pages, long long k_page_stride, const void* v_pages,
                        long long v_page_stride, const int* positions, const int* token_seq, const int* block_table, int table_stride,
                        const float* slopes, const float* mix, void* out, int tokens, int heads, int kv_heads, int key_dim, int value_dim,
                        int page_size, int window, float scale, size_t smem, int splits, float* partial, int keep_first, int gate_per_head,
                        const float* sinks, int v_row_stride, cudaStream_t stream) {
  auto kernel = mixed_heads_attention_kernel<T, ACC>;
  // room for a tile's keys and values of every key/value head behind the 32-bit part; without it rows are read from global memory
  const size_t tiles = (size_t)kv_heads * kMixKeys * ((size_t)staged_key_stride<T>(key_dim) + value_dim) * sizeof(T);
  const size_t with_tiles = (smem + 15) / 16 * 16 + tiles;
  const int staged = with_tiles <= 160 * 1024 ? 1 : 0;
  if (staged) smem = with_tiles;
  if (smem > 48 * 1024) {
    const cudaError_t set = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (set != cudaSuccess) return (int)set;
  }
  kernel<<<dim3(tokens, splits), kMixThreads, smem, stream>>>((const T*)rows, row_stride, gate_offset, (const T*)k_pages, k_page_stride, (const T*)v_pages,
                                                              v_page_stride, positions, token_seq, block_table, table_stride, slopes, mix, (T*)out, heads,
                                                              kv_heads, key_dim, value_dim, page_size, window, scale, partial, staged, keep_first, gate_per_head,
                                                              sinks, v_row_stride);
  if (splits > 1)
    merge_mixed_kernel<T><<<dim3(tokens, heads), value_dim >= 128 ? 128 : (value_dim > 32 ? 64 : 32), 0, stream>>>(partial, (const T*)rows, row_stride, gate_offset,
                                                                                                                  (T*)out, heads, value_dim, splits, gate_per_head, sinks);
  return (int)cudaGetLastError();
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_store_kv_planes(int dtype, const void* rows, int row_stride, int k_offset, int v_offset, const int* positions,
                                     const int* token_seq, const int* block_table, int table_stride, void* k_pages, long long k_page_stride,
                                     void* v_pages, long long v_page_stride, int tokens, int kv_heads, int key_dim, int value_dim, int page_size,
                                     cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dtype == TLIE_F32)
    store_kv_planes_kernel<float><<<tokens, 128, 0, stream>>>((const float*)rows, row_stride, k_offset, v_offset, positions, token_seq, block_table,
                                                              table_stride, (float*)k_pages, k_page_stride, (float*)v_pages, v_page_stride, kv_heads,
                                                              key_dim, value_dim, page_size);
  else
    store_kv_planes_kernel<__nv_bfloat16><<<tokens, 128, 0, stream>>>((const __nv_bfloat16*)rows, row_stride, k_offset, v_offset, positions, token_seq,
                                                                      block_table, table_stride, (__nv_bfloat16*)k_pages, k_page_stride,
                                                                      (__nv_bfloat16*)v_pages, v_page_stride, kv_heads, key_dim, value_dim, page_size);
  return (int)cudaGetLastError();
}

// ``q_bias`` / ``k_bias`` / ``v_bias`` null: none.  ``rot_dims`` 0 (then ``inv_freq`` may be null): nothing turns.
TLIE_EXPORT int tlie_rotary_store_planes(int dtype, void* rows, int row_stride, int k_offset, int v_offset, const float* q_bias, const float* k_bias, const float* v_bias,
                                         const float* inv_freq, int rot_dims, const int* positions, const int* token_seq, const int* block_table, int table_stride,
                                         void* k_pages, long long k_page_stride, void* v_pages, long long v_page_stride, int tokens, int heads, int kv_heads, int key_dim,
                                         int value_dim, int page_size, int write_cache, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > key_dim || rot_dims > 8192 || (rot_dims > 0 && inv_freq == nullptr)) return (int)cudaErrorInvalidValue;
  if (dtype == TLIE_F32)
    rotary_store_planes_kernel<float><<<tokens, 256, (size_t)rot_dims * sizeof(float), stream>>>((float*)rows, row_stride, k_offset, v_offset, q_bias, k_bias, v_bias, inv_freq, rot_dims, positions,
                                                                  token_seq, block_table, table_stride, (float*)k_pages, k_page_stride, (float*)v_pages, v_page_stride,
                                                                  heads, kv_heads, key_dim, value_dim, page_size, write_cache);
  else
    rotary_store_planes_kernel<__nv_bfloat16><<<tokens, 256, (size_t)rot_dims * sizeof(float), stream>>>((__nv_bfloat16*)rows, row_stride, k_offset, v_offset, q_bias, k_bias, v_bias, inv_freq, rot_dims,
                                                                          positions, token_seq, block_table, table_stride, (__nv_bfloat16*)k_pages, k_page_stride,
                                                                          (__nv_bfloat16*)v_pages, v_page_stride, heads, kv_heads, key_dim, value_dim, page_size,
                                                                          write_cache);
  return (int)cudaGetLastError();
}

// ``gate_offset`` < 0: no output gate.  ``slopes`` / ``mix`` null: no distance bias / heads left as they are.  ``splits`` > 1: every row's
// keys are dealt to that many CTAs (steps of few rows and long contexts); ``partial`` then holds tokens * splits * (heads * value_dim + 2 * heads) floats.
TLIE_EXPORT int tlie_mixed_heads_attention(int dtype, const void* rows, int row_stride, int gate_offset, const void* k_pages,
                                           long long k_page_stride, const void* v_pages, long long v_page_stride, const int* positions,
                                           const int* token_seq, const int* block_table, int table_stride, const float* slopes, const float* mix,
                                           void* out, int tokens, int heads, int kv_heads, int key_dim, int value_dim, int page_size, int window,
                                           float scale, int splits, float* partial, int keep_first, int gate_per_head, const float* sinks,
                                           int v_row_stride, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (keep_first < 0 || v_row_stride < value_dim) return (int)cudaErrorInvalidValue;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || key_dim <= 0 || value_dim <= 0 || splits < 1 || splits > 64 || (splits > 1 && partial == nullptr))
    return (int)cudaErrorInvalidValue;
  const int outputs = heads * value_dim;
  if (outputs > 32 * kMixThreads) return (int)cudaErrorInvalidValue;
  const size_t floats = (size_t)heads * key_dim + (mix ? (size_t)heads * heads : 0) + 2 * (size_t)heads * kMixKeys + 3 * (size_t)heads;
  const size_t smem = floats * sizeof(float) + 2 * kMixKeys * sizeof(long long);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
#define TLIE_MIXED(T, ACC)                                                                                                                    \
  return launch_mixed<T, ACC>(rows, row_stride, gate_offset, k_pages, k_page_stride, v_pages, v_page_stride, positions, token_seq, block_table, \
                              table_stride, slopes, mix, out, tokens, heads, kv_heads, key_dim, value_dim, page_size, window, scale, smem, splits, partial, \
                              keep_first, gate_per_head, sinks, v_row_stride, stream)
  if (dtype == TLIE_F32) {
    if (outputs <= 4 * kMixThreads) TLIE_MIXED(float, 4);
    if (outputs <= 8 * kMixThreads) TLIE_MIXED(float, 8);
    if (outputs <= 16 * kMixThreads) TLIE_MIXED(float, 16);
    TLIE_MIXED(float, 32);
  }
  if (outputs <= 4 * kMixThreads) TLIE_MIXED(__nv_bfloat16, 4);
  if (outputs <= 8 * kMixThreads) TLIE_MIXED(__nv_bfloat16, 8);
  if (outputs <= 16 * kMixThreads) TLIE_MIXED(__nv_bfloat16, 16);
  TLIE_MIXED(__nv_bfloat16, 32);
#undef TLIE_MIXED
}

// q (in place) and k divided by their root mean square per head, k into the key plane, the value columns into the value plane.
TLIE_EXPORT int tlie_normed_store(int dtype, void* rows, int row_stride, int k_offset, int v_offset, const float* q_weight, const float* k_weight, float eps,
                                  const int* positions, const int* token_seq, const int* block_table, int table_stride, void* k_pages, long long k_page_stride,
                                  void* v_pages, long long v_page_stride, int tokens, int heads, int kv_heads, int key_dim, int value_dim, int page_size,
                                  int write_cache, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dtype == TLIE_F32)
    normed_store_kernel<float><<<tokens, 128, 0, stream>>>((float*)rows, row_stride, k_offset, v_offset, q_weight, k_weight, eps, positions, token_seq, block_table,
                                                           table_stride, (float*)k_pages, k_page_stride, (float*)v_pages, v_page_stride, heads, kv_heads, key_dim,
                                                           value_dim, page_size, write_cache);
  else
    normed_store_kernel<__nv_bfloat16><<<tokens, 128, 0, stream>>>((__nv_bfloat16*)rows, row_stride, k_offset, v_offset, q_weight, k_weight, eps, positions, token_seq,
                                                                   block_table, table_stride, (__nv_bfloat16*)k_pages, k_page_stride, (__nv_bfloat16*)v_pages,
                                                                   v_page_stride, heads, kv_heads, key_dim, value_dim, page_size, write_cache);
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_latent_store(int dtype, const void* rows, int row_stride, int latent_offset, const float* weight, float eps, const float* inv_freq, int rot_dims,
                                  const int* positions, const int* token_seq, const int* block_table, int table_stride, void* pages, long long page_stride,
                                  int tokens, int heads, int plain, int rot, int rank, int page_size, int write_cache, void* queries, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rot_dims < 0 || rot_dims > rot || (rot_dims & 1) || (rot & 1)) return (int)cudaErrorInvalidValue;
  if (dtype == TLIE_F32)
    latent_store_kernel<float><<<tokens, 128, 0, stream>>>((const float*)rows, row_stride, latent_offset, weight, eps, inv_freq, rot_dims, positions, token_seq, block_table,
                                                           table_stride, (float*)pages, page_stride, heads, plain, rot, rank, page_size, write_cache, (float*)queries);
  else
    latent_store_kernel<__nv_bfloat16><<<tokens, 128, 0, stream>>>((const __nv_bfloat16*)rows, row_stride, latent_offset, weight, eps, inv_freq, rot_dims, positions, token_seq,
                                                                   block_table, table_stride, (__nv_bfloat16*)pages, page_stride, heads, plain, rot, rank, page_size,
                                                                   write_cache, (__nv_bfloat16*)queries);
  return (int)cudaGetLastError();
}

// The merge alone, for a kernel of another file that leaves a row's parts in the same layout (bfloat16 output, no gate).
TLIE_EXPORT int tlie_merge_parts(const float* partial, void* out, int tokens, int heads, int value_dim, int splits, const float* sinks, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (splits < 1 || splits > 64) return (int)cudaErrorInvalidValue;
  merge_mixed_kernel<__nv_bfloat16><<<dim3(tokens, heads), value_dim >= 128 ? 128 : (value_dim > 32 ? 64 : 32), 0, stream>>>(partial, nullptr, 0, -1, (__nv_bfloat16*)out, heads,
                                                                                                                          value_dim, splits, 0, sinks);
  return (int)cudaGetLastError();
}
