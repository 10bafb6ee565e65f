// A feed-forward of routed experts: every token goes through ``top`` of ``experts`` small gated feed-forwards, chosen by a router.
//
//   moe_route     per token: z = W_router x (32-bit), s = sigmoid(z), choice = s + correction.  Experts form ``groups`` equal groups
//                 of neighbours; a group's score is the sum of its two largest choice scores; only experts of the ``keep`` best
//                 groups can be chosen.  The ``top`` largest choice scores among them are chosen (ties: the lower index); their
//                 weights are s / (sum of the chosen s + 1e-20) * route_scale (``normalize`` 0: s * route_scale, the scores as they are).
//   moe_gate_up   per (token, chosen expert): act(W_gate x) * (W_up x), straight from the expert's rows (steps of few rows, and the
//                 32-bit path): a warp per output, the sums in a fixed order.
//   moe_down      per token: sum over its chosen experts of weight * W_down act, plus the shared branch if there is one.
//                 ``weight_input``: the weight multiplies what the expert reads instead (moe_gate_up scales the token as it loads it,
//                 moe_down adds the experts' outputs as they are).
//
// Expert weights are stacked: gate_up [experts][2 ff][width] (gate rows, then up rows), down [experts][width][ff].
// Activation codes: 0 silu, 1 gelu in its tanh form.
#include "common.cuh"

namespace tlie {

__device__ __forceinline__ float moe_act(float z, int kind) {
  if (kind == 1) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z / (1.0f + expf(-z));
}

// the lane's share of w . x: w a row of T in global memory, x 32-bit numbers in shared memory; 16 bytes at a time where rows allow it
__device__ __forceinline__ float lane_dot(const float* w, const float* x, int width, int lane, bool vector) {
  float sum = 0.0f;
  if (vector) {
    for (int d = lane * 4; d < width; d += 128) {
      const float4 a = *reinterpret_cast<const float4*>(w + d);
      sum = fmaf(a.x, x[d], sum);
      sum = fmaf(a.y, x[d + 1], sum);
      sum = fmaf(a.z, x[d + 2], sum);
      sum = fmaf(a.w, x[d + 3], sum);
    }
  } else {
    for (int d = lane; d < width; d += 32) sum = fmaf(w[d], x[d], sum);
  }
  return sum;
}
__device__ __forceinline__ float lane_dot(const __nv_bfloat16* w, const float* x, int width, int lane, bool vector) {
  float sum = 0.0f;
  if (vector) {
    for (int d = lane * 8; d < width; d += 256) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + d);
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __bfloat1622float2(pairs[i]);
        sum = fmaf(a.x, x[d + 2 * i], sum);
        sum = fmaf(a.y, x[d + 2 * i + 1], sum);
      }
    }
  } else {
    for (int d = lane; d < width; d += 32) sum = fmaf(__bfloat162float(w[d]), x[d], sum);
  }
  return sum;
}
// N rows against the same x at once: every pass of the loop has N independent 16-byte loads in flight per lane and reads its piece of x
// once for all of them (a row at a time left a warp with one row's loads in flight and a chain of dependent sums behind each).  Every
// row's sum is formed in the order lane_dot forms it, so the bits are the same.
template <int N>
__device__ __forceinline__ void lane_dot_n(const float* const (&w)[N], const float* x, int width, int lane, bool vector, float (&sums)[N]) {
#pragma unroll
  for (int r = 0; r < N; ++r) sums[r] = 0.0f;
  if (vector) {
    for (int d = lane * 4; d < width; d += 128) {
      float4 a[N];
#pragma unroll
      for (int r = 0; r < N; ++r) a[r] = *reinterpret_cast<const float4*>(w[r] + d);
      const float4 v = *reinterpret_cast<const float4*>(x + d);
#pragma unroll
      for (int r = 0; r < N; ++r) {
        sums[r] = fmaf(a[r].x, v.x, sums[r]);
        sums[r] = fmaf(a[r].y, v.y, sums[r]);
        sums[r] = fmaf(a[r].z, v.z, sums[r]);
        sums[r] = fmaf(a[r].w, v.w, sums[r]);
      }
    }
  } else {
#pragma unroll
    for (int r = 0; r < N; ++r) sums[r] = lane_dot(w[r], x, width, lane, false);
  }
}
template <int N>
__device__ __forceinline__ void lane_dot_n(const __nv_bfloat16* const (&w)[N], const float* x, int width, int lane, bool vector, float (&sums)[N]) {
#pragma unroll
  for (int r = 0; r < N; ++r) sums[r] = 0.0f;
  if (vector) {
    for (int d = lane * 8; d < width; d += 256) {
      uint4 raw[N];
#pragma unroll
      for (int r = 0; r < N; ++r) raw[r] = *reinterpret_cast<const uint4*>(w[r] + d);
      const float4 v0 = *reinterpret_cast<const float4*>(x + d), v1 = *reinterpret_cast<const float4*>(x + d + 4);
      const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
      for (int r = 0; r < N; ++r) {
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw[r]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 a = __bfloat1622float2(pairs[i]);
          sums[r] = fmaf(a.x, v[2 * i], sums[r]);
          sums[r] = fmaf(a.y, v[2 * i + 1], sums[r]);
        }
      }
    }
  } else {
#pragma unroll
    for (int r = 0; r < N; ++r) sums[r] = lane_dot(w[r], x, width, lane, false);
  }
}
// 16 bytes of a row as 32-bit numbers
__device__ __forceinline__ void load_piece(const float* p, float (&v)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w;
}
__device__ __forceinline__ void load_piece(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(pairs[i]);
    v[2 * i] = a.x, v[2 * i + 1] = a.y;
  }
}
// Two outputs x K inputs: row w[o][k] against x[k], all 2 K rows' loads of a pass in flight together; sums as lane_dot forms them.
template <int K, typename T>
__device__ __forceinline__ void lane_dot_sides(const T* const (&w)[2][K], const float* const (&x)[K], int width, int lane, bool vector, float (&sums)[2][K]) {
  constexpr int kPiece = 16 / (int)sizeof(T);
#pragma unroll
  for (int o = 0; o < 2; ++o)
#pragma unroll
    for (int k = 0; k < K; ++k) sums[o][k] = 0.0f;
  if (vector) {
    for (int d = lane * kPiece; d < width; d += 32 * kPiece) {
      float a[2][K][kPiece];
#pragma unroll
      for (int o = 0; o < 2; ++o)
#pragma unroll
        for (int k = 0; k < K; ++k) load_piece(w[o][k] + d, a[o][k]);
#pragma unroll
      for (int k = 0; k < K; ++k) {
#pragma unroll
        for (int i = 0; i < kPiece; ++i) {
          const float v = x[k][d + i];
          sums[0][k] = fmaf(a[0][k][i], v, sums[0][k]);
          sums[1][k] = fmaf(a[1][k][i], v, sums[1][k]);
        }
      }
    }
  } else {
#pragma unroll
    for (int o = 0; o < 2; ++o)
#pragma unroll
      for (int k = 0; k < K; ++k) sums[o][k] = lane_dot(w[o][k], x[k], width, lane, false);
  }
}
// The same for bfloat16 rows with the pieces kept as they were loaded (four registers each, not eight) until they are used: with the
// converted pieces the kernel took 102 registers and two CTAs an SM, sixteen warps, which left the loads in flight short of what memory needs.
template <int K>
__device__ __forceinline__ void lane_dot_sides(const __nv_bfloat16* const (&w)[2][K], const float* const (&x)[K], int width, int lane, bool vector, float (&sums)[2][K]) {
#pragma unroll
  for (int o = 0; o < 2; ++o)
#pragma unroll
    for (int k = 0; k < K; ++k) sums[o][k] = 0.0f;
  if (vector) {
    for (int d = lane * 8; d < width; d += 256) {
      uint4 raw[2][K];
#pragma unroll
      for (int o = 0; o < 2; ++o)
#pragma unroll
        for (int k = 0; k < K; ++k) raw[o][k] = *reinterpret_cast<const uint4*>(w[o][k] + d);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const __nv_bfloat162* p0 = reinterpret_cast<const __nv_bfloat162*>(&raw[0][k]);
        const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&raw[1][k]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 a0 = __bfloat1622float2(p0[i]), a1 = __bfloat1622float2(p1[i]);
          const float v0 = x[k][d + 2 * i], v1 = x[k][d + 2 * i + 1];
          sums[0][k] = fmaf(a0.x, v0, sums[0][k]);
          sums[1][k] = fmaf(a1.x, v0, sums[1][k]);
          sums[0][k] = fmaf(a0.y, v1, sums[0][k]);
          sums[1][k] = fmaf(a1.y, v1, sums[1][k]);
        }
      }
    }
  } else {
#pragma unroll
    for (int o = 0; o < 2; ++o)
#pragma unroll
      for (int k = 0; k < K; ++k) sums[o][k] = lane_dot(w[o][k], x[k], width, lane, false);
  }
}
template <typename T>
__device__ __forceinline__ bool rows_are_vectors(const T* base, int width) {
  return width % (16 / (int)sizeof(T)) == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
}

// the largest of values[0 .. n) over the warp, the lower index on ties; every lane gets the answer
__device__ __forceinline__ int warp_argmax(const float* values, int n, int lane, float& best_value) {
  float best = -INFINITY;
  int at = 0x7fffffff;
  for (int i = lane; i < n; i += 32)
    if (values[i] > best || at == 0x7fffffff) {
      best = values[i];
      at = i;
    }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, best, offset);
    const int other_at = __shfl_xor_sync(0xffffffffu, at, offset);
    if (other_at != 0x7fffffff && (at == 0x7fffffff || other > best || (other == best && other_at < at))) {
      best = other;
      at = other_at;
    }
  }
  best_value = best;
  return at;
}

constexpr int kRouteWarps = 4;

// One warp chooses a token's experts from s [experts] and choice [experts] (shared memory, written before); group_score [groups] is scratch.
__device__ __forceinline__ void route_select(float* s, float* choice, float* group_score, int* __restrict__ ids, float* __restrict__ weights, int t, int lane,
                                             int experts, int groups, int keep, int top, float route_scale, int normalize) {
  const int per = experts / groups;
  if (groups > 1 && keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      float first = -INFINITY, second = -INFINITY;
      for (int i = 0; i < per; ++i) {
        const float c = choice[g * per + i];
        if (c > first) {
          second = first;
          first = c;
        } else if (c > second) {
          second = c;
        }
      }
      group_score[g] = per > 1 ? first + second : first;
    }
    __syncwarp();
    // the ``keep`` best groups are marked by a score of +inf; the others' experts leave the choice
    for (int round = 0; round < keep; ++round) {
      float value;
      // groups already taken hold +inf and would win again: pick among the rest
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (group_score[g] != INFINITY && (at == 0x7fffffff || group_score[g] > best)) {
          best = group_score[g];
          at = g;
        }
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_at = __shfl_xor_sync(0xffffffffu, at, offset);
        if (other_at != 0x7fffffff && (at == 0x7fffffff || other > best || (other == best && other_at < at))) {
          best = other;
          at = other_at;
        }
      }
      (void)value;
      if (lane == 0 && at != 0x7fffffff) group_score[at] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (group_score[e / per] != INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.0f;
  for (int k = 0; k < top; ++k) {
    float value;
    const int e = warp_argmax(choice, experts, lane, value);
    if (lane == 0) {
      ids[(size_t)t * top + k] = e;
      weights[(size_t)t * top + k] = s[e];
      choice[e] = -INFINITY;
    }
    total += s[e];
    __syncwarp();
  }
  const float factor = normalize ? route_scale / (total + 1e-20f) : route_scale;   // not normalised: the scores as they are
  for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] *= factor;
}

// The general form: a warp per token; shared memory per warp: s [experts], choice [experts], group scores [groups]
template <typename T>
__global__ void __launch_bounds__(kRouteWarps * 32) moe_route_kernel(const T* __restrict__ x, const float* __restrict__ router, const float* __restrict__ correction,
                                                                     int* __restrict__ ids, float* __restrict__ weights, int tokens, int width, int experts,
                                                                     int groups, int keep, int top, float route_scale, int normalize) {
  extern __shared__ float route_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  if (t >= tokens) return;
  float* s = route_smem + (size_t)warp * (2 * experts + groups);
  float* choice = s + experts;
  float* group_score = choice + experts;
  const T* row = x + (size_t)t * width;
  for (int e = 0; e < experts; ++e) {
    const float* w = router + (size_t)e * width;
    float sum = 0.0f;
    for (int d = lane; d < width; d += 32) sum = fmaf(w[d], to_float(row[d]), sum);
    sum = warp_sum(sum);
    if (lane == 0) {
      const float score = 1.0f / (1.0f + expf(-sum));
      s[e] = score;
      choice[e] = score + (correction != nullptr ? correction[e] : 0.0f);
    }
  }
  __syncwarp();
  route_select(s, choice, group_score, ids, weights, t, lane, experts, groups, keep, top, route_scale, normalize);
}

constexpr int kRouteTiledWarps = 8;    // steps of many tokens (four share a CTA); a CTA of one token has 16 warps

// Rows of a multiple of 4 numbers: a CTA of eight warps per TOK tokens.  The tokens' rows wait in shared memory as 32-bit numbers; a warp
// takes every eighth expert and reads its row of the router once for all TOK tokens, 16 bytes a lane at a time, so that the router
// is read tokens / TOK times (out of L2) and a step of few tokens spreads over experts as well as tokens.  A token's sum runs over
// the columns in the same order whatever TOK is and whoever shares the CTA.  Then warp i chooses for token i as above.
// Shared memory: x [TOK][width], then per token s [experts], choice [experts], group scores [groups].
template <typename T, int TOK, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) moe_route_tiled_kernel(const T* __restrict__ x, const float* __restrict__ router,
                                                                                const float* __restrict__ correction, int* __restrict__ ids,
                                                                                float* __restrict__ weights, int tokens, int width, int experts, int groups, int keep,
                                                                                int top, float route_scale, int normalize) {
  extern __shared__ __align__(16) float route_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * TOK;
  float* xs = route_smem;
  float* tables = xs + (size_t)TOK * width;
  const int per_token = 2 * experts + groups;
#pragma unroll
  for (int i = 0; i < TOK; ++i) {
    const bool live = t0 + i < tokens;
    const T* row = x + (size_t)(live ? t0 + i : t0) * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x) xs[(size_t)i * width + d] = live ? to_float(row[d]) : 0.0f;
  }
  __syncthreads();
  // two experts of a warp side by side and four pieces of each ahead: a row at a time with one piece in flight made a step of few
  // tokens wait for memory once per 512 bytes of a row.  An expert past the end reads the last one again and writes nothing.
  for (int e0 = warp; e0 < experts; e0 += 2 * WARPS) {
    const int e1 = e0 + WARPS;
    const float* w0 = router + (size_t)e0 * width;
    const float* w1 = router + (size_t)min(e1, experts - 1) * width;
    float sum[2][TOK];
#pragma unroll
    for (int i = 0; i < TOK; ++i) sum[0][i] = sum[1][i] = 0.0f;
#pragma unroll 4
    for (int d = lane * 4; d < width; d += 128) {
      const float4 a0 = *reinterpret_cast<const float4*>(w0 + d);
      const float4 a1 = *reinterpret_cast<const float4*>(w1 + d);
#pragma unroll
      for (int i = 0; i < TOK; ++i) {
        const float4 b = *reinterpret_cast<const float4*>(xs + (size_t)i * width + d);
        sum[0][i] = fmaf(a0.x, b.x, sum[0][i]);
        sum[0][i] = fmaf(a0.y, b.y, sum[0][i]);
        sum[0][i] = fmaf(a0.z, b.z, sum[0][i]);
        sum[0][i] = fmaf(a0.w, b.w, sum[0][i]);
        sum[1][i] = fmaf(a1.x, b.x, sum[1][i]);
        sum[1][i] = fmaf(a1.y, b.y, sum[1][i]);
        sum[1][i] = fmaf(a1.z, b.z, sum[1][i]);
        sum[1][i] = fmaf(a1.w, b.w, sum[1][i]);
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int e = j == 0 ? e0 : e1;
      if (e >= experts) break;
      const float shift = correction != nullptr ? correction[e] : 0.0f;
#pragma unroll
      for (int i = 0; i < TOK; ++i) {
        const float z = warp_sum(sum[j][i]);
        if (lane == 0) {
          const float score = 1.0f / (1.0f + expf(-z));
          tables[(size_t)i * per_token + e] = score;
          tables[(size_t)i * per_token + experts + e] = score + shift;
        }
      }
    }
  }
  __syncthreads();
  for (int i = warp; i < TOK; i += WARPS) {
    if (t0 + i >= tokens) break;
    float* s = tables + (size_t)i * per_token;
    route_select(s, s + experts, s + 2 * experts, ids, weights, t0 + i, lane, experts, groups, keep, top, route_scale, normalize);
  }
}

constexpr int kMoeWarps = 8;
constexpr int kGateUpOutputs = 32;   // outputs of one CTA of the direct first half
constexpr int kDownOutputs = 32;

// grid (tokens * top, ceil(ff / 32)); act [tokens * top][ff]
template <typename T>
__global__ void __launch_bounds__(kMoeWarps * 32) moe_gate_up_kernel(const T* __restrict__ x, const T* __restrict__ gate_up, const int* __restrict__ ids,
                                                                     const float* __restrict__ input_weights, T* __restrict__ act, int width, int ff, int top, int kind) {
  extern __shared__ float moe_x[];
  const int slot = blockIdx.x, t = slot / top;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float scale = input_weights != nullptr ? input_weights[slot] : 1.0f;   // an expert that reads its token times the token's weight
  for (int d = threadIdx.x; d < width; d += blockDim.x) moe_x[d] = to_float(x[(size_t)t * width + d]) * scale;
  __syncthreads();
  const T* expert = gate_up + (size_t)ids[slot] * 2 * ff * width;
  const bool vector = rows_are_vectors(expert, width);
  // a warp's outputs (warp, warp + kMoeWarps, ...) four at a time: four gate rows and four up rows side by side.  Outputs past the end
  // read the last row again and store nothing.
  constexpr int kPerWarp = kGateUpOutputs / kMoeWarps;
  static_assert(kPerWarp == 4, "four outputs per warp");
  const T* rows[2 * kPerWarp];
  int f[kPerWarp];
#pragma unroll
  for (int j = 0; j < kPerWarp; ++j) {
    f[j] = blockIdx.y * kGateUpOutputs + warp + j * kMoeWarps;
    const int row = min(f[j], ff - 1);
    rows[2 * j] = expert + (size_t)row * width;
    rows[2 * j + 1] = expert + (size_t)(ff + row) * width;
  }
  float sums[2 * kPerWarp];
  lane_dot_n<2 * kPerWarp>(rows, moe_x, width, lane, vector, sums);
#pragma unroll
  for (int j = 0; j < kPerWarp; ++j) {
    const float g = warp_sum(sums[2 * j]);
    const float u = warp_sum(sums[2 * j + 1]);
    if (lane == 0 && f[j] < ff) act[(size_t)slot * ff + f[j]] = from_float<T>(moe_act(g, kind) * u);
  }
}

// grid (tokens, ceil(width / 32)); out[t] = sum_k weight_k * W_down[e_k] act[t, k]  (+ shared[t])
template <typename T>
__global__ void __launch_bounds__(kMoeWarps * 32, 4) moe_down_kernel(const T* __restrict__ act, const T* __restrict__ down, const int* __restrict__ ids,
                                                                  const float* __restrict__ weights, const T* __restrict__ shared, T* __restrict__ out, int width,
                                                                  int ff, int top) {
  extern __shared__ float moe_act_rows[];   // [top][ff]
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < top * ff; i += blockDim.x) moe_act_rows[i] = to_float(act[(size_t)t * top * ff + i]);
  __syncthreads();
  const bool vector = rows_are_vectors(down, ff);
  // two of a warp's outputs at a time, each with four chosen experts' rows side by side (eight rows in flight); experts past ``top``
  // read the last one's row again and are left out of the sum.  A token's experts are added in the order they were chosen.
  constexpr int kSide = 4;
  for (int i = warp; i < kDownOutputs; i += 2 * kMoeWarps) {
    int n[2];
    n[0] = blockIdx.y * kDownOutputs + i;
    n[1] = n[0] + kMoeWarps;
    if (n[0] >= width) break;
    float total[2] = {0.0f, 0.0f};
    for (int k0 = 0; k0 < top; k0 += kSide) {
      const T* rows[2][kSide];
      const float* inputs[kSide];
#pragma unroll
      for (int j = 0; j < kSide; ++j) {
        const int k = min(k0 + j, top - 1);
        const size_t expert = (size_t)ids[(size_t)t * top + k] * width;
        inputs[j] = moe_act_rows + (size_t)k * ff;
#pragma unroll
        for (int o = 0; o < 2; ++o) rows[o][j] = down + (expert + min(n[o], width - 1)) * ff;
      }
      float sums[2][kSide];
      lane_dot_sides<kSide>(rows, inputs, ff, lane, vector, sums);
#pragma unroll
      for (int j = 0; j < kSide; ++j) {
#pragma unroll
        for (int o = 0; o < 2; ++o) {
          const float dot = warp_sum(sums[o][j]);
          if (k0 + j < top) total[o] += (weights != nullptr ? weights[(size_t)t * top + k0 + j] : 1.0f) * dot;
        }
      }
    }
#pragma unroll
    for (int o = 0; o < 2; ++o) {
      if (n[o] >= width) continue;
      float value = total[o];
      if (shared != nullptr) value += to_float(shared[(size_t)t * width + n[o]]);
      if (lane == 0) out[(size_t)t * width + n[o]] = from_float<T>(value);
    }
  }
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_moe_route(int dtype, const void* x, const float* router, const float* correction, int* ids, float* weights, int tokens, int width, int experts,
                               int groups, int keep, int top, float route_scale, int normalize, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (experts <= 0 || groups <= 0 || experts % groups != 0 || keep <= 0 || keep > groups || top <= 0 || top > keep * (experts / groups))
    return (int)cudaErrorInvalidValue;
  const size_t tables = (size_t)(2 * experts + groups) * sizeof(float);
  if (width % 4 == 0 && (reinterpret_cast<uintptr_t>(router) & 15) == 0) {
    // few tokens: a CTA each, so that the step spreads over the SMs; many: four share a CTA and a reading of the router
    const int tok = tokens >= 4 * 2 * device_sm_count() ? 4 : 1;
    const size_t tiled = (size_t)tok * ((size_t)width * sizeof(float) + tables);
    if (tiled <= 200 * 1024) {
      const int blocks = (tokens + tok - 1) / tok;
      cudaError_t e = cudaSuccess;
#define TLIE_ROUTE_TILED(T, TOK)                                                                                                                          \
  do {                                                                                                                                                    \
    if (tiled > 48 * 1024) e = cudaFuncSetAttribute(moe_route_tiled_kernel<T, TOK, (TOK == 1 ? 16 : kRouteTiledWarps)>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tiled);             \
    if (e == cudaSuccess)                                                                                                                                 \
      moe_route_tiled_kernel<T, TOK, (TOK == 1 ? 16 : kRouteTiledWarps)><<<blocks, (TOK == 1 ? 16 : kRouteTiledWarps) * 32, tiled, stream>>>((const T*)x, router, correction, ids, weights, tokens, width, experts, groups, keep, \
                                                                                     top, route_scale, normalize);                                                  \
  } while (0)
      if (dtype == TLIE_F32) {
        if (tok == 4) TLIE_ROUTE_TILED(float, 4); else TLIE_ROUTE_TILED(float, 1);
      } else {
        if (tok == 4) TLIE_ROUTE_TILED(__nv_bfloat16, 4); else TLIE_ROUTE_TILED(__nv_bfloat16, 1);
      }
#undef TLIE_ROUTE_TILED
      return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
    }
  }
  const size_t smem = kRouteWarps * tables;
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  const int blocks = (tokens + kRouteWarps - 1) / kRouteWarps;
  if (dtype == TLIE_F32)
    moe_route_kernel<float><<<blocks, kRouteWarps * 32, smem, stream>>>((const float*)x, router, correction, ids, weights, tokens, width, experts, groups, keep, top, route_scale, normalize);
  else
    moe_route_kernel<__nv_bfloat16><<<blocks, kRouteWarps * 32, smem, stream>>>((const __nv_bfloat16*)x, router, correction, ids, weights, tokens, width, experts, groups,
                                                                              keep, top, route_scale, normalize);
  return (int)cudaGetLastError();
}

template <typename T>
static int launch_moe_experts(const void* x, const void* gate_up, const void* down, const int* ids, const float* weights, const void* shared, void* act, void* out,
                              int tokens, int width, int ff, int top, int kind, int weight_input, cudaStream_t stream) {
  const size_t x_smem = (size_t)width * sizeof(float), act_smem = (size_t)top * ff * sizeof(float);
  if (x_smem > 200 * 1024 || act_smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  cudaError_t e;
  if (x_smem > 48 * 1024) {
    e = cudaFuncSetAttribute(moe_gate_up_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)x_smem);
    if (e != cudaSuccess) return (int)e;
  }
  if (act_smem > 48 * 1024) {
    e = cudaFuncSetAttribute(moe_down_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)act_smem);
    if (e != cudaSuccess) return (int)e;
  }
  moe_gate_up_kernel<T><<<dim3(tokens * top, (ff + kGateUpOutputs - 1) / kGateUpOutputs), kMoeWarps * 32, x_smem, stream>>>(
      (const T*)x, (const T*)gate_up, ids, weight_input ? weights : nullptr, (T*)act, width, ff, top, kind);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  moe_down_kernel<T><<<dim3(tokens, (width + kDownOutputs - 1) / kDownOutputs), kMoeWarps * 32, act_smem, stream>>>(
      (const T*)act, (const T*)down, ids, weight_input ? nullptr : weights, (const T*)shared, (T*)out, width, ff, top);
  return (int)cudaGetLastError();
}

// ``act``: scratch [tokens * top, ff] of ``dtype``; ``shared`` [tokens, width] or null; ``out`` [tokens, width].  ``weight_input`` 1: a chosen expert reads
// the token times its weight and its output is added as it is (out[t] = sum_k expert_k(weight_k x[t])); 0: the weight multiplies the expert's output.
TLIE_EXPORT int tlie_moe_experts(int dtype, const void* x, const void* gate_up, const void* down, const int* ids, const float* weights, const void* shared, void* act,
                                 void* out, int tokens, int width, int ff, int top, int kind, int weight_input, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if ((long long)tokens * top > 2147483647LL / 2 || kind < 0 || kind > 1) return (int)cudaErrorInvalidValue;
  if (dtype == TLIE_F32) return launch_moe_experts<float>(x, gate_up, down, ids, weights, shared, act, out, tokens, width, ff, top, kind, weight_input, stream);
  return launch_moe_experts<__nv_bfloat16>(x, gate_up, down, ids, weights, shared, act, out, tokens, width, ff, top, kind, weight_input, stream);
}
