// Norms around a residual branch, for layers that normalise a sublayer's output before it joins the stream:
//
//   residual[t] += norm(y[t]) * post_weight          (if y is given)
//   out[r]       = norm(residual[rows[r]]) * next_weight   (if out is given; rows null: every row in order)
//
// in one kernel, a CTA per row.  ``centred`` 1: (x - mean) / sqrt(mean((x - mean)^2) + eps), the layer norm without a bias;
// 0: x / sqrt(mean(x^2) + eps).  ``groups`` > 1: the statistics are taken over each of that many equal consecutive parts of the row.  The row waits in shared memory as 32-bit numbers between the passes; mean, variance (of
// the deviations, after the mean is known), the sum into the stream and the second norm are 32-bit whatever y and out are
// stored as.  The order of a row's sums depends on the block size alone.
//
// stream_with_embedding: out[t] = [residual[t] | table[ids[t]] * scale] rounded to out's type: the operand of a product that
// mixes the stream with the embedding's output.
#include <cstdint>
#include "common.cuh"

namespace tlie {

constexpr int kNormThreads = 256;

__device__ __forceinline__ void row_statistics(const float* row, int width, int centred, float eps, float* scratch, float& mean, float& inv) {
  mean = 0.0f;
  if (centred) {
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) sum += row[i];
    mean = block_sum(sum, scratch) / (float)width;
  }
  float squares = 0.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float d = row[i] - mean;
    squares += d * d;
  }
  inv = 1.0f / sqrtf(block_sum(squares, scratch) / (float)width + eps);
}

// The same per group: a row cut into ``groups`` equal consecutive parts, each with statistics of its own, left in shared memory
// (``means`` and ``invs``, one entry per group) for all threads.  One group is the whole row, summed in the order it always was.
constexpr int kNormMaxGroups = 256;
__device__ __forceinline__ void group_statistics(const float* row, int width, int groups, int centred, float eps, float* scratch, float* means, float* invs) {
  const int part = width / groups;
  for (int g = 0; g < groups; ++g) {
    float mean, inv;
    row_statistics(row + g * part, part, centred, eps, scratch, mean, inv);
    if (threadIdx.x == 0) means[g] = mean, invs[g] = inv;
  }
  __syncthreads();
}

// eight neighbours of a row at once, 16 bytes a load: a row of a few thousand numbers is then one or two loads per thread, all of them
// in flight together, where a number per load made every pass of a step of few rows wait for memory several times over
__device__ __forceinline__ void load8(const float* src, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* src, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(pairs[i]);
    v[2 * i] = f.x, v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(float* dst, const float (&v)[8]) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* dst, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) pairs[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(dst) = raw;
}

// The same kernel for rows whose width is a multiple of 8 (every row then starts on a 16-byte boundary): thread t takes the runs of
// eight numbers t, t + block, ...  Which of the two kernels runs depends on the width alone, so a row's bits do not depend on the step.
template <typename TY, typename TO>
__global__ void __launch_bounds__(kNormThreads) branch_norm_wide_kernel(float* __restrict__ residual, const TY* __restrict__ y, const float* __restrict__ post_weight,
                                                                        const float* __restrict__ next_weight, TO* __restrict__ out, const int* __restrict__ rows,
                                                                        float eps, int centred, int width, int groups) {
  extern __shared__ __align__(16) float norm_row[];
  __shared__ float scratch[32];
  __shared__ float means[kNormMaxGroups], invs[kNormMaxGroups];
  const int source = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  float* stream = residual + (size_t)source * width;
  const int part = width / groups;   // a multiple of 8 here: a run of eight lies in one group
  float a[8], b[8], w[8];
  if (y != nullptr) {
    const TY* branch = y + (size_t)source * width;
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
      load8(branch + i, a);
      store8(norm_row + i, a);
    }
    __syncthreads();
    group_statistics(norm_row, width, groups, centred, eps, scratch, means, invs);
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {   // a thread's own runs again
      load8(stream + i, b);
      load8(post_weight + i, w);
      load8(norm_row + i, a);
      const float mean = means[i / part], inv = invs[i / part];
#pragma unroll
      for (int j = 0; j < 8; ++j) b[j] = b[j] + ((a[j] - mean) * inv) * w[j];
      store8(stream + i, b);
      store8(norm_row + i, b);
    }
  } else {
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
      load8(stream + i, b);
      store8(norm_row + i, b);
    }
  }
  if (out == nullptr) return;
  __syncthreads();
  group_statistics(norm_row, width, groups, centred, eps, scratch, means, invs);
  TO* dst = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
    load8(next_weight + i, w);
    load8(norm_row + i, a);
    const float mean = means[i / part], inv = invs[i / part];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = ((a[j] - mean) * inv) * w[j];
    store8(dst + i, a);
  }
}

template <typename TY, typename TO>
__global__ void __launch_bounds__(kNormThreads) branch_norm_kernel(float* __restrict__ residual, const TY* __restrict__ y, const float* __restrict__ post_weight,
                                                                   const float* __restrict__ next_weight, TO* __restrict__ out, const int* __restrict__ rows,
                                                                   float eps, int centred, int width, int groups) {
  extern __shared__ float norm_row[];
  __shared__ float scratch[32];
  __shared__ float means[kNormMaxGroups], invs[kNormMaxGroups];
  const int source = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  float* stream = residual + (size_t)source * width;
  const int part = width / groups;
  if (y != nullptr) {
    const TY* branch = y + (size_t)source * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) norm_row[i] = to_float(branch[i]);
    __syncthreads();
    group_statistics(norm_row, width, groups, centred, eps, scratch, means, invs);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {   // every thread rereads what it wrote itself
      const float v = stream[i] + ((norm_row[i] - means[i / part]) * invs[i / part]) * post_weight[i];
      stream[i] = v;
      norm_row[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) norm_row[i] = stream[i];
  }
  if (out == nullptr) return;
  __syncthreads();
  group_statistics(norm_row, width, groups, centred, eps, scratch, means, invs);
  TO* dst = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_float<TO>(((norm_row[i] - means[i / part]) * invs[i / part]) * next_weight[i]);
}

template <typename T>
__global__ void stream_with_embedding_kernel(const float* __restrict__ residual, const T* __restrict__ table, const int* __restrict__ ids, float scale,
                                             T* __restrict__ out, int width, int vocab, int* __restrict__ error_flag) {
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && error_flag != nullptr) atomicOr(error_flag, 2);
    id = 0;
  }
  const float* stream = residual + (size_t)row * width;
  const T* token = table + (size_t)id * width;
  T* dst = out + (size_t)row * 2 * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    dst[i] = from_float<T>(stream[i]);
    dst[width + i] = from_float<T>(to_float(token[i]) * scale);
  }
}

template <typename TY, typename TO>
static int launch_branch_norm(float* residual, const void* y, const float* post_weight, const float* next_weight, void* out, const int* rows, float eps,
                              int centred, int count, int width, int groups, cudaStream_t stream) {
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(branch_norm_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (width % 8 == 0 && (width / groups) % 8 == 0 && aligned(residual) && aligned(y) && aligned(post_weight) && aligned(next_weight) && aligned(out)) {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(branch_norm_wide_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    branch_norm_wide_kernel<TY, TO><<<count, kNormThreads, smem, stream>>>(residual, (const TY*)y, post_weight, next_weight, (TO*)out, rows, eps, centred, width, groups);
    return (int)cudaGetLastError();
  }
  branch_norm_kernel<TY, TO><<<count, kNormThreads, smem, stream>>>(residual, (const TY*)y, post_weight, next_weight, (TO*)out, rows, eps, centred, width, groups);
  return (int)cudaGetLastError();
}

}  // namespace tlie

using namespace tlie;

// ``count`` rows are worked on: all of the stream's, or with ``rows`` the listed ones (then y must be null: a gathered norm adds nothing).
// ``y`` and ``out`` are of ``dtype``; either may be null.
// ``groups``: the norms' statistics are taken over each of that many equal consecutive parts of a row (1: over the whole row).
TLIE_EXPORT int tlie_branch_norm(int dtype, float* residual, const void* y, const float* post_weight, const float* next_weight, void* out, const int* rows,
                                 float eps, int centred, int count, int width, int groups, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (groups < 1 || groups > kNormMaxGroups || width % groups != 0 || width <= 0 || (rows != nullptr && y != nullptr) || (y != nullptr && post_weight == nullptr) || (out != nullptr && next_weight == nullptr))
    return (int)cudaErrorInvalidValue;
  if (dtype == TLIE_F32) return launch_branch_norm<float, float>(residual, y, post_weight, next_weight, out, rows, eps, centred, count, width, groups, stream);
  return launch_branch_norm<__nv_bfloat16, __nv_bfloat16>(residual, y, post_weight, next_weight, out, rows, eps, centred, count, width, groups, stream);
}

TLIE_EXPORT int tlie_stream_with_embedding(int dtype, const float* residual, const void* table, const int* ids, float scale, void* out, int rows, int width,
                                           int vocab, int* error_flag, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == TLIE_F32)
    stream_with_embedding_kernel<float><<<rows, 256, 0, stream>>>(residual, (const float*)table, ids, scale, (float*)out, width, vocab, error_flag);
  else
    stream_with_embedding_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>(residual, (const __nv_bfloat16*)table, ids, scale, (__nv_bfloat16*)out, width, vocab, error_flag);
  return (int)cudaGetLastError();
}
