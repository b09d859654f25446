// Deterministic top-k per row: the first k indices of a stable descending sort (ties -> lower index).
// One CTA per row; the row is turned into 64-bit keys (descending-ordered score bits << 32 | index),
// bitonic-sorted in shared memory, and the first k indices are written out.  Bit-exact by construction:
// no floating-point arithmetic, no atomics.  Also holds the small cast kernel for the per-key outputs.
#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int kTopkThreads = 1024;
constexpr int kTopkMaxN = 16384;

__device__ __forceinline__ uint32_t descending_key(float f) {
  f += 0.f;  // -0 -> +0 so that equal values compare equal
  uint32_t u = __float_as_uint(f);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // monotone increasing in f
  return ~u;                                       // ascending sort of this = descending in f
}

__global__ void __launch_bounds__(kTopkThreads) topk_kernel(const float* __restrict__ scores, int32_t* __restrict__ idx,
                                                          int n, int n_pow2, int k) {
  extern __shared__ unsigned long long keys[];
  const float* row = scores + static_cast<int64_t>(blockIdx.x) * n;
  for (int i = threadIdx.x; i < n_pow2; i += kTopkThreads)
    keys[i] = (i < n) ? ((static_cast<unsigned long long>(descending_key(row[i])) << 32) | static_cast<uint32_t>(i))
                      : 0xFFFFFFFFFFFFFFFFull;
  __syncthreads();
  for (int size = 2; size <= n_pow2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < (n_pow2 >> 1); t += kTopkThreads) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool ascending = (lo & size) == 0;
        const unsigned long long a = keys[lo], b = keys[hi];
        if ((a > b) == ascending) {
          keys[lo] = b;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  int32_t* out = idx + static_cast<int64_t>(blockIdx.x) * k;
  for (int i = threadIdx.x; i < k; i += kTopkThreads) out[i] = static_cast<int32_t>(keys[i] & 0xFFFFFFFFull);
}

template <typename T>
__global__ void cast_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    dst[i] = static_cast<T>(src[i]);
}

// RoCo column variance from the two per-key sums: var_j = sum_p2_j / n_j - (sum_p_j / n_j)^2, n_j = the number of
// queries that can see key j (all S without a mask; S - max(0, j - past) with the causal one).  In place over sum_p2.
__global__ void roco_variance_kernel(const float* __restrict__ sum_p, float* __restrict__ sum_p2, int64_t total, int kv_len,
                                     int past, int S, int causal) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(i % kv_len);
    const int hidden = causal ? max(0, j - past) : 0;
    const float n = static_cast<float>(S - hidden);
    const float mean = sum_p[i] / n;
    sum_p2[i] = sum_p2[i] / n - mean * mean;
  }
}

}  // namespace

int launch_roco_variance(const float* sum_p, float* sum_p2, int64_t rows, int kv_len, int past, int S, int causal, cudaStream_t stream) {
  if (!sum_p || !sum_p2 || rows < 0 || kv_len <= 0 || S <= 0 || past < 0) return TB200_ERR_INVALID;
  if (rows == 0) return TB200_OK;
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  const int64_t total = rows * kv_len;
  int64_t blocks = (total + 255) / 256;
  if (blocks > st->num_sms * 16) blocks = st->num_sms * 16;
  roco_variance_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(sum_p, sum_p2, total, kv_len, past, S, causal);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

int launch_topk(const float* scores, int32_t* idx, int64_t rows, int n, int k, cudaStream_t stream) {
  if (scores == nullptr || idx == nullptr || rows < 0 || n <= 0 || k <= 0 || k > n) return TB200_ERR_INVALID;
  if (n > kTopkMaxN) return TB200_ERR_UNSUPPORTED;
  if (rows == 0) return TB200_OK;
  int n_pow2 = 2;
  while (n_pow2 < n) n_pow2 <<= 1;
  const size_t smem = static_cast<size_t>(n_pow2) * sizeof(unsigned long long);
  static bool attr_set[32] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 31]) {
    if (cudaFuncSetAttribute(topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTopkMaxN * 8) != cudaSuccess) return TB200_ERR_CUDA;
    attr_set[dev & 31] = true;
  }
  topk_kernel<<<static_cast<unsigned>(rows), kTopkThreads, smem, stream>>>(scores, idx, n, n_pow2, k);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

int launch_cast_f32(const float* src, void* dst, int64_t n, int dtype, cudaStream_t stream) {
  if (n == 0) return TB200_OK;
  if (!src || !dst) return TB200_ERR_INVALID;
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  int64_t blocks = (n + 255) / 256;
  if (blocks > st->num_sms * 16) blocks = st->num_sms * 16;
  if (dtype == TB200_BF16) cast_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(src, static_cast<__nv_bfloat16*>(dst), n);
  else if (dtype == TB200_F16) cast_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(src, static_cast<__half*>(dst), n);
  else return TB200_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

}  // namespace tb200

extern "C" int tb200_topk(const float* scores, int32_t* idx, int64_t rows, int n, int k, void* stream) {
  int status = TB200_OK;
  if (tb200::device_state(&status) == nullptr) return status;
  return tb200::launch_topk(scores, idx, rows, n, k, static_cast<cudaStream_t>(stream));
}
