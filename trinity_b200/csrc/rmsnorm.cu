// RMSNorm / row statistics: the bandwidth-bound kernel class.
// One CTA per row; 128-bit coalesced loads, the row is kept in registers between the
// sum-of-squares pass and the scale pass (one HBM read, one HBM write per element),
// warp-shuffle + one shared-memory hop for the reduction, fp32 accumulation.
#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int kThreads = 256;
constexpr int kCachedVecs = 4;  // 16-byte vectors a thread keeps in registers: rows up to 256*4*8 = 8192 elements

template <typename T>
__global__ void __launch_bounds__(kThreads) rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ weight,
                                                         T* __restrict__ y, float* __restrict__ inv_rms, int cols,
                                                         float eps, float divisor) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int nvec = cols >> 3;  // 8 elements per 16-byte vector
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
  uint4 cache[kCachedVecs];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kCachedVecs; ++i) {
    const int v = threadIdx.x + i * kThreads;
    if (v < nvec) {
      cache[i] = __ldg(xr + v);
      const uint32_t w[4] = {cache[i].x, cache[i].y, cache[i].z, cache[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Pack2<T>::unpack(w[j]);
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
    }
  }
  for (int v = threadIdx.x + kCachedVecs * kThreads; v < nvec; v += kThreads) {  // rows wider than the register cache
    const uint4 u = __ldg(xr + v);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = Pack2<T>::unpack(w[j]);
      ss = fmaf(f.x, f.x, ss);
      ss = fmaf(f.y, f.y, ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  __shared__ float warp_sums[kThreads / 32];
  if (lane_id() == 0) warp_sums[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) total += warp_sums[i];  // same order in every thread: deterministic
  const float r = rsqrtf(total / divisor + eps);
  if (inv_rms != nullptr && threadIdx.x == 0) inv_rms[row] = r;
  if (y == nullptr) return;

  uint4* yr = reinterpret_cast<uint4*>(y + row * cols);
  const uint4* wr = reinterpret_cast<const uint4*>(weight);
  auto scale_store = [&](int v, const uint4& u) {
    const uint32_t in[4] = {u.x, u.y, u.z, u.w};
    uint32_t out[4];
    uint4 g = make_uint4(0, 0, 0, 0);
    if (wr != nullptr) g = __ldg(wr + v);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = Pack2<T>::unpack(in[j]);
      f.x *= r;
      f.y *= r;
      if (wr != nullptr) {
        const float2 gf = Pack2<T>::unpack(gw[j]);
        f.x *= gf.x;
        f.y *= gf.y;
      }
      out[j] = Pack2<T>::pack(f.x, f.y);
    }
    yr[v] = make_uint4(out[0], out[1], out[2], out[3]);
  };
#pragma unroll
  for (int i = 0; i < kCachedVecs; ++i) {
    const int v = threadIdx.x + i * kThreads;
    if (v < nvec) scale_store(v, cache[i]);
  }
  for (int v = threadIdx.x + kCachedVecs * kThreads; v < nvec; v += kThreads) scale_store(v, __ldg(xr + v));
}

// Row statistic only (inv_rms[r] = rsqrt(mean(x[r,:]^2) + eps)): the norm-as-epilogue path reads x once and writes four
// bytes per row.  One WARP per row, warps walking the rows with a grid-wide stride; a lane keeps eight 16-byte loads in
// flight, so a few resident warps per SM cover the HBM latency -- a CTA per row (the kernel above) spends most of an
// 8 KiB row's time starting and ending CTAs.  The lane-order reduction is fixed: bit-identical run to run.
template <typename T>
__global__ void __launch_bounds__(256) row_stats_kernel(const T* __restrict__ x, float* __restrict__ inv_rms, int64_t rows, int cols,
                                                         float eps, float divisor) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int nvec = cols >> 3;
  for (int64_t row = warp0; row < rows; row += nwarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
    float ss = 0.f;
    for (int v0 = lane; v0 < nvec; v0 += 32 * 8) {
      uint4 u[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int v = v0 + 32 * i;
        u[i] = v < nvec ? __ldg(xr + v) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t w[4] = {u[i].x, u[i].y, u[i].z, u[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Pack2<T>::unpack(w[j]);
          ss = fmaf(f.x, f.x, ss);
          ss = fmaf(f.y, f.y, ss);
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) inv_rms[row] = rsqrtf(ss / divisor + eps);
  }
}

// out[k, :] = w[k, :] * g[k]: the norm weight folded into the rows of a (K, N) projection weight, so that
// (x * r * g) @ W = r * (x @ (diag(g) W)) and the weighted norm costs the projection nothing but its row scale.
template <typename T>
__global__ void fold_rows_kernel(const T* __restrict__ w, const T* __restrict__ g, T* __restrict__ out, int64_t k, int64_t nvec) {
  const int64_t total = k * nvec;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / nvec;
    const float gr = static_cast<float>(g[row]);
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(w) + i);
    const uint32_t in[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = Pack2<T>::unpack(in[j]);
      o[j] = Pack2<T>::pack(f.x * gr, f.y * gr);
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace

int launch_fold_rows(const void* w, const void* g, void* out, int64_t k, int64_t n, int dtype, cudaStream_t stream) {
  if (!w || !g || !out || k <= 0 || n <= 0 || (n & 7) != 0 || k > (1 << 30) || n > (1 << 30)) return TB200_ERR_INVALID;
  if (!aligned16(w) || !aligned16(out) || (reinterpret_cast<uintptr_t>(g) & 1) != 0) return TB200_ERR_INVALID;
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  const int64_t nvec = n / 8;
  int64_t blocks = (k * nvec + 255) / 256;
  if (blocks > st->num_sms * 16) blocks = st->num_sms * 16;
  if (dtype == TB200_BF16)
    fold_rows_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(g),
                                                                                    static_cast<__nv_bfloat16*>(out), k, nvec);
  else if (dtype == TB200_F16)
    fold_rows_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const __half*>(w), static_cast<const __half*>(g),
                                                                             static_cast<__half*>(out), k, nvec);
  else
    return TB200_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

int launch_rmsnorm(const void* x, const void* weight, void* y, float* inv_rms, int64_t rows, int64_t cols, float eps,
                   int dtype, cudaStream_t stream, int mean_divisor) {
  if (x == nullptr || (y == nullptr && inv_rms == nullptr)) return TB200_ERR_INVALID;
  if (rows < 0 || cols <= 0 || (cols & 7) != 0 || rows > 0x7fffffffLL || cols > (1 << 24)) return TB200_ERR_INVALID;
  if (!aligned16(x) || !aligned16(y) || !aligned16(weight)) return TB200_ERR_INVALID;
  if (rows == 0) return TB200_OK;
  const dim3 grid(static_cast<unsigned>(rows));
  const float divisor = static_cast<float>(mean_divisor > 0 ? mean_divisor : cols);
  if (y == nullptr && rows >= 64) {  // statistic only, enough rows to fill the machine with warps
    int status = TB200_OK;
    DeviceState* st = device_state(&status);
    if (!st) return status;
    int64_t blocks = (rows + 7) / 8;
    if (blocks > st->num_sms * 8) blocks = st->num_sms * 8;
    const dim3 sgrid(static_cast<unsigned>(blocks), 1, 1), sblock(256, 1, 1);
    cudaError_t e;
    if (dtype == TB200_BF16)
      e = launch_chained(row_stats_kernel<__nv_bfloat16>, sgrid, sblock, 0, stream, static_cast<const __nv_bfloat16*>(x), inv_rms, rows,
                         static_cast<int>(cols), eps, divisor);
    else if (dtype == TB200_F16)
      e = launch_chained(row_stats_kernel<__half>, sgrid, sblock, 0, stream, static_cast<const __half*>(x), inv_rms, rows,
                         static_cast<int>(cols), eps, divisor);
    else
      return TB200_ERR_UNSUPPORTED;
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
  }
  const dim3 block(kThreads, 1, 1);
  cudaError_t e;
  if (dtype == TB200_BF16) {
    e = launch_chained(rmsnorm_kernel<__nv_bfloat16>, grid, block, 0, stream, static_cast<const __nv_bfloat16*>(x),
                       static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(y), inv_rms, static_cast<int>(cols), eps, divisor);
  } else if (dtype == TB200_F16) {
    e = launch_chained(rmsnorm_kernel<__half>, grid, block, 0, stream, static_cast<const __half*>(x), static_cast<const __half*>(weight),
                       static_cast<__half*>(y), inv_rms, static_cast<int>(cols), eps, divisor);
  } else {
    return TB200_ERR_UNSUPPORTED;
  }
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

}  // namespace tb200

extern "C" int tb200_fold_norm_weight(const void* w, const void* norm_weight, void* w_out, int64_t k, int64_t n, int dtype, void* stream) {
  return tb200::launch_fold_rows(w, norm_weight, w_out, k, n, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int tb200_rmsnorm(const void* x, const void* weight, void* y, float* inv_rms, int64_t rows, int64_t cols,
                             float eps, int dtype, void* stream) {
  int status = TB200_OK;
  if (tb200::device_state(&status) == nullptr) return status;
  return tb200::launch_rmsnorm(x, weight, y, inv_rms, rows, cols, eps, dtype, static_cast<cudaStream_t>(stream));
}
