// Per-key score reductions of KeyFormer / RoCo: a key-stationary second pass over the attention
// probabilities.  For key j of head (b,h):
//     sum_p[j]  = sum_i p[i,j]          sum_p2[j] = sum_i p[i,j]^2          (RoCo)
//     sum_pt[j] = sum_i softmax_j((scale*s + noise)/tau)[i,j]               (KeyFormer)
// with p[i,j] = exp2(scale_log2 * s[i,j] - lse2[i]) from the row statistics the forward pass left behind.
//
// One CTA per (128-key tile, q head, batch element).  The scores are recomputed TRANSPOSED on the tensor
// core, S^T = K_tile Q_i^T, so that a TMEM lane is a key and its columns are the queries: the sum over
// queries is then a thread-local loop -- no atomics, no cross-thread reduction, run-to-run identical.
//   warp 0     TMA: the K tile once, then the Q tiles that can see it (two-deep ring)
//   warp 1     MMA: S^T into two 128-column TMEM buffers
//   warps 2-5  reduction: thread = key; log-sum-exp of the 128 queries of the tile staged in shared memory
#include <math.h>
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int BK_ = 128;  // keys per CTA
constexpr int BQ_ = 128;  // queries per step
constexpr int kThreads = 192;
constexpr int kTmemCols = 256;
constexpr float kLog2e = 1.4426950408889634f;

template <int D, bool NOISE> struct ScoreSmem {
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kNoiseBytes = 128 * 128 * 2;              // [2 chunks of 64 keys][128 queries][128 B], swizzled
  static constexpr int kKOff = 0;
  static constexpr int kQOff = kTileBytes;
  static constexpr int kNoiseOff = kQOff + 2 * kTileBytes;       // two-deep ring (KeyFormer only)
  static constexpr int kLseOff = kNoiseOff + (NOISE ? 2 * kNoiseBytes : 0);  // [2 buffers][2 statistics][128] fp32
  static constexpr int kBarOff = kLseOff + 2 * 2 * 128 * 4;
  static constexpr int kTotal = kBarOff + 128 + 1024;
};

struct ScoreParams {
  CUtensorMap map_q;
  CUtensorMap map_k;
  CUtensorMap map_noise;  // dims {past+S, S, B*Hq}; valid when noise_tma
  int noise_tma;
  int B, S, Hq, Hkv, past, kv_len, causal;
  float scale_log2, inv_tau;
  const float* lse2;
  const float* lse2t;
  const void* noise;
  float* sum_p;
  float* sum_p2;
  float* sum_pt;
  int* err;
};

__device__ __forceinline__ void bar_sync_reducers() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <typename T, int D, bool NOISE>
__global__ void __launch_bounds__(kThreads, 2) score_kernel(const __grid_constant__ ScoreParams p) {
  using L = ScoreSmem<D, NOISE>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* k_full = bars + 0;
  uint64_t* q_full = bars + 1;   // [2]
  uint64_t* q_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;   // [2]
  uint64_t* s_empty = bars + 7;  // [2]
  uint64_t* n_full = bars + 9;   // [2] noise tiles
  uint64_t* n_empty = bars + 11; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* lse_s = reinterpret_cast<float*>(smem + L::kLseOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * BK_;
  const int hq = blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int q_tiles = (p.S + BQ_ - 1) / BQ_;
  // first query tile that can see key k0+127 ... any key of this tile: query i sees key j iff j <= past + i
  int first_tile = 0;
  if (p.causal && k0 > p.past) first_tile = (k0 - p.past) / BQ_;
  const int nt = q_tiles - first_tile;

  if (threadIdx.x == 0) {
    mbar_init(k_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
      mbar_init(&n_full[i], 1);
      mbar_init(&n_empty[i], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const AbortCtx ctx{p.err, abort_flag};

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(k_full, L::kTileBytes);
#pragma unroll
      for (int dc = 0; dc < D / 64; ++dc)
        tma_load_3d(smem + L::kKOff + dc * (128 * 128), &p.map_k, k_full, dc * 64, k0, b * p.Hkv + hkv);
    }
    __syncwarp();
    for (int i = 0; i < nt; ++i) {
      const int st = i & 1;
      if (NOISE && p.noise_tma) {
        if (!mbar_wait(&n_empty[st], ((i >> 1) & 1) ^ 1, ctx, 306)) break;
        if (lane == 0) {
          mbar_arrive_expect_tx(&n_full[st], L::kNoiseBytes);
#pragma unroll
          for (int kc = 0; kc < 2; ++kc)
            tma_load_3d(smem + L::kNoiseOff + st * L::kNoiseBytes + kc * (128 * 128), &p.map_noise, &n_full[st], k0 + kc * 64,
                        (first_tile + i) * BQ_, b * p.Hq + hq);
        }
        __syncwarp();
      }
      if (!mbar_wait(&q_empty[st], ((i >> 1) & 1) ^ 1, ctx, 301)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&q_full[st], L::kTileBytes);
#pragma unroll
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_3d(smem + L::kQOff + st * L::kTileBytes + dc * (128 * 128), &p.map_q, &q_full[st], dc * 64,
                      (first_tile + i) * BQ_, b * p.Hq + hq);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc(IsBf16<T>::value, false, false, BK_, BQ_);
    const uint32_t k_s = smem_u32(smem + L::kKOff);
    bool ok = mbar_wait(k_full, 0, ctx, 302);
    for (int i = 0; ok && i < nt; ++i) {
      const int st = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      if (!mbar_wait(&q_full[st], ph, ctx, 303)) break;
      if (!mbar_wait(&s_empty[st], ph ^ 1, ctx, 304)) break;
      tc_fence_after();
      {  // all lanes converged, operands warp-uniform, one elected lane issues
        const uint64_t kd = make_smem_desc(k_s, 16, 1024);
        const uint64_t qd = make_smem_desc(smem_u32(smem + L::kQOff + st * L::kTileBytes), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t off = static_cast<uint64_t>(((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4);
          umma_ss_warp(tmem_base + st * BQ_, kd + off, qd + off, idesc, kk > 0 ? 1u : 0u);
        }
        umma_commit_warp(&s_full[st]);
        umma_commit_warp(&q_empty[st]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int r_in = quad * 32 + lane;
    const int kj = k0 + r_in;
    const bool key_ok = kj < p.kv_len;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const long long head_row0 = (static_cast<long long>(b) * p.Hq + hq) * p.S;
    float acc_p = 0.f, acc_p2 = 0.f, acc_pt = 0.f;
    for (int i = 0; i < nt; ++i) {
      const int st = i & 1;
      const int q0 = (first_tile + i) * BQ_;
      // stage the row statistics of this query tile (thread r loads query q0+r)
      {
        const int qi = q0 + r_in;
        lse_s[(st * 2 + 0) * 128 + r_in] = (qi < p.S) ? p.lse2[head_row0 + qi] : INFINITY;  // +inf -> p = 0
        if (NOISE) lse_s[(st * 2 + 1) * 128 + r_in] = (qi < p.S) ? p.lse2t[head_row0 + qi] : INFINITY;
      }
      bar_sync_reducers();
      if (!mbar_wait(&s_full[st], (i >> 1) & 1, ctx, 305)) break;
      tc_fence_after();
      if (NOISE && p.noise_tma) {
        if (!mbar_wait(&n_full[st], (i >> 1) & 1, ctx, 307)) break;
      }
      // this key's column of the swizzled noise tile: element (query c, key r_in)
      const uint8_t* n_col = smem + L::kNoiseOff + st * L::kNoiseBytes + (r_in >> 6) * (128 * 128) + (r_in & 7) * 2;
      const int n_unit = (r_in & 63) >> 3;
      const float nscale = kLog2e * p.inv_tau;
      const float* lse_q = lse_s + (st * 2 + 0) * 128;
      const float* lse_t = lse_s + (st * 2 + 1) * 128;
      // a query column c is visible to this key iff kj <= past + q0 + c
      const int c_min = p.causal ? max(0, kj - p.past - q0) : 0;
#pragma unroll 1
      for (int cc = 0; cc < BQ_ / 32; ++cc) {
        uint32_t s[32];
        tmem_ld_x32(tmem_base + st * BQ_ + lane_sel + cc * 32, s);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int c = cc * 32 + e;
          const bool vis = key_ok && (c >= c_min);
          const float t = __uint_as_float(s[e]) * p.scale_log2;
          if (!NOISE) {  // RoCo: sums of p and p^2
            const float pr = vis ? fast_exp2(t - lse_q[c]) : 0.f;
            acc_p += pr;
            acc_p2 = fmaf(pr, pr, acc_p2);
          } else {       // KeyFormer: only the perturbed probability is summed
            float nz = 0.f;
            if (p.noise_tma)
              nz = static_cast<float>(*reinterpret_cast<const T*>(n_col + c * 128 + ((n_unit ^ (c & 7)) << 4)));
            else if (vis && (q0 + c) < p.S)
              nz = static_cast<float>(static_cast<const T*>(p.noise)[(head_row0 + q0 + c) * p.kv_len + kj]);
            const float pt = vis ? fast_exp2(fmaf(nz, nscale, fmaf(t, p.inv_tau, -lse_t[c]))) : 0.f;
            acc_pt += pt;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&s_empty[st]);
      if (NOISE && p.noise_tma) mbar_arrive(&n_empty[st]);
    }
    if (key_ok) {
      const long long o = (static_cast<long long>(b) * p.Hq + hq) * p.kv_len + kj;
      if (p.sum_p) p.sum_p[o] = acc_p;
      if (p.sum_p2) p.sum_p2[o] = acc_p2;
      if (NOISE && p.sum_pt) p.sum_pt[o] = acc_pt;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, int D, bool NOISE>
int launch_one(const ScoreParams& p, dim3 grid, cudaStream_t stream) {
  static bool attr_set[32] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 31]) {
    if (cudaFuncSetAttribute(score_kernel<T, D, NOISE>, cudaFuncAttributeMaxDynamicSharedMemorySize, ScoreSmem<D, NOISE>::kTotal) != cudaSuccess)
      return TB200_ERR_CUDA;
    attr_set[dev & 31] = true;
  }
  score_kernel<T, D, NOISE><<<grid, kThreads, ScoreSmem<D, NOISE>::kTotal, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

template <typename T>
int launch_t(const ScoreParams& p, int D, bool noise, dim3 grid, cudaStream_t stream) {
  if (D == 128) return noise ? launch_one<T, 128, true>(p, grid, stream) : launch_one<T, 128, false>(p, grid, stream);
  if (D == 64) return noise ? launch_one<T, 64, true>(p, grid, stream) : launch_one<T, 64, false>(p, grid, stream);
  return TB200_ERR_UNSUPPORTED;
}

}  // namespace

int launch_score_colreduce(const ScoreLaunch& a, cudaStream_t stream) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  if (a.dtype != TB200_BF16 && a.dtype != TB200_F16) return TB200_ERR_UNSUPPORTED;
  if (a.B <= 0 || a.S <= 0 || a.Hq <= 0 || a.Hkv <= 0 || a.Hq % a.Hkv != 0 || a.past < 0 || a.cache_len < a.past + a.S)
    return TB200_ERR_INVALID;
  if (a.D != 64 && a.D != 128) return TB200_ERR_UNSUPPORTED;
  if (!a.q || !a.k_cache || !a.lse2) return TB200_ERR_INVALID;
  const bool noise = a.noise != nullptr;
  if (noise && (!a.lse2_perturbed || !a.sum_pt)) return TB200_ERR_INVALID;
  if (a.Hq > 65535 || a.B > 65535) return TB200_ERR_INVALID;

  ScoreParams p;
  memset(&p, 0, sizeof(p));
  p.B = a.B; p.S = a.S; p.Hq = a.Hq; p.Hkv = a.Hkv; p.past = a.past; p.kv_len = a.past + a.S; p.causal = a.causal;
  p.scale_log2 = a.sm_scale * kLog2e;
  p.inv_tau = 1.f / a.tau;
  p.lse2 = a.lse2;
  p.lse2t = a.lse2_perturbed;
  p.noise = a.noise;
  p.sum_p = a.sum_p;
  p.sum_p2 = a.sum_p2;
  p.sum_pt = a.sum_pt;
  p.err = st->err_word;
  const uint64_t D = static_cast<uint64_t>(a.D);
  {
    const uint64_t dims[3] = {D, static_cast<uint64_t>(a.S), static_cast<uint64_t>(a.B) * a.Hq};
    const uint64_t strides[2] = {D * 2, static_cast<uint64_t>(a.S) * D * 2};
    const uint32_t box[3] = {64, 128, 1};
    if ((status = make_tensor_map(&p.map_q, a.q, 3, dims, strides, box)) != TB200_OK) return status;
  }
  {
    const uint64_t dims[3] = {D, static_cast<uint64_t>(p.kv_len), static_cast<uint64_t>(a.B) * a.Hkv};
    const uint64_t strides[2] = {D * 2, static_cast<uint64_t>(a.cache_len) * D * 2};
    const uint32_t box[3] = {64, 128, 1};
    if ((status = make_tensor_map(&p.map_k, a.k_cache, 3, dims, strides, box)) != TB200_OK) return status;
  }
  if (noise && (p.kv_len & 7) == 0) {  // rows of the noise tensor are 16-byte aligned: tiles by TMA
    const uint64_t dims[3] = {static_cast<uint64_t>(p.kv_len), static_cast<uint64_t>(a.S), static_cast<uint64_t>(a.B) * a.Hq};
    const uint64_t strides[2] = {static_cast<uint64_t>(p.kv_len) * 2, static_cast<uint64_t>(a.S) * p.kv_len * 2};
    const uint32_t box[3] = {64, 128, 1};
    if ((status = make_tensor_map(&p.map_noise, a.noise, 3, dims, strides, box)) != TB200_OK) return status;
    p.noise_tma = 1;
  }
  const dim3 grid((p.kv_len + BK_ - 1) / BK_, a.Hq, a.B);
  if (a.dtype == TB200_BF16) return launch_t<__nv_bfloat16>(p, a.D, noise, grid, stream);
  return launch_t<__half>(p, a.D, noise, grid, stream);
}

}  // namespace tb200
