// Attention forward on tcgen05: O2 = softmax(scale * Q K^T [causal]) V with GQA/MQA, online softmax,
// and the per-row log-sum-exp the score kernels need afterwards.
//
// One CTA per (128-query tile, q head, batch element), 192 threads:
//   warp 0     TMA producer: Q tile once, then K and V tiles of 128 keys through two-deep rings
//   warp 1     MMA issuer:   S_j = Q K_j^T (128x128, fp32 in TMEM, two S buffers) and O += P_j V_j
//   warps 2-5  softmax:      thread = query row; S row from TMEM to registers, running max in the log2
//                            domain (the reference exponent is only moved when the row max grows by
//                            more than 2^8, so O in TMEM is rarely rescaled), P_j written to shared
//                            memory in the UMMA K-major 128B-swizzle layout, O rescaled in TMEM when needed
// S_{j+1} is issued before P_j V_j so the tensor core works while the softmax warps are busy.
// Q is (B,Hq,S,D); K/V are the caches (B,Hkv,cache_len,D) seen through a tensor map whose row extent is
// past+S, so rows beyond the valid length read as zeros; O2 is (B,S,Hq*D) (heads merged).
//
// KeyFormer (NOISE): the same pass also keeps the online log-sum-exp of (scale*s + noise)/tau per row.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int BQ = 128;   // queries per CTA
constexpr int BKV = 128;  // keys per step
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;  // log2 units

// With a noise tensor (KeyFormer) the K and V rings shrink to one stage each -- that pass is bound by its two
// exponentials per score, not by the loads -- and the room goes to a two-deep ring of noise tiles.
template <int D, bool NOISE> struct AttnSmem {
  static constexpr int kKVStages = NOISE ? 1 : 2;
  static constexpr int kQBytes = BQ * D * 2;
  static constexpr int kKVBytes = BKV * D * 2;
  static constexpr int kPBytes = BQ * BKV * 2;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQBytes;
  static constexpr int kVOff = kKOff + kKVStages * kKVBytes;
  static constexpr int kPOff = kVOff + kKVStages * kKVBytes;
  static constexpr int kNoiseOff = kPOff + kPBytes;             // [2][2 chunks of 64 keys][128 rows][128 B], swizzled
  static constexpr int kBarOff = kNoiseOff + (NOISE ? 2 * kPBytes : 0);
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

struct AttnParams {
  CUtensorMap map_q;  // dims {D, S, B*Hq}
  CUtensorMap map_k;  // dims {D, past+S, B*Hkv}, pitch cache_len*D
  CUtensorMap map_v;
  CUtensorMap map_noise;  // dims {past+S, S, B*Hq}; valid when noise_tma
  int noise_tma;          // the noise rows are 16-byte aligned: tiles come through TMA, else plain loads
  int B, S, Hq, Hkv, past, kv_len, causal;
  float scale_log2;   // sm_scale * log2(e)
  float inv_tau;
  void* o2;
  float* lse2;
  const void* noise;
  float* lse2_perturbed;
  int* err;
  long long wait_limit;  // cycles a bounded wait may last (tb200_set_wait_limit_cycles)
};

template <typename T, int D, bool NOISE>
__global__ void __launch_bounds__(kThreads, 1) attn_fwd_kernel(const __grid_constant__ AttnParams p) {
  using L = AttnSmem<D, NOISE>;
  constexpr int KVS = L::kKVStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* k_empty = bars + 3;  // [2]
  uint64_t* v_full = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;   // [2]
  uint64_t* s_empty = bars + 11; // [2]
  uint64_t* p_ready = bars + 13;
  uint64_t* pv_done = bars + 14;
  uint64_t* n_full = bars + 15;   // [2] noise tiles
  uint64_t* n_empty = bars + 17;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_tiles = (p.S + BQ - 1) / BQ;
  const int q_tile = q_tiles - 1 - blockIdx.x;  // longest (latest) tiles first
  const int q0 = q_tile * BQ;
  const int hq = blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = hq / (p.Hq / p.Hkv);
  // keys this tile can see
  int last_key = p.kv_len - 1;
  if (p.causal) last_key = min(last_key, p.past + min(q0 + BQ - 1, p.S - 1));
  const int nt = last_key / BKV + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
      mbar_init(&n_full[i], 1);
      mbar_init(&n_empty[i], 128);
    }
    mbar_init(p_ready, 128);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&p.map_q);
    tma_prefetch_desc(&p.map_k);
    tma_prefetch_desc(&p.map_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 2 * BKV;
  const AbortCtx ctx{p.err, abort_flag, p.wait_limit};

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, L::kQBytes);
#pragma unroll
      for (int dc = 0; dc < D / 64; ++dc)
        tma_load_3d(smem + L::kQOff + dc * (BQ * 128), &p.map_q, q_full, dc * 64, q0, b * p.Hq + hq);
    }
    __syncwarp();
    for (int j = 0; j < nt; ++j) {
      const int st = j % KVS;
      const uint32_t ph = (j / KVS) & 1;
      if (NOISE && p.noise_tma) {
        if (!mbar_wait(&n_empty[j & 1], ((j >> 1) & 1) ^ 1, ctx, 212)) break;
        if (lane == 0) {
          mbar_arrive_expect_tx(&n_full[j & 1], L::kPBytes);
#pragma unroll
          for (int kc = 0; kc < 2; ++kc)
            tma_load_3d(smem + L::kNoiseOff + (j & 1) * L::kPBytes + kc * (BQ * 128), &p.map_noise, &n_full[j & 1], j * BKV + kc * 64, q0,
                        b * p.Hq + hq);
        }
        __syncwarp();
      }
      if (!mbar_wait(&k_empty[st], ph ^ 1, ctx, 201)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&k_full[st], L::kKVBytes);
#pragma unroll
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_3d(smem + L::kKOff + st * L::kKVBytes + dc * (BKV * 128), &p.map_k, &k_full[st], dc * 64, j * BKV, b * p.Hkv + hkv);
      }
      __syncwarp();
      if (!mbar_wait(&v_empty[st], ph ^ 1, ctx, 202)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&v_full[st], L::kKVBytes);
#pragma unroll
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_3d(smem + L::kVOff + st * L::kKVBytes + dc * (BKV * 128), &p.map_v, &v_full[st], dc * 64, j * BKV, b * p.Hkv + hkv);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_s = make_idesc(IsBf16<T>::value, false, false, BQ, BKV);
    constexpr uint32_t idesc_o = make_idesc(IsBf16<T>::value, false, true, BQ, D);
    // All lanes run converged with warp-uniform operands; one elected lane issues (see common.cuh).
    const uint64_t qd = make_smem_desc(smem_u32(smem + L::kQOff), 16, 1024);
    const uint64_t pd = make_smem_desc(smem_u32(smem + L::kPOff), 16, 1024);
    auto issue_s = [&](int j) {  // S_j = Q K_j^T into S buffer j&1
      const uint64_t kd = make_smem_desc(smem_u32(smem + L::kKOff + (j % KVS) * L::kKVBytes), 16, 1024);
      const uint32_t d_tmem = tmem_base + (j & 1) * BKV;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint64_t off = static_cast<uint64_t>(((kk >> 2) * (BQ * 128) + (kk & 3) * 32) >> 4);
        umma_ss_warp(d_tmem, qd + off, kd + off, idesc_s, kk > 0 ? 1u : 0u);
      }
      umma_commit_warp(&s_full[j & 1]);
      umma_commit_warp(&k_empty[j % KVS]);
    };
    bool ok = mbar_wait(q_full, 0, ctx, 203) && mbar_wait(&k_full[0], 0, ctx, 204);
    if (ok) {
      tc_fence_after();
      issue_s(0);
    }
    for (int j = 0; ok && j < nt; ++j) {
      if (j + 1 < nt) {
        const int n1 = (j + 1) >> 1;
        if (!mbar_wait(&k_full[(j + 1) % KVS], ((j + 1) / KVS) & 1, ctx, 205)) break;
        if (!mbar_wait(&s_empty[(j + 1) & 1], (n1 & 1) ^ 1, ctx, 206)) break;
        tc_fence_after();
        issue_s(j + 1);
      }
      if (!mbar_wait(p_ready, j & 1, ctx, 207)) break;
      if (!mbar_wait(&v_full[j % KVS], (j / KVS) & 1, ctx, 208)) break;
      tc_fence_after();
      const uint64_t vd = make_smem_desc(smem_u32(smem + L::kVOff + (j % KVS) * L::kKVBytes), BKV * 128, 1024);  // MN-major
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk) {  // 16 keys per step: +32 B in P (K-major), +2048 B in V
        const uint64_t poff = static_cast<uint64_t>(((kk >> 2) * (BQ * 128) + (kk & 3) * 32) >> 4);
        umma_ss_warp(tmem_o, pd + poff, vd + static_cast<uint64_t>(kk * 128), idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
      }
      umma_commit_warp(&v_empty[j % KVS]);
      umma_commit_warp(pv_done);
    }
  } else {
    // ------------------------------------------------------------ softmax + output (warps 2..5)
    const int quad = warp & 3;
    const int r_in = quad * 32 + lane;
    const int qi = q0 + r_in;
    const bool row_ok = qi < p.S;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const int key_limit = p.causal ? min(p.past + qi, p.kv_len - 1) : p.kv_len - 1;  // last visible key of this row
    float m_use = -INFINITY, l = 0.f;
    float mt = -INFINITY, lt = 0.f;  // KeyFormer statistic
    const T* noise_row = nullptr;
    if (NOISE && row_ok)
      noise_row = static_cast<const T*>(p.noise) + ((static_cast<long long>(b) * p.Hq + hq) * p.S + qi) * p.kv_len;
    uint8_t* p_smem = smem + L::kPOff;
    bool ok = true;

    for (int j = 0; j < nt; ++j) {
      const int k0 = j * BKV;
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, ctx, 209)) { ok = false; break; }
      tc_fence_after();
      uint32_t s[BKV];
      {
        const uint32_t ts = tmem_base + (j & 1) * BKV + lane_sel;
        tmem_ld_x32(ts + 0, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_ld_x32(ts + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
        tmem_ld_x32(ts + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
        tmem_ld_x32(ts + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
        tmem_wait_ld();
      }
      tc_fence_before();
      mbar_arrive(&s_empty[j & 1]);  // the S buffer may be overwritten

      const bool need_mask = (k0 + BKV - 1 > key_limit);
      float rowmax = -INFINITY;
#pragma unroll
      for (int i = 0; i < BKV; ++i) {
        float t = __uint_as_float(s[i]) * p.scale_log2;
        if (need_mask && (k0 + i > key_limit)) t = -INFINITY;
        s[i] = __float_as_uint(t);
        rowmax = fmaxf(rowmax, t);
      }
      if (NOISE) {  // log-sum-exp of x = (scale*s + noise)/tau in the log2 domain, one sweep over the noise row:
        // the exponent reference mt only has to keep exp2(x - mt) inside fp32 range, so it is moved after the sweep
        // and only when the row's maximum ran more than 2^60 ahead of it; it starts at the noise-free row maximum.
        const uint8_t* n_smem = smem + L::kNoiseOff + (j & 1) * L::kPBytes;
        if (p.noise_tma) {
          if (!mbar_wait(&n_full[j & 1], (j >> 1) & 1, ctx, 213)) { ok = false; break; }
        }
        if (mt == -INFINITY && rowmax > -INFINITY) mt = rowmax * p.inv_tau;
        const float nscale = kLog2e * p.inv_tau;
        const float neg_ref = (mt == -INFINITY) ? 0.f : -mt;
        float tmax = -INFINITY, acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int u = 0; u < BKV / 8; ++u) {
          float nz[8];
          const int kbase = k0 + u * 8;
          if (p.noise_tma) {  // row r_in of the swizzled tile: 16-byte unit u lands at (u & 7) ^ (row & 7) of its 64-key chunk
            const uint4 q4 = *reinterpret_cast<const uint4*>(n_smem + (u >> 3) * (BQ * 128) + r_in * 128 + (((u & 7) ^ (r_in & 7)) << 4));
            const uint32_t w[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f2 = Pack2<T>::unpack(w[e]);
              nz[2 * e] = f2.x;
              nz[2 * e + 1] = f2.y;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)
              nz[e] = (row_ok && kbase + e < p.kv_len) ? static_cast<float>(noise_row[kbase + e]) : 0.f;
          }
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            const float x0 = fmaf(nz[e], nscale, fmaf(__uint_as_float(s[u * 8 + e]), p.inv_tau, neg_ref));  // -inf stays -inf
            const float x1 = fmaf(nz[e + 1], nscale, fmaf(__uint_as_float(s[u * 8 + e + 1]), p.inv_tau, neg_ref));
            tmax = max3(tmax, x0, x1);
            acc0 += fast_exp2(x0);
            acc1 += fast_exp2(x1);
          }
        }
        lt += acc0 + acc1;
        if (tmax > 60.f) {  // move the reference up to this row maximum
          lt *= fast_exp2(-tmax);
          mt += tmax;
        }
        if (p.noise_tma) mbar_arrive(&n_empty[j & 1]);
      }

      const float m_new = fmaxf(m_use, rowmax);
      const bool grow = m_new > m_use + kRescaleThreshold;  // also true on the first tile (m_use = -inf)
      float alpha = 1.f;
      if (grow) {
        alpha = fast_exp2(m_use - m_new);  // 0 on the first tile
        m_use = m_new;
      }
      const float mref = (m_use == -INFINITY) ? 0.f : m_use;
      float rowsum = 0.f;
      uint32_t pk[BKV / 2];
#pragma unroll
      for (int i = 0; i < BKV; i += 2) {
        const float p0 = fast_exp2(__uint_as_float(s[i]) - mref);
        const float p1 = fast_exp2(__uint_as_float(s[i + 1]) - mref);
        rowsum += p0 + p1;
        pk[i >> 1] = Pack2<T>::pack(p0, p1);
      }
      l = l * alpha + rowsum;

      // P_{j-1} V_{j-1} must have finished before P is overwritten or O is rescaled
      if (j > 0) {
        if (!mbar_wait(pv_done, (j - 1) & 1, ctx, 210)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow)) {
          uint32_t o[32];
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            tmem_ld_x32(tmem_o + lane_sel + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_x32(tmem_o + lane_sel + c * 32, o);
          }
          tmem_wait_st();
        }
      }
      // P row into shared memory: K-major, 128-byte swizzle (16-byte unit u of a row lands at u ^ (row & 7))
#pragma unroll
      for (int u = 0; u < BKV / 8; ++u) {
        uint8_t* dst = p_smem + (u >> 3) * (BQ * 128) + r_in * 128 + (((u & 7) ^ (r_in & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
    }

    if (ok && mbar_wait(pv_done, (nt - 1) & 1, ctx, 211)) {
      tc_fence_after();
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      T* orow = static_cast<T*>(p.o2) + ((static_cast<long long>(b) * p.S + qi) * p.Hq + hq) * D;
      uint32_t o[32];
      float v[32];
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        tmem_ld_x32(tmem_o + lane_sel + c * 32, o);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o[i]) * inv_l;
          uint4* d = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            d[i] = make_uint4(Pack2<T>::pack(v[8 * i], v[8 * i + 1]), Pack2<T>::pack(v[8 * i + 2], v[8 * i + 3]),
                              Pack2<T>::pack(v[8 * i + 4], v[8 * i + 5]), Pack2<T>::pack(v[8 * i + 6], v[8 * i + 7]));
        }
      }
      if (row_ok) {
        const long long ridx = (static_cast<long long>(b) * p.Hq + hq) * p.S + qi;
        if (p.lse2 != nullptr) p.lse2[ridx] = m_use + log2f(l);
        if (NOISE && p.lse2_perturbed != nullptr) p.lse2_perturbed[ridx] = mt + log2f(lt);
      }
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
int launch_one(const AttnParams& p, dim3 grid, cudaStream_t stream) {
  static bool attr_set[32] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 31]) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<T, D, NOISE>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<D, NOISE>::kTotal) != cudaSuccess)
      return TB200_ERR_CUDA;
    attr_set[dev & 31] = true;
  }
  attn_fwd_kernel<T, D, NOISE><<<grid, kThreads, AttnSmem<D, NOISE>::kTotal, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

template <typename T>
int launch_t(const AttnParams& p, int D, bool noise, dim3 grid, cudaStream_t stream) {
  if (D == 128) return noise ? launch_one<T, 128, true>(p, grid, stream) : launch_one<T, 128, false>(p, grid, stream);
  if (D == 64) return noise ? launch_one<T, 64, true>(p, grid, stream) : launch_one<T, 64, false>(p, grid, stream);
  return TB200_ERR_UNSUPPORTED;
}

}  // namespace

int launch_attn_fwd(const AttnLaunch& a, cudaStream_t stream) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  if (a.dtype != TB200_BF16 && a.dtype != TB200_F16) return TB200_ERR_UNSUPPORTED;
  if (a.B <= 0 || a.S <= 0 || a.Hq <= 0 || a.Hkv <= 0 || a.Hq % a.Hkv != 0 || a.past < 0 || a.cache_len < a.past + a.S)
    return TB200_ERR_INVALID;
  if (a.D != 64 && a.D != 128) return TB200_ERR_UNSUPPORTED;
  if (!a.q || !a.k_cache || !a.v_cache || !a.o2) return TB200_ERR_INVALID;
  if (!aligned16(a.q) || !aligned16(a.k_cache) || !aligned16(a.v_cache) || !aligned16(a.o2) || !aligned16(a.noise)) return TB200_ERR_INVALID;
  if (a.Hq > 65535 || a.B > 65535) return TB200_ERR_INVALID;
  if (!(a.sm_scale > 0.f)) return TB200_ERR_INVALID;  // the row maximum is taken before scaling
  // the two-tile persistent kernels, except for a noise tensor whose rows are not 16-byte aligned (no TMA tiles)
  if (a.noise == nullptr) return launch_attn_fwd_pingpong(a, stream);
  if (((a.past + a.S) & 7) == 0) return launch_attn_fwd_keyformer(a, stream);

  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.B = a.B; p.S = a.S; p.Hq = a.Hq; p.Hkv = a.Hkv; p.past = a.past; p.kv_len = a.past + a.S; p.causal = a.causal;
  p.scale_log2 = a.sm_scale * kLog2e;
  p.inv_tau = 1.f / a.tau;
  p.o2 = a.o2;
  p.lse2 = a.lse2;
  p.noise = a.noise;
  p.lse2_perturbed = a.lse2_perturbed;
  p.err = st->err_word;
  p.wait_limit = wait_limit_cycles();
  const uint64_t D = static_cast<uint64_t>(a.D);
  {
    const uint64_t dims[3] = {D, static_cast<uint64_t>(a.S), static_cast<uint64_t>(a.B) * a.Hq};
    const uint64_t strides[2] = {D * 2, static_cast<uint64_t>(a.S) * D * 2};
    const uint32_t box[3] = {64, BQ, 1};
    if ((status = make_tensor_map(&p.map_q, a.q, 3, dims, strides, box)) != TB200_OK) return status;
  }
  {
    const uint64_t dims[3] = {D, static_cast<uint64_t>(p.kv_len), static_cast<uint64_t>(a.B) * a.Hkv};
    const uint64_t strides[2] = {D * 2, static_cast<uint64_t>(a.cache_len) * D * 2};
    const uint32_t box[3] = {64, BKV, 1};
    if ((status = make_tensor_map(&p.map_k, a.k_cache, 3, dims, strides, box)) != TB200_OK) return status;
    if ((status = make_tensor_map(&p.map_v, a.v_cache, 3, dims, strides, box)) != TB200_OK) return status;
  }
  if (a.noise != nullptr && (p.kv_len & 7) == 0) {  // rows of the noise tensor are 16-byte aligned: tiles by TMA
    const uint64_t dims[3] = {static_cast<uint64_t>(p.kv_len), static_cast<uint64_t>(a.S), static_cast<uint64_t>(a.B) * a.Hq};
    const uint64_t strides[2] = {static_cast<uint64_t>(p.kv_len) * 2, static_cast<uint64_t>(a.S) * p.kv_len * 2};
    const uint32_t box[3] = {64, BQ, 1};
    if ((status = make_tensor_map(&p.map_noise, a.noise, 3, dims, strides, box)) != TB200_OK) return status;
    p.noise_tma = 1;
  }
  const dim3 grid((a.S + BQ - 1) / BQ, a.Hq, a.B);
  const bool noise = a.noise != nullptr;
  if (a.dtype == TB200_BF16) return launch_t<__nv_bfloat16>(p, a.D, noise, grid, stream);
  return launch_t<__half>(p, a.D, noise, grid, stream);
}

}  // namespace tb200
