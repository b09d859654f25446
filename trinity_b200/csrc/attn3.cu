// Attention forward, two query tiles per CTA, with the score MMA taken off the softmax's critical path.
//
// Same roles as attn2.cu (warp 0 TMA, warp 1 MMA, warps 2-5 / 6-9 softmax of query tile 0 / 1), but P_j goes through
// shared memory instead of being written back over S_j in tensor memory.  With S and P in different places the next
// score tile S_{j+1} = Q K_{j+1}^T can be issued as soon as the softmax warps have copied S_j into registers, i.e.
// while they are still exponentiating it, and the chain softmax(j) -> P V(j) -> S(j+1) -> softmax(j+1) that bounds
// attn2.cu shrinks to softmax(j) -> softmax(j+1).  Per key tile j the MMA warp issues
//     S0_{j+1}, S1_{j+1}   (each after its tile's S_j was consumed),   then P0_j V_j, P1_j V_j   (after each P is ready).
// Shared memory at D = 128: Q 2 x 32 KiB, K one 32 KiB stage (the load of K_{j+1} starts when S_j is done and has a whole
// softmax to arrive), V two stages, P 2 x 32 KiB  = 224 KiB.
// Tensor memory: S0 [0,128)  S1 [128,256)  O0 [256,256+D)  O1 [256+D,256+2D).
#include <math.h>
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kThreads = 320;
constexpr int kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;

template <int D> struct Smem3 {
  static constexpr int kKStages = (D == 64) ? 2 : 1;  // K_{j+1} is fetched as soon as S_j is done: one stage is enough
  static constexpr int kVStages = 2;                  // V_{j+1} must be on its way while P V_j still runs
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kPBytes = BQ * BKV * 2;
  static constexpr int kQOff = 0;                          // two query tiles
  static constexpr int kKOff = 2 * kTile;
  static constexpr int kVOff = kKOff + kKStages * kTile;
  static constexpr int kPOff = kVOff + kVStages * kTile;  // two P tiles, UMMA K-major 128B-swizzle layout
  static constexpr int kBarOff = kPOff + 2 * kPBytes;
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

struct Attn3Params {
  CUtensorMap map_q, map_k, map_v;
  int B, S, Hq, Hkv, past, kv_len, causal;
  float scale_log2;
  void* o2;
  float* lse2;
  int* err;
};

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 1) attn_fwd3_kernel(const __grid_constant__ Attn3Params p) {
  using L = Smem3<D>;
  constexpr int KS = L::kKStages, VS = L::kVStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2] per query tile
  uint64_t* s_taken = bars + 11;    // [2] per query tile: the softmax warps hold S_j in registers
  uint64_t* p_ready = bars + 13;    // [2] per query tile
  uint64_t* pv_done = bars + 15;    // [2] per query tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_blocks = (p.S + 2 * BQ - 1) / (2 * BQ);
  const int q0 = (n_blocks - 1 - blockIdx.x) * 2 * BQ;  // longest blocks first
  const int hq = blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = hq / (p.Hq / p.Hkv);
  int nt[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0t = q0 + t * BQ;
    int last_key = p.kv_len - 1;
    if (p.causal) last_key = min(last_key, p.past + min(q0t + BQ - 1, p.S - 1));
    nt[t] = (q0t < p.S) ? last_key / BKV + 1 : 0;
  }
  const int nt_max = max(nt[0], nt[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_taken[i], 128);
      mbar_init(&p_ready[i], 128);
      mbar_init(&pv_done[i], 1);
    }
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
  const AbortCtx ctx{p.err, abort_flag};

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 2 * L::kTile);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_3d(smem + L::kQOff + t * L::kTile + dc * (BQ * 128), &p.map_q, q_full, dc * 64, q0 + t * BQ, b * p.Hq + hq);
    }
    __syncwarp();
    for (int j = 0; j < nt_max; ++j) {
      const int ks = j % KS, vs = j % VS;
      if (!mbar_wait(&k_empty[ks], ((j / KS) & 1) ^ 1, ctx, 501)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&k_full[ks], L::kTile);
#pragma unroll
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_3d(smem + L::kKOff + ks * L::kTile + dc * (BKV * 128), &p.map_k, &k_full[ks], dc * 64, j * BKV, b * p.Hkv + hkv);
      }
      __syncwarp();
      if (!mbar_wait(&v_empty[vs], ((j / VS) & 1) ^ 1, ctx, 502)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&v_full[vs], L::kTile);
#pragma unroll
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_3d(smem + L::kVOff + vs * L::kTile + dc * (BKV * 128), &p.map_v, &v_full[vs], dc * 64, j * BKV, b * p.Hkv + hkv);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (all lanes converged, one elected lane issues)
    constexpr uint32_t idesc_s = make_idesc(IsBf16<T>::value, false, false, BQ, BKV);
    constexpr uint32_t idesc_o = make_idesc(IsBf16<T>::value, false, true, BQ, D);
    const uint32_t q_base = smem_u32(smem + L::kQOff);
    const uint32_t k_base = smem_u32(smem + L::kKOff);
    const uint32_t v_base = smem_u32(smem + L::kVOff);
    const uint32_t p_base = smem_u32(smem + L::kPOff);
    auto issue_s = [&](int t, int j) {  // S_t = Q_t K_j^T
      const uint64_t qd = make_smem_desc(q_base + t * L::kTile, 16, 1024);
      const uint64_t kd = make_smem_desc(k_base + (j % KS) * L::kTile, 16, 1024);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint64_t off = static_cast<uint64_t>(((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4);
        umma_ss_warp(tmem_base + t * BKV, qd + off, kd + off, idesc_s, kk > 0 ? 1u : 0u);
      }
      umma_commit_warp(&s_full[t]);
    };
    auto issue_pv = [&](int t, int j) {  // O_t += P_t V_j, both operands from shared memory
      const uint64_t pd = make_smem_desc(p_base + t * L::kPBytes, 16, 1024);
      const uint64_t vd = make_smem_desc(v_base + (j % VS) * L::kTile, BKV * 128, 1024);  // MN-major
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk) {
        const uint64_t poff = static_cast<uint64_t>(((kk >> 2) * (BQ * 128) + (kk & 3) * 32) >> 4);
        umma_ss_warp(tmem_base + 2 * BKV + t * D, pd + poff, vd + static_cast<uint64_t>(kk * 128), idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
      }
      umma_commit_warp(&pv_done[t]);
    };
    bool ok = mbar_wait(q_full, 0, ctx, 503) && mbar_wait(&k_full[0], 0, ctx, 504);
    if (ok) {
      tc_fence_after();
      if (nt[0] > 0) issue_s(0, 0);
      if (nt[1] > 0) issue_s(1, 0);
      umma_commit_warp(&k_empty[0]);
    }
    for (int j = 0; ok && j < nt_max; ++j) {
      // next score tiles first: they only need K_{j+1} and the S buffers, which the softmax warps free early
      if (j + 1 < nt_max) {
        if (!mbar_wait(&k_full[(j + 1) % KS], ((j + 1) / KS) & 1, ctx, 505)) break;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j + 1 < nt[t]) {
            if (!mbar_wait(&s_taken[t], j & 1, ctx, 506)) { ok = false; break; }
            tc_fence_after();
            issue_s(t, j + 1);
          }
        }
        if (!ok) break;
        umma_commit_warp(&k_empty[(j + 1) % KS]);
      }
      if (!mbar_wait(&v_full[j % VS], (j / VS) & 1, ctx, 507)) break;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (j < nt[t]) {
          if (!mbar_wait(&p_ready[t], j & 1, ctx, 508)) { ok = false; break; }
          tc_fence_after();
          issue_pv(t, j);
        }
      }
      if (!ok) break;
      umma_commit_warp(&v_empty[j % VS]);
    }
  } else {
    // ------------------------------------------------------------ softmax warpgroups (thread = query row)
    const int t = (warp - 2) >> 2;
    const int quad = warp & 3;
    const int r_in = quad * 32 + lane;
    const int qi = q0 + t * BQ + r_in;
    const bool row_ok = qi < p.S;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tmem_s = tmem_base + t * BKV + lane_sel;
    const uint32_t tmem_o = tmem_base + 2 * BKV + t * D + lane_sel;
    uint8_t* p_row = smem + L::kPOff + t * L::kPBytes + r_in * 128;  // this row inside each 64-key chunk of the P tile
    const int key_limit = p.causal ? min(p.past + qi, p.kv_len - 1) : p.kv_len - 1;
    const int my_nt = nt[t];
    float m_use = -INFINITY, l = 0.f;
    bool ok = true;

    for (int j = 0; j < my_nt; ++j) {
      const int k0 = j * BKV;
      if (!mbar_wait(&s_full[t], j & 1, ctx, 509)) { ok = false; break; }
      tc_fence_after();
      uint32_t s[BKV];
      tmem_ld_x32(tmem_s + 0, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld_x32(tmem_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_ld_x32(tmem_s + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
      tmem_ld_x32(tmem_s + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&s_taken[t]);  // S_j is in registers: the tensor core may write S_{j+1}

      if (k0 + BKV - 1 > key_limit) {  // tile touches the causal diagonal or the end of the keys
#pragma unroll
        for (int i = 0; i < BKV; ++i)
          if (k0 + i > key_limit) s[i] = 0xff800000u;  // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BKV; i += 8) {  // three-input max: one instruction per two elements, four chains
        mx0 = max3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        mx1 = max3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
        mx2 = max3(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
        mx3 = max3(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
      }
      const float rowmax = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_new = fmaxf(m_use, rowmax * p.scale_log2);
      const bool grow = m_new > m_use + kRescaleThreshold;  // true on the first tile (m_use = -inf)
      float alpha = 1.f;
      if (grow) {
        alpha = fast_exp2(m_use - m_new);
        m_use = m_new;
      }
      const float neg_mref = (m_use == -INFINITY) ? 0.f : -m_use;
      // packed fp32x2 arithmetic: one FMA and one ADD instruction per two elements
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 nm2 = make_float2(neg_mref, neg_mref);
      float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
      uint32_t pk[BKV / 2];
#pragma unroll
      for (int i = 0; i < BKV; i += 4) {
        const float2 t0 = __ffma2_rn(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), sc2, nm2);
        const float2 t1 = __ffma2_rn(make_float2(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3])), sc2, nm2);
        const float2 e0 = make_float2(fast_exp2(t0.x), fast_exp2(t0.y));
        const float2 e1 = make_float2(fast_exp2(t1.x), fast_exp2(t1.y));
        acc0 = __fadd2_rn(acc0, e0);
        acc1 = __fadd2_rn(acc1, e1);
        pk[i >> 1] = Pack2<T>::pack(e0.x, e0.y);
        pk[(i >> 1) + 1] = Pack2<T>::pack(e1.x, e1.y);
      }
      l = l * alpha + ((acc0.x + acc0.y) + (acc1.x + acc1.y));

      // P_{j-1} V_{j-1} of this tile must have finished before its P tile is overwritten or O is rescaled
      if (j > 0) {
        if (!mbar_wait(&pv_done[t], (j - 1) & 1, ctx, 510)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow)) {
          uint32_t o[32];
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            tmem_ld_x32(tmem_o + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_x32(tmem_o + c * 32, o);
          }
          tmem_wait_st();
        }
      }
      // P row into shared memory: K-major, 128-byte swizzle (16-byte unit u of a row lands at u ^ (row & 7))
#pragma unroll
      for (int u = 0; u < BKV / 8; ++u)
        *reinterpret_cast<uint4*>(p_row + (u >> 3) * (BQ * 128) + (((u & 7) ^ (r_in & 7)) << 4)) =
            make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_ready[t]);
    }

    if (ok && my_nt > 0 && mbar_wait(&pv_done[t], (my_nt - 1) & 1, ctx, 511)) {
      tc_fence_after();
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      T* orow = static_cast<T*>(p.o2) + ((static_cast<long long>(b) * p.S + qi) * p.Hq + hq) * D;
      uint32_t o[32];
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        tmem_ld_x32(tmem_o + c * 32, o);
        tmem_wait_ld();
        if (row_ok) {
          uint4* d = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            d[i] = make_uint4(Pack2<T>::pack(__uint_as_float(o[8 * i]) * inv_l, __uint_as_float(o[8 * i + 1]) * inv_l),
                              Pack2<T>::pack(__uint_as_float(o[8 * i + 2]) * inv_l, __uint_as_float(o[8 * i + 3]) * inv_l),
                              Pack2<T>::pack(__uint_as_float(o[8 * i + 4]) * inv_l, __uint_as_float(o[8 * i + 5]) * inv_l),
                              Pack2<T>::pack(__uint_as_float(o[8 * i + 6]) * inv_l, __uint_as_float(o[8 * i + 7]) * inv_l));
        }
      }
      if (row_ok && p.lse2 != nullptr) p.lse2[(static_cast<long long>(b) * p.Hq + hq) * p.S + qi] = m_use + log2f(l);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, int D>
int launch_one(const Attn3Params& p, dim3 grid, cudaStream_t stream) {
  static bool attr_set[32] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 31]) {
    if (cudaFuncSetAttribute(attn_fwd3_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem3<D>::kTotal) != cudaSuccess)
      return TB200_ERR_CUDA;
    attr_set[dev & 31] = true;
  }
  attn_fwd3_kernel<T, D><<<grid, kThreads, Smem3<D>::kTotal, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

}  // namespace

// Same contract as launch_attn_fwd without the KeyFormer statistic; arguments are validated by the caller.
int launch_attn_fwd_decoupled(const AttnLaunch& a, cudaStream_t stream) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  Attn3Params p;
  memset(&p, 0, sizeof(p));
  p.B = a.B; p.S = a.S; p.Hq = a.Hq; p.Hkv = a.Hkv; p.past = a.past; p.kv_len = a.past + a.S; p.causal = a.causal;
  p.scale_log2 = a.sm_scale * kLog2e;
  p.o2 = a.o2;
  p.lse2 = a.lse2;
  p.err = st->err_word;
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
  const dim3 grid((a.S + 2 * BQ - 1) / (2 * BQ), a.Hq, a.B);
  if (a.dtype == TB200_BF16) {
    return a.D == 128 ? launch_one<__nv_bfloat16, 128>(p, grid, stream) : launch_one<__nv_bfloat16, 64>(p, grid, stream);
  }
  return a.D == 128 ? launch_one<__half, 128>(p, grid, stream) : launch_one<__half, 64>(p, grid, stream);
}

}  // namespace tb200
