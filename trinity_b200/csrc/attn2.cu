// Attention forward, two query tiles per CTA ("ping-pong"): the kernel used when no noise tensor is involved.
//
// One CTA per (256 queries, q head, batch element), 320 threads (kHalves = 1):
//   warp 0      TMA producer: both Q tiles once, then K and V tiles of 128 keys through two-deep rings
//   warp 1      MMA issuer, in this order per key tile j:  P0_j V_j, S0_{j+1}, P1_j V_j, S1_{j+1}
//   warps 2-5   softmax of query tile 0          warps 6-9   softmax of query tile 1
// While one softmax warpgroup works on its S tile the tensor core serves the other tile, and each SM sub-partition
// holds two softmax warps whose MUFU / FMA / TMEM latencies overlap.  K and V tiles are fetched once for 256 queries.
//
// Tensor memory (512 columns): S0 [0,128)  S1 [128,256)  O0 [256,256+D)  O1 [256+D,256+2D).
// P_j (16-bit) is written back over the first 64 columns of its own S tile and is the A operand of P_j V_j straight
// from tensor memory (no shared-memory round trip).  MMAs issued by one thread complete in issue order, so S_{j+1}
// (issued after P_j V_j) cannot overwrite P_j early, and an arrival on s_full also means the previous P V is done.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
// Threads per query row in the softmax.  2 was measured slower on B200 (0.418 ms against 0.353 ms on the Llama-3-8B
// B8 S2048 prefill): the row-max exchange and the 96-register cap of a 576-thread CTA cost more than the extra warps hide.
constexpr int kHalves = 1;
constexpr int kThreads = 64 + 2 * 128 * kHalves;  // TMA warp, MMA warp, softmax warps of two query tiles
constexpr int kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;

template <int D> struct Smem2 {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kQOff = 0;                 // two query tiles
  static constexpr int kKOff = 2 * kTile;         // two stages
  static constexpr int kVOff = 4 * kTile;         // two stages
  static constexpr int kBarOff = 6 * kTile;
  static constexpr int kXchOff = kBarOff + 256;   // row max / row sum exchange between the threads of a row
  static constexpr int kTotal = kXchOff + 6 * 1024 + 1024;
};

struct Attn2Params {
  CUtensorMap map_q, map_k, map_v;
  int B, S, Hq, Hkv, past, kv_len, causal;
  float scale_log2;
  void* o2;
  float* lse2;
  int kv_splits;     // > 1: the key tiles are dealt out over this many CTAs, which leave partial results
  float* part_o;     // (kv_splits, B, Hq, S, D) fp32, unnormalised
  float* part_ml;    // (kv_splits, B, Hq, S, 2): exponent reference and row sum of each part
  int* err;
  long long* trace;  // timing probes (TB200_TRACE builds only)
};

#ifdef TB200_TRACE
#define TRACE(slot, cond) do { if ((cond) && p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) p.trace[(slot)] = clock64(); } while (0)
#else
#define TRACE(slot, cond) do { } while (0)
#endif

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 1) attn_fwd2_kernel(const __grid_constant__ Attn2Params p) {
  using L = Smem2<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2] per query tile
  uint64_t* p_ready = bars + 11;  // [2] per query tile
  uint64_t* pv_done = bars + 13;  // [2] per query tile
  uint64_t* row_xch = bars + 15;  // [2] per query tile: the threads of a row have published their partial
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_blocks = (p.S + 2 * BQ - 1) / (2 * BQ);
  const int blk = blockIdx.x / p.kv_splits;
  const int sp = blockIdx.x - blk * p.kv_splits;         // which share of the key tiles this CTA takes
  const int q0 = (n_blocks - 1 - blk) * 2 * BQ;          // longest blocks first
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
  // key tiles [j_begin, j_begin + nt[t]) of each query tile; local index j below, global j_begin + j for coordinates
  const int per_split = (max(nt[0], nt[1]) + p.kv_splits - 1) / p.kv_splits;
  const int j_begin = sp * per_split;
#pragma unroll
  for (int t = 0; t < 2; ++t) nt[t] = max(0, min(nt[t], j_begin + per_split) - j_begin);
  const int nt_max = max(nt[0], nt[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 128 * kHalves);
      mbar_init(&pv_done[i], 1);
      mbar_init(&row_xch[i], 128 * kHalves);
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
    if (lane == 0 && nt_max > 0) {
      mbar_arrive_expect_tx(q_full, 2 * L::kTile);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_3d(smem + L::kQOff + t * L::kTile + dc * (BQ * 128), &p.map_q, q_full, dc * 64, q0 + t * BQ, b * p.Hq + hq);
    }
    __syncwarp();
    for (int j = 0; j < nt_max; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&k_empty[st], ph ^ 1, ctx, 401)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&k_full[st], L::kTile);
#pragma unroll
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_3d(smem + L::kKOff + st * L::kTile + dc * (BKV * 128), &p.map_k, &k_full[st], dc * 64, (j_begin + j) * BKV, b * p.Hkv + hkv);
      }
      __syncwarp();
      if (!mbar_wait(&v_empty[st], ph ^ 1, ctx, 402)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&v_full[st], L::kTile);
#pragma unroll
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_3d(smem + L::kVOff + st * L::kTile + dc * (BKV * 128), &p.map_v, &v_full[st], dc * 64, (j_begin + j) * BKV, b * p.Hkv + hkv);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_s = make_idesc(IsBf16<T>::value, false, false, BQ, BKV);
    constexpr uint32_t idesc_o = make_idesc(IsBf16<T>::value, false, true, BQ, D);
    // All 32 lanes run this code converged with warp-uniform operands; one elected lane issues (see common.cuh).
    const uint32_t q_base = smem_u32(smem + L::kQOff);
    const uint32_t k_base = smem_u32(smem + L::kKOff);
    const uint32_t v_base = smem_u32(smem + L::kVOff);
    auto issue_s = [&](int t, int j) {  // S_t = Q_t K_j^T
      const uint64_t qd = make_smem_desc(q_base + t * L::kTile, 16, 1024);
      const uint64_t kd = make_smem_desc(k_base + (j & 1) * L::kTile, 16, 1024);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint64_t off = static_cast<uint64_t>(((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4);  // start-address field
        umma_ss_warp(tmem_base + t * BKV, qd + off, kd + off, idesc_s, kk > 0 ? 1u : 0u);
      }
      umma_commit_warp(&s_full[t]);
    };
    auto issue_pv = [&](int t, int j) {  // O_t += P_t V_j, P_t read from tensor memory
      const uint64_t vd = make_smem_desc(v_base + (j & 1) * L::kTile, BKV * 128, 1024);
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk)
        umma_ts_warp(tmem_base + 2 * BKV + t * D, tmem_base + t * BKV + kk * 8, vd + static_cast<uint64_t>((kk * 2048) >> 4), idesc_o,
                     (j > 0 || kk > 0) ? 1u : 0u);
      umma_commit_warp(&pv_done[t]);
    };
    bool ok = nt_max > 0 && mbar_wait(q_full, 0, ctx, 403) && mbar_wait(&k_full[0], 0, ctx, 404);
    if (ok) {
      tc_fence_after();
      if (nt[0] > 0) issue_s(0, 0);
      if (nt[1] > 0) issue_s(1, 0);
      umma_commit_warp(&k_empty[0]);
    }
    for (int j = 0; ok && j < nt_max; ++j) {
      if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1, ctx, 405)) break;
      bool k_ready = false;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (j < nt[t]) {
          if (!mbar_wait(&p_ready[t], j & 1, ctx, 406)) { ok = false; break; }
          tc_fence_after();
          TRACE(512 + (t * 32 + j) * 4 + 0, lane == 0 && j < 32);
          issue_pv(t, j);
          TRACE(512 + (t * 32 + j) * 4 + 1, lane == 0 && j < 32);
        }
        if (t == 1) umma_commit_warp(&v_empty[j & 1]);
        if (j + 1 < nt[t]) {
          if (!k_ready) {
            if (!mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, ctx, 407)) { ok = false; break; }
            tc_fence_after();
            k_ready = true;
          }
          issue_s(t, j + 1);
          TRACE(512 + (t * 32 + j) * 4 + 2, lane == 0 && j < 32);
        }
      }
      if (ok && j + 1 < nt_max) umma_commit_warp(&k_empty[(j + 1) & 1]);
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    // kHalves threads share a query row: thread (row, h) owns the S columns [h*CW, (h+1)*CW) of the row and the O
    // columns [h*D/kHalves, ...).  The two threads sit in different warps that may touch the same TMEM lanes
    // (warp % 4 is equal), which doubles the warps per SM sub-partition available to hide MUFU / FMA latency.
    constexpr int CW = BKV / kHalves;   // S columns per thread
    constexpr int OW = D / kHalves;     // O columns per thread
    const int sw = warp - 2;
    const int t = sw / (4 * kHalves);   // query tile
    const int h = (sw >> 2) % kHalves;  // column half
    const int quad = warp & 3;
    const int r_in = quad * 32 + lane;
    const int qi = q0 + t * BQ + r_in;
    const bool row_ok = qi < p.S;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tmem_s = tmem_base + t * BKV + lane_sel;
    const uint32_t tmem_o = tmem_base + 2 * BKV + t * D + h * OW + lane_sel;
    const int key_limit = p.causal ? min(p.past + qi, p.kv_len - 1) : p.kv_len - 1;
    const int my_nt = nt[t];
    float* xmax = reinterpret_cast<float*>(smem + L::kXchOff) + t * (2 * kHalves * 128);  // [parity][half][row]
    float* xsum = reinterpret_cast<float*>(smem + L::kXchOff) + 2 * (2 * kHalves * 128) + t * (kHalves * 128);
    float m_use = -INFINITY, l = 0.f;
    bool ok = true;

    for (int j = 0; j < my_nt; ++j) {
      const int k0 = (j_begin + j) * BKV + h * CW;
      TRACE((t * 32 + j) * 8 + 0, r_in == 0 && h == 0 && j < 32);
      if (!mbar_wait(&s_full[t], j & 1, ctx, 408)) { ok = false; break; }
      tc_fence_after();
      TRACE((t * 32 + j) * 8 + 1, r_in == 0 && h == 0 && j < 32);
      uint32_t s[CW];
#pragma unroll
      for (int c = 0; c < CW / 32; ++c) tmem_ld_x32(tmem_s + h * CW + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
      tmem_wait_ld();
      TRACE((t * 32 + j) * 8 + 2, r_in == 0 && h == 0 && j < 32);

      if (k0 + CW - 1 > key_limit) {  // these columns touch the causal diagonal or the end of the keys
#pragma unroll
        for (int i = 0; i < CW; ++i)
          if (k0 + i > key_limit) s[i] = 0xff800000u;  // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < CW; i += 8) {  // three-input max: one instruction per two elements, four chains
        mx0 = max3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        mx1 = max3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
        mx2 = max3(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
        mx3 = max3(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
      }
      float rowmax = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      if (kHalves > 1) {  // combine with the other half of the row (bounded wait, no bar.sync)
        float* slot = xmax + (j & 1) * (kHalves * 128);
        slot[h * 128 + r_in] = rowmax;
        mbar_arrive(&row_xch[t]);
        if (!mbar_wait(&row_xch[t], j & 1, ctx, 410)) { ok = false; break; }
        rowmax = fmaxf(rowmax, slot[(h ^ 1) * 128 + r_in]);
      }
      const float m_new = fmaxf(m_use, rowmax * p.scale_log2);
      const bool grow = m_new > m_use + kRescaleThreshold;  // true on the first tile (m_use = -inf)
      float alpha = 1.f;
      if (grow) {
        alpha = fast_exp2(m_use - m_new);
        m_use = m_new;
      }
      const float neg_mref = (m_use == -INFINITY) ? 0.f : -m_use;
      TRACE((t * 32 + j) * 8 + 3, r_in == 0 && h == 0 && j < 32);
      // packed fp32x2 arithmetic: one FMA and one ADD instruction per two elements
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 nm2 = make_float2(neg_mref, neg_mref);
      float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
      uint32_t pk[CW / 2];
#pragma unroll
      for (int i = 0; i < CW; i += 4) {
        const float2 t0 = __ffma2_rn(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), sc2, nm2);
        const float2 t1 = __ffma2_rn(make_float2(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3])), sc2, nm2);
        const float2 e0 = make_float2(fast_exp2(t0.x), fast_exp2(t0.y));
        const float2 e1 = make_float2(fast_exp2(t1.x), fast_exp2(t1.y));
        acc0 = __fadd2_rn(acc0, e0);
        acc1 = __fadd2_rn(acc1, e1);
        pk[i >> 1] = Pack2<T>::pack(e0.x, e0.y);
        pk[(i >> 1) + 1] = Pack2<T>::pack(e1.x, e1.y);
      }
      l = l * alpha + ((acc0.x + acc0.y) + (acc1.x + acc1.y));  // this thread's share of the row sum
      TRACE((t * 32 + j) * 8 + 4, r_in == 0 && h == 0 && j < 32);

      // s_full(j) arrived => P_{j-1} V_{j-1} of this tile has completed: O may be rescaled, P may be overwritten
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        uint32_t o[32];
#pragma unroll 1
        for (int c = 0; c < OW / 32; ++c) {
          tmem_ld_x32(tmem_o + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_x32(tmem_o + c * 32, o);
        }
      }
#pragma unroll
      for (int c = 0; c < CW / 64; ++c)  // 64 keys = 32 packed columns per store
        tmem_st_x32(tmem_s + h * (CW / 2) + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[c * 32]));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_ready[t]);
      TRACE((t * 32 + j) * 8 + 5, r_in == 0 && h == 0 && j < 32);
    }

    if (ok && my_nt > 0 && kHalves > 1) {  // total row sum
      xsum[h * 128 + r_in] = l;
      mbar_arrive(&row_xch[t]);
      ok = mbar_wait(&row_xch[t], my_nt & 1, ctx, 411);
      if (ok) l += xsum[(h ^ 1) * 128 + r_in];
    }
    if (p.kv_splits > 1) {
      // this CTA saw only a share of the keys: leave the unnormalised accumulator, its exponent reference and its row
      // sum; attn_combine_kernel merges the shares.  A share without keys leaves the neutral element.
      const long long prow = ((static_cast<long long>(sp) * p.B + b) * p.Hq + hq) * p.S + qi;
      const bool have = ok && my_nt > 0 && mbar_wait(&pv_done[t], (my_nt - 1) & 1, ctx, 409);
      if (have) tc_fence_after();
      uint32_t o[32];
#pragma unroll 1
      for (int c = 0; c < OW / 32; ++c) {
        if (have) {  // uniform over the warp
          tmem_ld_x32(tmem_o + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (row_ok) {
          uint4* d = reinterpret_cast<uint4*>(p.part_o + prow * D + h * OW + c * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i) d[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
      }
      if (row_ok && h == 0) {
        p.part_ml[prow * 2] = have ? m_use : -INFINITY;
        p.part_ml[prow * 2 + 1] = have ? l : 0.f;
      }
    } else if (ok && my_nt > 0 && mbar_wait(&pv_done[t], (my_nt - 1) & 1, ctx, 409)) {
      tc_fence_after();
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      T* orow = static_cast<T*>(p.o2) + ((static_cast<long long>(b) * p.S + qi) * p.Hq + hq) * D + h * OW;
      uint32_t o[32];
#pragma unroll 1
      for (int c = 0; c < OW / 32; ++c) {
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
      if (row_ok && h == 0 && p.lse2 != nullptr) p.lse2[(static_cast<long long>(b) * p.Hq + hq) * p.S + qi] = m_use + log2f(l);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Merge the shares of a key-split launch: one warp per (batch, head, query) row, lanes over the D columns.
template <typename T, int D>
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, T* __restrict__ o2,
                                    float* __restrict__ lse2, int splits, int B, int Hq, int S) {
  constexpr int V = D / 32;
  const long long rows = static_cast<long long>(B) * Hq * S;
  const int lane = threadIdx.x & 31;
  for (long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; row < rows;
       row += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(s * rows + row) * 2]);
    float l = 0.f, acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    for (int s = 0; s < splits; ++s) {  // fixed order: deterministic
      const float ms = part_ml[(s * rows + row) * 2];
      const float w = (ms == -INFINITY) ? 0.f : fast_exp2(ms - m);
      l = fmaf(w, part_ml[(s * rows + row) * 2 + 1], l);
      const float* po = part_o + (s * rows + row) * D + lane * V;
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = fmaf(w, po[i], acc[i]);
    }
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
    const int qi = static_cast<int>(row % S);
    const int hq = static_cast<int>((row / S) % Hq);
    const int b = static_cast<int>(row / (static_cast<long long>(S) * Hq));
    uint32_t* dst = reinterpret_cast<uint32_t*>(o2 + ((static_cast<long long>(b) * S + qi) * Hq + hq) * D + lane * V);
#pragma unroll
    for (int i = 0; i < V; i += 2) dst[i >> 1] = Pack2<T>::pack(acc[i] * inv_l, acc[i + 1] * inv_l);
    if (lane == 0 && lse2 != nullptr) lse2[row] = m + log2f(l);
  }
}

template <typename T, int D>
int launch_one(const Attn2Params& p, dim3 grid, cudaStream_t stream) {
  static bool attr_set[32] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 31]) {
    if (cudaFuncSetAttribute(attn_fwd2_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem2<D>::kTotal) != cudaSuccess)
      return TB200_ERR_CUDA;
    attr_set[dev & 31] = true;
  }
  attn_fwd2_kernel<T, D><<<grid, kThreads, Smem2<D>::kTotal, stream>>>(p);
  if (cudaGetLastError() != cudaSuccess) return TB200_ERR_CUDA;
  if (p.kv_splits > 1) {
    const long long rows = static_cast<long long>(p.B) * p.Hq * p.S;
    long long blocks = (rows * 32 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    attn_combine_kernel<T, D><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p.part_o, p.part_ml, static_cast<T*>(p.o2), p.lse2,
                                                                             p.kv_splits, p.B, p.Hq, p.S);
    if (cudaGetLastError() != cudaSuccess) return TB200_ERR_CUDA;
  }
  return TB200_OK;
}

}  // namespace

// With few (query block, head, batch) CTAs and many key tiles -- the decode shapes -- the key range is dealt out over
// several CTAs per block so that the SMs are filled; 1 = no split.
int attn_kv_splits(int B, int S, int Hq, int kv_len, int num_sms) {
  const long long ctas = static_cast<long long>((S + 2 * BQ - 1) / (2 * BQ)) * Hq * B;
  const int tiles = (kv_len + BKV - 1) / BKV;
  if (ctas * 2 > num_sms || tiles < 4) return 1;
  int s = static_cast<int>(num_sms / ctas);
  if (s > tiles / 2) s = tiles / 2;
  if (s > 16) s = 16;
  return s < 2 ? 1 : s;
}

// Same contract as launch_attn_fwd without the KeyFormer statistic; arguments are validated by the caller.
int launch_attn_fwd_pingpong(const AttnLaunch& a, cudaStream_t stream) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  Attn2Params p;
  memset(&p, 0, sizeof(p));
  p.B = a.B; p.S = a.S; p.Hq = a.Hq; p.Hkv = a.Hkv; p.past = a.past; p.kv_len = a.past + a.S; p.causal = a.causal;
  p.scale_log2 = a.sm_scale * kLog2e;
  p.o2 = a.o2;
  p.lse2 = a.lse2;
  p.kv_splits = (a.kv_splits > 1 && a.part_o != nullptr && a.part_ml != nullptr) ? a.kv_splits : 1;
  p.part_o = a.part_o;
  p.part_ml = a.part_ml;
  p.err = st->err_word;
#ifdef TB200_TRACE
  if (const char* tp = getenv("TB200_TRACE_PTR")) p.trace = reinterpret_cast<long long*>(strtoull(tp, nullptr, 0));
#endif
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
  const dim3 grid(((a.S + 2 * BQ - 1) / (2 * BQ)) * p.kv_splits, a.Hq, a.B);
  if (a.dtype == TB200_BF16) {
    return a.D == 128 ? launch_one<__nv_bfloat16, 128>(p, grid, stream) : launch_one<__nv_bfloat16, 64>(p, grid, stream);
  }
  return a.D == 128 ? launch_one<__half, 128>(p, grid, stream) : launch_one<__half, 64>(p, grid, stream);
}

}  // namespace tb200
