// Attention forward, two query tiles per CTA ("ping-pong"): the kernel used when no noise tensor is involved.
//
// Persistent: one CTA per SM walks work items (256 queries, q head, batch element[, share of the keys]), longest
// items first.  512 threads in four warpgroups, registers re-dealt between them with setmaxnreg (80 / 184 / 184 / 64):
//   warp 0      TMA producer: the two Q tiles of an item, then its K and V tiles of 128 keys through two-deep rings
//               that run on across items
//   warp 1      MMA issuer, in this order per key tile j:  P0_j V_j, S0_{j+1}, P1_j V_j, S1_{j+1}; in the last step of
//               an item the S_0 tiles of the NEXT item take the place of S_{j+1}     (warps 2-3 idle)
//   warps 4-7   softmax of query tile 0          warps 8-11  softmax of query tile 1
//   warps 12-15 output: when an item's last P V of a query tile is done, O leaves tensor memory, is normalised, staged
//               in shared memory and written with TMA stores -- while the softmax warpgroups are already on the next item
// While one softmax warpgroup works on its S tile the tensor core serves the other tile, and each SM sub-partition
// holds two softmax warps whose MUFU / FMA / TMEM latencies overlap.  K and V tiles are fetched once for 256 queries.
// Across items the pipeline does not drain: the Q tiles of item i+1 are in shared memory and its first S tiles in
// tensor memory before item i's output has left.
//
// Tensor memory (512 columns): S0 [0,128)  S1 [128,256)  O0 [256,256+D)  O1 [256+D,256+2D).
// P_j (16-bit) is written back over the first 64 columns of its own S tile and is the A operand of P_j V_j straight
// from tensor memory (no shared-memory round trip).  MMAs issued by one thread complete in issue order, so S_{j+1}
// (issued after P_j V_j) cannot overwrite P_j early, and an arrival on s_full also means the previous P V is done.
// The first P V of an item overwrites O, so it waits until the output warpgroup has read the previous item's O (o_free).
//
// One thread owns one query row.  (Two threads per row were measured slower on B200 -- 0.418 ms against 0.353 ms on
// the Llama-3-8B B8 S2048 prefill: the row-max exchange costs more than the extra warps hide -- and so was a variant
// with P staged in shared memory.)
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kThreads = 4 * 128;  // warpgroups: TMA + MMA (+2 idle warps), softmax of query tile 0, of tile 1, output
constexpr int kRegsControl = 80, kRegsSoftmax = 184, kRegsOutput = 64;  // (80 + 184 + 184 + 64) * 128 = 65536
constexpr int kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;

template <int D> struct Smem2 {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kQOff = 0;                 // two query tiles
  static constexpr int kKOff = 2 * kTile;         // two stages
  static constexpr int kVOff = 4 * kTile;         // two stages
  static constexpr int kOOff = 6 * kTile;         // one normalised output tile (16-bit) on its way to a TMA store
  static constexpr int kStatOff = 7 * kTile;      // 2 x 128 floats: the factor each row of O is multiplied with
  static constexpr int kBarOff = kStatOff + 1024;
  static constexpr int kTotal = kBarOff + 256 + 1024;
  static_assert(kTotal <= 232448, "more shared memory than an sm_100 CTA can have");
};

// Division by a value fixed for the launch as a multiply and a shift: decoding an item takes four divisions, and as
// emulated 32-bit divisions they cost each role about a thousand cycles per item.  Valid for n < 2^31.
struct FastDiv {
  uint32_t mul, shr, d;
};
inline FastDiv make_fastdiv(uint32_t d) {
  FastDiv f;
  f.d = d;
  uint32_t s = 0;
  while ((1ull << s) < d) ++s;
  f.shr = s;
  f.mul = static_cast<uint32_t>(((1ull << 32) * ((1ull << s) - d)) / d + 1);
  return f;
}
__device__ __forceinline__ int fdiv(int n, const FastDiv& f) {
  return static_cast<int>((__umulhi(static_cast<uint32_t>(n), f.mul) + static_cast<uint32_t>(n)) >> f.shr);
}

struct Attn2Params {
  CUtensorMap map_q, map_k, map_v, map_o;
  int B, S, Hq, Hkv, past, kv_len, causal;
  int n_blocks;      // blocks of 256 queries
  int n_items;       // n_blocks * kv_splits * Hq * B
  FastDiv d_per_blk, d_splits, d_hq, d_group;  // B * Hq * kv_splits, kv_splits, Hq, Hq / Hkv
  float scale_log2;
  void* o2;
  float* lse2;
  int kv_splits;     // > 1: the key tiles are dealt out over this many items, which leave partial results
  float* part_o;     // (kv_splits, B, Hq, S, D) fp32, unnormalised
  float* part_ml;    // (kv_splits, B, Hq, S, 2): exponent reference and row sum of each part
  int* err;
  long long wait_limit;  // cycles a bounded wait may last (tb200_set_wait_limit_cycles)
};

// One unit of work.  Items are numbered so that the longest (the last queries of a causal sequence) come first and
// the q heads that share a kv head are neighbours, i.e. run at the same time on neighbouring SMs.
struct Item {
  int q0, hq, b, hkv, sp;
  int j_begin;   // first key tile of this share
  int nt[2];     // key tiles of each query tile within the share (0: nothing to do)
  int nt_max;
};

__device__ __forceinline__ Item decode_item(const Attn2Params& p, int i) {
  Item it;
  it.nt[0] = it.nt[1] = it.nt_max = 0;
  it.q0 = it.hq = it.b = it.hkv = it.sp = it.j_begin = 0;
  if (i >= p.n_items) return it;
  const int blk = fdiv(i, p.d_per_blk);
  int rem = i - blk * static_cast<int>(p.d_per_blk.d);
  const int r1 = fdiv(rem, p.d_splits);
  it.sp = rem - r1 * p.kv_splits;
  it.b = fdiv(r1, p.d_hq);
  it.hq = r1 - it.b * p.Hq;
  it.hkv = fdiv(it.hq, p.d_group);
  it.q0 = (p.n_blocks - 1 - blk) * 2 * BQ;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0t = it.q0 + t * BQ;
    int last_key = p.kv_len - 1;
    if (p.causal) last_key = min(last_key, p.past + min(q0t + BQ - 1, p.S - 1));
    it.nt[t] = (q0t < p.S) ? last_key / BKV + 1 : 0;
  }
  if (p.kv_splits > 1) {
    const int per_split = fdiv(max(it.nt[0], it.nt[1]) + p.kv_splits - 1, p.d_splits);
    it.j_begin = it.sp * per_split;
#pragma unroll
    for (int t = 0; t < 2; ++t) it.nt[t] = max(0, min(it.nt[t], it.j_begin + per_split) - it.j_begin);
  }
  it.nt_max = max(it.nt[0], it.nt[1]);
  return it;
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 1) attn_fwd2_kernel(const __grid_constant__ Attn2Params p) {
  using L = Smem2<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars + 0;    // [2] per query tile
  uint64_t* q_empty = bars + 2;   // [2] per query tile: the last S of an item has read Q
  uint64_t* k_full = bars + 4;    // [2] ring
  uint64_t* k_empty = bars + 6;
  uint64_t* v_full = bars + 8;    // [2] ring
  uint64_t* v_empty = bars + 10;
  uint64_t* s_full = bars + 12;   // [2] per query tile
  uint64_t* p_ready = bars + 14;  // [2] per query tile
  uint64_t* pv_done = bars + 16;  // [2] per query tile
  uint64_t* o_free = bars + 18;   // [2] per query tile: the output warpgroup has read O of the item that finished
  uint64_t* stat_full = bars + 20;   // [2] per query tile: the softmax warpgroup has left the rows' output factors
  uint64_t* stat_empty = bars + 22;  // [2] per query tile: the output warpgroup has read them
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
  float* stat = reinterpret_cast<float*>(smem + L::kStatOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);   // one arrival per warp of the warpgroup
      mbar_init(&pv_done[i], 1);
      mbar_init(&o_free[i], 4);
      mbar_init(&stat_full[i], 4);
      mbar_init(&stat_empty[i], 4);
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
    tma_prefetch_desc(&p.map_o);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();  // q and the appended cache rows come from the kernel before this one
  const uint32_t tmem_base = *tmem_slot;
  const AbortCtx ctx{p.err, abort_flag, p.wait_limit};
  const int wg = warp >> 2;

  if (wg == 0) {
   warpgroup_regs_release<kRegsControl>();
   if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    uint32_t ring = 0;               // K/V tiles loaded so far: stage = ring & 1, use = ring >> 1
    uint32_t q_loads[2] = {0, 0};    // Q tiles loaded so far, per query tile
    bool ok = true;
    for (int i = blockIdx.x; ok && i < p.n_items; i += gridDim.x) {
      const Item it = decode_item(p, i);
      // order: Q0, K0, Q1, V0, then K1 V1 K2 V2 ...: the first S of query tile 0 needs only Q0 and K0
      for (int step = 0; ok && step < 2 * it.nt_max + 2; ++step) {
        if (step == 0 || step == 2) {
          const int t = step >> 1;
          const uint32_t loads = t == 0 ? q_loads[0] : q_loads[1];
          if ((t == 0 ? it.nt[0] : it.nt[1]) == 0) continue;
          if (loads > 0 && !mbar_wait(&q_empty[t], (loads - 1) & 1, ctx, 400)) { ok = false; break; }
          if (lane == 0) {
            mbar_arrive_expect_tx(&q_full[t], L::kTile);
#pragma unroll
            for (int dc = 0; dc < D / 64; ++dc)
              tma_load_3d(smem + L::kQOff + t * L::kTile + dc * (BQ * 128), &p.map_q, &q_full[t], dc * 64, it.q0 + t * BQ,
                          it.b * p.Hq + it.hq);
          }
          __syncwarp();
          if (t == 0) ++q_loads[0]; else ++q_loads[1];
          continue;
        }
        // steps 1, 3, 4, 5, ...  ->  K0, V0, K1, V1, ...
        const int kv = (step == 1) ? 0 : step - 2;  // 0: K0, 1: V0, 2: K1, ...
        const int j = kv >> 1;
        if (j >= it.nt_max) break;
        const bool is_v = (kv & 1) != 0;
        const uint32_t pos = ring + static_cast<uint32_t>(j);
        const uint32_t st = pos & 1, ph = (pos >> 1) & 1;
        uint64_t* full = is_v ? &v_full[st] : &k_full[st];
        uint64_t* empty = is_v ? &v_empty[st] : &k_empty[st];
        if (!mbar_wait(empty, ph ^ 1, ctx, is_v ? 402 : 401)) { ok = false; break; }
        if (lane == 0) {
          mbar_arrive_expect_tx(full, L::kTile);
          uint8_t* dst = smem + (is_v ? L::kVOff : L::kKOff) + st * L::kTile;
#pragma unroll
          for (int dc = 0; dc < D / 64; ++dc)
            tma_load_3d(dst + dc * (BKV * 128), is_v ? &p.map_v : &p.map_k, full, dc * 64, (it.j_begin + j) * BKV,
                        it.b * p.Hkv + it.hkv);
        }
        __syncwarp();
      }
      ring += static_cast<uint32_t>(it.nt_max);
    }
   } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_s = make_idesc(IsBf16<T>::value, false, false, BQ, BKV);
    constexpr uint32_t idesc_o = make_idesc(IsBf16<T>::value, false, true, BQ, D);
    // All 32 lanes run this code converged with warp-uniform operands; one elected lane issues (see common.cuh).
    const uint32_t q_base = smem_u32(smem + L::kQOff);
    const uint32_t k_base = smem_u32(smem + L::kKOff);
    const uint32_t v_base = smem_u32(smem + L::kVOff);
    uint32_t kpos = 0, vpos = 0;      // ring positions of the next K tile an S reads / the next V tile a P V reads
    uint32_t q_uses[2] = {0, 0};      // items whose Q tile has been waited for, per query tile
    uint32_t pv_count[2] = {0, 0};    // P V products issued, per query tile (= index of the next P)
    uint32_t o_items[2] = {0, 0};     // items that have started accumulating into O, per query tile
    bool ok = true;

    auto issue_s = [&](int t) {  // S_t = Q_t K^T with the K tile at ring position kpos
      const uint64_t qd = make_smem_desc(q_base + t * L::kTile, 16, 1024);
      const uint64_t kd = make_smem_desc(k_base + (kpos & 1) * L::kTile, 16, 1024);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint64_t off = static_cast<uint64_t>(((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4);  // start-address field
        umma_ss_warp(tmem_base + t * BKV, qd + off, kd + off, idesc_s, kk > 0 ? 1u : 0u);
      }
      umma_commit_warp(&s_full[t]);
    };
    auto issue_pv = [&](int t, bool accumulate) {  // O_t (+)= P_t V, P_t read from tensor memory, V at ring position vpos
      const uint64_t vd = make_smem_desc(v_base + (vpos & 1) * L::kTile, BKV * 128, 1024);
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk)
        umma_ts_warp(tmem_base + 2 * BKV + t * D, tmem_base + t * BKV + kk * 8, vd + static_cast<uint64_t>((kk * 2048) >> 4), idesc_o,
                     (accumulate || kk > 0) ? 1u : 0u);
      umma_commit_warp(&pv_done[t]);
    };
    bool k_ready = false;
    auto need_k = [&]() -> bool {  // the K tile at kpos has landed
      if (k_ready) return true;
      if (!mbar_wait(&k_full[kpos & 1], (kpos >> 1) & 1, ctx, 407)) return false;
      tc_fence_after();
      k_ready = true;
      return true;
    };
    auto k_step_done = [&]() {  // every S that reads the K tile at kpos has been issued
      if (k_ready) {
        umma_commit_warp(&k_empty[kpos & 1]);
        ++kpos;
        k_ready = false;
      }
    };
    // first S tiles of an item (Q just loaded, first K tile of the item)
    auto start_item = [&](const Item& it) -> bool {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (it.nt[t] == 0) continue;
        if (!mbar_wait(&q_full[t], q_uses[t] & 1, ctx, 403)) return false;
        ++q_uses[t];
        if (!need_k()) return false;
        tc_fence_after();
        issue_s(t);
        if (it.nt[t] == 1) umma_commit_warp(&q_empty[t]);
      }
      k_step_done();
      return true;
    };
    auto do_pv = [&](int t, int j) -> bool {
      if (j == 0) {
        if (o_items[t] > 0 && !mbar_wait(&o_free[t], (o_items[t] - 1) & 1, ctx, 410)) return false;
        ++o_items[t];
      }
      if (!mbar_wait(&p_ready[t], pv_count[t] & 1, ctx, 406)) return false;
      tc_fence_after();
      issue_pv(t, j > 0);
      ++pv_count[t];
      return true;
    };

    Item cur = decode_item(p, blockIdx.x);
    ok = start_item(cur);
    for (int i = blockIdx.x; ok && i < p.n_items; i += gridDim.x) {
      const Item nxt = decode_item(p, i + gridDim.x);
      if (cur.nt_max == 0) ok = start_item(nxt);
      for (int j = 0; ok && j < cur.nt_max; ++j) {
        if (!mbar_wait(&v_full[vpos & 1], (vpos >> 1) & 1, ctx, 405)) { ok = false; break; }
        tc_fence_after();
        if (j + 1 < cur.nt_max) {
          // Every barrier wait and every commit costs this warp about 200 cycles, and whatever stands between the
          // arrival of P_t and the issue of S_t(j+1) is on the critical path of query tile t: the K tile is waited
          // for before P, and the V stage is released after the last S.
          if (!need_k()) { ok = false; break; }
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j < cur.nt[t] && !do_pv(t, j)) { ok = false; break; }
            if (j + 1 < cur.nt[t]) {
              issue_s(t);
              if (j + 2 == cur.nt[t]) umma_commit_warp(&q_empty[t]);  // that was the item's last read of Q_t
            }
          }
          if (!ok) break;
          umma_commit_warp(&v_empty[vpos & 1]);
          k_step_done();
        } else {  // last step of the item: both P V first, then the first S tiles of the next item
#pragma unroll
          for (int t = 0; t < 2; ++t)
            if (j < cur.nt[t] && !do_pv(t, j)) { ok = false; break; }
          if (!ok) break;
          umma_commit_warp(&v_empty[vpos & 1]);
          ok = start_item(nxt);
        }
        ++vpos;
      }
      cur = nxt;
    }
   }
  } else if (wg == 1 || wg == 2) {
    // ------------------------------------------------------------ softmax warps: a thread owns a query row
    warpgroup_regs_take<kRegsSoftmax>();
    const int t = wg - 1;           // query tile
    const int quad = warp & 3;      // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may touch
    const int r_in = quad * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tmem_s = tmem_base + t * BKV + lane_sel;
    const uint32_t tmem_o = tmem_base + 2 * BKV + t * D + lane_sel;
    uint32_t s_count = 0;   // S tiles consumed so far by this query tile, over all items
    uint32_t handed = 0;    // items whose output factors have been handed to the output warpgroup
    bool ok = true;

    for (int i = blockIdx.x; ok && i < p.n_items; i += gridDim.x) {
      int my_nt, k_first, key_limit;
      {  // only what the key loop needs stays live through it; the item is decoded again for the output addresses
        const Item it = decode_item(p, i);
        my_nt = t == 0 ? it.nt[0] : it.nt[1];
        k_first = it.j_begin * BKV;
        const int qi = it.q0 + t * BQ + r_in;
        key_limit = p.causal ? min(p.past + qi, p.kv_len - 1) : p.kv_len - 1;
      }
      float m_use = -INFINITY, l = 0.f;

      for (int j = 0; j < my_nt; ++j, ++s_count) {
        const int k0 = k_first + j * BKV;
        if (!mbar_wait(&s_full[t], s_count & 1, ctx, 408)) { ok = false; break; }
        tc_fence_after();
        uint32_t s[BKV];
#pragma unroll
        for (int c = 0; c < BKV / 32; ++c) tmem_ld_x32(tmem_s + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
        tmem_wait_ld();

        if (k0 + BKV - 1 > key_limit) {  // these columns touch the causal diagonal or the end of the keys
#pragma unroll
          for (int c = 0; c < BKV; ++c)
            if (k0 + c > key_limit) s[c] = 0xff800000u;  // -inf
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < BKV; c += 8) {  // three-input max: one instruction per two elements, four chains
          mx0 = max3(mx0, __uint_as_float(s[c]), __uint_as_float(s[c + 1]));
          mx1 = max3(mx1, __uint_as_float(s[c + 2]), __uint_as_float(s[c + 3]));
          mx2 = max3(mx2, __uint_as_float(s[c + 4]), __uint_as_float(s[c + 5]));
          mx3 = max3(mx3, __uint_as_float(s[c + 6]), __uint_as_float(s[c + 7]));
        }
        const float rowmax = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        const float m_new = fmaxf(m_use, rowmax * p.scale_log2);
        const bool grow = m_new > m_use + kRescaleThreshold;  // true on the first tile (m_use = -inf)
        float alpha = 1.f;
        if (grow) {
          alpha = fast_exp2(m_use - m_new);
          m_use = m_new;
        }
        // s_full(j) arrived => P_{j-1} V_{j-1} of this tile has completed: O may be rescaled, P may be overwritten
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          uint32_t o[32];
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            tmem_ld_x32(tmem_o + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_x32(tmem_o + c * 32, o);
          }
        }
        const float neg_mref = (m_use == -INFINITY) ? 0.f : -m_use;
        // packed fp32x2 arithmetic: one FMA and one ADD instruction per two elements; P leaves in two halves of 64 keys
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
        const float2 nm2 = make_float2(neg_mref, neg_mref);
        float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int h = 0; h < BKV / 64; ++h) {
          uint32_t pk[32];
#pragma unroll
          for (int c = 0; c < 64; c += 4) {
            const int e = h * 64 + c;
            const float2 t0 = __ffma2_rn(make_float2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), sc2, nm2);
            const float2 t1 = __ffma2_rn(make_float2(__uint_as_float(s[e + 2]), __uint_as_float(s[e + 3])), sc2, nm2);
            const float2 e0 = make_float2(fast_exp2(t0.x), fast_exp2(t0.y));
            const float2 e1 = make_float2(fast_exp2(t1.x), fast_exp2(t1.y));
            acc0 = __fadd2_rn(acc0, e0);
            acc1 = __fadd2_rn(acc1, e1);
            pk[c >> 1] = Pack2<T>::pack(e0.x, e0.y);
            pk[(c >> 1) + 1] = Pack2<T>::pack(e1.x, e1.y);
          }
          tmem_st_x32(tmem_s + h * 32, pk);  // 64 keys = 32 packed columns
        }
        l = l * alpha + ((acc0.x + acc0.y) + (acc1.x + acc1.y));
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[t]);  // arrivals on one barrier serialise: one per warp, not per thread
      }
      if (!ok) break;

      // ---- end of the item: hand the factor each row of O is to be multiplied with to the output warpgroup (which
      //      waits for the last P V itself) and go on to the next item at once
      const Item it = decode_item(p, i);
      const int qi = it.q0 + t * BQ + r_in;
      const bool row_ok = qi < p.S;
      if (my_nt > 0) {
        if (handed > 0 && !mbar_wait(&stat_empty[t], (handed - 1) & 1, ctx, 411)) { ok = false; break; }
        stat[t * BQ + r_in] = (p.kv_splits > 1) ? 1.f : ((l > 0.f) ? 1.f / l : 0.f);
        __syncwarp();
        if (lane == 0) mbar_arrive(&stat_full[t]);
        ++handed;
      }
      if (p.kv_splits > 1) {
        // this item saw only a share of the keys: its unnormalised accumulator, exponent reference and row sum are
        // left for attn_combine_kernel.  A share without keys leaves the neutral element.
        const long long prow = ((static_cast<long long>(it.sp) * p.B + it.b) * p.Hq + it.hq) * p.S + qi;
        if (row_ok) {
          p.part_ml[prow * 2] = my_nt > 0 ? m_use : -INFINITY;
          p.part_ml[prow * 2 + 1] = my_nt > 0 ? l : 0.f;
          if (my_nt == 0) {
            uint4* d = reinterpret_cast<uint4*>(p.part_o + prow * D);
#pragma unroll
            for (int e = 0; e < D / 4; ++e) d[e] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      } else if (my_nt > 0 && row_ok && p.lse2 != nullptr) {
        p.lse2[(static_cast<long long>(it.b) * p.Hq + it.hq) * p.S + qi] = m_use + log2f(l);
      }
    }
  } else if (wg == 3) {
    // ------------------------------------------------------------ output warps: a thread owns a query row of O
    warpgroup_regs_release<kRegsOutput>();
    const int quad = warp & 3;
    const int r_in = quad * 32 + lane;
    const int tid = threadIdx.x - 3 * 128;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    uint8_t* stage = smem + L::kOOff;
    uint32_t pv_total[2] = {0, 0};   // P V products of each query tile up to the end of the current item
    uint32_t taken[2] = {0, 0};      // items whose factors have been taken, per query tile
    bool store_pending = false;
    bool ok = true;
    for (int i = blockIdx.x; ok && i < p.n_items; i += gridDim.x) {
      const Item it = decode_item(p, i);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int nt = t == 0 ? it.nt[0] : it.nt[1];
        if (nt == 0) continue;
        const uint32_t total = (t == 0 ? pv_total[0] : pv_total[1]) + static_cast<uint32_t>(nt);
        const uint32_t seen = t == 0 ? taken[0] : taken[1];
        if (t == 0) { pv_total[0] = total; ++taken[0]; } else { pv_total[1] = total; ++taken[1]; }
        if (!mbar_wait(&stat_full[t], seen & 1, ctx, 412)) { ok = false; break; }
        const float f = stat[t * BQ + r_in];
        __syncwarp();
        if (lane == 0) mbar_arrive(&stat_empty[t]);
        // The last P V of the item.  When the factors arrive, the P V before it is complete (the softmax warps saw the S
        // tile that was issued behind it), so the barrier is at most one phase behind the one waited for.
        if (!mbar_wait(&pv_done[t], (total - 1) & 1, ctx, 409)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_o = tmem_base + 2 * BKV + t * D + lane_sel;
        const int q0t = it.q0 + t * BQ;
        uint32_t o[32];
        if (p.kv_splits > 1) {
          const int qi = q0t + r_in;
          const long long prow = ((static_cast<long long>(it.sp) * p.B + it.b) * p.Hq + it.hq) * p.S + qi;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            tmem_ld_x32(tmem_o + c * 32, o);
            tmem_wait_ld();
            if (c == D / 32 - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&o_free[t]);
            }
            if (qi < p.S) {
              uint4* d = reinterpret_cast<uint4*>(p.part_o + prow * D + c * 32);
#pragma unroll
              for (int e = 0; e < 8; ++e) d[e] = make_uint4(o[4 * e], o[4 * e + 1], o[4 * e + 2], o[4 * e + 3]);
            }
          }
          continue;
        }
        if (store_pending) {  // the previous tile's TMA stores have read the staging tile
          if (tid == 0) tma_store_wait_read();
          named_barrier_sync(1, 128);
        }
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          tmem_ld_x32(tmem_o + c * 32, o);
          tmem_wait_ld();
          if (c == D / 32 - 1) {  // O has left tensor memory: the next item's first P V may overwrite it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_free[t]);
          }
          // row r_in of the 64-column box c / 2, 128-byte swizzle: 16-byte chunk k of a row sits at k ^ (row & 7)
          uint8_t* row = stage + (c >> 1) * (BQ * 128) + r_in * 128;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint4 v = make_uint4(Pack2<T>::pack(__uint_as_float(o[8 * k]) * f, __uint_as_float(o[8 * k + 1]) * f),
                                       Pack2<T>::pack(__uint_as_float(o[8 * k + 2]) * f, __uint_as_float(o[8 * k + 3]) * f),
                                       Pack2<T>::pack(__uint_as_float(o[8 * k + 4]) * f, __uint_as_float(o[8 * k + 5]) * f),
                                       Pack2<T>::pack(__uint_as_float(o[8 * k + 6]) * f, __uint_as_float(o[8 * k + 7]) * f));
            *reinterpret_cast<uint4*>(row + ((((c & 1) * 4 + k) ^ (r_in & 7)) << 4)) = v;
          }
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (tid == 0) {  // rows beyond S are clipped by the tensor map
#pragma unroll
          for (int dc = 0; dc < D / 64; ++dc) tma_store_3d(&p.map_o, stage + dc * (BQ * 128), it.hq * D + dc * 64, q0t, it.b);
          tma_store_commit();
        }
        store_pending = true;
      }
    }
    if (tid == 0) tma_store_wait_all();
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
  pdl_launch_dependents();
  pdl_wait();
  const long long rows = static_cast<long long>(B) * Hq * S;
  const int lane = threadIdx.x & 31;
  for (long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; row < rows;
       row += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    // all the shares' loads are in flight together (at most 16 shares): one trip to L2, not one per share
    constexpr int kMaxSplits = 16;
    float2 ml[kMaxSplits];
    float po[kMaxSplits][V];
#pragma unroll
    for (int s = 0; s < kMaxSplits; ++s) {
      const bool on = s < splits;
      ml[s] = on ? __ldcg(reinterpret_cast<const float2*>(part_ml + (s * rows + row) * 2)) : make_float2(-INFINITY, 0.f);
      const float* ps = part_o + ((on ? s : 0) * rows + row) * D + lane * V;
#pragma unroll
      for (int i = 0; i < V; ++i) po[s][i] = on ? __ldcg(ps + i) : 0.f;
    }
    float m = -INFINITY;
#pragma unroll
    for (int s = 0; s < kMaxSplits; ++s) m = fmaxf(m, ml[s].x);
    float l = 0.f, acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
#pragma unroll
    for (int s = 0; s < kMaxSplits; ++s) {  // fixed order: deterministic
      const float w = (ml[s].x == -INFINITY) ? 0.f : fast_exp2(ml[s].x - m);
      l = fmaf(w, ml[s].y, l);
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = fmaf(w, po[s][i], acc[i]);
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
int launch_one(const Attn2Params& p, dim3 grid, int num_sms, cudaStream_t stream) {
  static bool attr_set[32] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 31]) {
    if (cudaFuncSetAttribute(attn_fwd2_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem2<D>::kTotal) != cudaSuccess)
      return TB200_ERR_CUDA;
    attr_set[dev & 31] = true;
  }
  if (launch_chained(attn_fwd2_kernel<T, D>, grid, dim3(kThreads, 1, 1), Smem2<D>::kTotal, stream, p) != cudaSuccess) return TB200_ERR_CUDA;
  if (cudaGetLastError() != cudaSuccess) return TB200_ERR_CUDA;
  if (p.kv_splits > 1) {
    const long long rows = static_cast<long long>(p.B) * p.Hq * p.S;
    long long blocks = (rows * 32 + 255) / 256;
    if (blocks > num_sms * 8) blocks = num_sms * 8;
    if (launch_chained(attn_combine_kernel<T, D>, dim3(static_cast<unsigned>(blocks), 1, 1), dim3(256, 1, 1), 0, stream, p.part_o, p.part_ml,
                       static_cast<T*>(p.o2), p.lse2, p.kv_splits, p.B, p.Hq, p.S) != cudaSuccess)
      return TB200_ERR_CUDA;
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
  {  // o2 (B, S, Hq*D): a box is 128 query rows of one head's 64 columns; rows past S are clipped per batch element
    const uint64_t dims[3] = {static_cast<uint64_t>(a.Hq) * D, static_cast<uint64_t>(a.S), static_cast<uint64_t>(a.B)};
    const uint64_t strides[2] = {static_cast<uint64_t>(a.Hq) * D * 2, static_cast<uint64_t>(a.S) * a.Hq * D * 2};
    const uint32_t box[3] = {64, BQ, 1};
    if ((status = make_tensor_map(&p.map_o, a.o2, 3, dims, strides, box)) != TB200_OK) return status;
  }
  p.n_blocks = (a.S + 2 * BQ - 1) / (2 * BQ);
  const long long items = static_cast<long long>(p.n_blocks) * p.kv_splits * a.Hq * a.B;
  if (items > 0x7fffffffLL) return TB200_ERR_INVALID;
  p.n_items = static_cast<int>(items);
  p.d_per_blk = make_fastdiv(static_cast<uint32_t>(a.B) * a.Hq * p.kv_splits);
  p.d_splits = make_fastdiv(static_cast<uint32_t>(p.kv_splits));
  p.d_hq = make_fastdiv(static_cast<uint32_t>(a.Hq));
  p.d_group = make_fastdiv(static_cast<uint32_t>(a.Hq / a.Hkv));
  const dim3 grid(static_cast<unsigned>(p.n_items < st->num_sms ? p.n_items : st->num_sms), 1, 1);  // persistent: one CTA per SM
  if (a.dtype == TB200_BF16) {
    return a.D == 128 ? launch_one<__nv_bfloat16, 128>(p, grid, st->num_sms, stream) : launch_one<__nv_bfloat16, 64>(p, grid, st->num_sms, stream);
  }
  return a.D == 128 ? launch_one<__half, 128>(p, grid, st->num_sms, stream) : launch_one<__half, 64>(p, grid, st->num_sms, stream);
}

}  // namespace tb200
