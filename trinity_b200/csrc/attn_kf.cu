// KeyFormer attention forward: the persistent two-query-tile kernel of attn2.cu with 64-key steps, two S buffers
// per query tile and a ring of noise tiles.  Kept apart from attn2.cu because the extra generality cost the kernel
// without noise 5 % (measured on the same GPU); the structure is the same:
//
// Persistent: one CTA per SM walks work items (256 queries, q head, batch element[, share of the keys]), longest
// items first.  384 threads:
//   warp 0      TMA producer: the two Q tiles of an item, then its K and V tiles of BKV keys through two-deep rings
//               that run on across items
//   warp 1      MMA issuer, in this order per key tile j:  P0_j V_j, S0_{j+1}, P1_j V_j, S1_{j+1}; in the last step of
//               an item the S_0 tiles of the NEXT item take the place of S_{j+1}
//   warp 2      TMA producer of the noise tiles (KeyFormer only); warp 3 idles
//   warps 4-7   softmax of query tile 0          warps 8-11  softmax of query tile 1
// While one softmax warpgroup works on its S tile the tensor core serves the other tile, and each SM sub-partition
// holds two softmax warps whose MUFU / FMA / TMEM latencies overlap.  K and V tiles are fetched once for 256 queries.
// Across items the pipeline does not drain: while a warpgroup normalises and stores O of item i, the Q tiles of item
// i+1 are already in shared memory and its first S tile is in tensor memory.
//
// Tensor memory (512 columns): S0 [0,128)  S1 [128,256)  O0 [256,256+D)  O1 [256+D,256+2D).
// P_j (16-bit) is written back over the first 64 columns of its own S tile and is the A operand of P_j V_j straight
// from tensor memory (no shared-memory round trip).  MMAs issued by one thread complete in issue order, so S_{j+1}
// (issued after P_j V_j) cannot overwrite P_j early, and an arrival on s_full also means the previous P V is done.
// The first P V of an item overwrites O, so it waits until the warpgroup has read the previous item's O (o_free).
//
// KeyFormer (NOISE): the same pass keeps the online log-sum-exp of (scale*s + noise)/tau per row.  That is two
// exponentials per score, so the pass is bound by the special-function unit, not by the tensor core: it runs with
// BKV = 64, which leaves room for a six-deep ring of 128 x 64 noise tiles (the noise tensor is streamed from HBM
// once, so enough of it has to be in flight).
//
// One thread owns one query row.  (Two threads per row were measured slower on B200 -- 0.418 ms against 0.353 ms on
// the Llama-3-8B B8 S2048 prefill: the row-max exchange and the register cap of a 576-thread CTA cost more than the
// extra warps hide -- and so was a variant with P staged in shared memory.)
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int BQ = 128;
constexpr int kThreads = 128 + 2 * 128;  // TMA warp, MMA warp, noise TMA warp, idle warp, softmax warps of two query tiles
constexpr int kNoiseStages = 6;
constexpr int kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;

template <int D, int BKV, bool NOISE> struct Smem2 {
  static constexpr int kQTile = BQ * D * 2;
  static constexpr int kKVTile = BKV * D * 2;
  static constexpr int kNoiseTile = BQ * BKV * 2;                 // [128 queries][128 B] swizzled; BKV = 64 with noise
  static constexpr int kKVStages = (BKV == 64 && !NOISE) ? 4 : 2;
  static constexpr int kQOff = 0;                                 // two query tiles
  static constexpr int kKOff = 2 * kQTile;                        // ring
  static constexpr int kVOff = kKOff + kKVStages * kKVTile;       // ring
  static constexpr int kNoiseOff = kVOff + kKVStages * kKVTile;   // ring (KeyFormer only)
  static constexpr int kBarOff = kNoiseOff + (NOISE ? kNoiseStages * kNoiseTile : 0);
  static constexpr int kTotal = kBarOff + 512 + 1024;
  static_assert(!NOISE || BKV == 64, "a noise tile is one 128-byte-wide swizzled block");
};

// Division by a value fixed for the launch as a multiply and a shift (item decoding; valid for n < 2^31).
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
  CUtensorMap map_q, map_k, map_v;
  CUtensorMap map_noise;       // dims {past+S, S, B*Hq}, box {64, 128, 1} (KeyFormer)
  int bkv;                     // keys per step of the kernel this launch uses
  float inv_tau;
  float* lse2_perturbed;       // (B,Hq,S): log2-domain log-sum-exp of (scale*s + noise)/tau
  int B, S, Hq, Hkv, past, kv_len, causal;
  int n_blocks;      // blocks of 256 queries
  int n_items;       // n_blocks * kv_splits * Hq * B
  FastDiv d_per_blk, d_hq, d_group;  // B * Hq, Hq, Hq / Hkv
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
  const int blk = fdiv(i, p.d_per_blk);  // the key range is never split here (kv_splits = 1)
  const int rem = i - blk * static_cast<int>(p.d_per_blk.d);
  it.sp = 0;
  it.b = fdiv(rem, p.d_hq);
  it.hq = rem - it.b * p.Hq;
  it.hkv = fdiv(it.hq, p.d_group);
  it.q0 = (p.n_blocks - 1 - blk) * 2 * BQ;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0t = it.q0 + t * BQ;
    int last_key = p.kv_len - 1;
    if (p.causal) last_key = min(last_key, p.past + min(q0t + BQ - 1, p.S - 1));
    it.nt[t] = (q0t < p.S) ? last_key / p.bkv + 1 : 0;
  }
  it.j_begin = 0;
  it.nt_max = max(it.nt[0], it.nt[1]);
  return it;
}

template <typename T, int D, int BKV, bool NOISE>
__global__ void __launch_bounds__(kThreads, 1) attn_fwd2_kernel(const __grid_constant__ Attn2Params p) {
  using L = Smem2<D, BKV, NOISE>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  constexpr int KVS = L::kKVStages;
  // With 64-key steps an S tile takes 64 tensor-memory columns and every query tile gets two of them: S_{j+1} is
  // computed while the warpgroup still works on S_j / P_j, so the warpgroup never waits for the tensor core.
  constexpr int NB = (BKV == 64) ? 2 : 1;
  uint64_t* q_full = bars + 0;    // [2] per query tile
  uint64_t* q_empty = bars + 2;   // [2] per query tile: the last S of an item has read Q
  uint64_t* k_full = bars + 4;    // [KVS] ring
  uint64_t* k_empty = bars + 8;
  uint64_t* v_full = bars + 12;   // [KVS] ring
  uint64_t* v_empty = bars + 16;
  uint64_t* s_full = bars + 20;   // [2][2] per query tile and S buffer
  uint64_t* p_ready = bars + 24;  // [2][2] per query tile and S buffer
  uint64_t* pv_done = bars + 28;  // [2] per query tile
  uint64_t* o_free = bars + 30;   // [2] per query tile: the warpgroup has read O of the item it finished
  uint64_t* n_full = bars + 32;   // [kNoiseStages]
  uint64_t* n_empty = bars + 32 + kNoiseStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32 + 2 * kNoiseStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // Noise tiles whose load has been issued.  The two warpgroups take noise tiles from one ring and run out of step;
  // a warpgroup first waits here until its tile's barrier phase has been armed, so that it cannot mistake the
  // completed phase of the stage's previous tile for its own.
  volatile int* noise_issued = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&pv_done[i], 1);
      mbar_init(&o_free[i], 4);
    }
    for (int i = 0; i < KVS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);   // one arrival per warp of the warpgroup
    }
    for (int i = 0; i < kNoiseStages; ++i) {
      mbar_init(&n_full[i], 1);
      mbar_init(&n_empty[i], 4);
    }
    *abort_flag = 0;
    *noise_issued = 0;
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
  const AbortCtx ctx{p.err, abort_flag, p.wait_limit};
  // tensor-memory column of S buffer b of query tile t; O_t follows the four (or two) S tiles at column 256
  auto s_col = [](int t, int b) -> uint32_t { return static_cast<uint32_t>(NB == 2 ? (t * 2 + b) * 64 : t * 128); };
  constexpr uint32_t kOCol = 256;

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
            mbar_arrive_expect_tx(&q_full[t], L::kQTile);
#pragma unroll
            for (int dc = 0; dc < D / 64; ++dc)
              tma_load_3d(smem + L::kQOff + t * L::kQTile + dc * (BQ * 128), &p.map_q, &q_full[t], dc * 64, it.q0 + t * BQ,
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
        const uint32_t st = pos % KVS, ph = (pos / KVS) & 1;
        uint64_t* full = is_v ? &v_full[st] : &k_full[st];
        uint64_t* empty = is_v ? &v_empty[st] : &k_empty[st];
        if (!mbar_wait(empty, ph ^ 1, ctx, is_v ? 402 : 401)) { ok = false; break; }
        if (lane == 0) {
          mbar_arrive_expect_tx(full, L::kKVTile);
          uint8_t* dst = smem + (is_v ? L::kVOff : L::kKOff) + st * L::kKVTile;
#pragma unroll
          for (int dc = 0; dc < D / 64; ++dc)
            tma_load_3d(dst + dc * (BKV * 128), is_v ? &p.map_v : &p.map_k, full, dc * 64, (it.j_begin + j) * BKV,
                        it.b * p.Hkv + it.hkv);
        }
        __syncwarp();
      }
      ring += static_cast<uint32_t>(it.nt_max);
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ TMA producer of the noise tiles
    // ring order: per item, per key tile j, query tile 0 then 1 (where the tile still has keys at j)
    if (NOISE) {
      uint32_t n = 0;
      bool ok = true;
      for (int i = blockIdx.x; ok && i < p.n_items; i += gridDim.x) {
        const Item it = decode_item(p, i);
        for (int j = 0; ok && j < it.nt_max; ++j) {
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j >= (t == 0 ? it.nt[0] : it.nt[1])) continue;
            const uint32_t st = n % kNoiseStages;
            if (!mbar_wait(&n_empty[st], ((n / kNoiseStages) & 1) ^ 1, ctx, 412)) { ok = false; break; }
            if (lane == 0) {
              mbar_arrive_expect_tx(&n_full[st], L::kNoiseTile);
              tma_load_3d(smem + L::kNoiseOff + st * L::kNoiseTile, &p.map_noise, &n_full[st], (it.j_begin + j) * BKV, it.q0 + t * BQ,
                          it.b * p.Hq + it.hq);
              __threadfence_block();  // the armed barrier phase is visible before the count
              *noise_issued = static_cast<int>(n + 1);
            }
            __syncwarp();
            ++n;
          }
        }
      }
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
    uint32_t s_count[2] = {0, 0};     // S tiles issued, per query tile
    uint32_t o_items[2] = {0, 0};     // items that have started accumulating into O, per query tile
    bool ok = true;

    auto issue_s = [&](int t) {  // S_t = Q_t K^T with the K tile at ring position kpos
      const uint64_t qd = make_smem_desc(q_base + t * L::kQTile, 16, 1024);
      const uint64_t kd = make_smem_desc(k_base + (kpos % KVS) * L::kKVTile, 16, 1024);
      const int b = static_cast<int>(s_count[t] % NB);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {  // start-address field: 64-column chunk (rows x 128 B each), 32 B per 16 columns
        const uint64_t qoff = static_cast<uint64_t>(((kk >> 2) * (BQ * 128) + (kk & 3) * 32) >> 4);
        const uint64_t koff = static_cast<uint64_t>(((kk >> 2) * (BKV * 128) + (kk & 3) * 32) >> 4);
        umma_ss_warp(tmem_base + s_col(t, b), qd + qoff, kd + koff, idesc_s, kk > 0 ? 1u : 0u);
      }
      umma_commit_warp(&s_full[t * 2 + b]);
      ++s_count[t];
    };
    auto issue_pv = [&](int t, bool accumulate) {  // O_t (+)= P_t V, P_t read from tensor memory, V at ring position vpos
      const uint64_t vd = make_smem_desc(v_base + (vpos % KVS) * L::kKVTile, BKV * 128, 1024);
      const uint32_t p_col = s_col(t, static_cast<int>(pv_count[t] % NB));
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk)
        umma_ts_warp(tmem_base + kOCol + t * D, tmem_base + p_col + kk * 8, vd + static_cast<uint64_t>((kk * 2048) >> 4), idesc_o,
                     (accumulate || kk > 0) ? 1u : 0u);
      umma_commit_warp(&pv_done[t]);
    };
    bool k_ready = false;
    auto need_k = [&]() -> bool {  // the K tile at kpos has landed
      if (k_ready) return true;
      if (!mbar_wait(&k_full[kpos % KVS], (kpos / KVS) & 1, ctx, 407)) return false;
      tc_fence_after();
      k_ready = true;
      return true;
    };
    auto k_step_done = [&]() {  // every S that reads the K tile at kpos has been issued
      if (k_ready) {
        umma_commit_warp(&k_empty[kpos % KVS]);
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
      if (!mbar_wait(&p_ready[t * 2 + pv_count[t] % NB], (pv_count[t] / NB) & 1, ctx, 406)) return false;
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
        if (NB == 2 && j + 1 < cur.nt_max) {  // two S buffers: the next S tiles go first, they do not wait for P
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j + 1 < cur.nt[t]) {
              if (!need_k()) { ok = false; break; }
              issue_s(t);
              if (j + 2 == cur.nt[t]) umma_commit_warp(&q_empty[t]);  // that was the item's last read of Q_t
            }
          }
          if (!ok) break;
          k_step_done();
        }
        if (!mbar_wait(&v_full[vpos % KVS], (vpos / KVS) & 1, ctx, 405)) { ok = false; break; }
        tc_fence_after();
        if (NB == 2 && j + 1 < cur.nt_max) {
#pragma unroll
          for (int t = 0; t < 2; ++t)
            if (j < cur.nt[t] && !do_pv(t, j)) { ok = false; break; }
          if (!ok) break;
          umma_commit_warp(&v_empty[vpos % KVS]);
        } else if (j + 1 < cur.nt_max) {
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j < cur.nt[t] && !do_pv(t, j)) { ok = false; break; }
            if (t == 1) umma_commit_warp(&v_empty[vpos % KVS]);
            if (j + 1 < cur.nt[t]) {
              if (!need_k()) { ok = false; break; }
              issue_s(t);
              if (j + 2 == cur.nt[t]) umma_commit_warp(&q_empty[t]);  // that was the item's last read of Q_t
            }
          }
          if (!ok) break;
          k_step_done();
        } else {  // last step of the item: both P V first, then the first S tiles of the next item
#pragma unroll
          for (int t = 0; t < 2; ++t)
            if (j < cur.nt[t] && !do_pv(t, j)) { ok = false; break; }
          if (!ok) break;
          umma_commit_warp(&v_empty[vpos % KVS]);
          ok = start_item(nxt);
        }
        ++vpos;
      }
      cur = nxt;
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ softmax warps: a thread owns a query row
    const int t = (warp - 4) >> 2;  // query tile
    const int quad = warp & 3;      // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may touch
    const int r_in = quad * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tmem_o = tmem_base + kOCol + t * D + lane_sel;
    uint32_t s_count = 0;  // S tiles consumed so far by this query tile, over all items
    uint32_t n_base = 0;   // noise tiles of all earlier items (both query tiles)
    const float st_scale = p.scale_log2 * p.inv_tau;  // (scale*s + noise)/tau in the log2 domain
    const float nscale = kLog2e * p.inv_tau;
    bool ok = true;

    for (int i = blockIdx.x; ok && i < p.n_items; i += gridDim.x) {
      int my_nt, k_first, key_limit, n_min = 0;
      uint32_t n_item = 0;
      {  // only what the key loop needs stays live through it; the item is decoded again for the output addresses
        const Item it = decode_item(p, i);
        my_nt = t == 0 ? it.nt[0] : it.nt[1];
        n_min = min(it.nt[0], it.nt[1]);
        n_item = static_cast<uint32_t>(it.nt[0] + it.nt[1]);
        k_first = it.j_begin * BKV;
        const int qi = it.q0 + t * BQ + r_in;
        key_limit = p.causal ? min(p.past + qi, p.kv_len - 1) : p.kv_len - 1;
      }
      float m_use = -INFINITY, l = 0.f;
      float mt = -INFINITY, lt = 0.f;  // KeyFormer statistic

      for (int j = 0; j < my_nt; ++j, ++s_count) {
        const int k0 = k_first + j * BKV;
        const int sb = static_cast<int>(s_count % NB);
        const uint32_t tmem_s = tmem_base + s_col(t, sb) + lane_sel;
        if (!mbar_wait(&s_full[t * 2 + sb], (s_count / NB) & 1, ctx, 408)) { ok = false; break; }
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
        if (NOISE) {
          // log-sum-exp of x = (scale*s + noise)/tau in the log2 domain in one sweep over the noise row.  The exponent
          // reference mt only has to keep exp2(x - mt) inside fp32 range: it starts at the noise-free maximum of the
          // row's first tile and is moved, after a sweep, when the row's maximum ran more than 2^60 ahead of it.
          const uint32_t pos = n_base + static_cast<uint32_t>(j < n_min ? 2 * j + t : 2 * n_min + (j - n_min));
          const uint32_t stg = pos % kNoiseStages;
          bool armed = *noise_issued > static_cast<int>(pos);
          if (!armed) {
            const long long t0 = clock64();
            while (!(armed = *noise_issued > static_cast<int>(pos))) {
              if (*ctx.flag) break;
              if (clock64() - t0 > ctx.limit) {
                *ctx.flag = 1;
                atomicCAS(ctx.gerr, 0, 413);
                break;
              }
            }
          }
          if (!armed) { ok = false; break; }
          __threadfence_block();
          if (!mbar_wait(&n_full[stg], (pos / kNoiseStages) & 1, ctx, 414)) { ok = false; break; }
          // row r_in of the swizzled tile: 16-byte unit u lands at u ^ (row & 7)
          const uint8_t* n_row = smem + L::kNoiseOff + stg * L::kNoiseTile + r_in * 128;
          if (mt == -INFINITY && rowmax > -INFINITY) mt = rowmax * st_scale;
          const float neg_ref = (mt == -INFINITY) ? 0.f : -mt;
          const float2 ss2 = make_float2(st_scale, st_scale), ns2 = make_float2(nscale, nscale), nr2 = make_float2(neg_ref, neg_ref);
          float tmax0 = -INFINITY, tmax1 = -INFINITY;
          float2 ta0 = make_float2(0.f, 0.f), ta1 = make_float2(0.f, 0.f);
#pragma unroll
          for (int u = 0; u < BKV / 8; ++u) {
            const uint4 q4 = *reinterpret_cast<const uint4*>(n_row + ((u ^ (r_in & 7)) << 4));
            const uint32_t w[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int c = u * 8 + e * 2;
              const float2 x = __ffma2_rn(Pack2<T>::unpack(w[e]), ns2,
                                          __ffma2_rn(make_float2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), ss2, nr2));  // -inf stays -inf
              if (e & 1) tmax1 = max3(tmax1, x.x, x.y); else tmax0 = max3(tmax0, x.x, x.y);
              const float2 ex = make_float2(fast_exp2(x.x), fast_exp2(x.y));
              if (e & 1) ta1 = __fadd2_rn(ta1, ex); else ta0 = __fadd2_rn(ta0, ex);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&n_empty[stg]);  // the noise row is in registers
          lt += (ta0.x + ta0.y) + (ta1.x + ta1.y);
          const float tmax = fmaxf(tmax0, tmax1);
          if (tmax > 60.f) {  // move the reference up to this row maximum
            lt *= fast_exp2(-tmax);
            mt += tmax;
          }
        }
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
        for (int c = 0; c < BKV; c += 4) {
          const float2 t0 = __ffma2_rn(make_float2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), sc2, nm2);
          const float2 t1 = __ffma2_rn(make_float2(__uint_as_float(s[c + 2]), __uint_as_float(s[c + 3])), sc2, nm2);
          const float2 e0 = make_float2(fast_exp2(t0.x), fast_exp2(t0.y));
          const float2 e1 = make_float2(fast_exp2(t1.x), fast_exp2(t1.y));
          acc0 = __fadd2_rn(acc0, e0);
          acc1 = __fadd2_rn(acc1, e1);
          pk[c >> 1] = Pack2<T>::pack(e0.x, e0.y);
          pk[(c >> 1) + 1] = Pack2<T>::pack(e1.x, e1.y);
        }
        l = l * alpha + ((acc0.x + acc0.y) + (acc1.x + acc1.y));

        // O may be rescaled once P_{j-1} V_{j-1} of this tile has completed.  With one S buffer the arrival of S_j says
        // so; with two, S_j was issued before that product, and its barrier is waited for at every step (by now the
        // product is long done) so that the warpgroup never trails the barrier by more than one phase.
        if (NB == 2 && j > 0 && !mbar_wait(&pv_done[t], (s_count - 1) & 1, ctx, 415)) { ok = false; break; }
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          tc_fence_after();
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
#pragma unroll
        for (int c = 0; c < BKV / 64; ++c)  // 64 keys = 32 packed columns per store
          tmem_st_x32(tmem_s + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[c * 32]));
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[t * 2 + sb]);  // arrivals on one barrier serialise: one per warp, not per thread
      }
      if (!ok) break;

      // ---- end of the item: O leaves tensor memory first (which lets the next item's P V start), then goes out
      const bool have = my_nt > 0 && mbar_wait(&pv_done[t], (s_count - 1) & 1, ctx, 409);
      if (my_nt > 0 && !have) { ok = false; break; }
      const Item it = decode_item(p, i);
      const int qi = it.q0 + t * BQ + r_in;
      const bool row_ok = qi < p.S;
      if (p.kv_splits > 1) {
        // this item saw only a share of the keys: leave the unnormalised accumulator, its exponent reference and its
        // row sum; attn_combine_kernel merges the shares.  A share without keys leaves the neutral element.
        const long long prow = ((static_cast<long long>(it.sp) * p.B + it.b) * p.Hq + it.hq) * p.S + qi;
        if (have) tc_fence_after();
        uint32_t o[32];
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          if (have) {  // uniform over the warp
            tmem_ld_x32(tmem_o + c * 32, o);
            tmem_wait_ld();
            if (c == D / 32 - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&o_free[t]);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = 0u;
          }
          if (row_ok) {
            uint4* d = reinterpret_cast<uint4*>(p.part_o + prow * D + c * 32);
#pragma unroll
            for (int e = 0; e < 8; ++e) d[e] = make_uint4(o[4 * e], o[4 * e + 1], o[4 * e + 2], o[4 * e + 3]);
          }
        }
        if (row_ok) {
          p.part_ml[prow * 2] = have ? m_use : -INFINITY;
          p.part_ml[prow * 2 + 1] = have ? l : 0.f;
        }
      } else if (have) {
        tc_fence_after();
        const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
        uint32_t packed[D / 2];
        uint32_t o[32];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          tmem_ld_x32(tmem_o + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 16; ++e)
            packed[c * 16 + e] = Pack2<T>::pack(__uint_as_float(o[2 * e]) * inv_l, __uint_as_float(o[2 * e + 1]) * inv_l);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_free[t]);
        if (row_ok) {
          T* orow = static_cast<T*>(p.o2) + ((static_cast<long long>(it.b) * p.S + qi) * p.Hq + it.hq) * D;
          uint4* d = reinterpret_cast<uint4*>(orow);
#pragma unroll
          for (int e = 0; e < D / 8; ++e) d[e] = make_uint4(packed[4 * e], packed[4 * e + 1], packed[4 * e + 2], packed[4 * e + 3]);
          const long long ridx = (static_cast<long long>(it.b) * p.Hq + it.hq) * p.S + qi;
          if (p.lse2 != nullptr) p.lse2[ridx] = m_use + log2f(l);
          if (NOISE && p.lse2_perturbed != nullptr) p.lse2_perturbed[ridx] = mt + log2f(lt);
        }
      }
      n_base += n_item;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, int D, int BKV, bool NOISE>
int launch_variant(const Attn2Params& p, dim3 grid, cudaStream_t stream) {
  using L = Smem2<D, BKV, NOISE>;
  static bool attr_set[32] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 31]) {
    if (cudaFuncSetAttribute(attn_fwd2_kernel<T, D, BKV, NOISE>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess)
      return TB200_ERR_CUDA;
    attr_set[dev & 31] = true;
  }
  attn_fwd2_kernel<T, D, BKV, NOISE><<<grid, kThreads, L::kTotal, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

}  // namespace

// Same contract as launch_attn_fwd; arguments are validated by the caller.  The rows of the noise tensor must be
// 16-byte aligned (kv_len a multiple of 8); the key range is never split.
int launch_attn_fwd_keyformer(const AttnLaunch& a, cudaStream_t stream) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  Attn2Params p;
  memset(&p, 0, sizeof(p));
  p.B = a.B; p.S = a.S; p.Hq = a.Hq; p.Hkv = a.Hkv; p.past = a.past; p.kv_len = a.past + a.S; p.causal = a.causal;
  p.scale_log2 = a.sm_scale * kLog2e;
  p.o2 = a.o2;
  p.lse2 = a.lse2;
  if (a.noise == nullptr) return TB200_ERR_INVALID;
  // 64-key steps with two S buffers were also measured without noise: slower (B8 S2048 0.418 against 0.382 ms,
  // S4096 1.38 against 1.18 ms) -- an S tile of 64 columns re-reads Q from shared memory twice as often.
  p.bkv = 64;
  p.inv_tau = 1.f / a.tau;
  p.lse2_perturbed = a.lse2_perturbed;
  p.kv_splits = 1;
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
    const uint32_t box[3] = {64, static_cast<uint32_t>(p.bkv), 1};
    if ((status = make_tensor_map(&p.map_k, a.k_cache, 3, dims, strides, box)) != TB200_OK) return status;
    if ((status = make_tensor_map(&p.map_v, a.v_cache, 3, dims, strides, box)) != TB200_OK) return status;
  }
  {
    if ((p.kv_len & 7) != 0) return TB200_ERR_INVALID;
    const uint64_t dims[3] = {static_cast<uint64_t>(p.kv_len), static_cast<uint64_t>(a.S), static_cast<uint64_t>(a.B) * a.Hq};
    const uint64_t strides[2] = {static_cast<uint64_t>(p.kv_len) * 2, static_cast<uint64_t>(a.S) * p.kv_len * 2};
    const uint32_t box[3] = {64, BQ, 1};
    if ((status = make_tensor_map(&p.map_noise, a.noise, 3, dims, strides, box)) != TB200_OK) return status;
  }
  p.n_blocks = (a.S + 2 * BQ - 1) / (2 * BQ);
  const long long items = static_cast<long long>(p.n_blocks) * p.kv_splits * a.Hq * a.B;
  if (items > 0x7fffffffLL) return TB200_ERR_INVALID;
  p.n_items = static_cast<int>(items);
  p.d_per_blk = make_fastdiv(static_cast<uint32_t>(a.B) * a.Hq);
  p.d_hq = make_fastdiv(static_cast<uint32_t>(a.Hq));
  p.d_group = make_fastdiv(static_cast<uint32_t>(a.Hq / a.Hkv));
  const dim3 grid(static_cast<unsigned>(p.n_items < st->num_sms ? p.n_items : st->num_sms), 1, 1);  // persistent: one CTA per SM
  if (a.dtype == TB200_BF16) {
    return a.D == 128 ? launch_variant<__nv_bfloat16, 128, 64, true>(p, grid, stream) : launch_variant<__nv_bfloat16, 64, 64, true>(p, grid, stream);
  }
  return a.D == 128 ? launch_variant<__half, 128, 64, true>(p, grid, stream) : launch_variant<__half, 64, 64, true>(p, grid, stream);
}

}  // namespace tb200
