// Per-key score reductions of KeyFormer / RoCo: a key-stationary second pass over the attention
// probabilities.  For key j of head (b,h):
//     sum_p[j]  = sum_i p[i,j]          sum_p2[j] = sum_i p[i,j]^2          (RoCo)
//     sum_pt[j] = sum_i softmax_j((scale*s + noise)/tau)[i,j]               (KeyFormer)
// with p[i,j] = exp2(scale_log2 * s[i,j] - lse2[i]) from the row statistics the forward pass left behind.
//
// A work item is a (128-key tile, q head, batch element).  The scores are recomputed TRANSPOSED on the tensor
// core, S^T = K_tile Q_i^T, so that a TMEM lane is a key and its columns are the queries: the sum over
// queries is then a thread-local loop -- no atomics, run-to-run identical.  A CTA walks items (persistent, snake
// order over the CTAs; one CTA per item for RoCo at S > 2048, where the hardware's own scheduling balances best):
//   warp 0      TMA: the K tile of an item, then the Q tiles that can see it (ring of two to four tiles that runs on
//               across items)
//   warp 1      MMA: S^T into 128-column TMEM buffers (one per group for RoCo, two for KeyFormer)
//   warp 2      TMA (KeyFormer): the noise tiles through a ring of their own, three deep -- the pass streams the
//               noise tensor, and its waits must not hold up Q.  (Asking for tiles into L2 ahead of the ring was
//               measured to hurt: 0.39 / 0.73 / 1.40 ms without against 0.43 / 0.82 / 1.47 ms with 8 tiles of lead.)
//   warps 4-..  reduction, in two groups that take alternate query tiles.  The groups run out of step, so while
//               one waits for its next S^T tile, copies row statistics or loads from tensor memory, the other
//               keeps the special-function unit busy (with all warps in step those phases were measured to cost
//               as much as the exponentials).
//               RoCo: two groups of four warps, thread = key, and TWO CTAs per SM (384 threads, 104 KB of shared
//               memory, 256 tensor-memory columns each).
//               KeyFormer: two groups of eight warps, thread = (key, half of the tile's queries), one CTA per SM:
//               the noise ring takes the shared memory, and a group holds a noise stage while it works on a
//               tile, so with only three stages the tile has to be finished quickly.
//               The partial sums of an item are added in a fixed order by four of the warps, one item late (by
//               then they are complete: nobody waits for the slowest warp of an item).
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int BK_ = 128;  // keys per CTA
constexpr int BQ_ = 128;  // queries per step
constexpr int G = 2;  // reducer groups
template <bool NOISE> struct ScoreCfg {
  static constexpr int kReducerWarps = NOISE ? 16 : 8;
  static constexpr int kThreads = 128 + 32 * kReducerWarps;  // warps 0..3: K/Q producer, MMA issuer, noise producer, idle
  static constexpr int kCtasPerSm = NOISE ? 1 : 2;
  static constexpr int kGroupWarps = kReducerWarps / G;
  static constexpr int kParts = kGroupWarps / 4;      // warps of a group that share a quarter of the keys and split the queries
  static constexpr int kChunks = 4 / kParts;          // 32-query chunks each warp sums per tile
  static constexpr int kSBuffers = NOISE ? 4 : 2;     // S^T buffers in tensor memory
  static constexpr int kTmemCols = kSBuffers * 128;
  static constexpr int kLseBuffers = 3 * kSBuffers;
};
constexpr float kLog2e = 1.4426950408889634f;

template <int D, bool NOISE> struct ScoreSmem {
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kNoiseBytes = 128 * 128 * 2;              // [2 chunks of 64 keys][128 queries][128 B], swizzled
  static constexpr int kNoiseStages = 3;                         // what fits beside K and the Q ring at D = 128
  static constexpr int kQStages = (D == 128) ? 2 : 4;
  static constexpr int kKOff = 0;
  static constexpr int kQOff = kTileBytes;
  static constexpr int kNoiseOff = kQOff + kQStages * kTileBytes;  // ring (KeyFormer only)
  static constexpr int kLseOff = kNoiseOff + (NOISE ? kNoiseStages * kNoiseBytes : 0);  // [8 buffers][2 statistics][128] fp32
  static constexpr int kRedOff = kLseOff + ScoreCfg<NOISE>::kLseBuffers * 2 * 128 * 4;  // [3 sums][4 partial sums][128 keys] fp32
  static constexpr int kRedSums = NOISE ? 1 : 2;                 // KeyFormer: sum of p~; RoCo: sums of p and p^2
  static constexpr int kRedSlots = G * ScoreCfg<NOISE>::kParts;  // partial sums per key
  static constexpr int kRedItem = kRedSums * kRedSlots * 128;    // floats per item
  static constexpr int kBarOff = kRedOff + 2 * kRedItem * 4;     // two items' partial sums
  static constexpr int kTotal = kBarOff + 512 + 1024;
  static_assert(kTotal <= 232448 / ScoreCfg<NOISE>::kCtasPerSm - 1024 * (ScoreCfg<NOISE>::kCtasPerSm - 1), "shared memory of an SM");
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

struct ScoreParams {
  CUtensorMap map_q;
  CUtensorMap map_k;
  CUtensorMap map_noise;  // dims {past+S, S, B*Hq}; valid when noise_tma
  int noise_tma;
  int B, S, Hq, Hkv, past, kv_len, causal;
  int q_tiles;            // ceil(S / 128)
  int n_items;            // key tiles * Hq * B
  FastDiv d_hb, d_hq, d_group;  // Hq * B, Hq, Hq / Hkv
  float scale_log2, inv_tau;
  const float* lse2;
  const float* lse2t;
  const void* noise;
  float* sum_p;
  float* sum_p2;
  float* sum_pt;
  int* err;
  long long wait_limit;  // cycles a bounded wait may last (tb200_set_wait_limit_cycles)
};

// One unit of work: a tile of 128 keys of one (q head, batch element) and the query tiles that can see it.  Items are
// numbered with the key tiles in ascending order, i.e. under a causal mask the longest first.
struct ScoreItem {
  int k0, hq, b, hkv, first_tile, nt;
};
__device__ __forceinline__ ScoreItem decode_score_item(const ScoreParams& p, int i) {
  ScoreItem it;
  it.k0 = it.hq = it.b = it.hkv = it.first_tile = it.nt = 0;
  if (i >= p.n_items) return it;
  const int kt = fdiv(i, p.d_hb);
  const int rem = i - kt * static_cast<int>(p.d_hb.d);
  it.b = fdiv(rem, p.d_hq);
  it.hq = rem - it.b * p.Hq;
  it.hkv = fdiv(it.hq, p.d_group);
  it.k0 = kt * BK_;
  // first query tile that can see any key of this tile: query i sees key j iff j <= past + i
  if (p.causal && it.k0 > p.past) it.first_tile = (it.k0 - p.past) / BQ_;
  it.nt = p.q_tiles - it.first_tile;
  return it;
}

// The items a CTA takes: in round r the CTAs take items [r G, (r+1) G), forwards in even rounds and backwards in odd
// ones.  Items are sorted longest first, so plain round-robin would hand CTA 0 the longest item of every round; the
// snake order keeps the CTAs' sums within about 1 % of each other.
__device__ __forceinline__ int score_item_of_round(const ScoreParams& p, int round) {
  const int n_ctas = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
  const int i = round * n_ctas + ((round & 1) ? n_ctas - 1 - c : c);  // n_items < 2^30: no overflow
  return min(i, p.n_items);                                           // n_items: nothing left for this CTA
}

// Persistent: a CTA walks items; the Q ring, the S^T buffers, the noise ring and the statistics buffers are indexed by
// a count of query tiles that runs on across items, so that nothing drains between items except the K tile (one
// buffer: the next item's keys are fetched when the last S^T of the current item has been computed, while the reducers
// are still a tile or two behind).
template <typename T, int D, bool NOISE>
__global__ void __launch_bounds__(ScoreCfg<NOISE>::kThreads, ScoreCfg<NOISE>::kCtasPerSm)
score_kernel(const __grid_constant__ ScoreParams p) {
  using L = ScoreSmem<D, NOISE>;
  using C = ScoreCfg<NOISE>;
  constexpr int kGroupWarps = C::kGroupWarps, kParts = C::kParts, kChunks = C::kChunks;
  constexpr int SB = C::kSBuffers, LB = C::kLseBuffers;
  constexpr int kNoiseStages = L::kNoiseStages;
  constexpr int QS = L::kQStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* k_full = bars + 0;
  uint64_t* q_full = bars + 1;   // [QS]
  uint64_t* q_empty = bars + 5;  // [QS]
  uint64_t* s_full = bars + 9;   // [4]
  uint64_t* s_empty = bars + 13; // [4]
  uint64_t* n_full = bars + 17;  // [kNoiseStages] noise tiles
  uint64_t* n_empty = bars + 17 + kNoiseStages;
  uint64_t* lse_ready = bars + 17 + 2 * kNoiseStages;  // [LB] the row statistics of a query tile are staged
  uint64_t* red_done = lse_ready + 12;                // [2] every reducer warp has published its partial sums of an item
  uint64_t* red_free = red_done + 2;                  // [2] the partial sums of an item have been added up
  uint64_t* k_free = red_free + 2;                    // the MMAs of an item have read the K tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(k_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // Noise tiles whose load has been issued.  The reducer groups run out of step and a ring stage serves tiles of
  // different groups in turn, so a group could reach the stage's barrier a whole phase early and mistake the
  // previous tile's completed phase for its own; it first waits here until its tile's phase has been armed.
  volatile int* noise_issued = abort_flag + 1;
  float* lse_s = reinterpret_cast<float*>(smem + L::kLseOff);
  float* red_s = reinterpret_cast<float*>(smem + L::kRedOff);  // [2 items][sums][slots][128 keys]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(k_full, 1);
    mbar_init(k_free, 1);
    for (int i = 0; i < QS; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < SB; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], kGroupWarps);  // one arrival per warp of the group that owns the tile
    }
    for (int i = 0; i < kNoiseStages; ++i) {
      mbar_init(&n_full[i], 1);
      mbar_init(&n_empty[i], kGroupWarps);
    }
    for (int i = 0; i < LB; ++i) mbar_init(&lse_ready[i], kGroupWarps);  // the warps of the owning group
    for (int i = 0; i < 2; ++i) {
      mbar_init(&red_done[i], C::kReducerWarps);
      mbar_init(&red_free[i], 4);  // the four warps that add the partial sums up
    }
    *abort_flag = 0;
    *noise_issued = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&p.map_q);
    tma_prefetch_desc(&p.map_k);
    if (NOISE) tma_prefetch_desc(&p.map_noise);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const AbortCtx ctx{p.err, abort_flag, p.wait_limit};

  if (warp == 0) {
    // ------------------------------------------------------------ TMA: K tile of each item, Q tiles through the ring
    uint32_t n = 0, items = 0;
    bool ok = true;
    for (int round = 0; ok; ++round, ++items) {
      const int i = score_item_of_round(p, round);
      if (i >= p.n_items) break;
      const ScoreItem it = decode_score_item(p, i);
      if (items > 0 && !mbar_wait(k_free, (items - 1) & 1, ctx, 311)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(k_full, L::kTileBytes);
#pragma unroll
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_3d(smem + L::kKOff + dc * (128 * 128), &p.map_k, k_full, dc * 64, it.k0, it.b * p.Hkv + it.hkv);
      }
      __syncwarp();
      for (int t = 0; t < it.nt; ++t, ++n) {
        const uint32_t st = n % QS;
        if (!mbar_wait(&q_empty[st], ((n / QS) & 1) ^ 1, ctx, 301)) { ok = false; break; }
        if (lane == 0) {
          mbar_arrive_expect_tx(&q_full[st], L::kTileBytes);
#pragma unroll
          for (int dc = 0; dc < D / 64; ++dc)
            tma_load_3d(smem + L::kQOff + st * L::kTileBytes + dc * (128 * 128), &p.map_q, &q_full[st], dc * 64,
                        (it.first_tile + t) * BQ_, it.b * p.Hq + it.hq);
        }
        __syncwarp();
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ TMA: noise tiles (KeyFormer), a ring of their own
    if (NOISE && p.noise_tma) {
      uint32_t n = 0;
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int i = score_item_of_round(p, round);
        if (i >= p.n_items) break;
        const ScoreItem it = decode_score_item(p, i);
        for (int t = 0; t < it.nt; ++t, ++n) {
          const uint32_t st = n % kNoiseStages;
          if (!mbar_wait(&n_empty[st], ((n / kNoiseStages) & 1) ^ 1, ctx, 306)) { ok = false; break; }
          if (lane == 0) {
            mbar_arrive_expect_tx(&n_full[st], L::kNoiseBytes);
#pragma unroll
            for (int kc = 0; kc < 2; ++kc)
              tma_load_3d(smem + L::kNoiseOff + st * L::kNoiseBytes + kc * (128 * 128), &p.map_noise, &n_full[st], it.k0 + kc * 64,
                          (it.first_tile + t) * BQ_, it.b * p.Hq + it.hq);
            __threadfence_block();  // the armed barrier phase is visible before the count
            *noise_issued = static_cast<int>(n + 1);
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA: S^T = K_tile Q_t^T
    constexpr uint32_t idesc = make_idesc(IsBf16<T>::value, false, false, BK_, BQ_);
    const uint32_t k_s = smem_u32(smem + L::kKOff);
    uint32_t n = 0, items = 0;
    bool ok = true;
    for (int round = 0; ok; ++round, ++items) {
      const int i = score_item_of_round(p, round);
      if (i >= p.n_items) break;
      const ScoreItem it = decode_score_item(p, i);
      if (!mbar_wait(k_full, items & 1, ctx, 302)) break;
      for (int t = 0; t < it.nt; ++t, ++n) {
        const uint32_t st = n % SB, qs = n % QS;
        if (!mbar_wait(&q_full[qs], (n / QS) & 1, ctx, 303)) { ok = false; break; }
        if (!mbar_wait(&s_empty[st], ((n / SB) & 1) ^ 1, ctx, 304)) { ok = false; break; }
        tc_fence_after();
        {  // all lanes converged, operands warp-uniform, one elected lane issues
          const uint64_t kd = make_smem_desc(k_s, 16, 1024);
          const uint64_t qd = make_smem_desc(smem_u32(smem + L::kQOff + qs * L::kTileBytes), 16, 1024);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t off = static_cast<uint64_t>(((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4);
            umma_ss_warp(tmem_base + st * BQ_, kd + off, qd + off, idesc, kk > 0 ? 1u : 0u);
          }
          umma_commit_warp(&s_full[st]);
          umma_commit_warp(&q_empty[qs]);
        }
      }
      if (ok) umma_commit_warp(k_free);  // arrives when the item's last S^T is done: the K tile may be replaced
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ reducers
    const int quad = warp & 3;               // quarter of the TMEM lanes (keys) this warp may read
    const int grp = ((warp - 4) >> 2) % G;   // which tiles this warp takes: those whose running count n has n % G == grp
    const int part = (warp - 4) / (4 * G);   // which of the tile's query columns it sums: [part, part + 1) * 128 / kParts
    const int cg = grp * kParts + part;      // slot of its partial sums
    const int r_in = quad * 32 + lane;       // key within the tile; also the query row whose statistics it stages
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const float nscale = kLog2e * p.inv_tau;
    const float st_scale = p.scale_log2 * p.inv_tau;
    // The first 128 threads of a group stage lse2 of the queries of the group's tile, the last 128 (the same ones when
    // the group has four warps) the perturbed statistic of KeyFormer; within an item the values are fetched three of the
    // group's tiles ahead: a tile takes about as long as one trip to L2.  +inf for rows past the end makes their
    // probability 0.
    // There are three times as many statistics buffers as S^T buffers; buffer n % LB is written again for tile n + LB
    // by the same group.  A warp that is there has been handed the S^T buffer of tile n + 2 LB / 3, which is given out
    // only after every warp of the group released tile n + LB / 3, i.e. is done with tile n (whose statistics are read
    // while it is summed): no warp runs more than one phase of a buffer's barrier ahead of another.
    const bool stage_a = part == 0, stage_b = NOISE && part == kParts - 1;
    uint32_t n_base = 0, items = 0;
    bool ok = true;
    long long prev_o = 0;   // output index of this thread's key in the previous item
    bool prev_ok = false;
    // add the partial sums of item `item` (all warps have published them once red_done completes) and store them
    auto add_up = [&](uint32_t item, long long o, bool key_valid) -> bool {
      const uint32_t b2 = item & 1;
      const float* red = red_s + b2 * L::kRedItem;
      if (!mbar_wait(&red_done[b2], (item >> 1) & 1, ctx, 309)) return false;
      if (key_valid) {
        float tsum[L::kRedSums];
#pragma unroll
        for (int w = 0; w < L::kRedSums; ++w) {
          tsum[w] = red[(w * L::kRedSlots + 0) * 128 + r_in];
#pragma unroll
          for (int slot = 1; slot < L::kRedSlots; ++slot) tsum[w] += red[(w * L::kRedSlots + slot) * 128 + r_in];
        }
        if (NOISE) {
          if (p.sum_pt) p.sum_pt[o] = tsum[0];
        } else {
          if (p.sum_p) p.sum_p[o] = tsum[0];
          if (p.sum_p2) p.sum_p2[o] = tsum[L::kRedSums - 1];
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_free[b2]);
      return true;
    };
    for (int round = 0; ok; ++round, ++items) {
      const int i = score_item_of_round(p, round);
      if (i >= p.n_items) break;
      const ScoreItem it = decode_score_item(p, i);
      const int kj = it.k0 + r_in;
      const bool key_ok = kj < p.kv_len;
      const long long head_row0 = (static_cast<long long>(it.b) * p.Hq + it.hq) * p.S;
      float acc_p = 0.f, acc_p2 = 0.f, acc_pt = 0.f;
      // this group's tiles of the item: t0, t0 + G, ...
      const int t0 = static_cast<int>((grp + G - n_base % G) % G);
      auto fetch_stat = [&](const float* src, int tile) -> float {
        const int qi = (it.first_tile + tile) * BQ_ + r_in;
        return (tile < it.nt && qi < p.S) ? src[head_row0 + qi] : INFINITY;
      };
      float sa0 = 0.f, sa1 = 0.f, sa2 = 0.f, sb0 = 0.f, sb1 = 0.f, sb2 = 0.f;
      if (stage_a) {
        sa0 = fetch_stat(p.lse2, t0);
        sa1 = fetch_stat(p.lse2, t0 + G);
        sa2 = fetch_stat(p.lse2, t0 + 2 * G);
      }
      if (stage_b) {
        sb0 = fetch_stat(p.lse2t, t0);
        sb1 = fetch_stat(p.lse2t, t0 + G);
        sb2 = fetch_stat(p.lse2t, t0 + 2 * G);
      }
      for (int t = t0; t < it.nt; t += G) {
        const uint32_t n = n_base + static_cast<uint32_t>(t);
        const uint32_t st = n % SB, lb = n % LB;
        const int q0 = (it.first_tile + t) * BQ_;
        if (stage_a) lse_s[(lb * 2 + 0) * 128 + r_in] = sa0;
        if (stage_b) lse_s[(lb * 2 + 1) * 128 + r_in] = sb0;
        __syncwarp();
        if (lane == 0) mbar_arrive(&lse_ready[lb]);  // arrivals on one barrier serialise: one per warp
        if (stage_a) {
          sa0 = sa1;
          sa1 = sa2;
          sa2 = fetch_stat(p.lse2, t + 3 * G);
        }
        if (stage_b) {
          sb0 = sb1;
          sb1 = sb2;
          sb2 = fetch_stat(p.lse2t, t + 3 * G);
        }
        if (!mbar_wait(&s_full[st], (n / SB) & 1, ctx, 305)) { ok = false; break; }
        tc_fence_after();
        if (!mbar_wait(&lse_ready[lb], (n / LB) & 1, ctx, 308)) { ok = false; break; }
        const uint32_t ns = n % kNoiseStages;
        if (NOISE && p.noise_tma) {
          bool armed = *noise_issued > static_cast<int>(n);
          if (!armed) {
            const long long c0 = clock64();
            while (!(armed = *noise_issued > static_cast<int>(n))) {
              if (*ctx.flag) break;
              if (clock64() - c0 > ctx.limit) {
                *ctx.flag = 1;
                atomicCAS(ctx.gerr, 0, 310);
                break;
              }
            }
          }
          if (!armed) { ok = false; break; }
          __threadfence_block();
          if (!mbar_wait(&n_full[ns], (n / kNoiseStages) & 1, ctx, 307)) { ok = false; break; }
        }
#pragma unroll 1
        for (int ch = 0; ch < kChunks; ++ch) {  // this warp's query columns, 32 at a time
          const int cb = (part * kChunks + ch) * 32;
          uint32_t s[32];
          tmem_ld_x32(tmem_base + st * BQ_ + lane_sel + cb, s);
          // this key's column of the swizzled noise tile: element (query c, key r_in)
          const uint8_t* n_col = smem + L::kNoiseOff + ns * L::kNoiseBytes + (r_in >> 6) * (128 * 128) + (cb) * 128 + (r_in & 7) * 2;
          const int n_unit = (r_in & 63) >> 3;
          // the statistic of these 32 queries, read four at a time where it is used
          const float4* lq4 = reinterpret_cast<const float4*>(lse_s + (lb * 2 + (NOISE ? 1 : 0)) * 128 + cb);
          // query column c of the tile is visible to this key iff kj <= past + q0 + c; only tiles on the diagonal mask
          const int c_min = (p.causal ? kj - p.past - q0 : 0) - cb;
          const bool mask_tile = !key_ok || c_min > 0;
          tmem_wait_ld();
          if (ch == kChunks - 1) {  // the last of this warp's S^T columns is in registers: the buffer may be overwritten
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[st]);
          }
          // Tiles off the causal diagonal (and with all keys valid) take the branch without per-element tests; the
          // arithmetic is packed two queries per instruction.  Sums run over fixed positions: identical from run to run.
          const bool plain = !__any_sync(0xffffffffu, mask_tile) && (!NOISE || p.noise_tma);
          if (plain) {
            float2 a1 = make_float2(0.f, 0.f), a2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int e4 = 0; e4 < 8; ++e4) {
              const float2 nl[2] = {make_float2(-lq4[e4].x, -lq4[e4].y), make_float2(-lq4[e4].z, -lq4[e4].w)};
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int e = e4 * 4 + u * 2;
                const float2 sv = make_float2(__uint_as_float(s[e]), __uint_as_float(s[e + 1]));
                float2 x;
                if (!NOISE) {
                  x = __ffma2_rn(sv, make_float2(p.scale_log2, p.scale_log2), nl[u]);
                } else {
                  const float2 nz = make_float2(
                      static_cast<float>(*reinterpret_cast<const T*>(n_col + e * 128 + ((n_unit ^ (e & 7)) << 4))),
                      static_cast<float>(*reinterpret_cast<const T*>(n_col + (e + 1) * 128 + ((n_unit ^ ((e + 1) & 7)) << 4))));
                  x = __ffma2_rn(nz, make_float2(nscale, nscale), __ffma2_rn(sv, make_float2(st_scale, st_scale), nl[u]));
                }
                const float2 pr = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                a1 = __fadd2_rn(a1, pr);
                if (!NOISE) a2 = __ffma2_rn(pr, pr, a2);
              }
            }
            if (!NOISE) {
              acc_p += a1.x + a1.y;
              acc_p2 += a2.x + a2.y;
            } else {
              acc_pt += a1.x + a1.y;
            }
          } else {
#pragma unroll
            for (int e4 = 0; e4 < 8; ++e4) {
              const float lq[4] = {lq4[e4].x, lq4[e4].y, lq4[e4].z, lq4[e4].w};
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int e = e4 * 4 + u;
                const float sv = __uint_as_float(s[e]);
                const bool hidden = !key_ok || e < c_min;
                if (!NOISE) {  // RoCo: sums of p and p^2
                  const float pr = hidden ? 0.f : fast_exp2(fmaf(sv, p.scale_log2, -lq[u]));
                  acc_p += pr;
                  acc_p2 = fmaf(pr, pr, acc_p2);
                } else {       // KeyFormer: only the perturbed probability is summed
                  float nz = 0.f;
                  if (p.noise_tma)
                    nz = static_cast<float>(*reinterpret_cast<const T*>(n_col + e * 128 + ((n_unit ^ (e & 7)) << 4)));
                  else if (!hidden && (q0 + cb + e) < p.S)
                    nz = static_cast<float>(static_cast<const T*>(p.noise)[(head_row0 + q0 + cb + e) * p.kv_len + kj]);
                  const float pt = hidden ? 0.f : fast_exp2(fmaf(nz, nscale, fmaf(sv, st_scale, -lq[u])));
                  acc_pt += pt;
                }
              }
            }
          }
        }
        if (NOISE && p.noise_tma) {
          __syncwarp();
          if (lane == 0) mbar_arrive(&n_empty[ns]);
        }
      }
      if (!ok) break;
      n_base += static_cast<uint32_t>(it.nt);

      // ---- end of the item: the partial sums of a key are added in a fixed order.  Two buffers: a warp that is done
      // goes on to the next item, and the four warps that do the adding take the PREVIOUS item's sums at this point --
      // those are complete by now, so nobody waits for the slowest warp of the item just finished.  Before a buffer is
      // written again the sums of two items ago have been read (red_free).
      const uint32_t rb = items & 1;
      float* red = red_s + rb * L::kRedItem;  // [sum][slot][key]
      if (items >= 2 && !mbar_wait(&red_free[rb], ((items >> 1) - 1) & 1, ctx, 312)) break;
      if (NOISE) {
        red[cg * 128 + r_in] = acc_pt;
      } else {
        red[(0 * L::kRedSlots + cg) * 128 + r_in] = acc_p;
        red[(1 * L::kRedSlots + cg) * 128 + r_in] = acc_p2;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_done[rb]);
      if (cg == 0) {
        if (items >= 1 && !add_up(items - 1, prev_o, prev_ok)) break;
        prev_o = (static_cast<long long>(it.b) * p.Hq + it.hq) * p.kv_len + kj;
        prev_ok = key_ok;
      }
    }
    if (ok && cg == 0 && items >= 1) add_up(items - 1, prev_o, prev_ok);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
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
  score_kernel<T, D, NOISE><<<grid, ScoreCfg<NOISE>::kThreads, ScoreSmem<D, NOISE>::kTotal, stream>>>(p);
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
  p.wait_limit = wait_limit_cycles();
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
  const long long items = static_cast<long long>((p.kv_len + BK_ - 1) / BK_) * a.Hq * a.B;
  if (items > 0x3fffffffLL) return TB200_ERR_INVALID;
  p.n_items = static_cast<int>(items);
  p.q_tiles = (a.S + BQ_ - 1) / BQ_;
  p.d_hb = make_fastdiv(static_cast<uint32_t>(a.Hq) * a.B);
  p.d_hq = make_fastdiv(static_cast<uint32_t>(a.Hq));
  p.d_group = make_fastdiv(static_cast<uint32_t>(a.Hq / a.Hkv));
  const int slots = st->num_sms * (noise ? ScoreCfg<true>::kCtasPerSm : ScoreCfg<false>::kCtasPerSm);  // persistent CTAs
  // Long items (many query tiles per key tile) amortise the start and end of a CTA, and the hardware's own scheduling
  // of one CTA per item balances them best; with short items the persistent walk wins (measured for RoCo: -4 % at
  // S = 2048, +1.5 % at 4096, +4.5 % at 8192; for KeyFormer -15 %, -9 %, -4 %).
  const bool persistent = noise || p.q_tiles <= 16;  // KeyFormer: one CTA per SM, nothing else hides a CTA's start and end
  const dim3 grid(static_cast<unsigned>((persistent && p.n_items > slots) ? slots : p.n_items), 1, 1);
  if (a.dtype == TB200_BF16) return launch_t<__nv_bfloat16>(p, a.D, noise, grid, stream);
  return launch_t<__half>(p, a.D, noise, grid, stream);
}

}  // namespace tb200
