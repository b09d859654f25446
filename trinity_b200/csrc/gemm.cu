// Fused GEMM on tcgen05: C = epilogue(A[M,K] @ B[K,N]), 16-bit operands, fp32 accumulation in TMEM.
//
// Persistent, warp-specialised kernel, one CTA per SM, 192 threads:
//   warp 0      TMA producer: A tile (128 x 64, K-major) and four B boxes (64 K-rows x 64 columns each,
//               MN-major because the weights are stored (K,N) row-major) into a 4-stage ring
//   warp 1      MMA issuer: one thread issues tcgen05.mma 128x256x16, accumulators in TMEM
//               (two 256-column accumulators, so the epilogue of tile i overlaps the main loop of tile i+1)
//   warps 2-5   epilogue: tcgen05.ld (thread = output row, 32 columns at a time) -> fused epilogue -> global
// With at least one 256-row tile per pair of SMs the kernel is launched as clusters of two CTAs that share a
// 256 x 256 tile (tcgen05.mma.cta_group::2, see PAIR below); otherwise CTAs work alone.  No load is multicast:
// every CTA fetches its own operand boxes; reuse comes from L2, for which the tile order walks groups of
// row-tiles across all column tiles.
//
// The four B boxes of a stage may come from different weight tensors:
//   GEMM_STORE / GEMM_PARTIAL  one source, 256 consecutive columns
//   GEMM_SWIGLU                gate columns [n0,n0+128) and up columns [n0,n0+128) -> silu(g)*u, 128 wide
//   GEMM_QKV                   tiles walk Wq, then Wk, then Wv; the epilogue splits heads, optionally
//                              RMS-normalises each head of q and k, writes q head-major and appends k, v
//                              to the caches
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;         // 16 KiB
constexpr int kBChunkBytes = BK * 64 * 2;    // 8 KiB: 64 K-rows of 64 columns
constexpr int kBBytes = 4 * kBChunkBytes;    // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kBarrierBytes = 256;
constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;  // + slack to align the ring to 1 KiB
// GEMM_PEER: two staged boxes of 128 rows x 64 columns, 1 KiB-aligned (their swizzle is a function of the address),
// behind the barrier block padded to 1 KiB
constexpr int kPeerStageOff = kStages * kStageBytes + 1024;
constexpr int kPeerSmemBytes = kPeerStageOff + 2 * BM * 128 + 1024;
static_assert(kPeerSmemBytes <= 232448, "more shared memory than an sm_100 CTA can have");
constexpr int kThreads = 192;
constexpr int kGroupRows = 4096;  // rows of A whose tiles are walked across all column tiles before moving down
constexpr int kTmemCols = 512;
// CTA-pair variant (cta_group::2): two CTAs of a cluster share one 256 x 256 tile.  Each CTA stages its own 128 A
// rows and HALF of the B columns (two boxes), so a stage is 32 KiB and six stages fit where four did.
constexpr int kStagesPair = 6;
constexpr int kStageBytesPair = kABytes + 2 * kBChunkBytes;
static_assert(kStagesPair * kStageBytesPair == kStages * kStageBytes, "both variants use the same shared-memory size");

struct GemmParams {
  CUtensorMap map_a;
  CUtensorMap map_b[3];
  int M, K, k_blocks, split_k, kb_per_split;
  int n_src;
  int src_n[3];       // columns of each source
  int src_tile0[4];   // first column-tile of each source (prefix sums); [n_src] = number of column tiles
  int tile_n;         // output columns per tile (256, or 128 for SwiGLU)
  int m_tiles, n_tiles, total_units;
  int group_m;        // row-tiles per L2 group
  int mt_rotation;    // GEMM_PEER: row-tile this rank's walk starts at; 0 otherwise
  int owner_tiles;    // GEMM_PEER: row-tiles per owner when the walk is dealt out over the owners in rounds; 0 otherwise
  int rows64;         // M <= 64: the tile is 64 rows tall (tcgen05.mma with M = 64, A boxes of 64 rows): half the tensor-core
                      // work of a 128-row tile that is half padding -- these shapes run under the power cap, where that work
                      // costs SM clock -- and all four epilogue warps get rows (16 each) instead of two (32 each)
  int kv_merged;      // GEMM_QKV with at most 128 columns each of Wk and Wv: one tile holds both (K in accumulator
                      // columns [0,128), V in [128,256)) instead of two tiles that are three quarters empty
  int* err;
  long long wait_limit;  // cycles a bounded wait may last (tb200_set_wait_limit_cycles)
  // epilogue
  const float* row_scale;
  void* C;
  long long ldc;
  const void* residual;
  long long ldr;
  void* C2;
  int act;
  void* q_out;
  void* k_cache;
  void* v_cache;
  int S, Hq, Hkv, D, past, cache_len, qknorm;
  float qk_eps;
  const void* q_norm_weight;
  const void* k_norm_weight;
  float* partial;
  long long ldp;
  int world, rank, rows_per_rank;
  CUtensorMap map_peer[kMaxPeers];   // GEMM_PEER: this rank's slot of every rank's staging buffer, (rows_per_rank, N)
  unsigned* peer_counter[kMaxPeers];
};

struct Unit {
  int m0, src, n0, kb_begin, kb_end, split;
};

template <bool PAIR>
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, const AbortCtx& ctx, int code) {
  if (PAIR) return mbar_wait_cluster(bar, parity, ctx, code);
  return mbar_wait(bar, parity, ctx, code);
}

// rank: position of this CTA in its pair (0 when CTAs work alone); a pair's tile is 2 * BM rows tall.
template <bool PAIR>
__device__ __forceinline__ Unit decode_unit(const GemmParams& p, int u, int rank) {
  Unit r;
  const int tile = u / p.split_k;
  r.split = u - tile * p.split_k;
  // Groups of p.group_m row-tiles walk all column tiles before moving down: the group's slice of A stays in L2
  // while the weights stream by (see launch_gemm for its size).
  const int kGroupM = p.group_m;
  const int per_group = kGroupM * p.n_tiles;
  const int g = tile / per_group;
  const int rem = tile - g * per_group;
  const int rows_here = min(kGroupM, p.m_tiles - g * kGroupM);
  const int nt = rem / rows_here;
  int mt = g * kGroupM + (rem - nt * rows_here);
  // GEMM_PEER: at any time the ranks send to different owners (a permutation over the links, not all to the same one).
  // In rounds: position k * world + j of the walk is row-tile k of owner (rank + j) mod world, so that after round k
  // EVERY owner has row-tile k from every rank and can reduce it while the projection goes on with round k + 1.
  // (Row-tiles that do not divide among the owners: one rotation, every rank starting at its own rows.)
  if (p.owner_tiles > 0) {
    const int k = mt / p.world, j = mt - k * p.world;
    int owner = p.rank + j;
    if (owner >= p.world) owner -= p.world;
    mt = owner * p.owner_tiles + k;
  } else {
    mt += p.mt_rotation;
    if (mt >= p.m_tiles) mt -= p.m_tiles;
  }
  r.m0 = PAIR ? (mt * 2 + rank) * BM : mt * BM;
  int src = 0;
  while (src + 1 < p.n_src && nt >= p.src_tile0[src + 1]) ++src;
  if (p.tile_n != BN) src = 0;  // SwiGLU: both sources are walked together
  r.src = src;
  r.n0 = (nt - p.src_tile0[src]) * p.tile_n;
  r.kb_begin = r.split * p.kb_per_split;
  r.kb_end = min(p.k_blocks, r.kb_begin + p.kb_per_split);
  return r;
}

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
// x * sigmoid(x) with the approximate exponential and reciprocal (a few ulp, far inside a 16-bit result): the exact
// division is a twenty-instruction sequence, and with one tile per CTA (few-token FFN) nothing hides the epilogue.
__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.f + __expf(-x)); }

template <typename T>
__device__ __forceinline__ void store32(T* dst, const float (&v)[32]) {
  uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    d[i] = make_uint4(Pack2<T>::pack(v[8 * i + 0], v[8 * i + 1]), Pack2<T>::pack(v[8 * i + 2], v[8 * i + 3]),
                      Pack2<T>::pack(v[8 * i + 4], v[8 * i + 5]), Pack2<T>::pack(v[8 * i + 6], v[8 * i + 7]));
  }
}
// columns valid in steps of 8 (every N is a multiple of 8)
template <typename T>
__device__ __forceinline__ void store32_clipped(T* dst, const float (&v)[32], int valid) {
  uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (8 * i < valid)
      d[i] = make_uint4(Pack2<T>::pack(v[8 * i + 0], v[8 * i + 1]), Pack2<T>::pack(v[8 * i + 2], v[8 * i + 3]),
                        Pack2<T>::pack(v[8 * i + 4], v[8 * i + 5]), Pack2<T>::pack(v[8 * i + 6], v[8 * i + 7]));
  }
}

template <typename T, int MODE, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ GemmParams p) {
  constexpr int NST = PAIR ? kStagesPair : kStages;
  constexpr int NCH = PAIR ? 2 : 4;  // B boxes this CTA stages
  constexpr int SB = kABytes + NCH * kBChunkBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + NST * SB);
  uint64_t* empty = full + NST;
  uint64_t* tfull = empty + NST;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_launch_dependents();  // the next kernel of the stream waits for this one's completion before it reads or writes
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = PAIR ? static_cast<int>(cluster_ctarank()) : 0;
  const int unit0 = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int unit_step = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], PAIR ? 8 : 4);  // one arrival per epilogue warp (of both CTAs of a pair, on the leader)
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    if (PAIR) {  // the same warp of both CTAs of the pair allocates together
      tmem_alloc_pair(tmem_slot, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, kTmemCols);
      tmem_relinquish();
    }
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&p.map_a);
    for (int s = 0; s < p.n_src; ++s) tma_prefetch_desc(&p.map_b[s]);
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all(); else __syncthreads();  // a pair's barriers must exist before its peer signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const AbortCtx ctx{p.err, abort_flag, p.wait_limit};

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // One lane issues the boxes of a stage: the weights' (B) when with_b, the activations' (A) when with_a.
    auto issue = [&](const Unit& t, int kb, int stage, bool with_a, bool with_b) {
      uint8_t* sa = smem + stage * SB;
      uint8_t* sb = sa + kABytes;
      if (PAIR) {
        // both CTAs' boxes are counted on the leader's barrier; the leader announces the pair's bytes
        const uint32_t fb = mapa_u32(smem_u32(&full[stage]), 0);
        if (with_b) {
          if (rank == 0) mbar_arrive_expect_tx(&full[stage], 2 * SB);
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            const int g = rank * NCH + c;  // box of the pair's 256-column B tile
            int src = t.src, col = t.n0 + 64 * g;
            if (MODE == GEMM_SWIGLU) { src = g >> 1; col = t.n0 + 64 * (g & 1); }
            if (MODE == GEMM_QKV && p.kv_merged && t.src == 1) { src = 1 + (g >> 1); col = 64 * (g & 1); }
            tma_load_2d_pair(sb + c * kBChunkBytes, &p.map_b[src], fb, col, kb * BK);
          }
        }
        if (with_a) tma_load_2d_pair(sa, &p.map_a, fb, kb * BK, t.m0);
      } else {
        if (with_b) {
          mbar_arrive_expect_tx(&full[stage], p.rows64 ? SB - kABytes / 2 : SB);   // a 64-row A box is half the bytes
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            int src = t.src, col = t.n0 + 64 * c;
            if (MODE == GEMM_SWIGLU) { src = c >> 1; col = t.n0 + 64 * (c & 1); }
            if (MODE == GEMM_QKV && p.kv_merged && t.src == 1) { src = 1 + (c >> 1); col = 64 * (c & 1); }
            tma_load_2d(sb + c * kBChunkBytes, &p.map_b[src], &full[stage], col, kb * BK);
          }
        }
        if (with_a) tma_load_2d(sa, &p.map_a, &full[stage], kb * BK, t.m0);
      }
    };
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // The weights are written by no kernel of the call this launch belongs to, so the first stages' B boxes are
    // requested before the wait for the kernel before this one; A, which that kernel may still be writing, after.
    int prefilled = 0;
    if (unit0 < p.total_units) {
      const Unit t = decode_unit<PAIR>(p, unit0, rank);
      prefilled = min(NST, t.kb_end - t.kb_begin);
      if (lane == 0)
        for (int i = 0; i < prefilled; ++i) issue(t, t.kb_begin + i, i, false, true);
      pdl_wait();
      if (lane == 0)
        for (int i = 0; i < prefilled; ++i) issue(t, t.kb_begin + i, i, true, false);
      __syncwarp();
      stage = prefilled == NST ? 0 : prefilled;
      phase = prefilled == NST ? 1 : 0;
    } else {
      pdl_wait();
    }
    for (int u = unit0; ok && u < p.total_units; u += unit_step) {
      const Unit t = decode_unit<PAIR>(p, u, rank);
      for (int kb = t.kb_begin + (u == unit0 ? prefilled : 0); kb < t.kb_end; ++kb) {
        if (!wait_bar<PAIR>(&empty[stage], phase ^ 1, ctx, 101)) { ok = false; break; }
        if (lane == 0) issue(t, kb, stage, true, true);
        __syncwarp();
        if (++stage == NST) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ------------------------------------------------------------ MMA issuer (a pair's leader issues for both CTAs)
    constexpr uint32_t idesc_full = make_idesc(IsBf16<T>::value, /*a_mn=*/false, /*b_mn=*/true, PAIR ? 2 * BM : BM, BN);
    constexpr uint32_t idesc_64 = make_idesc(IsBf16<T>::value, false, true, 64, BN);
    const uint32_t idesc = (!PAIR && p.rows64) ? idesc_64 : idesc_full;
    pdl_wait();
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    bool ok = true;
    for (int u = unit0; ok && u < p.total_units; u += unit_step) {
      const Unit t = decode_unit<PAIR>(p, u, rank);
      if (!wait_bar<PAIR>(&tempty[acc], acc_phase ^ 1, ctx, 102)) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = t.kb_begin; kb < t.kb_end; ++kb) {
        if (!wait_bar<PAIR>(&full[stage], phase, ctx, 103)) { ok = false; break; }
        tc_fence_after();
        {  // all lanes converged, operands warp-uniform, one elected lane issues
          const uint32_t a0 = smem_u32(smem + stage * SB);
          const uint64_t ad = make_smem_desc(a0, 16, 1024);
          const uint64_t bd = make_smem_desc(a0 + kABytes, kBChunkBytes, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {  // K-major A: +32 B per 16 K; MN-major B: +16 K-rows (2048 B); in 16-byte units
            const uint32_t accum = (kb > t.kb_begin || k > 0) ? 1u : 0u;
            if (PAIR) umma_ss_pair_warp(d_tmem, ad + static_cast<uint64_t>(k * 2), bd + static_cast<uint64_t>(k * 128), idesc, accum);
            else umma_ss_warp(d_tmem, ad + static_cast<uint64_t>(k * 2), bd + static_cast<uint64_t>(k * 128), idesc, accum);
          }
          if (PAIR) {  // the arrivals land on the same barrier of both CTAs
            umma_commit_pair_warp(&empty[stage]);
            if (kb == t.kb_end - 1) umma_commit_pair_warp(&tfull[acc]);
          } else {
            umma_commit_warp(&empty[stage]);                       // frees the stage when these MMAs have read it
            if (kb == t.kb_end - 1) umma_commit_warp(&tfull[acc]);  // accumulator complete
          }
        }
        if (++stage == NST) { stage = 0; phase ^= 1; }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may read
    pdl_wait();
    int acc = 0;
    uint32_t acc_phase = 0;
    unsigned* peer_pending = nullptr;  // GEMM_PEER: the counter the last tile has yet to arrive on
    uint32_t peer_boxes = 0;           // GEMM_PEER: boxes staged so far
    for (int u = unit0; u < p.total_units; u += unit_step) {
      const Unit t = decode_unit<PAIR>(p, u, rank);
      if (!wait_bar<PAIR>(&tfull[acc], acc_phase, ctx, 104)) break;
      tc_fence_after();
      // A 128-row accumulator has row i in TMEM lane i.  A 64-row one (M = 64) has rows [16 q, 16 q + 16) in the first
      // sixteen lanes of quadrant q: every epilogue warp owns sixteen rows, its upper sixteen lanes hold nothing.
      const int row = p.rows64 ? t.m0 + quad * 16 + (lane & 15) : t.m0 + quad * 32 + lane;
      const bool row_ok = row < p.M && (!p.rows64 || lane < 16);
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      const float rs = (p.row_scale != nullptr && row_ok) ? p.row_scale[row] : 1.f;
      uint32_t r[32];
      float v[32];

      if (MODE == GEMM_STORE) {
        const int n_total = p.src_n[0];
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col = t.n0 + c * 32;
          if (col >= n_total) break;  // warp-uniform
          tmem_ld_x32(taddr + c * 32, r);
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float f = __uint_as_float(r[i]) * rs;
              if (p.act == 1) f = gelu_erf(f);
              v[i] = f;
            }
            const int valid = min(32, n_total - col);
            if (p.C2 != nullptr) store32_clipped<T>(static_cast<T*>(p.C2) + row * p.ldc + col, v, valid);
            if (p.residual != nullptr) {
              const uint4* rp = reinterpret_cast<const uint4*>(static_cast<const T*>(p.residual) + row * p.ldr + col);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if (8 * i < valid) {
                  const uint4 q4 = __ldg(rp + i);
                  const uint32_t w[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 f2 = Pack2<T>::unpack(w[j]);
                    v[8 * i + 2 * j] += f2.x;
                    v[8 * i + 2 * j + 1] += f2.y;
                  }
                }
              }
            }
            store32_clipped<T>(static_cast<T*>(p.C) + row * p.ldc + col, v, valid);
          }
        }
      } else if (MODE == GEMM_SWIGLU) {
        const int n_total = p.src_n[0];
        uint32_t r2[32];
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          const int col = t.n0 + c * 32;
          if (col >= n_total) break;
          tmem_ld_x32(taddr + c * 32, r);         // gate
          tmem_ld_x32(taddr + 128 + c * 32, r2);  // up
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = silu(__uint_as_float(r[i]) * rs) * (__uint_as_float(r2[i]) * rs);
            store32_clipped<T>(static_cast<T*>(p.C) + row * p.ldc + col, v, min(32, n_total - col));
          }
        }
      } else if (MODE == GEMM_PEER) {
        // The CTA's 128 rows of this tile lie in one 128-row block of one owner.  The four epilogue warps stage the
        // tile as 16-bit values, 64 columns at a time, in two alternating shared-memory boxes, and one thread sends
        // each box into the owner's staging buffer (its own memory or a peer's over NVLink) with a TMA store -- whole
        // 128-byte lines on the wire.  The arrival on the owner's counter for a tile is sent when the NEXT tile's
        // epilogue starts (or after the loop): by then its stores have long completed, nobody waits for the link.
        const int n_total = p.src_n[0];
        const int owner = t.m0 / p.rows_per_rank;
        const int local0 = t.m0 - owner * p.rows_per_rank;
        const bool leader = warp == 2 && lane == 0;
        uint8_t* stage = smem + kPeerStageOff;   // two boxes of 128 rows x 64 columns x 2 bytes
        if (leader && peer_pending != nullptr) {
          tma_store_wait_all();
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(peer_pending) : "memory");
          peer_pending = nullptr;
        }
#pragma unroll 1
        for (int cb = 0; cb < BN / 64; ++cb) {
          const int col = t.n0 + cb * 64;
          if (col >= n_total) break;  // uniform over the four warps
          uint8_t* box = stage + (peer_boxes & 1) * (BM * 128);
          if (peer_boxes >= 2) {  // the store that last used this box has read it
            if (leader) tma_store_wait_read_but_one();
            named_barrier_sync(1, 128);
          }
          ++peer_boxes;
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            tmem_ld_x32(taddr + cb * 64 + cc * 32, r);
            tmem_wait_ld();
            // row (quad * 32 + lane) of the box, 128-byte swizzle: 16-byte chunk k of a row sits at k ^ (row & 7)
            const int rr = quad * 32 + lane;
            uint8_t* rowp = box + rr * 128;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint4 v4 = make_uint4(Pack2<T>::pack(__uint_as_float(r[8 * k]), __uint_as_float(r[8 * k + 1])),
                                          Pack2<T>::pack(__uint_as_float(r[8 * k + 2]), __uint_as_float(r[8 * k + 3])),
                                          Pack2<T>::pack(__uint_as_float(r[8 * k + 4]), __uint_as_float(r[8 * k + 5])),
                                          Pack2<T>::pack(__uint_as_float(r[8 * k + 6]), __uint_as_float(r[8 * k + 7])));
              *reinterpret_cast<uint4*>(rowp + (((cc * 4 + k) ^ (rr & 7)) << 4)) = v4;
            }
          }
          fence_proxy_async_smem();
          named_barrier_sync(1, 128);
          if (leader) {  // columns past n_total are clipped by the tensor map
            tma_store_2d(&p.map_peer[owner], box, col, local0);
            tma_store_commit();
          }
        }
        if (leader) peer_pending = p.peer_counter[owner] + (local0 >> 7);
      } else if (MODE == GEMM_PARTIAL) {
        int n_total = 0, col_base = 0;
        for (int s = 0; s < p.n_src; ++s) {
          if (s < t.src) col_base += p.src_n[s];
        }
        n_total = p.src_n[t.src];
        float* prow = p.partial + (static_cast<long long>(t.split) * p.M + row) * p.ldp + col_base;
        // A warp none of whose 32 rows exist (few-token blocks: most of the tile) reads nothing.  The others take 64
        // columns per step, both loads in flight before the wait: with one tile per CTA nothing hides this loop.
        const bool warp_has_rows = t.m0 + quad * (p.rows64 ? 16 : 32) < p.M;
        uint32_t r2[32];
#pragma unroll 1
        for (int c = 0; warp_has_rows && c < BN / 64; ++c) {
          const int col = t.n0 + c * 64;
          if (col >= n_total) break;
          tmem_ld_x32(taddr + c * 64, r);
          tmem_ld_x32(taddr + c * 64 + 32, r2);
          tmem_wait_ld();
          if (row_ok) {
            const int valid = min(64, n_total - col);
            uint4* d = reinterpret_cast<uint4*>(prow + col);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (4 * i < valid) d[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (32 + 4 * i < valid) d[8 + i] = make_uint4(r2[4 * i], r2[4 * i + 1], r2[4 * i + 2], r2[4 * i + 3]);
          }
        }
      } else {  // GEMM_QKV
        const int D = p.D;
        const int b = row_ok ? row / p.S : 0;
        const int s_in = row_ok ? row - b * p.S : 0;
        const bool merged = p.kv_merged && t.src == 1;   // K in accumulator columns [0,128), V in [128,256)
        const int heads_all = (merged ? BN / 2 : BN) / D;  // heads per source in this tile
#pragma unroll 1
        for (int hx = 0; hx < (merged ? 2 : 1) * heads_all; ++hx) {
          const int part = hx / heads_all, hh_in = hx - part * heads_all;
          const int psrc = t.src + part;
          const int n_total = p.src_n[psrc];
          const bool norm_this = p.qknorm && psrc < 2;
          const T* nw = static_cast<const T*>(psrc == 0 ? p.q_norm_weight : p.k_norm_weight);
          const int col_h = (merged ? 0 : t.n0) + hh_in * D;
          if (col_h >= n_total) continue;
          const int head = col_h / D;
          const int hh = part * heads_all + hh_in;  // position of the head in the accumulator: column hh * D
          float scale = rs;
          if (norm_this) {  // pass 1: sum of squares over the head's D columns (thread-local: a thread owns a row)
            float ss = 0.f;
            for (int c = 0; c < D / 32; ++c) {
              tmem_ld_x32(taddr + hh * D + c * 32, r);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float f = __uint_as_float(r[i]) * rs;
                ss = fmaf(f, f, ss);
              }
            }
            scale = rs * rsqrtf(ss / static_cast<float>(D) + p.qk_eps);
          }
          T* dst;
          if (psrc == 0) {
            dst = static_cast<T*>(p.q_out) + ((static_cast<long long>(b) * p.Hq + head) * p.S + s_in) * D;
          } else {
            T* cache = static_cast<T*>(psrc == 1 ? p.k_cache : p.v_cache);
            dst = cache + ((static_cast<long long>(b) * p.Hkv + head) * p.cache_len + p.past + s_in) * D;
          }
          for (int c = 0; c < D / 32; ++c) {
            tmem_ld_x32(taddr + hh * D + c * 32, r);
            tmem_wait_ld();
            if (row_ok) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * scale;
              if (norm_this && nw != nullptr) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  const float2 g = Pack2<T>::unpack(*reinterpret_cast<const uint32_t*>(nw + c * 32 + i));
                  v[i] *= g.x;
                  v[i + 1] *= g.y;
                }
              }
              store32<T>(dst + c * 32, v);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));
        else mbar_arrive(&tempty[acc]);
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (MODE == GEMM_PEER && warp == 2 && lane == 0) {
      tma_store_wait_all();
      if (peer_pending != nullptr) asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(peer_pending) : "memory");
    }
  }

  tc_fence_before();
  if (PAIR) cluster_sync_all(); else __syncthreads();  // neither CTA of a pair leaves while its peer may still reach it
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ split-K finish
template <typename T, bool GATED>
__global__ void splitk_finish_kernel(SplitKFinish f) {
  pdl_launch_dependents();
  pdl_wait();
  // slices whose loads are in flight together: one slice at a time costs a trip to L2 each.  Sixteen cover the slice
  // counts the library chooses in one trip (the 64-token down projection has nine); half as many with a gate
  // tensor beside, whose loads double the registers
  constexpr int kBatch = GATED ? 8 : 16;
  const int64_t groups_per_row = f.N / 8;
  const int64_t total = static_cast<int64_t>(f.M) * groups_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / groups_per_row;
    const int col = static_cast<int>(i - row * groups_per_row) * 8;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const float* p0 = f.partial + row * f.ldp + col;
    const int64_t slice = static_cast<int64_t>(f.M) * f.ldp;
    for (int s0 = 0; s0 < f.split_k; s0 += kBatch) {  // fixed order: deterministic
      float4 x[kBatch][2], y[kBatch][2];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const bool on = s0 + j < f.split_k;
        const float* p = p0 + (on ? s0 + j : 0) * slice;
        x[j][0] = on ? __ldcg(reinterpret_cast<const float4*>(p)) : make_float4(0.f, 0.f, 0.f, 0.f);
        x[j][1] = on ? __ldcg(reinterpret_cast<const float4*>(p + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (GATED) {
          y[j][0] = on ? __ldcg(reinterpret_cast<const float4*>(p + f.N)) : make_float4(0.f, 0.f, 0.f, 0.f);
          y[j][1] = on ? __ldcg(reinterpret_cast<const float4*>(p + f.N + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        a[0] += x[j][0].x; a[1] += x[j][0].y; a[2] += x[j][0].z; a[3] += x[j][0].w;
        a[4] += x[j][1].x; a[5] += x[j][1].y; a[6] += x[j][1].z; a[7] += x[j][1].w;
        if (GATED) {
          b[0] += y[j][0].x; b[1] += y[j][0].y; b[2] += y[j][0].z; b[3] += y[j][0].w;
          b[4] += y[j][1].x; b[5] += y[j][1].y; b[6] += y[j][1].z; b[7] += y[j][1].w;
        }
      }
    }
    const float rs = f.row_scale ? f.row_scale[row] : 1.f;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float x = a[j] * rs;
      if (GATED) x = silu(x) * (b[j] * rs);
      if (f.act == 1) x = gelu_erf(x);
      v[j] = x;
    }
    if (f.C2)
      *reinterpret_cast<uint4*>(static_cast<T*>(f.C2) + row * f.ldc + col) =
          make_uint4(Pack2<T>::pack(v[0], v[1]), Pack2<T>::pack(v[2], v[3]), Pack2<T>::pack(v[4], v[5]), Pack2<T>::pack(v[6], v[7]));
    if (f.residual) {
      const uint4 q4 = *reinterpret_cast<const uint4*>(static_cast<const T*>(f.residual) + row * f.ldr + col);
      const uint32_t w[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f2 = Pack2<T>::unpack(w[j]);
        v[2 * j] += f2.x;
        v[2 * j + 1] += f2.y;
      }
    }
    *reinterpret_cast<uint4*>(static_cast<T*>(f.C) + row * f.ldc + col) =
        make_uint4(Pack2<T>::pack(v[0], v[1]), Pack2<T>::pack(v[2], v[3]), Pack2<T>::pack(v[4], v[5]), Pack2<T>::pack(v[6], v[7]));
  }
}

// ------------------------------------------------------------------ split-K finish of a QKV projection
// One warp per (token row, head of q | k | v): the lanes cover the head's D columns, sum the K slices in a fixed
// order, apply the row scale and the optional per-head RMSNorm (warp reduction), and write to q / the caches.
template <typename T, int D>
__global__ void qkv_finish_kernel(QkvFinish f) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = D / 32;  // columns per lane
  const int heads = f.Hq + 2 * f.Hkv;
  const long long ldp = static_cast<long long>(heads) * D;
  const int lane = threadIdx.x & 31;
  const long long items = static_cast<long long>(f.M) * heads;
  for (long long it = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; it < items;
       it += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    const int row = static_cast<int>(it / heads);
    const int slot = static_cast<int>(it - static_cast<long long>(row) * heads);
    float v[V];
#pragma unroll
    for (int i = 0; i < V; ++i) v[i] = 0.f;
    const float* src = f.partial + row * ldp + static_cast<long long>(slot) * D + lane * V;
    for (int s0 = 0; s0 < f.split_k; s0 += 8) {   // eight slices' loads in flight together; the order of the sum is fixed
      float x[8][V];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool on = s0 + j < f.split_k;
        const float* ps = src + static_cast<long long>(on ? s0 + j : 0) * f.M * ldp;
#pragma unroll
        for (int i = 0; i < V; ++i) x[j][i] = on ? __ldcg(ps + i) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < V; ++i) v[i] += x[j][i];
    }
    const float rs = f.row_scale ? f.row_scale[row] : 1.f;
#pragma unroll
    for (int i = 0; i < V; ++i) v[i] *= rs;
    const int which = slot < f.Hq ? 0 : (slot < f.Hq + f.Hkv ? 1 : 2);
    const int head = which == 0 ? slot : (which == 1 ? slot - f.Hq : slot - f.Hq - f.Hkv);
    if (f.qknorm && which < 2) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < V; ++i) ss = fmaf(v[i], v[i], ss);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float r = rsqrtf(ss / static_cast<float>(D) + f.qk_eps);
      const T* w = static_cast<const T*>(which == 0 ? f.q_norm_weight : f.k_norm_weight);
#pragma unroll
      for (int i = 0; i < V; ++i) v[i] *= r * (w ? static_cast<float>(w[lane * V + i]) : 1.f);
    }
    const int b = row / f.S, s_in = row - b * f.S;
    T* dst;
    if (which == 0) dst = static_cast<T*>(f.q_out) + ((static_cast<long long>(b) * f.Hq + head) * f.S + s_in) * D;
    else dst = static_cast<T*>(which == 1 ? f.k_cache : f.v_cache) + ((static_cast<long long>(b) * f.Hkv + head) * f.cache_len + f.past + s_in) * D;
    uint32_t* d32 = reinterpret_cast<uint32_t*>(dst + lane * V);
#pragma unroll
    for (int i = 0; i < V; i += 2) d32[i >> 1] = Pack2<T>::pack(v[i], v[i + 1]);
  }
}

// PAIR: the grid is made of clusters of two CTAs; `slots` is the SM count for single CTAs and is replaced by the
// number of pairs the device can hold at once (asked of the runtime once per device) for pairs.
template <typename T, int MODE, bool PAIR>
int launch_mode(const GemmParams& p, int slots, cudaStream_t stream) {
  static bool attr_set[32] = {};
  static int max_pairs[32] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attr[2];
  constexpr int kSmem = MODE == GEMM_PEER ? kPeerSmemBytes : kSmemBytes;
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = stream;
  cfg.attrs = attr;
  if (PAIR) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.numAttrs = 1;
  }
  if (!attr_set[dev & 31]) {
    if (cudaFuncSetAttribute(gemm_kernel<T, MODE, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess)
      return TB200_ERR_CUDA;
    if (PAIR) {
      cfg.gridDim = dim3(static_cast<unsigned>(slots / 2 * 2), 1, 1);
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_kernel<T, MODE, PAIR>, &cfg) != cudaSuccess || n < 1) return TB200_ERR_CUDA;
      max_pairs[dev & 31] = n < slots / 2 ? n : slots / 2;
    }
    attr_set[dev & 31] = true;
  }
  int ctas = slots;
  if (PAIR) ctas = 2 * max_pairs[dev & 31];
  if (PAIR) ctas = p.total_units * 2 < ctas ? p.total_units * 2 : ctas;
  else ctas = p.total_units < ctas ? p.total_units : ctas;
  cfg.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
  if (chain_next_launch()) {  // not the first kernel of the call: may start while the kernel before it drains
    attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
    ++cfg.numAttrs;
  }
  if (cudaLaunchKernelEx(&cfg, gemm_kernel<T, MODE, PAIR>, p) != cudaSuccess) return TB200_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

template <typename T, bool PAIR>
int launch_typed(const GemmParams& p, int mode, int slots, cudaStream_t stream) {
  switch (mode) {
    case GEMM_STORE: return launch_mode<T, GEMM_STORE, PAIR>(p, slots, stream);
    case GEMM_SWIGLU: return launch_mode<T, GEMM_SWIGLU, PAIR>(p, slots, stream);
    case GEMM_QKV: return launch_mode<T, GEMM_QKV, PAIR>(p, slots, stream);
    case GEMM_PARTIAL: return launch_mode<T, GEMM_PARTIAL, PAIR>(p, slots, stream);
    case GEMM_PEER: return launch_mode<T, GEMM_PEER, PAIR>(p, slots, stream);
    default: return TB200_ERR_UNSUPPORTED;
  }
}

// Pairs halve the B bytes each SM stages (measured +1.3 .. +4 % on 16384-row projections); they pay off when
// there is a 256-row tile for every pair of SMs, so decode-size M keeps single CTAs.
bool use_pair(int M, long long pair_units, int num_sms) {
  if (M < 2 * BM) return false;
  return pair_units >= num_sms / 2;
}

}  // namespace

int launch_gemm(const GemmLaunch& g, cudaStream_t stream) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  if (g.dtype != TB200_BF16 && g.dtype != TB200_F16) return TB200_ERR_UNSUPPORTED;
  if (g.A == nullptr || g.M < 0 || g.K <= 0 || (g.K & 7) != 0 || g.n_src < 1 || g.n_src > 3) return TB200_ERR_INVALID;
  if (!aligned16(g.A)) return TB200_ERR_INVALID;
  if (g.M == 0) return TB200_OK;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = g.M;
  p.K = g.K;
  p.k_blocks = (g.K + BK - 1) / BK;
  p.split_k = (g.mode == GEMM_PARTIAL) ? g.split_k : 1;
  if (p.split_k < 1 || p.split_k > p.k_blocks) return TB200_ERR_INVALID;
  p.kb_per_split = (p.k_blocks + p.split_k - 1) / p.split_k;
  p.split_k = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;  // no empty slice
  p.n_src = g.n_src;
  p.tile_n = (g.mode == GEMM_SWIGLU) ? 128 : BN;
  int tiles = 0;
  for (int s = 0; s < g.n_src; ++s) {
    if (g.B[s] == nullptr || g.N[s] <= 0 || (g.N[s] & 7) != 0 || !aligned16(g.B[s])) return TB200_ERR_INVALID;
    p.src_n[s] = g.N[s];
    p.src_tile0[s] = tiles;
    if (g.mode == GEMM_SWIGLU) {
      if (s == 0) tiles += (g.N[0] + 127) / 128;
    } else {
      tiles += (g.N[s] + BN - 1) / BN;
    }
  }
  if (g.mode == GEMM_SWIGLU && (g.n_src != 2 || g.N[0] != g.N[1])) return TB200_ERR_INVALID;
  if (g.mode == GEMM_QKV) {
    if (g.n_src != 3 || (g.D != 64 && g.D != 128) || g.S <= 0 || g.M % g.S != 0) return TB200_ERR_INVALID;
    if (g.N[0] != g.Hq * g.D || g.N[1] != g.Hkv * g.D || g.N[2] != g.Hkv * g.D) return TB200_ERR_INVALID;
    if (g.q_out == nullptr || g.k_cache == nullptr || g.v_cache == nullptr || g.past < 0 || g.cache_len < g.past + g.S)
      return TB200_ERR_INVALID;
    if (!aligned16(g.q_out) || !aligned16(g.k_cache) || !aligned16(g.v_cache)) return TB200_ERR_INVALID;
  }
  if (g.mode == GEMM_STORE || g.mode == GEMM_SWIGLU) {
    if (g.C == nullptr || !aligned16(g.C) || (g.ldc & 7) != 0 || !aligned16(g.residual) || (g.ldr & 7) != 0) return TB200_ERR_INVALID;
  }
  if (g.mode == GEMM_PARTIAL && (g.partial == nullptr || !aligned16(g.partial))) return TB200_ERR_INVALID;
  if (g.mode == GEMM_PEER) {
    if (g.n_src != 1 || g.world < 1 || g.world > kMaxPeers || g.rank < 0 || g.rank >= g.world) return TB200_ERR_INVALID;
    if (g.rows_per_rank <= 0 || (g.rows_per_rank & 127) != 0 || static_cast<long long>(g.rows_per_rank) * g.world != g.M) return TB200_ERR_INVALID;
    for (int r = 0; r < g.world; ++r)
      if (g.peer_stage[r] == nullptr || !aligned16(g.peer_stage[r]) || g.peer_counter[r] == nullptr || !aligned4(g.peer_counter[r]))
        return TB200_ERR_INVALID;
  }
  if (g.mode == GEMM_QKV && g.N[1] <= BN / 2 && g.N[2] <= BN / 2) {  // MQA / small GQA: K and V share one tile
    p.kv_merged = 1;
    tiles = p.src_tile0[1] + 1;
    p.src_tile0[2] = tiles;  // no tile of its own for Wv
  }
  for (int s = g.n_src; s < 4; ++s) p.src_tile0[s] = tiles;
  p.src_tile0[g.n_src] = tiles;
  p.n_tiles = tiles;
  const bool pair = use_pair(g.M, static_cast<long long>((g.M + 2 * BM - 1) / (2 * BM)) * tiles * p.split_k, st->num_sms);
  p.m_tiles = pair ? (g.M + 2 * BM - 1) / (2 * BM) : (g.M + BM - 1) / BM;
  // 4096 rows of A per group.  At K = 4096 that slice is 32 MiB and stays in the half of L2 next to each die while
  // the weights stream by (with 8192 rows the Llama QKV projection read 908 MB from DRAM, with 4096 rows 430 MB);
  // a sweep of 2..32 row-tiles on the K = 14336 and K = 18176 projections of the FFNs also had its best times here.
  p.group_m = kGroupRows / (pair ? 2 * BM : BM);
  if (p.group_m > p.m_tiles) p.group_m = p.m_tiles;
  const long long units = static_cast<long long>(p.m_tiles) * p.n_tiles * p.split_k;
  if (units > 0x7fffffffLL) return TB200_ERR_INVALID;
  p.total_units = static_cast<int>(units);
  p.err = st->err_word;
  p.wait_limit = wait_limit_cycles();
  p.row_scale = g.row_scale;
  p.C = g.C;
  p.ldc = g.ldc;
  p.residual = g.residual;
  p.ldr = g.ldr;
  p.C2 = g.C2;
  p.act = g.act;
  p.q_out = g.q_out;
  p.k_cache = g.k_cache;
  p.v_cache = g.v_cache;
  p.S = g.S; p.Hq = g.Hq; p.Hkv = g.Hkv; p.D = g.D; p.past = g.past; p.cache_len = g.cache_len;
  p.qknorm = g.qknorm;
  p.qk_eps = g.qk_eps;
  p.q_norm_weight = g.q_norm_weight;
  p.k_norm_weight = g.k_norm_weight;
  p.partial = g.partial;
  p.world = g.world; p.rank = g.rank; p.rows_per_rank = g.rows_per_rank;
  for (int r = 0; r < kMaxPeers; ++r) p.peer_counter[r] = g.peer_counter[r];
  if (g.mode == GEMM_PEER) {
    if (g.world > 1 && p.m_tiles % g.world == 0 && g.rows_per_rank % (pair ? 2 * BM : BM) == 0) p.owner_tiles = p.m_tiles / g.world;
    else p.mt_rotation = static_cast<int>(static_cast<long long>(g.rank) * p.m_tiles / g.world);
    for (int r = 0; r < g.world; ++r) {  // this rank's slot of rank r's staging buffer: (rows_per_rank, N) 16-bit values
      const uint64_t dims[2] = {static_cast<uint64_t>(g.N[0]), static_cast<uint64_t>(g.rows_per_rank)};
      const uint64_t strides[1] = {static_cast<uint64_t>(g.N[0]) * 2};
      const uint32_t box[2] = {64, BM};
      const uint8_t* slot = static_cast<const uint8_t*>(g.peer_stage[r]) + static_cast<size_t>(g.rank) * g.rows_per_rank * g.N[0] * 2;
      if ((status = make_tensor_map(&p.map_peer[r], slot, 2, dims, strides, box)) != TB200_OK) return status;
    }
  }
  long long ldp = 0;
  for (int s = 0; s < g.n_src; ++s) ldp += g.N[s];
  p.ldp = ldp;

  {
    p.rows64 = (!pair && g.M <= 64 && g.mode != GEMM_PEER) ? 1 : 0;
    const uint64_t dims[2] = {static_cast<uint64_t>(g.K), static_cast<uint64_t>(g.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(g.K) * 2};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(p.rows64 ? 64 : BM)};
    if ((status = make_tensor_map(&p.map_a, g.A, 2, dims, strides, box)) != TB200_OK) return status;
  }
  for (int s = 0; s < g.n_src; ++s) {
    const uint64_t dims[2] = {static_cast<uint64_t>(g.N[s]), static_cast<uint64_t>(g.K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(g.N[s]) * 2};
    const uint32_t box[2] = {64, BK};
    if ((status = make_tensor_map(&p.map_b[s], g.B[s], 2, dims, strides, box)) != TB200_OK) return status;
  }
  if (pair) {
    if (g.dtype == TB200_BF16) return launch_typed<__nv_bfloat16, true>(p, g.mode, st->num_sms, stream);
    return launch_typed<__half, true>(p, g.mode, st->num_sms, stream);
  }
  if (g.dtype == TB200_BF16) return launch_typed<__nv_bfloat16, false>(p, g.mode, st->num_sms, stream);
  return launch_typed<__half, false>(p, g.mode, st->num_sms, stream);
}

int launch_splitk_finish(const SplitKFinish& f, cudaStream_t stream) {
  if (f.M <= 0 || f.N <= 0 || (f.N & 7) != 0 || f.partial == nullptr || f.C == nullptr) return TB200_ERR_INVALID;
  // the kernel moves 16 bytes at a time through every one of these
  if (!aligned16(f.partial) || !aligned16(f.C) || !aligned16(f.C2) || !aligned16(f.residual) || (f.ldp & 3) != 0 || (f.ldc & 7) != 0 ||
      (f.ldr & 7) != 0)
    return TB200_ERR_INVALID;
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  const int64_t total = static_cast<int64_t>(f.M) * (f.N / 8);
  const int threads = 256;
  int64_t blocks = (total + threads - 1) / threads;
  if (blocks > st->num_sms * 8) blocks = st->num_sms * 8;
  const dim3 grid(static_cast<unsigned>(blocks), 1, 1), block(threads, 1, 1);
  cudaError_t e;
  if (f.dtype == TB200_BF16)
    e = f.gated ? launch_chained(splitk_finish_kernel<__nv_bfloat16, true>, grid, block, 0, stream, f)
                : launch_chained(splitk_finish_kernel<__nv_bfloat16, false>, grid, block, 0, stream, f);
  else if (f.dtype == TB200_F16)
    e = f.gated ? launch_chained(splitk_finish_kernel<__half, true>, grid, block, 0, stream, f)
                : launch_chained(splitk_finish_kernel<__half, false>, grid, block, 0, stream, f);
  else return TB200_ERR_UNSUPPORTED;
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

int launch_qkv_finish(const QkvFinish& f, cudaStream_t stream) {
  if (f.M <= 0 || f.split_k < 1 || !f.partial || !f.q_out || !f.k_cache || !f.v_cache || (f.D != 64 && f.D != 128) || f.S <= 0)
    return TB200_ERR_INVALID;
  if (!aligned16(f.partial) || !aligned16(f.q_out) || !aligned16(f.k_cache) || !aligned16(f.v_cache)) return TB200_ERR_INVALID;
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  const long long items = static_cast<long long>(f.M) * (f.Hq + 2 * f.Hkv);
  long long blocks = (items * 32 + 255) / 256;
  if (blocks > st->num_sms * 8) blocks = st->num_sms * 8;
  const dim3 grid(static_cast<unsigned>(blocks), 1, 1), block(256, 1, 1);
  cudaError_t e;
  if (f.dtype == TB200_BF16) {
    e = f.D == 128 ? launch_chained(qkv_finish_kernel<__nv_bfloat16, 128>, grid, block, 0, stream, f)
                   : launch_chained(qkv_finish_kernel<__nv_bfloat16, 64>, grid, block, 0, stream, f);
  } else if (f.dtype == TB200_F16) {
    e = f.D == 128 ? launch_chained(qkv_finish_kernel<__half, 128>, grid, block, 0, stream, f)
                   : launch_chained(qkv_finish_kernel<__half, 64>, grid, block, 0, stream, f);
  } else {
    return TB200_ERR_UNSUPPORTED;
  }
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

// ====================================================================================================
// Split-K GEMM whose scratch lives in the library image (no device allocation anywhere on the path).
//
// Some hosts of this library may not allocate device memory: an inference server that hands every byte
// of HBM to its own pool at start-up, or a plugin running inside someone else's allocator, cannot let a
// callee reach for cudaMalloc.  For them the fp32 partial sums of the K slices go into the fixed array
// below instead of a caller- or library-allocated workspace.  Every GPU that loads the library carries
// the array (kStaticScratchBytes) until the process exits.
//
// `g_static_scratch` is a DEVICE symbol.  In host code its name is only a handle: the device address is
// fetched once per device with cudaGetSymbolAddress (that device current) and it is that address that is
// passed to the kernels.  Bounded-wait expiries of this path are reported in the library's one error word
// (tb200_device_status), like those of every other entry point.
constexpr size_t kStaticScratchBytes = 16u << 20;  // 16 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];

namespace {

std::mutex g_static_mu;
float* g_static_ptr[32] = {};

// First call on a device: resolve the symbol's device address (under a lock: two host threads may make their first
// call at the same time).  Allocates nothing.
int static_scratch_ptr(int dev, float** out) {
  if (dev < 0 || dev >= 32) return TB200_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return TB200_ERR_CUDA;
    g_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_ptr[dev];
  return TB200_OK;
}

}  // namespace

int gemm_splitk_static(const tb200_gemm_args* a, cudaStream_t stream) {
  if (a == nullptr) return TB200_ERR_INVALID;
  if (a->dtype != TB200_BF16 && a->dtype != TB200_F16) return TB200_ERR_UNSUPPORTED;
  if (a->m < 0 || a->n <= 0 || a->k <= 0 || (a->n & 7) || (a->k & 7)) return TB200_ERR_INVALID;
  if (a->m > (1 << 30) || a->n > (1 << 30) || a->k > (1 << 30)) return TB200_ERR_INVALID;
  if (!a->a || !a->b || !a->c || (a->act != 0 && a->act != 1) || a->split_k < 0) return TB200_ERR_INVALID;
  if (!aligned16(a->a) || !aligned16(a->b) || !aligned16(a->b2) || !aligned16(a->c) || !aligned16(a->residual)) return TB200_ERR_INVALID;
  if (a->m == 0) return TB200_OK;
  int status = TB200_OK;
  DeviceState* st = device_state(&status);   // allocates nothing: SM count + the address of the error word
  if (!st) return status;
  float* scratch = nullptr;
  if ((status = static_scratch_ptr(st->device, &scratch)) != TB200_OK) return status;

  const int M = static_cast<int>(a->m), N = static_cast<int>(a->n), K = static_cast<int>(a->k);
  const bool gated = a->b2 != nullptr;
  const int n_src = gated ? 2 : 1;
  // even one slice must fit; checked in 64 bits before any tile arithmetic in int
  const unsigned long long one_slice = static_cast<unsigned long long>(a->m) * n_src * static_cast<unsigned long long>(a->n) * sizeof(float);
  if (one_slice > kStaticScratchBytes) return TB200_ERR_SCRATCH_LIMIT;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M;
  p.K = K;
  p.k_blocks = (K + BK - 1) / BK;
  p.m_tiles = (M + BM - 1) / BM;
  p.group_m = p.m_tiles;  // decode-size M: one group
  p.n_tiles = n_src * ((N + BN - 1) / BN);
  const long long tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;   // >= 1, bounded by the 16 MiB check above
  int split = a->split_k;
  if (split == 0) {  // as many slices as fill the SMs once, at least four K blocks each
    split = static_cast<int>(st->num_sms / tiles);
    if (split > p.k_blocks / 4) split = p.k_blocks / 4;
    if (split > 32) split = 32;
    if (split < 1) split = 1;
  }
  if (split > p.k_blocks) split = p.k_blocks;
  p.kb_per_split = (p.k_blocks + split - 1) / split;
  p.split_k = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;
  if (one_slice * static_cast<unsigned long long>(p.split_k) > kStaticScratchBytes) return TB200_ERR_SCRATCH_LIMIT;
  p.n_src = n_src;
  p.tile_n = BN;
  for (int s = 0; s < n_src; ++s) {
    p.src_n[s] = N;
    p.src_tile0[s] = s * ((N + BN - 1) / BN);
  }
  for (int s = n_src; s < 4; ++s) p.src_tile0[s] = p.n_tiles;
  p.total_units = static_cast<int>(tiles) * p.split_k;
  p.err = st->err_word;
  p.wait_limit = wait_limit_cycles();
  p.partial = scratch;
  p.ldp = static_cast<long long>(n_src) * N;
  {
    p.rows64 = M <= 64 ? 1 : 0;
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(K) * 2};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(p.rows64 ? 64 : BM)};
    if ((status = make_tensor_map(&p.map_a, a->a, 2, dims, strides, box)) != TB200_OK) return status;
  }
  const void* srcs[2] = {a->b, a->b2};
  for (int s = 0; s < n_src; ++s) {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(N) * 2};
    const uint32_t box[2] = {64, BK};
    if ((status = make_tensor_map(&p.map_b[s], srcs[s], 2, dims, strides, box)) != TB200_OK) return status;
  }
  ChainScope chain;   // the finish kernel may start while the slices drain; it waits for them before it reads
  status = (a->dtype == TB200_BF16) ? launch_typed<__nv_bfloat16, false>(p, GEMM_PARTIAL, st->num_sms, stream)
                                    : launch_typed<__half, false>(p, GEMM_PARTIAL, st->num_sms, stream);
  if (status != TB200_OK) return status;
  SplitKFinish f;
  f.dtype = a->dtype;
  f.M = M;
  f.N = N;
  f.split_k = p.split_k;
  f.partial = scratch;
  f.ldp = p.ldp;
  f.gated = gated ? 1 : 0;
  f.act = a->act;
  f.row_scale = a->row_scale;
  f.residual = a->residual;
  f.ldr = N;
  f.C = a->c;
  f.ldc = N;
  return launch_splitk_finish(f, stream);
}

}  // namespace tb200

extern "C" int tb200_gemm_static_scratch(const tb200_gemm_args* args, void* stream) {
  return tb200::gemm_splitk_static(args, static_cast<cudaStream_t>(stream));
}
