// softmax(Q K^T) V for decode-sized query blocks: at most 16 new tokens per sequence on a cache of `past` keys -- the
// reference's own benchmark point (M = 16 on 1024 cached keys, benchmark/vanilla_llama_benchmark.py:32-37).
//
// Sixteen query rows are an eighth of a 128-row tcgen05 tile and the whole problem is a few hundred MFLOP on a few MB
// of cache: what it costs is launches and hand-offs, not arithmetic.  So this path is ONE kernel where the general
// path has three (split-K finish of the projection, attention over key shares, merge of the shares), and it has no
// pipeline to fill: m16n8k16 warp MMAs on registers, every warp an independent stream over its own keys.
//
//   grid     one cluster of C CTAs (C = 1, 2, 4 or 8) per (batch, q head); CTA r of a cluster walks share r of the
//            cached keys; 256 threads, one CTA per SM
//   prologue (when the projection left fp32 K-slice sums) every CTA finishes q of its head, and 16 / C of the block's
//            new k and v rows, which it sends into the shared memory of the last share's CTA: slices summed in a
//            fixed order, row scale, optional per-head RMSNorm -- what qkv_finish_kernel does.  The first q head of
//            each group also appends those rows to the caches.  The loads of the cached keys are already in flight
//            by then: they are issued before the wait for the projection kernel, which does not write them.
//   main     warp w takes the 16-key chunks w, w+8, ... of the share: TMA boxes into its own three-deep ring, one
//            mbarrier per stage (no CTA-wide barrier), S = Q K^T (Q fragments stay in registers), online softmax in
//            the log2 domain, O += P V with P taken straight from the S accumulators
//   merge    the eight warps' (m, l, O) through shared memory, then the C shares through distributed shared memory:
//            CTA r of the cluster reads column slice r of every share, in rank order, and writes those columns of O2
// Nothing goes through global scratch and nothing waits on another CTA except at the cluster's barriers.
// Every order of summation is fixed: results are bit-identical from run to run.
//
// Bound: launch and memory latency (K and V of the cache once per q head: 17 MB at the benchmark point, 3 us of HBM
// time).
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int kDecWarps = 8;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kDecRows = 16;     // query rows of a block (S <= 16; the rest are zero)
constexpr int kDecChunk = 16;    // keys per warp step
constexpr int kDecStages = 3;    // chunks in flight per warp: at the benchmark point (two or three chunks per warp) all of them, before q is even finished
constexpr float kLog2e = 1.4426950408889634f;

struct DecodeParams {
  const void* q;            // (B,Hq,S,D), or null when `partial` holds the projection's K-slice sums
  const float* partial;     // (split, B*S, (Hq + 2 Hkv) * D)
  int split;
  const float* row_scale;   // per token, or null
  int qknorm;
  float qk_eps;
  const void* q_norm_weight;
  const void* k_norm_weight;
  void* k_cache;            // (B,Hkv,cache_len,D); rows [past, past+S) are written here when partial != null
  void* v_cache;
  void* o2;                 // (B,S,Hq*D)
  float* lse2;              // (B,Hq,S) or null
  int B, S, Hq, Hkv, past, cache_len, causal;
  int n_cached;             // keys read from the caches: past (+ S when the projection has already appended them)
  int shares, keys_per_share;
  float scale_log2;
  CUtensorMap map_k, map_v;   // (B * Hkv, n_cached, D): boxes of 16 keys x 64 columns, 128-byte swizzle, zero fill past n_cached
  int* err;
  long long wait_limit;
};

template <int D>
struct DecSmem {
  static constexpr int kRow = D * 2 + 16;                       // bytes per row of q: 16 bytes of padding keep ldmatrix off bank conflicts
  static constexpr int kQ = 0;                                  // [16] rows of q
  // K and V chunks arrive by TMA as boxes of 16 keys x 64 columns (2 KiB, rows of 128 bytes, 128-byte swizzle: the
  // 16-byte piece j of row r sits at j ^ (r & 7)): a chunk is D / 64 boxes, 1 KiB-aligned
  static constexpr int kBoxBytes = kDecChunk * 128;
  static constexpr int kChunkBytes = (D / 64) * kBoxBytes;
  static constexpr int kRing = (kQ + kDecRows * kRow + 1023) / 1024 * 1024;   // per warp: kDecStages x (K chunk, V chunk)
  static constexpr int kWarpRing = kDecStages * 2 * kChunkBytes;
  static constexpr int kRingEnd = kRing + kDecWarps * kWarpRing;
  static constexpr int kBars = kRingEnd;                        // uint64 [warps][stages] + the abort flag
  static constexpr int kTotal = kBars + kDecWarps * kDecStages * 8 + 16 + 1024;   // + slack to align the base to 1 KiB
  // In the CTA of the last share (sliced projection) the last warp's ring holds the block's own k and v rows (one chunk).
  // The merge buffers alias the rings (used after every warp has drained its ring):
  static constexpr int kWarpO = kRing;                                  // float [warps][16][D]
  static constexpr int kWarpML = kWarpO + kDecWarps * kDecRows * D * 4; // float [warps][16][2]
  static constexpr int kCtaO = kWarpML + kDecWarps * kDecRows * 2 * 4;  // float [16][D]: this share's result
  static constexpr int kCtaML = kCtaO + kDecRows * D * 4;       // float [16][2]
  static_assert(kCtaML + kDecRows * 2 * 4 <= kRingEnd, "the merge buffers must fit where the rings were");
  // byte offset, within a chunk, of the 16-byte piece `piece` (0 .. D/8) of key row `row`
  static __device__ __forceinline__ uint32_t piece_offset(int row, int piece) {
    return static_cast<uint32_t>((piece >> 3) * kBoxBytes + row * 128 + (((piece & 7) ^ (row & 7)) << 4));
  }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (IsBf16<T>::value)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// The cluster's barrier in its two halves; every thread of every CTA executes both, in this order, once per phase.
// The relaxed arrival publishes nothing (it only says "I am here"), so it does not wait for this thread's stores.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ float2 ld_cluster_f32x2(uint32_t cluster_addr) {
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(cluster_addr) : "memory");
  return v;
}

// The K slices of CPT consecutive columns, summed in a fixed order.  Two steps, so that a thread can have the loads of
// several rows in flight before it consumes any: begin() issues the loads of the first kBatch slices (one slice at a
// time would cost a trip to L2 each), end() adds them up and fetches whatever slices are left.
template <int CPT>
struct SliceSum {
  static constexpr int kBatch = CPT >= 32 ? 4 : 8;
  float4 buf[kBatch][CPT / 4];
  const float* src;
  long long stride;
  int split;
  __device__ __forceinline__ void load(int s0) {
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const bool on = s0 + j < split;
      const float4* ps = reinterpret_cast<const float4*>(src + (on ? s0 + j : 0) * stride);
#pragma unroll
      for (int i = 0; i < CPT / 4; ++i) buf[j][i] = on ? __ldcg(ps + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  __device__ __forceinline__ void add(float (&v)[CPT]) {
#pragma unroll
    for (int j = 0; j < kBatch; ++j)
#pragma unroll
      for (int i = 0; i < CPT / 4; ++i) {
        v[4 * i] += buf[j][i].x; v[4 * i + 1] += buf[j][i].y; v[4 * i + 2] += buf[j][i].z; v[4 * i + 3] += buf[j][i].w;
      }
  }
  __device__ __forceinline__ void begin(const float* src_, long long stride_, int split_) {
    src = src_; stride = stride_; split = split_;
    load(0);
  }
  __device__ __forceinline__ void end(float (&v)[CPT]) {
#pragma unroll
    for (int i = 0; i < CPT; ++i) v[i] = 0.f;
    add(v);
    for (int s0 = kBatch; s0 < split; s0 += kBatch) {
      load(s0);
      add(v);
    }
  }
};

// One row of one head out of the projection's K-slice sums: TPR consecutive lanes own the row, CPT = D / TPR columns
// each, starting at column c0.  begin() starts the loads; end() sums the slices, applies the row scale and (norm) the
// per-head RMSNorm with its weight, and returns the row's values packed to 16 bits.  A row that does not exist
// (live == false) comes out as zeros.  slot: the head's position among the Hq + 2 Hkv heads of a partial row.
template <typename T, int D, int TPR>
struct RowFinish {
  static constexpr int CPT = D / TPR;
  SliceSum<CPT> sum;
  __device__ __forceinline__ void begin(const DecodeParams& p, int b, int row, bool live, int slot, int c0) {
    const long long ldp = static_cast<long long>(p.Hq + 2 * p.Hkv) * D;
    const long long tokens = static_cast<long long>(p.B) * p.S;
    sum.begin(p.partial + (static_cast<long long>(b) * p.S + (live ? row : 0)) * ldp + static_cast<long long>(slot) * D + c0, tokens * ldp,
              live ? p.split : 0);
  }
  __device__ __forceinline__ void end(const DecodeParams& p, int b, int row, bool live, int c0, bool norm, const T* norm_weight,
                                      uint32_t (&w)[CPT / 2]) {
    float v[CPT];
    sum.end(v);
    const float rs = (live && p.row_scale) ? p.row_scale[static_cast<long long>(b) * p.S + row] : 1.f;
#pragma unroll
    for (int i = 0; i < CPT; ++i) v[i] *= rs;
    if (norm) {  // warp-uniform
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < CPT; ++i) ss = fmaf(v[i], v[i], ss);
#pragma unroll
      for (int o = 1; o < TPR; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float r = live ? rsqrtf(ss / static_cast<float>(D) + p.qk_eps) : 0.f;
#pragma unroll
      for (int i = 0; i < CPT; ++i) v[i] *= r * (norm_weight ? static_cast<float>(norm_weight[c0 + i]) : 1.f);
    }
#pragma unroll
    for (int i = 0; i < CPT / 2; ++i) w[i] = Pack2<T>::pack(v[2 * i], v[2 * i + 1]);
  }
};

// One 16-key chunk: s = scale * Q K^T (masked), online softmax update of (m, l, o), o += P V.
// kbase / vbase: shared-memory addresses of the chunk's K and V rows; key0: index of the chunk's first key among ALL
// keys of the sequence (for the causal test); n_valid: keys of the chunk that exist.
template <typename T, int D>
__device__ __forceinline__ void chunk_step(const uint32_t (&qf)[D / 16][4], uint32_t kbase, uint32_t vbase, int key0, int n_valid,
                                           const DecodeParams& p, float (&m)[2], float (&l)[2], float (&o)[D / 8][4]) {
  using L = DecSmem<D>;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  float s[2][4];
#pragma unroll
  for (int nb = 0; nb < 2; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[nb][i] = 0.f;
  {  // matrices of one ldmatrix.x4: (keys 0-7, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 0-7), (keys 8-15, d 8-15) of a 16-wide k step
    const int mat = lane >> 3, r = lane & 7;
    const int krow = (mat >> 1) * 8 + r;   // this lane's row address: key krow, columns (2 ks + (mat & 1)) * 8 ...
    // even and odd k steps into accumulators of their own: four chains of D / 32 dependent MMAs instead of two of D / 16
    float s2[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int i = 0; i < 4; ++i) s2[nb][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ks += 2) {
      uint32_t kf[4], kg[4];
      ldmatrix_x4(kf, kbase + L::piece_offset(krow, 2 * ks + (mat & 1)));
      ldmatrix_x4(kg, kbase + L::piece_offset(krow, 2 * ks + 2 + (mat & 1)));
      mma_16816<T>(s[0], qf[ks], kf[0], kf[1]);
      mma_16816<T>(s[1], qf[ks], kf[2], kf[3]);
      mma_16816<T>(s2[0], qf[ks + 1], kg[0], kg[1]);
      mma_16816<T>(s2[1], qf[ks + 1], kg[2], kg[3]);
    }
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[nb][i] += s2[nb][i];
  }
  // thread (g, t) holds rows g (i = 0, 1) and g + 8 (i = 2, 3), keys nb * 8 + 2 t + (i & 1)
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nb = 0; nb < 2; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int key = nb * 8 + 2 * t + (i & 1);
      const int row = g + (i >> 1) * 8;
      bool ok = key < n_valid;
      if (p.causal) ok = ok && (key0 + key <= p.past + row);
      const float x = ok ? s[nb][i] * p.scale_log2 : -INFINITY;
      s[nb][i] = x;
      mx[i >> 1] = fmaxf(mx[i >> 1], x);
    }
  uint32_t pf[4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    const float m_new = fmaxf(m[h], mx[h]);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;   // a row with no visible key so far: every p is 0
    const float alpha = fast_exp2(m[h] - m_use);            // m[h] = -inf -> 0
    m[h] = m_new;
    float psum = 0.f;
    float pv[4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float e = fast_exp2(s[nb][h * 2 + j] - m_use);
        pv[nb * 2 + j] = e;
        psum += e;
      }
    l[h] = fmaf(l[h], alpha, psum);   // this thread's share of the row sum; the quad is added up at the end
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) {
      o[nb][h * 2] *= alpha;
      o[nb][h * 2 + 1] *= alpha;
    }
    // A fragment of P (16 rows x 16 keys): a0 = row g keys 2t,2t+1; a1 = row g+8; a2 = row g keys 8+2t..; a3 = row g+8
    pf[h] = Pack2<T>::pack(pv[0], pv[1]);
    pf[2 + h] = Pack2<T>::pack(pv[2], pv[3]);
  }
  {  // matrices of one transposed ldmatrix.x4: (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15)
    const int mat = lane >> 3, r = lane & 7;
    const int vrow = (mat & 1) * 8 + r;
#pragma unroll
    for (int nb = 0; nb < D / 8; nb += 2) {
      uint32_t vf[4];
      ldmatrix_x4_trans(vf, vbase + L::piece_offset(vrow, nb + (mat >> 1)));
      mma_16816<T>(o[nb], pf, vf[0], vf[1]);
      mma_16816<T>(o[nb + 1], pf, vf[2], vf[3]);
    }
  }
}


// C: CTAs per cluster = shares of the cached keys per (batch, q head).
template <typename T, int D, int C>
__global__ void __launch_bounds__(kDecThreads) attn_decode_kernel(const __grid_constant__ DecodeParams p) {
  using L = DecSmem<D>;
  constexpr int kRow = L::kRow;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  pdl_launch_dependents();
  const bool from_partial = p.partial != nullptr;
  if (from_partial) cluster_arrive_relaxed();   // "this CTA runs": a peer may write its shared memory after waiting for this
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int share = static_cast<int>(blockIdx.x) % C;   // = rank in the cluster
  const int head_lin = static_cast<int>(blockIdx.x) / C;
  const int b = head_lin / p.Hq, hq = head_lin - b * p.Hq;
  const int group = p.Hq / p.Hkv;
  const int hkv = hq / group;
  // The CTA of the last share also takes the block's own keys, which its peers finish into its shared memory: its
  // last warp keeps out of the cached chunks, gives its ring to those rows and processes them.
  const bool new_keys_here = from_partial && share == C - 1;
  const int chunk_warps = new_keys_here ? kDecWarps - 1 : kDecWarps;
  T* kc = static_cast<T*>(p.k_cache) + (static_cast<long long>(b) * p.Hkv + hkv) * p.cache_len * D;
  T* vc = static_cast<T*>(p.v_cache) + (static_cast<long long>(b) * p.Hkv + hkv) * p.cache_len * D;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars) + warp * kDecStages;   // this warp's, one per stage
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kBars + kDecWarps * kDecStages * 8);
  const AbortCtx ctx{p.err, abort_flag, p.wait_limit};
  if (lane == 0) {   // every warp sets up its own barriers: no CTA-wide barrier before its first load
    for (int st = 0; st < kDecStages; ++st) mbar_init(&bars[st], 1);
    if (warp == 0) {
      *abort_flag = 0;
      tma_prefetch_desc(&p.map_k);
      tma_prefetch_desc(&p.map_v);
    }
    fence_mbar_init();
  }
  __syncwarp();

  // ---- the cached keys of this share: start the first chunks before q is touched.  With a sliced projection the
  //      kernel before this one writes only its K-slice sums: the cached rows are older than the call, and their
  //      loads need not wait for that kernel.  (An unsliced projection appends the new rows itself: wait first.)
  if (!from_partial) pdl_wait();
  const int k_begin = min(p.n_cached, share * p.keys_per_share);
  const int k_end = min(p.n_cached, k_begin + p.keys_per_share);
  const int n_chunks = (k_end - k_begin + kDecChunk - 1) / kDecChunk;   // of the CTA; warp w takes chunks w, w + chunk_warps, ...
  uint8_t* ring = smem + L::kRing + warp * L::kWarpRing;
  auto load_chunk = [&](int c, int stage) {   // one lane; c: chunk index within the share
    const int key0 = k_begin + c * kDecChunk;
    uint8_t* ks = ring + stage * 2 * L::kChunkBytes;
    uint8_t* vs = ks + L::kChunkBytes;
    mbar_arrive_expect_tx(&bars[stage], 2 * L::kChunkBytes);   // rows past n_cached arrive as zeros and count
#pragma unroll
    for (int dc = 0; dc < D / 64; ++dc) {
      tma_load_3d(ks + dc * L::kBoxBytes, &p.map_k, &bars[stage], dc * 64, key0, b * p.Hkv + hkv);
      tma_load_3d(vs + dc * L::kBoxBytes, &p.map_v, &bars[stage], dc * 64, key0, b * p.Hkv + hkv);
    }
  };
  int issued = 0;
  if (warp < chunk_warps) {
    for (; issued < kDecStages; ++issued) {
      const int c = warp + chunk_warps * issued;
      if (c < n_chunks && lane == 0) load_chunk(c, issued);
    }
  }
  if (from_partial) pdl_wait();   // the K-slice sums come from the kernel before this one

  // ---- q (and this CTA's part of the new k, v rows) out of the K-slice sums, or q as the projection left it
  if (from_partial) {
    // q: sixteen consecutive lanes per row.  New rows [share * 16 / C, (share + 1) * 16 / C) of k (threads [0, D/2))
    // and v (threads [D/2, D)): into the shared memory of the last share's CTA, and -- from the first q head of a
    // group -- into the caches.  The loads of both are in flight before either is consumed.
    constexpr int kQTpr = kDecThreads / kDecRows, kQCpt = D / kQTpr;
    constexpr int kRowsHere = kDecRows / C;
    constexpr int kKvTpr = C * D / 32, kKvCpt = 32 / C;
    const int q_row = threadIdx.x / kQTpr, q_c0 = (threadIdx.x % kQTpr) * kQCpt;
    const bool kv_thread = threadIdx.x < D;   // whole warps
    const int is_v = kv_thread ? threadIdx.x / (D / 2) : 0;
    const int kv_idx = threadIdx.x - is_v * (D / 2);
    const int kv_row = share * kRowsHere + kv_idx / kKvTpr, kv_c0 = (kv_idx % kKvTpr) * kKvCpt;
    const bool kv_live = kv_row < p.S;
    RowFinish<T, D, kQTpr> fq;
    RowFinish<T, D, kKvTpr> fkv;
    fq.begin(p, b, q_row, q_row < p.S, hq, q_c0);
    if (kv_thread) fkv.begin(p, b, kv_row, kv_live, p.Hq + (is_v ? p.Hkv : 0) + hkv, kv_c0);
    {
      uint32_t w[kQCpt / 2];
      fq.end(p, b, q_row, q_row < p.S, q_c0, p.qknorm != 0, static_cast<const T*>(p.q_norm_weight), w);
      uint2* ds = reinterpret_cast<uint2*>(smem + L::kQ + q_row * kRow + q_c0 * 2);
#pragma unroll
      for (int i = 0; i < kQCpt / 4; ++i) ds[i] = make_uint2(w[2 * i], w[2 * i + 1]);
    }
    cluster_wait();   // every CTA of the cluster has started
    if (kv_thread) {
      uint32_t w[kKvCpt / 2];
      fkv.end(p, b, kv_row, kv_live, kv_c0, !is_v && p.qknorm != 0, static_cast<const T*>(p.k_norm_weight), w);
      // the layout a TMA box would have: 8-byte half i of the row's 16-byte piece (kv_c0 + 4 i) / 8
      const uint32_t chunk = mapa_u32(smem_u32(smem + L::kRing + (kDecWarps - 1) * L::kWarpRing + is_v * L::kChunkBytes), C - 1);
#pragma unroll
      for (int i = 0; i < kKvCpt / 4; ++i) {
        const int col = kv_c0 + 4 * i;
        const uint32_t dst = chunk + L::piece_offset(kv_row, col >> 3) + (col & 4) * 2;
        asm volatile("st.shared::cluster.v2.b32 [%0], {%1, %2};" ::"r"(dst), "r"(w[2 * i]), "r"(w[2 * i + 1]) : "memory");
      }
      cluster_arrive();   // "my rows are written"; waited for below.  Before the cache append: the arrival must not wait for it
      if (kv_live && hq == hkv * group) {
        uint2* dg = reinterpret_cast<uint2*>((is_v ? vc : kc) + static_cast<long long>(p.past + kv_row) * D + kv_c0);
#pragma unroll
        for (int i = 0; i < kKvCpt / 4; ++i) dg[i] = make_uint2(w[2 * i], w[2 * i + 1]);
      }
    } else {
      cluster_arrive();
    }
  } else {
    const T* q = static_cast<const T*>(p.q) + (static_cast<long long>(b) * p.Hq + hq) * p.S * D;
    constexpr int kVecs = D / 8;
    for (int i = threadIdx.x; i < kDecRows * kVecs; i += kDecThreads) {
      const int r = i / kVecs, v = i - r * kVecs;
      uint4 x = make_uint4(0, 0, 0, 0);
      if (r < p.S) x = *reinterpret_cast<const uint4*>(q + static_cast<long long>(r) * D + v * 8);
      *reinterpret_cast<uint4*>(smem + L::kQ + r * kRow + v * 16) = x;
    }
  }
  __syncthreads();

  uint32_t qf[D / 16][4];
  {  // A fragments of Q: matrices (rows 0-7, d 0-7), (rows 8-15, d 0-7), (rows 0-7, d 8-15), (rows 8-15, d 8-15)
    const int mat = lane >> 3, r = lane & 7;
    const uint32_t lane_addr = smem_u32(smem + L::kQ) + ((mat & 1) * 8 + r) * kRow + (mat >> 1) * 16;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) ldmatrix_x4(qf[ks], lane_addr + ks * 32);
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int nb = 0; nb < D / 8; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[nb][i] = 0.f;

  // ---- main loop over this warp's chunks
  if (warp < chunk_warps) {
    int stage = 0;
    uint32_t parity = 0;
    for (int c = warp; c < n_chunks; c += chunk_warps) {
      if (!mbar_wait(&bars[stage], parity, ctx, 700)) break;   // gave up: the barriers below are still passed
      const int key0 = k_begin + c * kDecChunk;
      const uint32_t kbase = smem_u32(ring + stage * 2 * L::kChunkBytes);
      chunk_step<T, D>(qf, kbase, kbase + L::kChunkBytes, key0, min(kDecChunk, k_end - key0), p, m, l, o);
      __syncwarp();   // every lane has read the stage
      const int cn = warp + chunk_warps * issued;   // refill it
      if (cn < n_chunks && lane == 0) load_chunk(cn, stage);
      ++issued;
      if (++stage == kDecStages) { stage = 0; parity ^= 1; }
    }
  }
  if (from_partial) {
    cluster_wait();   // every CTA's new rows have landed in the last share's shared memory
    if (new_keys_here && warp == kDecWarps - 1) {
      const uint32_t kbase = smem_u32(ring);
      chunk_step<T, D>(qf, kbase, kbase + L::kChunkBytes, p.past, p.S, p, m, l, o);
    }
  }

  // ---- merge the warps
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  __syncthreads();   // every warp is done with its ring: the merge buffers alias it
  {
    float* wo = reinterpret_cast<float*>(smem + L::kWarpO) + warp * kDecRows * D;
    float* wml = reinterpret_cast<float*>(smem + L::kWarpML) + warp * kDecRows * 2;
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) {
      *reinterpret_cast<float2*>(wo + g * D + nb * 8 + 2 * t) = make_float2(o[nb][0], o[nb][1]);
      *reinterpret_cast<float2*>(wo + (g + 8) * D + nb * 8 + 2 * t) = make_float2(o[nb][2], o[nb][3]);
    }
    if (t == 0) {
      wml[g * 2] = m[0]; wml[g * 2 + 1] = l[0];
      wml[(g + 8) * 2] = m[1]; wml[(g + 8) * 2 + 1] = l[1];
    }
  }
  __syncthreads();
  {
    constexpr int TPR = kDecThreads / kDecRows, CPT = D / TPR;
    const int row = threadIdx.x / TPR, c0 = (threadIdx.x % TPR) * CPT;
    const float* wml = reinterpret_cast<const float*>(smem + L::kWarpML);
    float mw[kDecWarps], lw[kDecWarps];
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float2 x = *reinterpret_cast<const float2*>(wml + (w * kDecRows + row) * 2);
      mw[w] = x.x; lw[w] = x.y;
      mm = fmaxf(mm, x.x);
    }
    const float m_use = mm == -INFINITY ? 0.f : mm;
    float ll = 0.f, acc[CPT];
#pragma unroll
    for (int i = 0; i < CPT; ++i) acc[i] = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {   // fixed order
      const float f = fast_exp2(mw[w] - m_use);
      ll = fmaf(f, lw[w], ll);
      const float4* wo = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(smem + L::kWarpO) + (w * kDecRows + row) * D + c0);
#pragma unroll
      for (int i = 0; i < CPT / 4; ++i) {
        const float4 x = wo[i];
        acc[4 * i] = fmaf(f, x.x, acc[4 * i]); acc[4 * i + 1] = fmaf(f, x.y, acc[4 * i + 1]);
        acc[4 * i + 2] = fmaf(f, x.z, acc[4 * i + 2]); acc[4 * i + 3] = fmaf(f, x.w, acc[4 * i + 3]);
      }
    }
    float4* co = reinterpret_cast<float4*>(reinterpret_cast<float*>(smem + L::kCtaO) + row * D + c0);
#pragma unroll
    for (int i = 0; i < CPT / 4; ++i) co[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
    if (threadIdx.x % TPR == 0) *reinterpret_cast<float2*>(reinterpret_cast<float*>(smem + L::kCtaML) + row * 2) = make_float2(mm, ll);
  }

  // ---- merge the shares of the cluster: CTA r finishes columns [r * D / C, (r + 1) * D / C) of every row.  All the
  //      remote loads of an output pair are independent: one trip through the cluster's network, not one per share.
  cluster_arrive();
  cluster_wait();
  {
    constexpr int kCols = D / C, kPairs = kCols / 2;
    const uint32_t o_local = smem_u32(smem + L::kCtaO), ml_local = smem_u32(smem + L::kCtaML);
    for (int e = threadIdx.x; e < kDecRows * kPairs; e += kDecThreads) {
      const int row = e / kPairs, col = share * kCols + 2 * (e - row * kPairs);
      if (row >= p.S) continue;
      float2 ml[C], ov[C];
#pragma unroll
      for (int r = 0; r < C; ++r) {
        ml[r] = ld_cluster_f32x2(mapa_u32(ml_local + row * 8, r));
        ov[r] = ld_cluster_f32x2(mapa_u32(o_local + (row * D + col) * 4, r));
      }
      float mm = -INFINITY;
#pragma unroll
      for (int r = 0; r < C; ++r) mm = fmaxf(mm, ml[r].x);
      const float m_use = mm == -INFINITY ? 0.f : mm;
      float ll = 0.f, acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int r = 0; r < C; ++r) {   // rank order: fixed
        const float f = fast_exp2(ml[r].x - m_use);
        ll = fmaf(f, ml[r].y, ll);
        acc0 = fmaf(f, ov[r].x, acc0);
        acc1 = fmaf(f, ov[r].y, acc1);
      }
      const float inv = ll > 0.f ? 1.f / ll : 0.f;
      *reinterpret_cast<uint32_t*>(static_cast<T*>(p.o2) + ((static_cast<long long>(b) * p.S + row) * p.Hq + hq) * D + col) =
          Pack2<T>::pack(acc0 * inv, acc1 * inv);
      if (p.lse2 != nullptr && col == 0) p.lse2[(static_cast<long long>(b) * p.Hq + hq) * p.S + row] = mm + log2f(ll);
    }
  }
  cluster_arrive_relaxed();   // nobody's shared memory goes away while a peer still reads it
  cluster_wait();
}

template <typename T, int D, int C>
int launch_one(const DecodeParams& p, cudaStream_t stream) {
  static bool attr_set[32] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 31]) {
    if (cudaFuncSetAttribute(attn_decode_kernel<T, D, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecSmem<D>::kTotal) != cudaSuccess)
      return TB200_ERR_CUDA;
    attr_set[dev & 31] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(p.B * p.Hq * C), 1, 1);
  cfg.blockDim = dim3(kDecThreads, 1, 1);
  cfg.dynamicSmemBytes = DecSmem<D>::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = C;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (chain_next_launch()) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  if (cudaLaunchKernelEx(&cfg, attn_decode_kernel<T, D, C>, p) != cudaSuccess) return TB200_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

template <typename T, int D>
int launch_shares(const DecodeParams& p, cudaStream_t stream) {
  switch (p.shares) {
    case 1: return launch_one<T, D, 1>(p, stream);
    case 2: return launch_one<T, D, 2>(p, stream);
    case 4: return launch_one<T, D, 4>(p, stream);
    case 8: return launch_one<T, D, 8>(p, stream);
    default: return TB200_ERR_INVALID;
  }
}

}  // namespace

bool attn_decode_applies(int B, int S, int Hq, int D) {
  return S >= 1 && S <= kDecRows && (D == 64 || D == 128) && static_cast<long long>(B) * Hq <= (1 << 20);
}

int launch_attn_decode(const AttnDecodeLaunch& a, cudaStream_t stream) {
  if (!attn_decode_applies(a.B, a.S, a.Hq, a.D)) return TB200_ERR_UNSUPPORTED;
  if (a.dtype != TB200_BF16 && a.dtype != TB200_F16) return TB200_ERR_UNSUPPORTED;
  if (a.Hkv <= 0 || a.Hq % a.Hkv != 0 || a.past < 0 || a.cache_len < a.past + a.S) return TB200_ERR_INVALID;
  if ((a.q == nullptr) == (a.partial == nullptr) || !a.k_cache || !a.v_cache || !a.o2) return TB200_ERR_INVALID;
  if (a.partial != nullptr && a.split < 1) return TB200_ERR_INVALID;
  if (!aligned16(a.q) || !aligned16(a.partial) || !aligned16(a.k_cache) || !aligned16(a.v_cache) || !aligned16(a.o2) ||
      !aligned16(a.q_norm_weight) || !aligned16(a.k_norm_weight) || !aligned4(a.row_scale) || !aligned4(a.lse2))
    return TB200_ERR_INVALID;
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  DecodeParams p;
  memset(&p, 0, sizeof(p));
  p.q = a.q; p.partial = a.partial; p.split = a.split; p.row_scale = a.row_scale;
  p.qknorm = a.qknorm; p.qk_eps = a.qk_eps; p.q_norm_weight = a.q_norm_weight; p.k_norm_weight = a.k_norm_weight;
  p.k_cache = a.k_cache; p.v_cache = a.v_cache; p.o2 = a.o2; p.lse2 = a.lse2;
  p.B = a.B; p.S = a.S; p.Hq = a.Hq; p.Hkv = a.Hkv; p.past = a.past; p.cache_len = a.cache_len; p.causal = a.causal;
  p.n_cached = a.partial != nullptr ? a.past : a.past + a.S;
  p.scale_log2 = a.sm_scale * kLog2e;
  // shares: one CTA per SM at most (a CTA's rings take most of an SM's shared memory), at least a chunk per warp in
  // every share, a power of two up to 8 (the portable cluster size)
  const long long heads = static_cast<long long>(a.B) * a.Hq;
  int shares = 1;
  while (shares < 8 && heads * shares * 2 <= st->num_sms && p.n_cached >= kDecWarps * kDecChunk * shares * 2) shares *= 2;
  p.shares = shares;
  const int per = (p.n_cached + shares - 1) / shares;
  p.keys_per_share = (per + kDecChunk - 1) / kDecChunk * kDecChunk;
  p.err = st->err_word;
  p.wait_limit = wait_limit_cycles();
  {  // rows past n_cached read as zeros; an empty cache still needs a map with one row (no box of it is ever loaded)
    const uint64_t D = static_cast<uint64_t>(a.D);
    const uint64_t dims[3] = {D, static_cast<uint64_t>(p.n_cached > 0 ? p.n_cached : 1), static_cast<uint64_t>(a.B) * a.Hkv};
    const uint64_t strides[2] = {D * 2, static_cast<uint64_t>(a.cache_len) * D * 2};
    const uint32_t box[3] = {64, kDecChunk, 1};
    if ((status = make_tensor_map(&p.map_k, a.k_cache, 3, dims, strides, box)) != TB200_OK) return status;
    if ((status = make_tensor_map(&p.map_v, a.v_cache, 3, dims, strides, box)) != TB200_OK) return status;
  }
  if (a.dtype == TB200_BF16) return a.D == 128 ? launch_shares<__nv_bfloat16, 128>(p, stream) : launch_shares<__nv_bfloat16, 64>(p, stream);
  return a.D == 128 ? launch_shares<__half, 128>(p, stream) : launch_shares<__half, 64>(p, stream);
}

}  // namespace tb200
