// KV-cache eviction, the step after the per-key scores and the top-k of the KeyFormer / RoCo blocks: keep the cache
// positions an index list names (plus, optionally, the most recent ones) and pack them, in ascending position order,
// to the front of a destination cache.  The reference emits the scores (`C_out`, `C_out1/2`) and stops there; the
// cache layout is its `(H, P+M, D)` (convert_eval_rms.py:82-83) with an optional leading batch axis.
//
// Bound: HBM.  Algorithmic bytes = kept positions x head_dim x element size x 2 tensors x (read + write).
//
// One CTA packs a span of 64 x G destination positions of one cache row (one (batch, kv head)); G (1..16) grows with
// the amount of work so that the per-CTA preamble below is paid once per several groups while the grid still fills
// the SMs.  The CTA rebuilds the row's keep-bitmap in shared memory from the index list (the list is a few KB and
// stays in L2; duplicates and out-of-range entries fall out of the bitmap for free), counts the kept positions before
// each bitmap word (a block-wide exclusive scan), finds the source positions of its slots, and moves their K and V
// vectors with 16-byte loads and stores, all loads of a thread in flight before its first store.  No atomics on global memory, no floating-point arithmetic: the result is bit-exact and
// the same on every run.
#include <cstdlib>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int kEvictThreads = 256;
constexpr int kEvictSlots = 64;          // destination positions per group: one round of loads and stores of a CTA
constexpr int kEvictMaxGroups = 16;      // groups per CTA
constexpr int kEvictMaxWords = 8192;     // bitmap words: up to 262144 cache positions per row

struct EvictParams {
  const int32_t* idx;   // (rows, n_idx)
  const uint4* k_src;
  const uint4* v_src;
  uint4* k_dst;
  uint4* v_dst;
  int32_t* kept_pos;    // (rows, max_keep) or null
  int32_t* new_len;     // (rows) or null
  int n_idx, kv_len, keep_recent, words, max_keep, groups;
  long long src_pitch, dst_pitch;  // 16-byte units per cache row of the source / destination
};

// The keep-bitmap of cache row `row` in shared memory (index list united with the recent window) and the block-wide
// exclusive count of kept positions: returns the number of kept positions before the run of words [*w_begin, *w_end)
// this thread owns; *total (shared) holds the row's count.  Ends with a barrier: bitmap and *total are readable.
__device__ __forceinline__ uint32_t keep_bitmap(const EvictParams& p, long long row, uint32_t* bitmap, uint32_t* warp_sums,
                                                uint32_t* total, int* w_begin_out, int* w_end_out) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int w = tid; w < p.words; w += kEvictThreads) {
    // the recent window [kv_len - keep_recent, kv_len) is written as whole-word masks
    const int lo = max(p.kv_len - p.keep_recent, 0) - w * 32, hi = p.kv_len - w * 32;
    uint32_t m = 0u;
    if (hi > 0 && lo < 32) {
      const uint32_t upto_hi = hi >= 32 ? 0xffffffffu : ((1u << hi) - 1u);
      const uint32_t below_lo = lo <= 0 ? 0u : ((1u << lo) - 1u);
      m = upto_hi & ~below_lo;
    }
    bitmap[w] = m;
  }
  __syncthreads();
  const int32_t* my_idx = p.idx + row * p.n_idx;
  for (int i = tid; i < p.n_idx; i += kEvictThreads) {
    const int pos = my_idx[i];
    if (pos >= 0 && pos < p.kv_len) atomicOr(&bitmap[pos >> 5], 1u << (pos & 31));
  }
  __syncthreads();

  // exclusive prefix count over the words: a contiguous run of words per thread, then a scan of the 256 run totals
  const int per_thread = (p.words + kEvictThreads - 1) / kEvictThreads;
  const int w_begin = min(tid * per_thread, p.words), w_end = min(w_begin + per_thread, p.words);
  uint32_t mine = 0;
  for (int w = w_begin; w < w_end; ++w) mine += __popc(bitmap[w]);
  uint32_t incl = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += up;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    uint32_t v = lane < kEvictThreads / 32 ? warp_sums[lane] : 0u;
    uint32_t s = v;
#pragma unroll
    for (int d = 1; d < kEvictThreads / 32; d <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, s, d);
      if (lane >= d) s += up;
    }
    if (lane < kEvictThreads / 32) warp_sums[lane] = s - v;  // exclusive
    if (lane == kEvictThreads / 32 - 1) *total = s;
  }
  __syncthreads();
  *w_begin_out = w_begin;
  *w_end_out = w_end;
  return warp_sums[warp] + incl - mine;
}

// VEC: 16-byte units per position (head_dim * 2 / 16)
template <int VEC>
__global__ void __launch_bounds__(kEvictThreads) kv_compact_kernel(const EvictParams p) {
  extern __shared__ uint32_t evict_smem[];
  uint32_t* bitmap = evict_smem;  // [words]
  __shared__ int src_pos[kEvictSlots * kEvictMaxGroups];
  __shared__ uint32_t warp_sums[kEvictThreads / 32];
  __shared__ uint32_t total_s;

  const int tid = threadIdx.x;
  const long long row = blockIdx.y;
  const int span = p.groups * kEvictSlots;
  const int slot0 = blockIdx.x * span;

  for (int s = tid; s < span; s += kEvictThreads) src_pos[s] = -1;
  int w_begin, w_end;
  uint32_t run = keep_bitmap(p, row, bitmap, warp_sums, &total_s, &w_begin, &w_end);
  for (int w = w_begin; w < w_end; ++w) {
    const uint32_t bits = bitmap[w];
    const uint32_t cnt = __popc(bits);
    // the slots this CTA packs are [slot0, slot0 + span): record where they come from
    if (cnt != 0u && run + cnt > static_cast<uint32_t>(slot0) && run < static_cast<uint32_t>(slot0 + span)) {
      uint32_t rest = bits;
      uint32_t dest = run;
      while (rest != 0u) {
        const int b = __ffs(rest) - 1;
        rest &= rest - 1u;
        const int s = static_cast<int>(dest) - slot0;
        if (s >= 0 && s < span) src_pos[s] = w * 32 + b;
        ++dest;
      }
    }
    run += cnt;
  }
  __syncthreads();
  const int n_kept = static_cast<int>(total_s);
  if (blockIdx.x == 0 && tid == 0 && p.new_len != nullptr) p.new_len[row] = n_kept;
  if (p.kept_pos != nullptr)
    for (int s = tid; s < span && slot0 + s < p.max_keep; s += kEvictThreads)
      p.kept_pos[row * p.max_keep + slot0 + s] = src_pos[s];  // -1 beyond the kept count
  const int n_span = min(max(n_kept - slot0, 0), span);

  // move K and V: 64 positions x VEC units per tensor, every load of a thread issued before its first store
  constexpr int kUnits = kEvictSlots * VEC;
  constexpr int kPerThread = kUnits / kEvictThreads;
  static_assert(kUnits % kEvictThreads == 0, "units must divide over the threads");
  const uint4* ks = p.k_src + row * p.src_pitch;
  const uint4* vs = p.v_src + row * p.src_pitch;
  for (int g0 = 0; g0 < n_span; g0 += kEvictSlots) {
    const int n_here = min(n_span - g0, kEvictSlots);
    uint4* kd = p.k_dst + row * p.dst_pitch + static_cast<long long>(slot0 + g0) * VEC;
    uint4* vd = p.v_dst + row * p.dst_pitch + static_cast<long long>(slot0 + g0) * VEC;
    uint4 kreg[kPerThread], vreg[kPerThread];
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int u = tid + i * kEvictThreads;
      const int s = u / VEC, v = u % VEC;
      if (s < n_here) {
        const long long off = static_cast<long long>(src_pos[g0 + s]) * VEC + v;
        kreg[i] = __ldg(ks + off);
        vreg[i] = __ldg(vs + off);
      }
    }
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int u = tid + i * kEvictThreads;
      if (u / VEC < n_here) {
        kd[u] = kreg[i];
        vd[u] = vreg[i];
      }
    }
  }
}

// The same packing inside the source caches.  A packed position never lies behind its source (slot j <= p_j), so a
// row can be packed front to back by ONE CTA: rounds of 128 slots, every load of a round done (block barrier) before
// its first store; a later round's sources lie behind everything earlier rounds wrote.  Slots that are already in
// place (the kept prefix of a row) are neither read nor written.  One CTA per row: the grid fills the GPU only with
// a few hundred cache rows, which is what a batch of sequences has.
constexpr int kInplaceSlots = 128;

template <int VEC>
__global__ void __launch_bounds__(kEvictThreads) kv_compact_inplace_kernel(const EvictParams p) {
  extern __shared__ uint32_t evict_smem[];
  uint32_t* bitmap = evict_smem;  // [words]
  __shared__ int src_pos[kInplaceSlots];
  __shared__ uint32_t warp_sums[kEvictThreads / 32];
  __shared__ uint32_t total_s;

  const int tid = threadIdx.x;
  const long long row = blockIdx.x;
  int w_begin, w_end;
  const uint32_t run0 = keep_bitmap(p, row, bitmap, warp_sums, &total_s, &w_begin, &w_end);
  const int n_kept = static_cast<int>(total_s);
  uint32_t run_end = run0;  // kept positions before the end of this thread's run of words
  for (int w = w_begin; w < w_end; ++w) run_end += __popc(bitmap[w]);
  if (tid == 0 && p.new_len != nullptr) p.new_len[row] = n_kept;
  if (p.kept_pos != nullptr) {
    uint32_t dest = run0;
    for (int w = w_begin; w < w_end; ++w)
      for (uint32_t rest = bitmap[w]; rest != 0u; rest &= rest - 1u) p.kept_pos[row * p.max_keep + dest++] = w * 32 + __ffs(rest) - 1;
    for (int s = n_kept + tid; s < p.max_keep; s += kEvictThreads) p.kept_pos[row * p.max_keep + s] = -1;
  }

  constexpr int kUnits = kInplaceSlots * VEC;
  constexpr int kPerThread = kUnits / kEvictThreads;
  uint4* kc = p.k_dst + row * p.dst_pitch;
  uint4* vc = p.v_dst + row * p.dst_pitch;
  for (int g0 = 0; g0 < n_kept; g0 += kInplaceSlots) {
    // sources of the slots [g0, g0 + 128): every thread whose run of words holds some of them walks that run
    if (run_end > static_cast<uint32_t>(g0) && run0 < static_cast<uint32_t>(g0 + kInplaceSlots)) {
      uint32_t dest = run0;
      for (int w = w_begin; w < w_end; ++w)
        for (uint32_t rest = bitmap[w]; rest != 0u; rest &= rest - 1u, ++dest) {
          const int s = static_cast<int>(dest) - g0;
          if (s >= 0 && s < kInplaceSlots) src_pos[s] = w * 32 + __ffs(rest) - 1;
        }
    }
    __syncthreads();
    const int n_here = min(n_kept - g0, kInplaceSlots);
    uint4 kreg[kPerThread], vreg[kPerThread];
    bool move[kPerThread];
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int u = tid + i * kEvictThreads;
      const int s = u / VEC, v = u % VEC;
      move[i] = s < n_here && src_pos[s] != g0 + s;
      if (move[i]) {
        const long long off = static_cast<long long>(src_pos[s]) * VEC + v;
        kreg[i] = kc[off];  // plain loads: this kernel writes the tensor it reads
        vreg[i] = vc[off];
      }
    }
    __syncthreads();  // every source of the round is in registers before a slot of the round is overwritten
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      if (move[i]) {
        const long long off = static_cast<long long>(g0) * VEC + tid + i * kEvictThreads;
        kc[off] = kreg[i];
        vc[off] = vreg[i];
      }
    }
  }
}

int dev_of() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev;
}

bool overlaps(const void* a, size_t an, const void* b, size_t bn) {
  const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
  return a0 < b0 + bn && b0 < a0 + an;
}

}  // namespace

int launch_kv_compact(const tb200_kv_compact_args& a, cudaStream_t stream) {
  if (a.dtype != TB200_BF16 && a.dtype != TB200_F16) return TB200_ERR_UNSUPPORTED;
  if (a.head_dim != 64 && a.head_dim != 128) return TB200_ERR_UNSUPPORTED;
  if (a.rows < 0 || a.kv_len < 0 || a.n_idx < 0 || a.keep_recent < 0) return TB200_ERR_INVALID;
  if (a.src_cache_len < a.kv_len) return TB200_ERR_INVALID;
  const long long max_keep = tb200_kv_compact_max_keep(&a);
  if (a.dst_cache_len < max_keep) return TB200_ERR_INVALID;
  if (a.rows == 0 || max_keep == 0) {
    if (a.rows > 0 && a.new_len != nullptr && cudaMemsetAsync(a.new_len, 0, sizeof(int32_t) * a.rows, stream) != cudaSuccess) return TB200_ERR_CUDA;
    return TB200_OK;
  }
  if (!a.k_src || !a.v_src || !a.k_dst || !a.v_dst || (a.n_idx > 0 && !a.idx)) return TB200_ERR_INVALID;
  const int words = (a.kv_len + 31) / 32;
  if (words > kEvictMaxWords) return TB200_ERR_UNSUPPORTED;
  const size_t row_bytes = static_cast<size_t>(a.head_dim) * 2;
  const size_t src_bytes = static_cast<size_t>(a.rows) * a.src_cache_len * row_bytes;
  const size_t dst_bytes = static_cast<size_t>(a.rows) * a.dst_cache_len * row_bytes;
  // In place: exactly the same caches as source and destination.  Any other overlap is refused: CTAs of the
  // out-of-place kernel read positions other CTAs of the row may already have overwritten.
  const bool in_place = a.k_dst == a.k_src && a.v_dst == a.v_src && a.dst_cache_len == a.src_cache_len &&
                        !overlaps(a.k_src, src_bytes, a.v_src, src_bytes);
  if (!in_place && (overlaps(a.k_src, src_bytes, a.k_dst, dst_bytes) || overlaps(a.v_src, src_bytes, a.v_dst, dst_bytes) ||
      overlaps(a.k_src, src_bytes, a.v_dst, dst_bytes) || overlaps(a.v_src, src_bytes, a.k_dst, dst_bytes) ||
      overlaps(a.k_dst, dst_bytes, a.v_dst, dst_bytes)))
    return TB200_ERR_INVALID;
  const uintptr_t align = reinterpret_cast<uintptr_t>(a.k_src) | reinterpret_cast<uintptr_t>(a.v_src) |
                          reinterpret_cast<uintptr_t>(a.k_dst) | reinterpret_cast<uintptr_t>(a.v_dst);
  if (align & 15u) return TB200_ERR_INVALID;

  EvictParams p;
  p.idx = a.idx;
  p.k_src = static_cast<const uint4*>(a.k_src);
  p.v_src = static_cast<const uint4*>(a.v_src);
  p.k_dst = static_cast<uint4*>(a.k_dst);
  p.v_dst = static_cast<uint4*>(a.v_dst);
  p.kept_pos = a.kept_pos;
  p.new_len = a.new_len;
  p.n_idx = a.n_idx;
  p.kv_len = a.kv_len;
  p.keep_recent = a.keep_recent;
  p.words = words;
  p.max_keep = static_cast<int>(max_keep);
  const int vec = a.head_dim * 2 / 16;
  p.src_pitch = static_cast<long long>(a.src_cache_len) * vec;
  p.dst_pitch = static_cast<long long>(a.dst_cache_len) * vec;

  const size_t smem = static_cast<size_t>(words) * sizeof(uint32_t);
  static bool attr_set[32] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 31]) {
    if (cudaFuncSetAttribute(kv_compact_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kEvictMaxWords * 4) != cudaSuccess ||
        cudaFuncSetAttribute(kv_compact_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kEvictMaxWords * 4) != cudaSuccess ||
        cudaFuncSetAttribute(kv_compact_inplace_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kEvictMaxWords * 4) != cudaSuccess ||
        cudaFuncSetAttribute(kv_compact_inplace_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kEvictMaxWords * 4) != cudaSuccess)
      return TB200_ERR_CUDA;
    attr_set[dev & 31] = true;
  }
  if (in_place) {  // one CTA per row along grid.x: no limit on the number of rows
    p.groups = 0;
    if (vec == 16) kv_compact_inplace_kernel<16><<<static_cast<unsigned>(a.rows), kEvictThreads, smem, stream>>>(p);
    else kv_compact_inplace_kernel<8><<<static_cast<unsigned>(a.rows), kEvictThreads, smem, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
  }

  // groups per CTA: the preamble costs about as much as one group per 2048 indices, so take two groups per 2048
  // indices (measured best on a B200: 2 up to 4096 indices, 4 at 8192), but leave at least four CTAs per SM
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  const int num_sms = st->num_sms;
  const long long groups_per_row = (max_keep + kEvictSlots - 1) / kEvictSlots;
  const long long fill = groups_per_row * a.rows / (4LL * num_sms);
  long long groups = (a.n_idx + 2047) / 2048;
  groups = groups < 2 ? 2 : groups;
  groups = groups > fill ? fill : groups;
  groups = groups < 1 ? 1 : (groups > kEvictMaxGroups ? kEvictMaxGroups : groups);
  p.groups = static_cast<int>(groups);
  if (a.rows > 65535) return TB200_ERR_UNSUPPORTED;  // rows run along grid.y
  const dim3 grid(static_cast<unsigned>((groups_per_row + groups - 1) / groups), static_cast<unsigned>(a.rows));
  if (vec == 16) kv_compact_kernel<16><<<grid, kEvictThreads, smem, stream>>>(p);
  else kv_compact_kernel<8><<<grid, kEvictThreads, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

}  // namespace tb200

extern "C" int64_t tb200_kv_compact_max_keep(const tb200_kv_compact_args* a) {
  if (a == nullptr || a->kv_len < 0 || a->n_idx < 0 || a->keep_recent < 0) return 0;
  const int64_t want = static_cast<int64_t>(a->n_idx) + a->keep_recent;
  return want < a->kv_len ? want : a->kv_len;
}

extern "C" int tb200_kv_compact(const tb200_kv_compact_args* args, void* stream) {
  if (args == nullptr) return TB200_ERR_INVALID;
  int status = TB200_OK;
  if (tb200::device_state(&status) == nullptr) return status;
  return tb200::launch_kv_compact(*args, static_cast<cudaStream_t>(stream));
}
