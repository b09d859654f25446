// Host-side declarations shared by the translation units of libtrinity_b200.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#include "../../include/trinity_b200.h"

namespace tb200 {

// Per-device state created by the first call on that device (outside any stream capture): the SM count and
// the device address of the error word.  Creating it allocates nothing: the error word is a device symbol
// inside the library image, looked up with cudaGetSymbolAddress.
struct DeviceState {
  int device = -1;
  int num_sms = 0;
  int* err_word = nullptr;  // device address of the 4-byte error word, zero when healthy
};
// Returns nullptr (and sets *status) if the state cannot be created.
DeviceState* device_state(int* status);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda dependency).
// 2D/3D row-major tensors of 16-bit elements, 128-byte swizzle, zero fill outside the bounds.
//   dims[0] is the contiguous (inner) extent in elements; strides_bytes[i] is the pitch of dims[i+1].
int make_tensor_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box);

// Cycles after which a bounded device-side wait gives up (tb200_set_wait_limit_cycles); copied into the
// parameters of every kernel launch.
long long wait_limit_cycles();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3) == 0; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---------------------------------------------------------------- chained launches (runtime.cu)
// Within one call of the library the kernels after the first are launched with programmatic stream serialisation
// (see pdl_wait in common.cuh): their set-up and their weight prefetch overlap the tail of the kernel before.  The
// FIRST kernel of a call is launched the ordinary way, so that everything written before the call -- its arguments,
// weights included -- is complete before any kernel of the call starts.  A ChainScope marks the extent of a call on
// the calling thread; outside one, and with tb200_set_chained_launch(0), every launch is an ordinary one.
struct ChainScope {
  ChainScope();
  ~ChainScope();
};
// Whether the launch about to be made may carry the attribute; marks the call's first launch as done.
bool chain_next_launch();

template <typename... KArgs, typename... Args>
cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (chain_next_launch()) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Args&&>(args)...);
}

// ---------------------------------------------------------------- rmsnorm.cu
// mean_divisor: the sum of squares is divided by this instead of cols when > 0 (the reference's Falcon
// tail hard-codes 4544, baseline/ffn_ref.py:121).
int launch_rmsnorm(const void* x, const void* weight, void* y, float* inv_rms, int64_t rows, int64_t cols,
                   float eps, int dtype, cudaStream_t stream, int mean_divisor = 0);

int launch_fold_rows(const void* w, const void* g, void* out, int64_t k, int64_t n, int dtype, cudaStream_t stream);

// ---------------------------------------------------------------- gemm.cu
enum GemmMode {
  GEMM_STORE = 0,    // c = act(acc * row_scale) + residual
  GEMM_SWIGLU = 1,   // two B sources of equal width: c = silu(acc0 * rs) * (acc1 * rs)
  GEMM_QKV = 2,      // three B sources (Wq, Wk, Wv): head split, optional per-head RMSNorm, cache append
  GEMM_PARTIAL = 3,  // fp32 partial sums of one K slice into the workspace
  GEMM_PEER = 4      // tensor-parallel partial product: every 128-row block of the result goes, as 16-bit values, into the
                     // staging buffer of the rank that owns those rows (a peer pointer), followed by an arrival on that
                     // rank's counter for the block; peer.cu sums the ranks' contributions
};
constexpr int kMaxPeers = 8;
struct GemmLaunch {
  int dtype = TB200_BF16;
  int mode = GEMM_STORE;
  int M = 0, K = 0;
  const void* A = nullptr;          // (M,K), pitch K
  int n_src = 1;
  const void* B[3] = {nullptr, nullptr, nullptr};  // (K, N[i]), pitch N[i]
  int N[3] = {0, 0, 0};
  const float* row_scale = nullptr;
  // GEMM_STORE / GEMM_SWIGLU
  void* C = nullptr;
  int64_t ldc = 0;
  const void* residual = nullptr;
  int64_t ldr = 0;
  void* C2 = nullptr;               // optional: the value before the residual is added (pitch ldc)
  int act = 0;
  // GEMM_QKV
  void* q_out = nullptr;            // (B,Hq,S,D)
  void* k_cache = nullptr;          // (B,Hkv,cache_len,D)
  void* v_cache = nullptr;
  int S = 0, Hq = 0, Hkv = 0, D = 0, past = 0, cache_len = 0;
  int qknorm = 0;
  float qk_eps = 0.f;
  const void* q_norm_weight = nullptr;
  const void* k_norm_weight = nullptr;
  // GEMM_PARTIAL
  int split_k = 1;
  float* partial = nullptr;         // (split_k, M, sum N[i])
  // GEMM_PEER: rows [r * rows_per_rank, (r + 1) * rows_per_rank) belong to rank r; rank r's staging buffer holds
  // (world, rows_per_rank, N[0]) 16-bit values, slot `rank` is this rank's; counters are one uint32 per 128 owned rows
  int world = 1, rank = 0, rows_per_rank = 0;
  void* peer_stage[kMaxPeers] = {};
  unsigned* peer_counter[kMaxPeers] = {};
};
int launch_gemm(const GemmLaunch& g, cudaStream_t stream);

// Sum the K slices and apply the epilogue: out = act(sum * row_scale) [silu-gated by the second half] + residual.
struct SplitKFinish {
  int dtype = TB200_BF16;
  int M = 0, N = 0;                 // N = output width
  int split_k = 1;
  const float* partial = nullptr;   // (split_k, M, ldp)
  int64_t ldp = 0;                  // N, or 2N when gated
  int gated = 0;                    // columns [0,N) = gate, [N,2N) = up
  int act = 0;
  const float* row_scale = nullptr;
  const void* residual = nullptr;
  int64_t ldr = 0;
  void* C = nullptr;
  int64_t ldc = 0;
  void* C2 = nullptr;               // optional: the value before the residual is added
};
int launch_splitk_finish(const SplitKFinish& f, cudaStream_t stream);

// Sum the K slices of a QKV projection and apply its epilogue (row scale, head split, optional per-head RMSNorm,
// q head-major, k and v appended to the caches): the decode-size counterpart of GEMM_QKV.
struct QkvFinish {
  int dtype = TB200_BF16;
  int M = 0, split_k = 1;
  const float* partial = nullptr;   // (split_k, M, (Hq + 2 Hkv) * D)
  const float* row_scale = nullptr;
  void* q_out = nullptr;
  void* k_cache = nullptr;
  void* v_cache = nullptr;
  int S = 0, Hq = 0, Hkv = 0, D = 0, past = 0, cache_len = 0;
  int qknorm = 0;
  float qk_eps = 0.f;
  const void* q_norm_weight = nullptr;
  const void* k_norm_weight = nullptr;
};
int launch_qkv_finish(const QkvFinish& f, cudaStream_t stream);

// ---------------------------------------------------------------- attn.cu
struct AttnLaunch {
  int dtype = TB200_BF16;
  int B = 0, S = 0, Hq = 0, Hkv = 0, D = 0, past = 0, cache_len = 0;
  int causal = 0;
  float sm_scale = 1.f;
  const void* q = nullptr;          // (B,Hq,S,D)
  const void* k_cache = nullptr;    // (B,Hkv,cache_len,D)
  const void* v_cache = nullptr;
  void* o2 = nullptr;               // (B,S,Hq*D)
  float* lse2 = nullptr;            // (B,Hq,S): log2-domain log-sum-exp of scale*s
  // KeyFormer: second statistic over (scale*s + noise)/tau
  const void* noise = nullptr;      // (B,Hq,S,past+S)
  float tau = 1.f;
  float* lse2_perturbed = nullptr;  // (B,Hq,S)
  // decode shapes: key range split over CTAs (attn_kv_splits); partial results in caller-provided workspace
  int kv_splits = 1;
  float* part_o = nullptr;          // (kv_splits,B,Hq,S,D) fp32
  float* part_ml = nullptr;         // (kv_splits,B,Hq,S,2) fp32
};
int launch_attn_fwd(const AttnLaunch& a, cudaStream_t stream);
// attn2.cu: two query tiles per CTA; chosen by launch_attn_fwd when there is no noise tensor
int launch_attn_fwd_pingpong(const AttnLaunch& a, cudaStream_t stream);
int attn_kv_splits(int B, int S, int Hq, int kv_len, int num_sms);
// attn_kf.cu: the same kernel with the KeyFormer statistic (noise tiles by TMA; kv_len a multiple of 8)
int launch_attn_fwd_keyformer(const AttnLaunch& a, cudaStream_t stream);

// ---------------------------------------------------------------- attn_dec.cu
// Decode-sized query blocks (S <= 16, no KeyFormer / RoCo statistic): one kernel takes the projection's K-slice sums
// (or a finished q with the caches already appended), finishes q and the new k, v rows, appends them to the caches and
// computes softmax(Q K^T) V with the key shares merged inside a cluster.
struct AttnDecodeLaunch {
  int dtype = TB200_BF16;
  int B = 0, S = 0, Hq = 0, Hkv = 0, D = 0, past = 0, cache_len = 0;
  int causal = 0;
  float sm_scale = 1.f;
  const void* q = nullptr;          // (B,Hq,S,D); exactly one of q / partial
  const float* partial = nullptr;   // (split, B*S, (Hq + 2 Hkv) * D) fp32 K-slice sums of the QKV projection
  int split = 1;
  const float* row_scale = nullptr;
  int qknorm = 0;
  float qk_eps = 0.f;
  const void* q_norm_weight = nullptr;
  const void* k_norm_weight = nullptr;
  void* k_cache = nullptr;
  void* v_cache = nullptr;
  void* o2 = nullptr;
  float* lse2 = nullptr;            // optional
};
bool attn_decode_applies(int B, int S, int Hq, int D);
int launch_attn_decode(const AttnDecodeLaunch& a, cudaStream_t stream);

// ---------------------------------------------------------------- score.cu
struct ScoreLaunch {
  int dtype = TB200_BF16;
  int B = 0, S = 0, Hq = 0, Hkv = 0, D = 0, past = 0, cache_len = 0;
  int causal = 0;
  float sm_scale = 1.f;
  const void* q = nullptr;
  const void* k_cache = nullptr;
  const float* lse2 = nullptr;
  const void* noise = nullptr;      // KeyFormer
  float tau = 1.f;
  const float* lse2_perturbed = nullptr;
  float* sum_p = nullptr;           // (B,Hq,past+S) or NULL
  float* sum_p2 = nullptr;
  float* sum_pt = nullptr;          // KeyFormer
};
int launch_score_colreduce(const ScoreLaunch& s, cudaStream_t stream);

// ---------------------------------------------------------------- topk.cu / misc
int launch_topk(const float* scores, int32_t* idx, int64_t rows, int n, int k, cudaStream_t stream);
int launch_roco_variance(const float* sum_p, float* sum_p2, int64_t rows, int kv_len, int past, int S, int causal, cudaStream_t stream);
int launch_cast_f32(const float* src, void* dst, int64_t n, int dtype, cudaStream_t stream);

// ---------------------------------------------------------------- evict.cu
int launch_kv_compact(const tb200_kv_compact_args& a, cudaStream_t stream);

}  // namespace tb200
