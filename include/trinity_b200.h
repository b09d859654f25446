/* trinity_b200 -- C ABI of the B200 (sm_100a) fused transformer blocks.
 *
 * The library replaces the device code behind the "generated module" operator API of
 * youngchan2/Trinity: a Python module exposing TENSOR_PARAMS, BLOCK_PARAMS and
 * forward(*tensors, block_*=16) (codegen/TritonGen.py:543-716), whose forward() launches the
 * Triton kernels kernel_0..kernel_k that TritonGen emitted.  Here forward() calls ONE of the entry
 * points below instead.  All pointers are DEVICE pointers borrowed for the duration of the call;
 * tensors are row-major and contiguous; `stream` is a cudaStream_t passed as void*.
 *
 * Conventions: return 0 (TB200_OK) or a negative tb200_status; never throw; never allocate device
 * memory (the only device state the library owns -- a 4-byte error word and the 16 MiB array of
 * tb200_gemm_static_scratch -- are device symbols inside the library image); never synchronise the
 * device, except tb200_device_status and tb200_attn_forward_timed, which say so.  The first call on a
 * device looks up that device's properties and symbol addresses and must run outside stream capture;
 * after it every entry point is safe under CUDA-graph capture.  Workspace is supplied by the caller and
 * sized by the *_workspace_bytes() queries.  Argument checks (null, shape, 16-byte alignment of every
 * tensor pointer, 4-byte alignment of the fp32 / int32 ones) are done on the host before anything is
 * launched: a call that returns an error has launched nothing.  tb200_*_check() run those checks alone
 * (no device needed).
 */
#ifndef TRINITY_B200_H_
#define TRINITY_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  TB200_OK = 0,
  TB200_ERR_INVALID = -1,        /* null pointer, bad shape, misaligned pointer */
  TB200_ERR_UNSUPPORTED = -2,    /* a legal request this build has no kernel for */
  TB200_ERR_CUDA = -3,           /* a CUDA runtime/driver call failed */
  TB200_ERR_WORKSPACE = -4,      /* workspace missing or too small */
  TB200_ERR_DEVICE_TIMEOUT = -5, /* a bounded device-side wait gave up (see tb200_device_status) */
  TB200_ERR_SCRATCH_LIMIT = -6   /* tb200_gemm_static_scratch: the partial sums exceed the built-in array */
} tb200_status;

typedef enum { TB200_F16 = 0, TB200_BF16 = 1, TB200_F32 = 2 } tb200_dtype;

const char* tb200_strerror(int status);
/* Library/ABI version: major*1000 + minor. */
int tb200_version(void);
/* Reads (and clears) the device-side error word of the current device; 0 = no kernel gave up a wait.
 * Every kernel of the library, tb200_gemm_static_scratch's included, reports there.
 * Synchronises the device -- a debugging / test aid, not part of the hot path. */
int tb200_device_status(int* code_out);
/* Every device-side wait (mbarrier, flag) is bounded: after this many SM cycles the waiting kernel records a
 * code in the error word, lets all its roles leave their loops, frees its tensor memory and returns
 * (TB200_ERR_DEVICE_TIMEOUT from tb200_device_status).  Default 4e9 (about 2 s); applies to launches made
 * after the call; process-wide.  No counterpart in the reference (Triton kernels have no such waits). */
int tb200_set_wait_limit_cycles(long long cycles);
long long tb200_get_wait_limit_cycles(void);
/* Within one call (tb200_gemm, tb200_attn_forward, tb200_ffn_forward ...) the kernels after the first are launched
 * with programmatic stream serialisation: each starts while the one before it drains, sets up, prefetches its
 * weights, and waits (griddepcontrol.wait) before it touches anything a kernel of the call writes.  The first
 * kernel of a call is an ordinary launch, so the call's arguments are complete before it starts.  Works inside
 * stream capture.  0 switches this off (every launch ordinary), non-zero on (the default); returns the previous
 * setting; process-wide.  The reference has no counterpart (its Triton kernels are launched one by one). */
int tb200_set_chained_launch(int enabled);
/* Test aid: launches a one-CTA kernel whose only mbarrier is never armed, with the given limit (1e3..2e9
 * cycles), through the same bounded-wait code as the compute kernels.  The wait runs out, the kernel
 * returns, and the next tb200_device_status reports TB200_ERR_DEVICE_TIMEOUT with code 900. */
int tb200_selftest_wait_timeout(long long limit_cycles, void* stream);

/* ---------------------------------------------------------------------------------------------
 * RMSNorm: y[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps) [* weight].
 * Replaces the standalone RMSNorm kernels of evaluation/ffn/ffn_falcon/rms_ref.py:13-71; math of
 * baseline/ref_rms.py:101-102 (reference point: weight = NULL, eps = 0).
 * y may be NULL (statistics only); inv_rms (fp32, one per row) may be NULL.  cols % 8 == 0. */
int tb200_rmsnorm(const void* x, const void* weight, void* y, float* inv_rms, int64_t rows, int64_t cols,
                  float eps, int dtype, void* stream);
/* w_out[k, :] = w[k, :] * norm_weight[k] over a (k, n) projection weight: folds an RMSNorm weight into the
 * projection that follows the norm, once per model load, because (x * r * g) @ W = r * (x @ (diag(g) W)).  With
 * the folded weights and TB200_ATTN_NORM_FOLDED / TB200_FFN_NORM_FOLDED the weighted norm is what the weight-free
 * one is in the reference optimizer's own rewrite (evaluation/prenorm/prenorm_falcon_benchmark579.py:86-88): a row
 * statistic and a per-row scale in the projection's epilogue; no normalised copy of x is written.  n % 8 == 0;
 * w_out may not alias w. */
int tb200_fold_norm_weight(const void* w, const void* norm_weight, void* w_out, int64_t k, int64_t n, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Fused GEMM  C = epilogue(A[m,k] @ B[k,n]),  16-bit inputs, fp32 accumulation on tcgen05/TMEM.
 * The building block behind the k-loops of every emitted kernel (e.g.
 * evaluation/ffn/ffn_llama/ffn_llama_benchmark2248.py:19-62 "O2*WO + X", :80-130 gate/up + SiLU,
 * :148-185 down projection).  Epilogue, in this order:  acc *= row_scale[m]  (norm-as-epilogue,
 * evaluation/prenorm/prenorm_falcon_benchmark579.py:86-88);  dual: silu(acc_b) * acc_b2  (SwiGLU);
 * act: 1 = exact-erf GELU;  + residual[m,n]. */
typedef struct {
  int dtype;               /* TB200_F16 or TB200_BF16: a, b, b2, c, residual */
  int act;                 /* 0 none, 1 GELU (erf) */
  int64_t m, n, k;         /* n % 8 == 0, k % 8 == 0 */
  const void* a;           /* (m,k) */
  const void* b;           /* (k,n) */
  const void* b2;          /* (k,n) or NULL: when set, c = silu(a@b) * (a@b2) */
  void* c;                 /* (m,n) */
  const float* row_scale;  /* (m) or NULL */
  const void* residual;    /* (m,n) or NULL */
  int split_k;             /* 0 = let the library choose; 1 = never split; >1 = that many K slices */
  void* workspace;         /* needed when K is split (fp32 partial sums) */
  size_t workspace_bytes;
} tb200_gemm_args;
size_t tb200_gemm_workspace_bytes(const tb200_gemm_args* args);
int tb200_gemm(const tb200_gemm_args* args, void* stream);
/* The host-side argument checks of tb200_gemm alone: nothing is launched, no device is needed. */
int tb200_gemm_check(const tb200_gemm_args* args);
/* No counterpart in the reference.  The same GEMM + epilogue as tb200_gemm, always computed as K slices
 * whose fp32 partial sums go into a 16 MiB array that is part of the library image, so that the call
 * performs NO device allocation at all (tb200_gemm takes a caller-allocated workspace for them).  Meant for hosts that are not allowed to
 * allocate: a server that gave all of HBM to its own pool, or code running under a foreign allocator.
 *   - args->workspace / workspace_bytes are ignored; split_k 0 lets the library choose.
 *   - split_k * m * n * 4 bytes (twice that with b2) must fit in 16 MiB, else TB200_ERR_SCRATCH_LIMIT.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, under a lock);
 *     make that call before starting any stream capture.
 *   - A bounded wait that runs out is reported through tb200_device_status, as for every other entry point.
 *   - All calls on a device share the one array: two calls that may run concurrently on the GPU (different
 *     streams) race on it.  Calls on one stream are ordered and safe.  Nothing in the array needs clearing
 *     between calls: every partial sum that is read has been written by the same call. */
int tb200_gemm_static_scratch(const tb200_gemm_args* args, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Tensor-parallel row-parallel projection with its all-reduce done by the kernels over peer memory (NVLink):
 * out = sum over ranks of (a_r @ b_r) [+ residual], every rank ending with the full (m, n) result.  No counterpart in
 * the reference, which has no multi-GPU path; it stands where "tb200_gemm, then ncclAllReduce" would, for the down
 * projection of a tensor-parallel FFN (a: this rank's columns of the activated inner tensor, (m, k_local); b: this
 * rank's rows of W_down, (k_local, n)).  One process per GPU; `world` <= 8 ranks on one NVSwitch domain.
 *   - Rank r owns rows [r*m/world, (r+1)*m/world) of the result; m % (128*world) == 0.
 *   - stage[q], out[q], sync[q] are rank q's buffers as seen from THIS process: this rank's own allocations for
 *     q == rank, peer mappings (tb200_ipc_open of what rank q exported) otherwise.  stage: tb200_peer_stage_bytes;
 *     out: m*n 16-bit values; sync: tb200_peer_sync_bytes, zeroed once when the communicator is set up.
 *   - epoch: 1 for the first call on these buffers, then 2, 3, ... -- the same on all ranks; the buffers serve ONE
 *     shape (m, n, world).  All ranks must make the call (it ends with a rank-to-rank completion exchange); `out` of a
 *     call must have been consumed, on this stream, before the next call.
 *   - Every device-side wait on a peer is bounded (tb200_set_wait_limit_cycles); a rank that never arrives shows up as
 *     TB200_ERR_DEVICE_TIMEOUT in tb200_device_status, code 601 (contributions) or 602 (completion).
 *   - The sum is taken in rank order in fp32 from the ranks' 16-bit partial products: the same bits on every run and
 *     on every rank. */
typedef struct {
  int dtype;                 /* TB200_F16 or TB200_BF16 */
  int world, rank;
  int64_t m, n, k;           /* k = this rank's share of the contraction */
  const void* a;             /* (m, k) */
  const void* b;             /* (k, n) */
  const void* residual;      /* (m, n) or NULL: added once, by the row's owner (identical on all ranks) */
  void* stage[8];
  void* out[8];
  void* sync[8];
  uint32_t epoch;
} tb200_peer_gemm_args;
size_t tb200_peer_stage_bytes(int64_t m, int64_t n);
size_t tb200_peer_sync_bytes(int64_t m, int world);
int tb200_gemm_peer_reduce(const tb200_peer_gemm_args* args, void* stream);
/* CUDA IPC plumbing for the buffers above (one process per GPU): export a device pointer as a 64-byte handle plus its
 * offset inside the underlying allocation; open what another process exported; close it again. */
int tb200_ipc_export(const void* ptr, void* handle64, int64_t* offset_out);
int tb200_ipc_open(const void* handle64, int64_t offset, void** ptr_out);
int tb200_ipc_close(void* ptr, int64_t offset);

/* ---------------------------------------------------------------------------------------------
 * Fused attention block -- replaces kernel_0/kernel_1 of the emitted attention modules:
 *   Vanilla   evaluation/vanilla/vanilla_falcon_benchmark28173.py:19-144  (baseline/ref_rms.py:44-82)
 *   PreNorm   evaluation/prenorm/prenorm_falcon_benchmark579.py:19-120    (ref_rms.py:100-126)
 *   QKNorm    evaluation/qknorm/qknorm_falcon_benchmark1350.py:19-116     (ref_rms.py:237-265)
 *   KeyFormer evaluation/keyformer/keyformer_falcon_benchmark4358.py:19-147 (ref_rms.py:146-171)
 *   RoCo      evaluation/roco/roco_falcon_benchmark1620.py:19-141         (ref_rms.py:333-357)
 * [x -> RMSNorm] -> q,k,v = x@W{q,k,v} -> split heads -> [per-head RMSNorm of q,k] -> append k,v to the
 * cache rows [past,past+seq) -> softmax(scale * q@K^T [causal]) @ V -> merge heads into o2; optional
 * per-key reductions and top-k.  Reference parameter point: batch 1, n_kv_heads == n_q_heads,
 * sm_scale 1, no CAUSAL flag, all weights NULL, eps 0, tau 1.5. */
enum {
  TB200_ATTN_PRENORM = 1,    /* RMSNorm over hidden before the projections */
  TB200_ATTN_QKNORM = 2,     /* per-head RMSNorm of q and k (normalised k is what is cached) */
  TB200_ATTN_CAUSAL = 4,     /* query i sees keys <= past + i */
  TB200_ATTN_KEYFORMER = 8,  /* c_out[b,h,j] = sum_i softmax_j((scale*s + noise)/tau)[i,j] */
  TB200_ATTN_ROCO = 16,      /* c_out1 = sum_i p[i,j], c_out2 = sum_i p[i,j]^2 (what the reference's kernels emit) */
  TB200_ATTN_NORM_FOLDED = 64, /* with PRENORM: wq, wk, wv already carry the norm weight (tb200_fold_norm_weight);
                                norm_weight is ignored, only the row statistic is computed before the projection */
  TB200_ATTN_ROCO_VARIANCE = 32 /* with ROCO: c_out2 = sum_i p^2 / n_j - (c_out1 / n_j)^2, the column variance over the n_j
                                queries that can see key j (S, or S - max(0, j - past) under the causal mask); c_out1 stays
                                the column sum, which is also what top-k ranks.  No counterpart in the reference. */
};
typedef struct {
  int dtype;                 /* TB200_F16 / TB200_BF16: x, weights, caches, o2, norm weights, noise */
  int flags;
  int batch, seq, hidden;    /* B, S (new tokens per sequence), N */
  int n_q_heads, n_kv_heads, head_dim; /* head_dim 64 or 128 */
  int past;                  /* P: rows already valid in the caches */
  int cache_len;             /* rows allocated per head in the caches, >= past + seq */
  float sm_scale, norm_eps, qk_eps, tau;
  const void* x;             /* (B,S,N) */
  const void* wq;            /* (N, Hq*D) */
  const void* wk;            /* (N, Hkv*D) */
  const void* wv;            /* (N, Hkv*D) */
  void* k_cache;             /* (B,Hkv,cache_len,D); rows [past,past+seq) are written */
  void* v_cache;
  void* o2;                  /* (B,S,Hq*D) */
  const void* norm_weight;   /* (N) or NULL */
  const void* q_norm_weight; /* (D) or NULL */
  const void* k_norm_weight; /* (D) or NULL */
  const void* noise;         /* (B,Hq,S,past+seq), KEYFORMER */
  void* c_out;               /* (B,Hq,past+seq), KEYFORMER */
  void* c_out1;              /* (B,Hq,past+seq), ROCO */
  void* c_out2;
  int aux_dtype;             /* dtype of c_out*: TB200_F32 or the 16-bit dtype */
  int topk;                  /* 0 = none; else indices of the k largest per-key scores per (b,h): */
  int32_t* topk_idx;         /* (B,Hq,topk), stable descending (ties -> lower index); key = c_out
                                (KEYFORMER) or c_out1 (ROCO) as fp32 before any narrowing */
  void* workspace;
  size_t workspace_bytes;
} tb200_attn_args;
size_t tb200_attn_workspace_bytes(const tb200_attn_args* args);
int tb200_attn_forward(const tb200_attn_args* args, void* stream);
/* The host-side argument checks of tb200_attn_forward alone (workspace excepted): nothing is launched. */
int tb200_attn_check(const tb200_attn_args* args);
/* Measuring aid with no counterpart in the reference (its harness times whole forward() calls,
 * benchmark/vanilla_llama_benchmark.py:277-294): the same block, with CUDA events recorded on `stream`
 * between its stages; waits for the stream and returns the stage durations in milliseconds:
 * [0] RMSNorm prologue, [1] QKV projection, [2] attention, [3] per-key reductions + top-k.
 * Creates and destroys events: not for use under graph capture. */
int tb200_attn_forward_timed(const tb200_attn_args* args, void* stream, float* stage_ms);

/* ---------------------------------------------------------------------------------------------
 * Fused FFN block -- replaces kernel_0..2 of evaluation/ffn/ffn_llama/ffn_llama_benchmark2248.py:19-258
 * and kernel_0..4 of evaluation/ffn/ffn_falcon/ffn_benchmark428.py:19-233 (baseline/ffn_ref.py:24-52,
 * :86-123):  a = [o2 @ wo + residual_x | x];  h = [RMSNorm(a) | a];
 * ff2 = act(h @ w_gate [, h @ w_up]) @ w_down;  [o_ff = ff2 + h; o_ff_norm = RMSNorm(o_ff)]. */
enum { TB200_FFN_SWIGLU = 0, TB200_FFN_GELU = 1 };
enum {
  TB200_FFN_NORM = 1,        /* RMSNorm of a before the up projections */
  TB200_FFN_FALCON_TAIL = 2, /* o_ff = ff2 + h, o_ff_norm = o_ff / sqrt(sum(o_ff^2)/tail_divisor) */
  TB200_FFN_NORM_FOLDED = 4  /* with NORM: w_gate (and w_up) already carry the norm weight (tb200_fold_norm_weight);
                                not with FALCON_TAIL, whose residual is the normalised h itself */
};
typedef struct {
  int dtype;
  int act;                   /* TB200_FFN_SWIGLU or TB200_FFN_GELU */
  int flags;
  int64_t tokens, hidden, inner; /* M, N, P */
  float norm_eps;
  int tail_divisor;          /* 0 = hidden (the reference hard-codes 4544) */
  const void* x;             /* (M,N): the block input, or the residual when wo is set */
  const void* o2;            /* (M,N) or NULL: attention output fed through wo */
  const void* wo;            /* (N,N) or NULL */
  const void* norm_weight;   /* (N) or NULL */
  const void* w_gate;        /* (N,P): WFF1b (SwiGLU gate) or W1 (GELU) */
  const void* w_up;          /* (N,P): WFF1a; NULL for GELU */
  const void* w_down;        /* (P,N): WFF2 */
  void* ff2;                 /* (M,N) out */
  void* attn_o2;             /* (M,N) out or NULL: a */
  void* ff1;                 /* (M,P) out or NULL: activated inner tensor (else kept in workspace) */
  void* o_ff_norm;           /* (M,N) out, FALCON_TAIL */
  void* workspace;
  size_t workspace_bytes;
} tb200_ffn_args;
size_t tb200_ffn_workspace_bytes(const tb200_ffn_args* args);
int tb200_ffn_forward(const tb200_ffn_args* args, void* stream);
/* The host-side argument checks of tb200_ffn_forward alone (workspace excepted): nothing is launched. */
int tb200_ffn_check(const tb200_ffn_args* args);
/* tb200_attn_forward(attn) followed by tb200_ffn_forward(ffn) as ONE call: the FFN block must consume the attention
 * block's output (ffn->o2 == attn->o2, ffn->wo given, tokens = batch * seq, equal dtype and hidden size).  The
 * two blocks form one launch chain (tb200_set_chained_launch): the output projection is launched while the
 * attention kernel drains and has its first weight tiles in flight when o2 is complete.  Results are those of the
 * two separate calls, bit for bit.  Every argument check of both blocks is made before the first launch.
 * Replaces the reference's pair of generated modules run back to back (the attention module of
 * evaluation/prenorm/prenorm_falcon_benchmark579.py:115-120 feeding the FFN module of
 * evaluation/ffn/ffn_llama/ffn_llama_benchmark2248.py:45-62). */
int tb200_layer_forward(const tb200_attn_args* attn, const tb200_ffn_args* ffn, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Deterministic top-k over the last axis of scores (rows, n) fp32: idx[r,:] = the first k entries of
 * a stable descending sort (ties -> lower index).  New relative to the reference (which never
 * selects keys); n <= 16384, 1 <= k <= n. */
int tb200_topk(const float* scores, int32_t* idx, int64_t rows, int n, int k, void* stream);

/* ---------------------------------------------------------------------------------------------
 * KV-cache eviction: pack the cache positions an index list names to the front of a destination
 * cache.  New relative to the reference: its KeyFormer / RoCo modules emit the per-key scores
 * (`C_out`, `C_out1`, `C_out2`: evaluation/keyformer/keyformer_falcon_benchmark4358.py:19-147,
 * evaluation/roco/roco_falcon_benchmark1620.py:19-141) and nothing consumes them; this is the
 * consumer, on the reference's cache layout `(H, P+M, D)` (convert_eval_rms.py:82-83) with rows =
 * batch * kv heads.
 *
 * For every cache row r: keep = { idx[r,i] : 0 <= idx[r,i] < kv_len } united with the recent
 * window [kv_len - keep_recent, kv_len); the kept positions p_0 < p_1 < ... (ascending, duplicates
 * counted once) give k_dst[r, j, :] = k_src[r, p_j, :], v likewise, new_len[r] = their count,
 * kept_pos[r, j] = p_j and -1 for j >= new_len[r].  Destination positions >= new_len[r] are left
 * untouched.  idx may hold several lists per row (GQA: the lists of the q heads of a group, one
 * after the other: n_idx = group * k) - a position any of them names is kept.  Bit-exact, no
 * workspace.  In place: pass k_dst == k_src, v_dst == v_src and dst_cache_len == src_cache_len
 * (one CTA per row packs front to back); any other overlap of source and destination is refused.
 * head_dim 64 or 128, 16-bit elements, kv_len <= 262144, rows <= 65535 (out of place),
 * dst_cache_len >= tb200_kv_compact_max_keep(). */
typedef struct {
  int dtype;                 /* TB200_F16 or TB200_BF16 (only the element size matters) */
  int rows;                  /* batch * kv heads */
  int head_dim;
  int kv_len;                /* valid positions per source row */
  int src_cache_len;         /* positions per source row (row pitch) */
  int dst_cache_len;         /* positions per destination row */
  int n_idx;                 /* indices per row */
  int keep_recent;           /* the last keep_recent positions are kept whatever idx says */
  const int32_t* idx;        /* (rows, n_idx); entries outside [0, kv_len) are ignored */
  const void* k_src;         /* (rows, src_cache_len, head_dim) */
  const void* v_src;
  void* k_dst;               /* (rows, dst_cache_len, head_dim) */
  void* v_dst;
  int32_t* kept_pos;         /* (rows, tb200_kv_compact_max_keep()) out, or NULL */
  int32_t* new_len;          /* (rows) out, or NULL */
} tb200_kv_compact_args;
/* min(kv_len, n_idx + keep_recent): the most positions a row can keep, and the width of kept_pos. */
int64_t tb200_kv_compact_max_keep(const tb200_kv_compact_args* args);
int tb200_kv_compact(const tb200_kv_compact_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TRINITY_B200_H_ */
