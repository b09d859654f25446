// extern "C" entry points that chain the kernels into the fused blocks: tb200_gemm, tb200_attn_forward,
// tb200_ffn_forward and their workspace queries.  Everything is launched on the caller's stream, nothing is
// allocated and nothing synchronises.
#include <string.h>

#include "internal.h"

namespace tb200 {

namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kTopkMaxKeys = 16384;   // launch_topk sorts one row in shared memory

// How many K slices for a weight-streaming (few row-tiles) GEMM: as many as brings the number of work
// units close to a whole number of waves over the SMs, at least 4 K-blocks per slice.
int choose_split(int M, int n_tiles, int K, int num_sms) {
  const long long m_tiles = (M + kBM - 1) / kBM;
  const long long tiles = m_tiles * n_tiles;   // 64-bit: the product of two tile counts can pass 2^31
  const int k_blocks = (K + kBK - 1) / kBK;
  if (tiles < 1 || tiles * 2 > num_sms || k_blocks < 8) return 1;
  int s = static_cast<int>(num_sms / tiles);
  if (s > k_blocks / 4) s = k_blocks / 4;
  if (s > 32) s = 32;
  return s < 1 ? 1 : s;
}

struct Carver {  // bump allocator over the caller's workspace, 256-byte granules
  uint8_t* base;
  size_t used = 0;
  explicit Carver(void* p) : base(static_cast<uint8_t*>(p)) {}
  void* take(size_t bytes) {
    void* p = base ? base + used : nullptr;
    used += align_up(bytes, 256);
    return p;
  }
};

int dtype_ok(int dtype) { return dtype == TB200_BF16 || dtype == TB200_F16; }

// ----------------------------------------------------------------------------------------- gemm
struct GemmPlan {
  int split = 1;
  size_t partial_bytes = 0;
};
GemmPlan plan_gemm(const tb200_gemm_args* a, int num_sms) {
  GemmPlan pl;
  const bool gated = a->b2 != nullptr;
  const int n_tiles = gated ? 2 * static_cast<int>((a->n + kBN - 1) / kBN) : static_cast<int>((a->n + kBN - 1) / kBN);
  int s = a->split_k;
  if (s == 0) s = choose_split(static_cast<int>(a->m), n_tiles, static_cast<int>(a->k), num_sms);
  const int k_blocks = static_cast<int>((a->k + kBK - 1) / kBK);
  if (s > k_blocks) s = k_blocks;
  if (s < 1) s = 1;
  pl.split = s;
  if (s > 1) pl.partial_bytes = static_cast<size_t>(s) * a->m * (gated ? 2 : 1) * a->n * sizeof(float);
  return pl;
}

// One GEMM with its epilogue, split over K when that fills the machine better.  `partial` may be null when
// split == 1.
int run_gemm(int dtype, int M, int N, int K, const void* A, const void* B, const void* B2, void* C, void* C2,
             const float* row_scale, const void* residual, int act, int split, float* partial, cudaStream_t stream) {
  const bool gated = B2 != nullptr;
  if (split <= 1) {
    GemmLaunch g;
    g.dtype = dtype;
    g.mode = gated ? GEMM_SWIGLU : GEMM_STORE;
    g.M = M; g.K = K; g.A = A;
    g.n_src = gated ? 2 : 1;
    g.B[0] = B; g.N[0] = N;
    if (gated) { g.B[1] = B2; g.N[1] = N; }
    g.row_scale = row_scale;
    g.C = C; g.ldc = N; g.C2 = C2;
    g.residual = residual; g.ldr = N;
    g.act = act;
    if (gated && (residual != nullptr || act != 0 || C2 != nullptr)) return TB200_ERR_UNSUPPORTED;
    return launch_gemm(g, stream);
  }
  GemmLaunch g;
  g.dtype = dtype;
  g.mode = GEMM_PARTIAL;
  g.M = M; g.K = K; g.A = A;
  g.n_src = gated ? 2 : 1;
  g.B[0] = B; g.N[0] = N;
  if (gated) { g.B[1] = B2; g.N[1] = N; }
  g.split_k = split;
  g.partial = partial;
  int status = launch_gemm(g, stream);
  if (status != TB200_OK) return status;
  // launch_gemm may have merged empty slices: recompute the slice count the same way
  const int k_blocks = (K + kBK - 1) / kBK;
  const int per = (k_blocks + split - 1) / split;
  const int real_split = (k_blocks + per - 1) / per;
  SplitKFinish f;
  f.dtype = dtype;
  f.M = M; f.N = N;
  f.split_k = real_split;
  f.partial = partial;
  f.ldp = gated ? 2LL * N : N;
  f.gated = gated ? 1 : 0;
  f.act = act;
  f.row_scale = row_scale;
  f.residual = residual; f.ldr = N;
  f.C = C; f.ldc = N; f.C2 = C2;
  return launch_splitk_finish(f, stream);
}

int check_gemm(const tb200_gemm_args* a) {
  if (a == nullptr || !dtype_ok(a->dtype)) return a ? TB200_ERR_UNSUPPORTED : TB200_ERR_INVALID;
  if (a->m < 0 || a->n <= 0 || a->k <= 0 || (a->n & 7) || (a->k & 7)) return TB200_ERR_INVALID;
  if (a->m > (1 << 30) || a->n > (1 << 30) || a->k > (1 << 30)) return TB200_ERR_INVALID;
  if (!a->a || !a->b || !a->c) return TB200_ERR_INVALID;
  if (a->act != 0 && a->act != 1) return TB200_ERR_INVALID;
  // every pointer a kernel touches with 16-byte accesses (TMA, uint4 loads and stores), whichever path is taken
  if (!aligned16(a->a) || !aligned16(a->b) || !aligned16(a->b2) || !aligned16(a->c) || !aligned16(a->residual)) return TB200_ERR_INVALID;
  if (!aligned4(a->row_scale)) return TB200_ERR_INVALID;
  return TB200_OK;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" {

int tb200_gemm_check(const tb200_gemm_args* a) { return check_gemm(a); }

size_t tb200_gemm_workspace_bytes(const tb200_gemm_args* a) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st || check_gemm(a) != TB200_OK) return 0;
  return align_up(plan_gemm(a, st->num_sms).partial_bytes, 256);
}

int tb200_gemm(const tb200_gemm_args* a, void* stream) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  if ((status = check_gemm(a)) != TB200_OK) return status;
  if (a->m == 0) return TB200_OK;
  ChainScope chain;
  GemmPlan pl = plan_gemm(a, st->num_sms);
  if (pl.split > 1 && (a->workspace == nullptr || a->workspace_bytes < pl.partial_bytes)) {
    if (a->split_k > 1) return TB200_ERR_WORKSPACE;  // the caller asked for slices but gave no room
    pl.split = 1;
  }
  if (pl.split > 1 && !aligned16(a->workspace)) return TB200_ERR_INVALID;
  return run_gemm(a->dtype, static_cast<int>(a->m), static_cast<int>(a->n), static_cast<int>(a->k), a->a, a->b, a->b2, a->c,
                  nullptr, a->row_scale, a->residual, a->act, pl.split, static_cast<float*>(a->workspace),
                  static_cast<cudaStream_t>(stream));
}

// ----------------------------------------------------------------------------------------- attention
static int check_attn(const tb200_attn_args* a) {
  if (a == nullptr) return TB200_ERR_INVALID;
  if (!dtype_ok(a->dtype)) return TB200_ERR_UNSUPPORTED;
  if (a->batch <= 0 || a->seq <= 0 || a->hidden <= 0 || (a->hidden & 7)) return TB200_ERR_INVALID;
  if (a->n_q_heads <= 0 || a->n_kv_heads <= 0 || a->n_q_heads % a->n_kv_heads) return TB200_ERR_INVALID;
  if (a->head_dim != 64 && a->head_dim != 128) return TB200_ERR_UNSUPPORTED;
  if (a->past < 0 || a->cache_len < a->past + a->seq) return TB200_ERR_INVALID;
  if (static_cast<int64_t>(a->batch) * a->seq > (1LL << 30)) return TB200_ERR_INVALID;
  if (!a->x || !a->wq || !a->wk || !a->wv || !a->k_cache || !a->v_cache || !a->o2) return TB200_ERR_INVALID;
  if ((a->flags & TB200_ATTN_KEYFORMER) && (!a->noise || !a->c_out || !(a->tau > 0.f))) return TB200_ERR_INVALID;
  if ((a->flags & TB200_ATTN_ROCO) && (!a->c_out1 || !a->c_out2)) return TB200_ERR_INVALID;
  if ((a->flags & TB200_ATTN_ROCO_VARIANCE) && !(a->flags & TB200_ATTN_ROCO)) return TB200_ERR_INVALID;
  if ((a->flags & (TB200_ATTN_KEYFORMER | TB200_ATTN_ROCO)) && a->aux_dtype != TB200_F32 && a->aux_dtype != a->dtype)
    return TB200_ERR_INVALID;
  if (a->topk < 0 || a->topk > a->past + a->seq) return TB200_ERR_INVALID;
  if (a->topk > 0 && (!a->topk_idx || !(a->flags & (TB200_ATTN_KEYFORMER | TB200_ATTN_ROCO)))) return TB200_ERR_INVALID;
  // requests no kernel exists for are refused here, before the first launch has touched the caches or o2
  if ((a->flags & TB200_ATTN_KEYFORMER) && (a->flags & TB200_ATTN_ROCO)) return TB200_ERR_UNSUPPORTED;
  if (a->topk > 0 && a->past + a->seq > kTopkMaxKeys) return TB200_ERR_UNSUPPORTED;
  if (!(a->sm_scale > 0.f)) return TB200_ERR_INVALID;
  const void* wide[] = {a->x, a->wq, a->wk, a->wv, a->k_cache, a->v_cache, a->o2, a->norm_weight, a->q_norm_weight,
                        a->k_norm_weight, a->noise};
  for (const void* ptr : wide)
    if (!aligned16(ptr)) return TB200_ERR_INVALID;
  const void* narrow[] = {a->c_out, a->c_out1, a->c_out2, a->topk_idx};
  for (const void* ptr : narrow)
    if (!aligned4(ptr)) return TB200_ERR_INVALID;
  return TB200_OK;
}

int tb200_attn_check(const tb200_attn_args* a) { return check_attn(a); }

struct AttnWs {
  void* q;
  void* x_norm;
  float* inv_rms;
  float* lse2;
  float* lse2t;
  float* sum_a;  // fp32 staging of c_out / c_out1 when the caller's tensors are 16-bit
  float* sum_b;
  float* partial;  // fp32 K-slice sums of the QKV projection (decode sizes only)
  int split_qkv;
  int kv_splits;   // attention over a split key range (decode sizes only)
  float* part_o;
  float* part_ml;
  size_t bytes;
};
static AttnWs carve_attn(const tb200_attn_args* a, void* base, int num_sms) {
  Carver c(base);
  AttnWs w;
  const size_t T = static_cast<size_t>(a->batch) * a->seq;
  const size_t rows = static_cast<size_t>(a->batch) * a->n_q_heads * a->seq;
  const size_t keys = static_cast<size_t>(a->batch) * a->n_q_heads * (a->past + a->seq);
  const bool prenorm = a->flags & TB200_ATTN_PRENORM;
  const bool aux = a->flags & (TB200_ATTN_KEYFORMER | TB200_ATTN_ROCO);
  // the normalised activations are only materialised for a norm weight that has not been folded into the projections
  const bool materialise = prenorm && a->norm_weight && !(a->flags & TB200_ATTN_NORM_FOLDED);
  w.q = c.take(rows * a->head_dim * 2);
  w.x_norm = materialise ? c.take(T * a->hidden * 2) : nullptr;
  w.inv_rms = (prenorm && !materialise) ? static_cast<float*>(c.take(T * 4)) : nullptr;
  w.lse2 = static_cast<float*>(c.take(rows * 4));
  w.lse2t = (a->flags & TB200_ATTN_KEYFORMER) ? static_cast<float*>(c.take(rows * 4)) : nullptr;
  const bool stage = aux && a->aux_dtype != TB200_F32;
  w.sum_a = stage ? static_cast<float*>(c.take(keys * 4)) : nullptr;
  w.sum_b = (stage && (a->flags & TB200_ATTN_ROCO)) ? static_cast<float*>(c.take(keys * 4)) : nullptr;
  // few tokens (decode): the projection streams the weights, so K is cut into slices until the SMs are filled
  const int n_tiles = (a->n_q_heads * a->head_dim + kBN - 1) / kBN + 2 * ((a->n_kv_heads * a->head_dim + kBN - 1) / kBN);
  w.split_qkv = choose_split(static_cast<int>(T), n_tiles, a->hidden, num_sms);
  w.partial = w.split_qkv > 1
                  ? static_cast<float*>(c.take(static_cast<size_t>(w.split_qkv) * T * (a->n_q_heads + 2 * a->n_kv_heads) * a->head_dim * 4))
                  : nullptr;
  w.kv_splits = (a->flags & TB200_ATTN_KEYFORMER) ? 1 : attn_kv_splits(a->batch, a->seq, a->n_q_heads, a->past + a->seq, num_sms);
  w.part_o = w.kv_splits > 1 ? static_cast<float*>(c.take(static_cast<size_t>(w.kv_splits) * rows * a->head_dim * 4)) : nullptr;
  w.part_ml = w.kv_splits > 1 ? static_cast<float*>(c.take(static_cast<size_t>(w.kv_splits) * rows * 2 * 4)) : nullptr;
  w.bytes = c.used;
  return w;
}

size_t tb200_attn_workspace_bytes(const tb200_attn_args* a) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st || check_attn(a) != TB200_OK) return 0;
  return carve_attn(a, nullptr, st->num_sms).bytes;
}

// ev: null, or 5 events recorded on the stream at the stage boundaries
static int attn_forward_impl(const tb200_attn_args* a, void* stream_, cudaEvent_t* ev) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  if ((status = check_attn(a)) != TB200_OK) return status;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->workspace == nullptr || !aligned16(a->workspace)) return TB200_ERR_WORKSPACE;
  const AttnWs w = carve_attn(a, a->workspace, st->num_sms);
  if (a->workspace_bytes < w.bytes) return TB200_ERR_WORKSPACE;
  ChainScope chain;
  const int T = a->batch * a->seq;
  const int D = a->head_dim;

  // 1. RMSNorm prologue.  Without a weight, or with the weight folded into the rows of Wq, Wk, Wv
  //    (TB200_ATTN_NORM_FOLDED), only the row statistic is computed and the scale is applied in the projection's
  //    epilogue; with an unfolded weight the normalised activations are materialised.
  const void* A = a->x;
  const float* row_scale = nullptr;
  if (ev) cudaEventRecord(ev[0], stream);
  if (a->flags & TB200_ATTN_PRENORM) {
    if (w.x_norm) {
      status = launch_rmsnorm(a->x, a->norm_weight, w.x_norm, nullptr, T, a->hidden, a->norm_eps, a->dtype, stream);
      A = w.x_norm;
    } else {
      status = launch_rmsnorm(a->x, nullptr, nullptr, w.inv_rms, T, a->hidden, a->norm_eps, a->dtype, stream);
      row_scale = w.inv_rms;
    }
    if (status != TB200_OK) return status;
  }
  // 2. QKV projection with head split, optional per-head norm and cache append in the epilogue.
  //    A block of at most 16 new tokens without a per-key statistic takes the one-kernel decode path after it.
  const bool decode_path = !(a->flags & (TB200_ATTN_KEYFORMER | TB200_ATTN_ROCO)) && attn_decode_applies(a->batch, a->seq, a->n_q_heads, D);
  AttnDecodeLaunch dec;
  if (ev) cudaEventRecord(ev[1], stream);
  {
    GemmLaunch g;
    g.dtype = a->dtype;
    g.mode = GEMM_QKV;
    g.M = T; g.K = a->hidden; g.A = A;
    g.n_src = 3;
    g.B[0] = a->wq; g.N[0] = a->n_q_heads * D;
    g.B[1] = a->wk; g.N[1] = a->n_kv_heads * D;
    g.B[2] = a->wv; g.N[2] = a->n_kv_heads * D;
    g.row_scale = row_scale;
    g.q_out = w.q; g.k_cache = a->k_cache; g.v_cache = a->v_cache;
    g.S = a->seq; g.Hq = a->n_q_heads; g.Hkv = a->n_kv_heads; g.D = D; g.past = a->past; g.cache_len = a->cache_len;
    g.qknorm = (a->flags & TB200_ATTN_QKNORM) ? 1 : 0;
    g.qk_eps = a->qk_eps;
    g.q_norm_weight = a->q_norm_weight;
    g.k_norm_weight = a->k_norm_weight;
    if (w.split_qkv > 1) {  // K slices into fp32 partial sums, then one small kernel with the same epilogue
      g.mode = GEMM_PARTIAL;
      g.row_scale = nullptr;
      g.split_k = w.split_qkv;
      g.partial = w.partial;
      if ((status = launch_gemm(g, stream)) != TB200_OK) return status;
      const int k_blocks = (a->hidden + kBK - 1) / kBK, per = (k_blocks + w.split_qkv - 1) / w.split_qkv;
      if (decode_path) {  // the slices are summed, normalised and appended by the attention kernel itself
        dec.partial = w.partial;
        dec.split = (k_blocks + per - 1) / per;
        dec.row_scale = row_scale;
      } else {
        QkvFinish f;
        f.dtype = a->dtype;
        f.M = T;
        f.split_k = (k_blocks + per - 1) / per;
        f.partial = w.partial;
        f.row_scale = row_scale;
        f.q_out = w.q; f.k_cache = a->k_cache; f.v_cache = a->v_cache;
        f.S = a->seq; f.Hq = a->n_q_heads; f.Hkv = a->n_kv_heads; f.D = D; f.past = a->past; f.cache_len = a->cache_len;
        f.qknorm = g.qknorm; f.qk_eps = a->qk_eps;
        f.q_norm_weight = a->q_norm_weight; f.k_norm_weight = a->k_norm_weight;
        if ((status = launch_qkv_finish(f, stream)) != TB200_OK) return status;
      }
    } else {
      if ((status = launch_gemm(g, stream)) != TB200_OK) return status;
      dec.q = w.q;
    }
    dec.qknorm = g.qknorm;
    dec.qk_eps = a->qk_eps;
    dec.q_norm_weight = a->q_norm_weight;
    dec.k_norm_weight = a->k_norm_weight;
  }
  // 3. softmax(QK^T)V
  if (ev) cudaEventRecord(ev[2], stream);
  if (decode_path) {
    dec.dtype = a->dtype;
    dec.B = a->batch; dec.S = a->seq; dec.Hq = a->n_q_heads; dec.Hkv = a->n_kv_heads; dec.D = D; dec.past = a->past; dec.cache_len = a->cache_len;
    dec.causal = (a->flags & TB200_ATTN_CAUSAL) ? 1 : 0;
    dec.sm_scale = a->sm_scale;
    dec.k_cache = a->k_cache; dec.v_cache = a->v_cache; dec.o2 = a->o2;
    if ((status = launch_attn_decode(dec, stream)) != TB200_OK) return status;
  } else {
    AttnLaunch f;
    f.dtype = a->dtype;
    f.B = a->batch; f.S = a->seq; f.Hq = a->n_q_heads; f.Hkv = a->n_kv_heads; f.D = D; f.past = a->past; f.cache_len = a->cache_len;
    f.causal = (a->flags & TB200_ATTN_CAUSAL) ? 1 : 0;
    f.sm_scale = a->sm_scale;
    f.q = w.q; f.k_cache = a->k_cache; f.v_cache = a->v_cache; f.o2 = a->o2;
    f.lse2 = w.lse2;
    f.kv_splits = w.kv_splits; f.part_o = w.part_o; f.part_ml = w.part_ml;
    if (a->flags & TB200_ATTN_KEYFORMER) {
      f.noise = a->noise;
      f.tau = a->tau;
      f.lse2_perturbed = w.lse2t;
    }
    if ((status = launch_attn_fwd(f, stream)) != TB200_OK) return status;
  }
  // 4. per-key reductions (second pass) and top-k
  if (ev) cudaEventRecord(ev[3], stream);
  if (a->flags & (TB200_ATTN_KEYFORMER | TB200_ATTN_ROCO)) {
    const bool kf = a->flags & TB200_ATTN_KEYFORMER, rc = a->flags & TB200_ATTN_ROCO;
    const bool stage = a->aux_dtype != TB200_F32;
    const int64_t keys = static_cast<int64_t>(a->batch) * a->n_q_heads * (a->past + a->seq);
    auto run_pass = [&](bool with_noise, float* sp, float* sp2, float* spt) {
      ScoreLaunch s;
      s.dtype = a->dtype;
      s.B = a->batch; s.S = a->seq; s.Hq = a->n_q_heads; s.Hkv = a->n_kv_heads; s.D = D; s.past = a->past; s.cache_len = a->cache_len;
      s.causal = (a->flags & TB200_ATTN_CAUSAL) ? 1 : 0;
      s.sm_scale = a->sm_scale;
      s.q = w.q; s.k_cache = a->k_cache; s.lse2 = w.lse2;
      if (with_noise) { s.noise = a->noise; s.tau = a->tau; s.lse2_perturbed = w.lse2t; }
      s.sum_p = sp; s.sum_p2 = sp2; s.sum_pt = spt;
      return launch_score_colreduce(s, stream);
    };
    const float* topk_key = nullptr;
    if (kf) {
      float* dst = stage ? w.sum_a : static_cast<float*>(a->c_out);
      if ((status = run_pass(true, nullptr, nullptr, dst)) != TB200_OK) return status;
      if (stage && (status = launch_cast_f32(dst, a->c_out, keys, a->aux_dtype, stream)) != TB200_OK) return status;
      topk_key = dst;
    } else {
      float* d1 = stage ? w.sum_a : static_cast<float*>(a->c_out1);
      float* d2 = stage ? w.sum_b : static_cast<float*>(a->c_out2);
      if ((status = run_pass(false, d1, d2, nullptr)) != TB200_OK) return status;
      if (a->flags & TB200_ATTN_ROCO_VARIANCE) {
        status = launch_roco_variance(d1, d2, static_cast<int64_t>(a->batch) * a->n_q_heads, a->past + a->seq, a->past, a->seq,
                                      (a->flags & TB200_ATTN_CAUSAL) ? 1 : 0, stream);
        if (status != TB200_OK) return status;
      }
      if (stage) {
        if ((status = launch_cast_f32(d1, a->c_out1, keys, a->aux_dtype, stream)) != TB200_OK) return status;
        if ((status = launch_cast_f32(d2, a->c_out2, keys, a->aux_dtype, stream)) != TB200_OK) return status;
      }
      topk_key = d1;
    }
    if (a->topk > 0) {
      status = launch_topk(topk_key, a->topk_idx, static_cast<int64_t>(a->batch) * a->n_q_heads, a->past + a->seq, a->topk, stream);
      if (status != TB200_OK) return status;
    }
  }
  if (ev) cudaEventRecord(ev[4], stream);
  return TB200_OK;
}

int tb200_attn_forward(const tb200_attn_args* a, void* stream) { return attn_forward_impl(a, stream, nullptr); }

int tb200_attn_forward_timed(const tb200_attn_args* a, void* stream, float* stage_ms) {
  if (stage_ms == nullptr) return TB200_ERR_INVALID;
  cudaEvent_t ev[5];
  for (int i = 0; i < 5; ++i)
    if (cudaEventCreate(&ev[i]) != cudaSuccess) return TB200_ERR_CUDA;
  int status = attn_forward_impl(a, stream, ev);
  if (status == TB200_OK && cudaEventSynchronize(ev[4]) != cudaSuccess) status = TB200_ERR_CUDA;
  for (int i = 0; i < 4; ++i) {
    stage_ms[i] = 0.f;
    if (status == TB200_OK && cudaEventElapsedTime(&stage_ms[i], ev[i], ev[i + 1]) != cudaSuccess) status = TB200_ERR_CUDA;
  }
  for (int i = 0; i < 5; ++i) cudaEventDestroy(ev[i]);
  return status;
}

// ----------------------------------------------------------------------------------------- FFN
static int check_ffn(const tb200_ffn_args* a) {
  if (a == nullptr) return TB200_ERR_INVALID;
  if (!dtype_ok(a->dtype)) return TB200_ERR_UNSUPPORTED;
  if (a->tokens <= 0 || a->hidden <= 0 || a->inner <= 0 || (a->hidden & 7) || (a->inner & 7)) return TB200_ERR_INVALID;
  if (a->tokens > (1 << 30) || a->hidden > (1 << 24) || a->inner > (1 << 24)) return TB200_ERR_INVALID;
  if (a->act != TB200_FFN_SWIGLU && a->act != TB200_FFN_GELU) return TB200_ERR_INVALID;
  if (!a->x || !a->w_gate || !a->w_down || !a->ff2) return TB200_ERR_INVALID;
  if (a->act == TB200_FFN_SWIGLU && !a->w_up) return TB200_ERR_INVALID;
  if ((a->wo == nullptr) != (a->o2 == nullptr)) return TB200_ERR_INVALID;
  if ((a->flags & TB200_FFN_FALCON_TAIL) && !a->o_ff_norm) return TB200_ERR_INVALID;
  if ((a->flags & TB200_FFN_NORM_FOLDED) && (a->flags & TB200_FFN_FALCON_TAIL)) return TB200_ERR_UNSUPPORTED;  // the tail adds h itself
  const void* ptrs[] = {a->x, a->o2, a->wo, a->norm_weight, a->w_gate, a->w_up, a->w_down, a->ff2, a->attn_o2, a->ff1, a->o_ff_norm};
  for (const void* ptr : ptrs)
    if (!aligned16(ptr)) return TB200_ERR_INVALID;
  return TB200_OK;
}

int tb200_ffn_check(const tb200_ffn_args* a) { return check_ffn(a); }

struct FfnWs {
  void* attn_o2;
  void* h;
  float* inv_rms;
  void* ff1;
  void* o_ff;
  float* partial;
  int split_wo, split_up, split_down;
  size_t bytes;
};
static FfnWs carve_ffn(const tb200_ffn_args* a, void* base, int num_sms) {
  Carver c(base);
  FfnWs w;
  const size_t M = a->tokens, N = a->hidden, P = a->inner;
  const bool norm = a->flags & TB200_FFN_NORM, tail = a->flags & TB200_FFN_FALCON_TAIL;
  const bool gated = a->act == TB200_FFN_SWIGLU;
  w.attn_o2 = (a->wo && !a->attn_o2) ? c.take(M * N * 2) : a->attn_o2;
  // h is materialised when the norm has a weight that is not folded into w_gate / w_up, or when the tail needs it as
  // a residual
  const bool folded = a->flags & TB200_FFN_NORM_FOLDED;
  w.h = (norm && ((a->norm_weight && !folded) || tail)) ? c.take(M * N * 2) : nullptr;
  w.inv_rms = (norm && !w.h) ? static_cast<float*>(c.take(M * 4)) : nullptr;
  w.ff1 = a->ff1 ? a->ff1 : c.take(M * P * 2);
  w.o_ff = tail ? c.take(M * N * 2) : nullptr;
  const int n_tiles_n = static_cast<int>((N + kBN - 1) / kBN), n_tiles_p = static_cast<int>((P + kBN - 1) / kBN);
  w.split_wo = a->wo ? choose_split(static_cast<int>(M), n_tiles_n, static_cast<int>(N), num_sms) : 1;
  w.split_up = choose_split(static_cast<int>(M), (gated ? 2 : 1) * n_tiles_p, static_cast<int>(N), num_sms);
  w.split_down = choose_split(static_cast<int>(M), n_tiles_n, static_cast<int>(P), num_sms);
  size_t pb = 0;
  if (w.split_wo > 1) pb = w.split_wo * M * N * 4;
  if (w.split_up > 1 && w.split_up * M * (gated ? 2 : 1) * P * 4 > pb) pb = w.split_up * M * (gated ? 2 : 1) * P * 4;
  if (w.split_down > 1 && w.split_down * M * N * 4 > pb) pb = w.split_down * M * N * 4;
  w.partial = pb ? static_cast<float*>(c.take(pb)) : nullptr;
  w.bytes = c.used;
  return w;
}

size_t tb200_ffn_workspace_bytes(const tb200_ffn_args* a) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st || check_ffn(a) != TB200_OK) return 0;
  return carve_ffn(a, nullptr, st->num_sms).bytes;
}

int tb200_ffn_forward(const tb200_ffn_args* a, void* stream_) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  if ((status = check_ffn(a)) != TB200_OK) return status;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const FfnWs w = carve_ffn(a, a->workspace, st->num_sms);
  if (w.bytes > 0 && (a->workspace == nullptr || a->workspace_bytes < w.bytes || !aligned16(a->workspace))) return TB200_ERR_WORKSPACE;
  const int M = static_cast<int>(a->tokens), N = static_cast<int>(a->hidden), P = static_cast<int>(a->inner);
  const bool norm = a->flags & TB200_FFN_NORM, tail = a->flags & TB200_FFN_FALCON_TAIL;
  ChainScope chain;

  // a = o2 @ wo + x
  const void* act_in = a->x;
  if (a->wo) {
    status = run_gemm(a->dtype, M, N, N, a->o2, a->wo, nullptr, w.attn_o2, nullptr, nullptr, a->x, 0, w.split_wo, w.partial, stream);
    if (status != TB200_OK) return status;
    act_in = w.attn_o2;
  }
  // h = RMSNorm(a): materialised, or folded into the next GEMM's epilogue as a per-row scale
  const void* h = act_in;
  const float* row_scale = nullptr;
  if (norm) {
    if (w.h) {
      status = launch_rmsnorm(act_in, a->norm_weight, w.h, nullptr, M, N, a->norm_eps, a->dtype, stream);
      h = w.h;
    } else {
      status = launch_rmsnorm(act_in, nullptr, nullptr, w.inv_rms, M, N, a->norm_eps, a->dtype, stream);
      row_scale = w.inv_rms;
    }
    if (status != TB200_OK) return status;
  }
  // ff1 = silu(h @ w_gate) * (h @ w_up)   or   gelu(h @ w_gate)
  if (a->act == TB200_FFN_SWIGLU)
    status = run_gemm(a->dtype, M, P, N, h, a->w_gate, a->w_up, w.ff1, nullptr, row_scale, nullptr, 0, w.split_up, w.partial, stream);
  else
    status = run_gemm(a->dtype, M, P, N, h, a->w_gate, nullptr, w.ff1, nullptr, row_scale, nullptr, 1, w.split_up, w.partial, stream);
  if (status != TB200_OK) return status;
  // ff2 = ff1 @ w_down  [o_ff = ff2 + h]
  if (!tail) return run_gemm(a->dtype, M, N, P, w.ff1, a->w_down, nullptr, a->ff2, nullptr, nullptr, nullptr, 0, w.split_down, w.partial, stream);
  status = run_gemm(a->dtype, M, N, P, w.ff1, a->w_down, nullptr, w.o_ff, a->ff2, nullptr, h, 0, w.split_down, w.partial, stream);
  if (status != TB200_OK) return status;
  return launch_rmsnorm(w.o_ff, nullptr, a->o_ff_norm, nullptr, M, N, 0.f, a->dtype, stream, a->tail_divisor);
}

// The attention block and the FFN block that consumes its o2, as one launch chain: the FFN's first projection is
// launched while the attention kernel still runs, sets up and requests its first weight boxes, and waits for o2.
// Everything either block would refuse is refused here before the first launch.
int tb200_layer_forward(const tb200_attn_args* attn, const tb200_ffn_args* ffn, void* stream) {
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  if ((status = check_attn(attn)) != TB200_OK) return status;
  if ((status = check_ffn(ffn)) != TB200_OK) return status;
  if (ffn->o2 == nullptr || ffn->o2 != attn->o2 || ffn->dtype != attn->dtype || ffn->hidden != attn->hidden ||
      ffn->tokens != static_cast<int64_t>(attn->batch) * attn->seq || attn->n_q_heads * attn->head_dim != attn->hidden)
    return TB200_ERR_INVALID;
  if (attn->workspace == nullptr || !aligned16(attn->workspace) || attn->workspace_bytes < carve_attn(attn, nullptr, st->num_sms).bytes)
    return TB200_ERR_WORKSPACE;
  const size_t ffn_need = carve_ffn(ffn, nullptr, st->num_sms).bytes;
  if (ffn_need > 0 && (ffn->workspace == nullptr || !aligned16(ffn->workspace) || ffn->workspace_bytes < ffn_need)) return TB200_ERR_WORKSPACE;
  ChainScope chain;
  if ((status = attn_forward_impl(attn, stream, nullptr)) != TB200_OK) return status;
  return tb200_ffn_forward(ffn, stream);
}

}  // extern "C"
