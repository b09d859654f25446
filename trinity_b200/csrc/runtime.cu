// Per-device state, tensor-map encoding and the status helpers of the C ABI.
#include <atomic>
#include <mutex>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

// The device error word: a DEVICE symbol, one instance per GPU that loads the library.  In host code the name is only
// a handle; its device address is looked up once per device (that device current) with cudaGetSymbolAddress and
// handed to every kernel.  Being part of the library image it costs no allocation.
static __device__ int g_err_word;

namespace {
constexpr int kMaxDevices = 32;
DeviceState g_states[kMaxDevices];
bool g_ready[kMaxDevices];
std::mutex g_mu;
std::atomic<long long> g_wait_limit{4000000000LL};   // = kDefaultWaitLimitCycles of common.cuh

std::atomic<int> g_chained{1};
thread_local int t_chain_depth = 0;      // ChainScopes open on this thread (a call may be made of calls)
thread_local bool t_chain_first = true;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
}  // namespace

ChainScope::ChainScope() {
  if (t_chain_depth++ == 0) t_chain_first = true;   // only the outermost scope starts a chain
}
ChainScope::~ChainScope() { --t_chain_depth; }
bool chain_next_launch() {
  const bool chained = t_chain_depth > 0 && !t_chain_first && g_chained.load(std::memory_order_relaxed) != 0;
  t_chain_first = false;
  return chained;
}

DeviceState* device_state(int* status) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *status = TB200_ERR_CUDA;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_ready[dev]) return &g_states[dev];
  DeviceState& st = g_states[dev];
  st.device = dev;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
    *status = TB200_ERR_CUDA;
    return nullptr;
  }
  if (prop.major != 10) {  // the kernels are sm_100a only; there is no fallback
    *status = TB200_ERR_UNSUPPORTED;
    return nullptr;
  }
  st.num_sms = prop.multiProcessorCount;
  void* err = nullptr;
  if (cudaGetSymbolAddress(&err, g_err_word) != cudaSuccess || err == nullptr) {
    *status = TB200_ERR_CUDA;
    return nullptr;
  }
  st.err_word = static_cast<int*>(err);
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
        qres != cudaDriverEntryPointSuccess) {
      *status = TB200_ERR_CUDA;
      return nullptr;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  g_ready[dev] = true;
  return &st;
}

long long wait_limit_cycles() { return g_wait_limit.load(std::memory_order_relaxed); }

// A kernel whose only job is to run one bounded wait to its end: one CTA, one mbarrier that nothing ever arms.  It
// goes through the same mbar_wait / AbortCtx code as the compute kernels: the wait gives up after `limit` cycles,
// records `code` in the device error word, raises the CTA's abort flag, and the kernel returns normally.
__global__ void wait_selftest_kernel(int* err, long long limit, int code, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const AbortCtx ctx{err, &abort_flag, limit};
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait(&bar, 0, ctx, code);   // phase 0 never completes
  __syncthreads();
  if (threadIdx.x == 0 && gave_up != nullptr) *gave_up = (!ok && abort_flag) ? 1 : 0;
}

int make_tensor_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box) {
  if (!g_encode) return TB200_ERR_CUDA;
  cuuint64_t gdim[5];
  cuuint64_t gstride[5];
  cuuint32_t gbox[5];
  cuuint32_t estride[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    estride[i] = 1;
    if (i + 1 < rank) gstride[i] = strides_bytes[i];
  }
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim,
                        gstride, gbox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TB200_OK : TB200_ERR_CUDA;
}

}  // namespace tb200

extern "C" {

const char* tb200_strerror(int status) {
  switch (status) {
    case TB200_OK: return "ok";
    case TB200_ERR_INVALID: return "invalid argument (null pointer, unsupported shape or misaligned pointer)";
    case TB200_ERR_UNSUPPORTED: return "unsupported request or device (sm_100a only, no fallback)";
    case TB200_ERR_CUDA: return "a CUDA call failed";
    case TB200_ERR_WORKSPACE: return "workspace missing or too small";
    case TB200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case TB200_ERR_SCRATCH_LIMIT: return "the problem needs more scratch than the library's built-in 16 MiB array";
    default: return "unknown status";
  }
}

int tb200_version(void) { return 1000; }

int tb200_device_status(int* code_out) {
  int status = TB200_OK;
  tb200::DeviceState* st = tb200::device_state(&status);
  if (!st) return status;
  if (cudaDeviceSynchronize() != cudaSuccess) return TB200_ERR_CUDA;
  int code = 0;
  if (cudaMemcpy(&code, st->err_word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return TB200_ERR_CUDA;
  if (code != 0) cudaMemset(st->err_word, 0, sizeof(int));
  if (code_out) *code_out = code;
  return code == 0 ? TB200_OK : TB200_ERR_DEVICE_TIMEOUT;
}

int tb200_set_wait_limit_cycles(long long cycles) {
  if (cycles < 1000) return TB200_ERR_INVALID;
  tb200::g_wait_limit.store(cycles, std::memory_order_relaxed);
  return TB200_OK;
}

long long tb200_get_wait_limit_cycles(void) { return tb200::wait_limit_cycles(); }

int tb200_set_chained_launch(int enabled) { return tb200::g_chained.exchange(enabled ? 1 : 0, std::memory_order_relaxed); }

int tb200_selftest_wait_timeout(long long limit_cycles, void* stream) {
  if (limit_cycles < 1000 || limit_cycles > 2000000000LL) return TB200_ERR_INVALID;   // at most about a second
  int status = TB200_OK;
  tb200::DeviceState* st = tb200::device_state(&status);
  if (!st) return status;
  tb200::wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(st->err_word, limit_cycles, 900, nullptr);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

}  // extern "C"
