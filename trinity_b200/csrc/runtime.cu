// Per-device state, tensor-map encoding and the status helpers of the C ABI.
#include <mutex>

#include "internal.h"

namespace tb200 {

namespace {
constexpr int kMaxDevices = 32;
DeviceState g_states[kMaxDevices];
bool g_ready[kMaxDevices];
std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
}  // namespace

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
  if (cudaMalloc(&st.err_word, sizeof(int)) != cudaSuccess || cudaMemset(st.err_word, 0, sizeof(int)) != cudaSuccess) {
    *status = TB200_ERR_CUDA;
    return nullptr;
  }
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

// Resolve cuTensorMapEncodeTiled without creating the per-device state (no device allocation).
int ensure_tensor_map_encoder() {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_encode) return TB200_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
      qres != cudaDriverEntryPointSuccess)
    return TB200_ERR_CUDA;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return TB200_OK;
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

}  // extern "C"
