// Tensor-parallel down projection with its all-reduce done by the kernels themselves over peer memory (NVLink through
// NVSwitch), in place of "GEMM, then ncclAllReduce" -- the reference has no multi-GPU path at all; this replaces the
// one collective of the row-parallel projection in a tensor-parallel FFN.
//
// Every rank owns M / world consecutive rows of the (M, N) result.
//   1. gemm_kernel<GEMM_PEER> computes this rank's partial product and, tile by tile while its main loop runs on,
//      sends each 128-row block as 16-bit values into the staging buffer of the block's OWNER -- TMA stores from shared
//      memory to a peer pointer, whole lines on the wire -- then arrives on the owner's counter for that block
//      (red.release.sys, once the stores are complete).  The exchange a reduce-scatter would do after the GEMM
//      travels during it.
//      The ranks walk the row tiles in rounds (tile k of owner r, r+1, ... in round k), so after round k every owner
//      has tile k from everybody.
//   2. reduce_broadcast_kernel, launched behind the projection with programmatic stream serialisation, is resident
//      beside it while it runs; every CTA waits (bounded) per owned block until all ranks' warps have arrived, sums
//      the `world` staged contributions in rank order in fp32 (deterministic), adds the optional residual, rounds once
//      and writes the block into EVERY rank's result buffer (the all-gather, again plain peer stores).  Its last CTA
//      tells every peer that this rank's rows are complete and waits (bounded) for the same word from all peers, so
//      that when the kernel ends on a rank, that rank's whole result is in place and every owner has finished reading
//      its staging buffer -- the next call may overwrite it.
// A peer's memory is only ever WRITTEN (tiled stores from shared memory, plain stores, reductions on counters and
// flags); no load of any kind reads it; every wait has a cycle limit after which the
// kernel records a code in the error word and returns.
//
// Counters and flags only ever grow: a communicator is used for ONE shape (M, N, world), call after call, and the
// host passes the values they must reach in this call.
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace tb200 {

namespace {

constexpr int kRbThreads = 256;
constexpr int kRbRows = 128;      // rows per counter (one row block of the GEMM)
constexpr int kRbCols = 256;      // columns per CTA

struct ReduceParams {
  int world, rank, rows_per_rank, N;
  const void* stage;               // this rank's staging buffer: (world, rows_per_rank, N)
  const void* residual;            // (M, N) or null: added once, by the owner
  void* out[kMaxPeers];            // every rank's (M, N) result buffer
  unsigned* counter;               // this rank's counters, one per 128 owned rows
  unsigned counter_target;         // what a counter reaches when all ranks' warps have arrived for this call
  unsigned* ticket;                // this rank's CTA ticket
  unsigned ticket_last;            // the ticket the last CTA of this call draws
  unsigned* done[kMaxPeers];       // every rank's (world) words: done[r][q] = last call rank q completed
  unsigned epoch;
  int* err;
  long long wait_limit;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Wait until *p >= target (wrap-safe), at most `limit` cycles.  One thread calls it.
__device__ __forceinline__ bool wait_reaches(const unsigned* p, unsigned target, long long limit, int* err, int code) {
  const long long t0 = clock64();
  while (static_cast<int>(ld_acquire_sys(p) - target) < 0) {
    if (clock64() - t0 > limit) {
      atomicCAS(err, 0, code);
      return false;
    }
    __nanosleep(64);
  }
  return true;
}

template <typename T>
__global__ void __launch_bounds__(kRbThreads) reduce_broadcast_kernel(const ReduceParams p) {
  __shared__ int go;
  const int col_slices = (p.N + kRbCols - 1) / kRbCols;
  const int rb = blockIdx.x / col_slices;                 // row block of this rank's rows
  const int cs = blockIdx.x - rb * col_slices;
  if (threadIdx.x == 0) go = wait_reaches(p.counter + rb, p.counter_target, p.wait_limit, p.err, 601) ? 1 : 0;
  __syncthreads();
  if (go) {
    const int col0 = cs * kRbCols;
    const int vec_per_row = min(kRbCols, p.N - col0) / 8;
    const long long slot = static_cast<long long>(p.rows_per_rank) * p.N;
    for (int i = threadIdx.x; i < kRbRows * vec_per_row; i += kRbThreads) {
      const int r = i / vec_per_row;
      const int c = col0 + (i - r * vec_per_row) * 8;
      const int local_row = rb * kRbRows + r;
      const long long off = static_cast<long long>(local_row) * p.N + c;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int q = 0; q < p.world; ++q) {                  // rank order: the same sum on every run
        const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.stage) + q * slot + off);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Pack2<T>::unpack(w[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      const long long goff = (static_cast<long long>(p.rank) * p.rows_per_rank + local_row) * p.N + c;
      if (p.residual != nullptr) {
        const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.residual) + goff);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Pack2<T>::unpack(w[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      const uint4 v = make_uint4(Pack2<T>::pack(acc[0], acc[1]), Pack2<T>::pack(acc[2], acc[3]), Pack2<T>::pack(acc[4], acc[5]),
                                 Pack2<T>::pack(acc[6], acc[7]));
      for (int q = 0; q < p.world; ++q) {                  // own copy first, then the peers', starting with the neighbour
        const int dst = (p.rank + q) % p.world;
        *reinterpret_cast<uint4*>(static_cast<T*>(p.out[dst]) + goff) = v;
      }
    }
  }
  // ---- the last CTA of this rank announces completion to every rank and waits for every rank's announcement
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned ticket = atomicAdd(p.ticket, 1u);
    if (ticket == p.ticket_last) {
      __threadfence_system();
      for (int q = 0; q < p.world; ++q) st_release_sys(p.done[q] + p.rank, p.epoch);
      for (int q = 0; q < p.world; ++q)
        if (!wait_reaches(p.done[p.rank] + q, p.epoch, p.wait_limit, p.err, 602)) break;
    }
  }
  // This kernel is launched while the projection before it still runs (see tb200_gemm_peer_reduce) and takes its
  // order from the counters, not from that kernel's completion; it must still not END before the projection has.
  pdl_wait();
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" {

size_t tb200_peer_stage_bytes(int64_t m, int64_t n) { return (m > 0 && n > 0) ? static_cast<size_t>(m) * n * 2 : 0; }

size_t tb200_peer_sync_bytes(int64_t m, int world) {
  // counters: one per 128 rows of a rank's share; ticket: 1; done: `world` words; rounded up to 256 bytes each
  if (m <= 0 || world < 1 || world > kMaxPeers) return 0;
  return 3 * 256 + align_up(static_cast<size_t>(m / world / 128 + 1) * 4, 256);
}

int tb200_gemm_peer_reduce(const tb200_peer_gemm_args* a, void* stream_) {
  if (a == nullptr) return TB200_ERR_INVALID;
  if (a->dtype != TB200_BF16 && a->dtype != TB200_F16) return TB200_ERR_UNSUPPORTED;
  if (a->world < 1 || a->world > kMaxPeers || a->rank < 0 || a->rank >= a->world) return TB200_ERR_INVALID;
  if (a->m <= 0 || a->n <= 0 || a->k <= 0 || (a->n & 7) || (a->k & 7) || a->m > (1 << 30) || a->n > (1 << 30) || a->k > (1 << 30))
    return TB200_ERR_INVALID;
  if (a->m % (128LL * a->world) != 0) return TB200_ERR_UNSUPPORTED;   // whole 128-row blocks per rank
  if (!a->a || !a->b || !aligned16(a->a) || !aligned16(a->b) || !aligned16(a->residual) || a->epoch == 0) return TB200_ERR_INVALID;
  for (int r = 0; r < a->world; ++r)
    if (!a->stage[r] || !a->out[r] || !a->sync[r] || !aligned16(a->stage[r]) || !aligned16(a->out[r]) || (reinterpret_cast<uintptr_t>(a->sync[r]) & 255))
      return TB200_ERR_INVALID;
  int status = TB200_OK;
  DeviceState* st = device_state(&status);
  if (!st) return status;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int rows_per_rank = static_cast<int>(a->m / a->world);
  const int n_tiles = static_cast<int>((a->n + 255) / 256);
  // layout of a rank's sync block: [0,256) ticket, [256,512) done words, [512,768) spare, [768,...) block counters
  auto ticket_of = [&](int r) { return reinterpret_cast<unsigned*>(a->sync[r]); };
  auto done_of = [&](int r) { return reinterpret_cast<unsigned*>(static_cast<uint8_t*>(a->sync[r]) + 256); };
  auto counters_of = [&](int r) { return reinterpret_cast<unsigned*>(static_cast<uint8_t*>(a->sync[r]) + 768); };

  ChainScope chain;
  GemmLaunch g;
  g.dtype = a->dtype;
  g.mode = GEMM_PEER;
  g.M = static_cast<int>(a->m); g.K = static_cast<int>(a->k); g.A = a->a;
  g.n_src = 1;
  g.B[0] = a->b; g.N[0] = static_cast<int>(a->n);
  g.world = a->world; g.rank = a->rank; g.rows_per_rank = rows_per_rank;
  for (int r = 0; r < a->world; ++r) {
    g.peer_stage[r] = a->stage[r];
    g.peer_counter[r] = counters_of(r);
  }
  if ((status = launch_gemm(g, stream)) != TB200_OK) return status;

  ReduceParams p;
  memset(&p, 0, sizeof(p));
  p.world = a->world; p.rank = a->rank; p.rows_per_rank = rows_per_rank; p.N = static_cast<int>(a->n);
  p.stage = a->stage[a->rank];
  p.residual = a->residual;
  for (int r = 0; r < a->world; ++r) {
    p.out[r] = a->out[r];
    p.done[r] = done_of(r);
  }
  p.counter = counters_of(a->rank);
  // arrivals per block and call: every rank, once per column tile
  p.counter_target = a->epoch * static_cast<unsigned>(a->world * n_tiles);
  const int col_slices = static_cast<int>((a->n + kRbCols - 1) / kRbCols);
  const unsigned ctas = static_cast<unsigned>(rows_per_rank / kRbRows * col_slices);
  p.ticket = ticket_of(a->rank);
  p.ticket_last = a->epoch * ctas - 1;
  p.epoch = a->epoch;
  p.err = st->err_word;
  p.wait_limit = wait_limit_cycles();
  // Chained to the projection: its CTAs (256 threads, no shared memory) become resident beside the projection's while
  // that kernel runs -- all of whose CTAs are resident by then, so it never waits for an SM -- and each reduces its
  // block as soon as the block's counter says that every rank's contribution has landed.
  cudaError_t e;
  if (a->dtype == TB200_BF16) e = launch_chained(reduce_broadcast_kernel<__nv_bfloat16>, dim3(ctas, 1, 1), dim3(kRbThreads, 1, 1), 0, stream, p);
  else e = launch_chained(reduce_broadcast_kernel<__half>, dim3(ctas, 1, 1), dim3(kRbThreads, 1, 1), 0, stream, p);
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

// ---- CUDA IPC plumbing for hosts that run one process per GPU: export a device allocation, open a peer's.
int tb200_ipc_export(const void* ptr, void* handle64, int64_t* offset_out) {
  if (!ptr || !handle64 || !offset_out) return TB200_ERR_INVALID;
  CUdeviceptr base = 0;
  size_t size = 0;
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return TB200_ERR_CUDA;
  if (reinterpret_cast<RangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return TB200_ERR_CUDA;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) return TB200_ERR_CUDA;
  static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
  memcpy(handle64, &h, 64);
  *offset_out = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return TB200_OK;
}

int tb200_ipc_open(const void* handle64, int64_t offset, void** ptr_out) {
  if (!handle64 || !ptr_out || offset < 0) return TB200_ERR_INVALID;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* base = nullptr;
  if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return TB200_ERR_CUDA;
  *ptr_out = static_cast<uint8_t*>(base) + offset;
  return TB200_OK;
}

int tb200_ipc_close(void* ptr, int64_t offset) {
  if (!ptr) return TB200_ERR_INVALID;
  return cudaIpcCloseMemHandle(static_cast<uint8_t*>(ptr) - offset) == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}

}  // extern "C"
