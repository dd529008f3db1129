// Peer-memory plumbing for one NVSwitch domain: a symmetric heap per GPU that
// every other rank maps through CUDA IPC, plus the flag kernels that order
// peer stores against their consumers.
//
// Flags are 32-bit counters in the heap. A producer publishes with
// st.release.sys after its data stores; a consumer polls with ld.acquire.sys.
// Every poll loop has an iteration limit: when it runs out the kernel writes
// HDIT_ERR_PEER_TIMEOUT and the index of the silent peer into the device status
// block and returns, so a lost rank turns into a host-side error instead of a
// hung GPU. Loads and stores are plain peer accesses -- no multimem, no TMA
// multicast.
#include <cuda_runtime.h>
#include <string.h>

#include "host_common.h"

namespace hdit {
namespace {

constexpr int kMaxPeers = 8;
constexpr int kWherePeerBarrier = 100;
constexpr int kWherePeerWait = 101;

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct BarrierParams {
  int32_t* peer_slot[kMaxPeers];  // address, in peer p's heap, of the counter this rank bumps
  const int32_t* my_slot[kMaxPeers];  // address, in this rank's heap, of the counter peer p bumps
  int n;
  int me;
  int32_t epoch;
  int32_t* epoch_counter;  // when set: the epoch is read from (and advanced in) device memory
  unsigned max_spins;
  int32_t* status;
};

// One warp: lane p signals peer p, then waits for peer p's signal.
__global__ void peer_barrier_kernel(const __grid_constant__ BarrierParams p) {
  const int lane = threadIdx.x;
  __shared__ int abort_flag;
  if (lane == 0) abort_flag = 0;
  // A counter in device memory keeps the barrier replayable from a CUDA graph: every execution
  // advances the epoch by itself instead of carrying a value baked in at capture time.
  int32_t epoch = p.epoch;
  if (p.epoch_counter != nullptr) {
    if (lane == 0) {
      epoch = *p.epoch_counter + 1;
      *p.epoch_counter = epoch;
    }
    epoch = __shfl_sync(0xffffffffu, epoch, 0);
  }
  __syncwarp();
  if (lane < p.n && lane != p.me) {
    __threadfence_system();
    st_release_sys(p.peer_slot[lane], epoch);
    bool seen = false;
    for (unsigned i = 0; i < p.max_spins; ++i) {
      // counters only grow; ">=" also accepts a peer that is already one barrier ahead
      if (ld_acquire_sys(p.my_slot[lane]) - epoch >= 0) {
        seen = true;
        break;
      }
      __nanosleep(64);
    }
    if (!seen) report_failure(p.status, &abort_flag, HDIT_ERR_PEER_TIMEOUT, kWherePeerBarrier, lane);
  }
}

// With `counter` (a device int32 of the calling rank) the sequence number is taken from it and advanced by the
// kernel itself, so a captured CUDA graph containing the call stays replayable; `value` is then ignored.
__global__ void peer_signal_kernel(int32_t* flag, int32_t value, int32_t* counter) {
  if (threadIdx.x == 0) {
    if (counter != nullptr) {
      value = *counter + 1;
      *counter = value;
    }
    __threadfence_system();
    st_release_sys(flag, value);
  }
}

__global__ void peer_wait_kernel(const int32_t* flag, int32_t value, unsigned max_spins, int32_t* status, int tag,
                                 int32_t* counter) {
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    if (counter != nullptr) {
      value = *counter + 1;
      *counter = value;
    }
    bool seen = false;
    for (unsigned i = 0; i < max_spins; ++i) {
      if (ld_acquire_sys(flag) - value >= 0) {
        seen = true;
        break;
      }
      __nanosleep(64);
    }
    if (!seen) report_failure(status, &abort_flag, HDIT_ERR_PEER_TIMEOUT, kWherePeerWait, tag);
  }
}

}  // namespace
}  // namespace hdit

extern "C" int hdit_heap_alloc(int64_t bytes, void** out) {
  using namespace hdit;
  if (out == nullptr || bytes <= 0) return set_error(HDIT_ERR_BAD_ARG, "bad heap size or null out");
  void* p = nullptr;
  HDIT_CUDA_OK(cudaMalloc(&p, static_cast<size_t>(bytes)));
  cudaError_t e = cudaMemset(p, 0, static_cast<size_t>(bytes));
  if (e != cudaSuccess) {
    cudaFree(p);
    return set_error(HDIT_ERR_CUDA, "cudaMemset(heap): %s", cudaGetErrorString(e));
  }
  HDIT_CUDA_OK(cudaDeviceSynchronize());
  *out = p;
  return HDIT_OK;
}

extern "C" int hdit_heap_free(void* ptr) {
  using namespace hdit;
  if (ptr == nullptr) return HDIT_OK;
  HDIT_CUDA_OK(cudaFree(ptr));
  return HDIT_OK;
}

extern "C" int hdit_ipc_export(void* ptr, unsigned char handle[64]) {
  using namespace hdit;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (ptr == nullptr || handle == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null pointer");
  cudaIpcMemHandle_t h;
  HDIT_CUDA_OK(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle, &h, 64);
  return HDIT_OK;
}

extern "C" int hdit_ipc_open(const unsigned char handle[64], void** out) {
  using namespace hdit;
  if (handle == nullptr || out == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  HDIT_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return HDIT_OK;
}

extern "C" int hdit_ipc_close(void* ptr) {
  using namespace hdit;
  if (ptr == nullptr) return HDIT_OK;
  HDIT_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return HDIT_OK;
}

extern "C" int hdit_peer_barrier(int32_t* const* peer_slots, const int32_t* const* my_slots, int n, int me,
                                 int32_t epoch, int32_t* epoch_counter, int64_t max_spins, void* stream) {
  using namespace hdit;
  if (n < 1 || n > kMaxPeers || me < 0 || me >= n) return set_error(HDIT_ERR_BAD_ARG, "bad group size or index");
  if (n == 1) return HDIT_OK;
  if (peer_slots == nullptr || my_slots == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null slot table");
  BarrierParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < n; ++i) {
    if (i != me && (peer_slots[i] == nullptr || my_slots[i] == nullptr))
      return set_error(HDIT_ERR_NOT_INITIALISED, "peer %d is not mapped", i);
    p.peer_slot[i] = peer_slots[i];
    p.my_slot[i] = my_slots[i];
  }
  p.n = n;
  p.me = me;
  p.epoch = epoch;
  p.epoch_counter = epoch_counter;
  p.max_spins = static_cast<unsigned>(max_spins > 0 ? (max_spins > 0xffffffffLL ? 0xffffffffLL : max_spins) : 1);
  p.status = device_status_ptr();
  if (p.status == nullptr) return HDIT_ERR_CUDA;
  peer_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}

extern "C" int hdit_peer_signal(int32_t* flag, int32_t value, int32_t* seq_counter, void* stream) {
  using namespace hdit;
  if (flag == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null flag");
  peer_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flag, value, seq_counter);
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}

extern "C" int hdit_peer_wait(const int32_t* flag, int32_t value, int32_t* seq_counter, int64_t max_spins, int32_t tag,
                              void* stream) {
  using namespace hdit;
  if (flag == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null flag");
  int32_t* status = device_status_ptr();
  if (status == nullptr) return HDIT_ERR_CUDA;
  const unsigned spins = static_cast<unsigned>(max_spins > 0 ? (max_spins > 0xffffffffLL ? 0xffffffffLL : max_spins) : 1);
  peer_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flag, value, spins, status, tag, seq_counter);
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}
