// Host-side helpers shared by the C-ABI translation units: thread-local error
// text, CUDA error mapping, and the per-device status block that kernels write
// to when one of their bounded waits runs out.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/hdit.h"

namespace hdit {

// printf-style; stores the text for hdit_last_error() and returns `code`.
int set_error(int code, const char* fmt, ...);

// Device pointer (valid on the current device) of the int32[16] status block.
// Lazily created; returns nullptr and sets the error text on failure.
int32_t* device_status_ptr();

#define HDIT_CUDA_OK(expr)                                                                       \
  do {                                                                                           \
    cudaError_t _e = (expr);                                                                     \
    if (_e != cudaSuccess)                                                                       \
      return ::hdit::set_error(HDIT_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                               __FILE__, __LINE__);                                              \
  } while (0)

// Device-side: record the first failure of this launch and raise the CTA abort flag.
__device__ __forceinline__ void report_failure(int32_t* status, volatile int* abort_flag, int code, int where,
                                               int iter) {
  *abort_flag = 1;
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = static_cast<int32_t>(blockIdx.x);
    status[2] = where;
    status[3] = iter;
    __threadfence_system();
  }
}

}  // namespace hdit
