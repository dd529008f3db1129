// Library-wide host state: version, thread-local error text, and the
// per-device status block kernels report into.
#include <mutex>
#include <string.h>

#include "host_common.h"

namespace hdit {
namespace {

constexpr int kMaxDevices = 64;
thread_local char g_error[512] = "";

// Kernels record the first failed bounded wait of a launch here. A file-scope
// device array needs no allocation; its device address is looked up once per device.
__device__ int32_t g_dev_status[16];
int32_t* g_status_ptr[kMaxDevices] = {nullptr};
std::mutex g_status_mutex;

}  // namespace

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int32_t* device_status_ptr() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error(HDIT_ERR_CUDA, "cudaGetDevice failed or device index out of range");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (g_status_ptr[dev] == nullptr) {
    void* d = nullptr;
    e = cudaGetSymbolAddress(&d, g_dev_status);
    if (e != cudaSuccess) {
      set_error(HDIT_ERR_CUDA, "cudaGetSymbolAddress(status block): %s", cudaGetErrorString(e));
      return nullptr;
    }
    g_status_ptr[dev] = static_cast<int32_t*>(d);
  }
  return g_status_ptr[dev];
}

}  // namespace hdit

extern "C" int hdit_version(void) { return 100; }

extern "C" const char* hdit_last_error(void) { return hdit::g_error; }

extern "C" int hdit_device_status(int device, int32_t out[4], int clear) {
  using namespace hdit;
  if (out == nullptr || device < 0 || device >= kMaxDevices) return set_error(HDIT_ERR_BAD_ARG, "bad device or null out");
  int32_t* ptr = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_status_mutex);
    ptr = g_status_ptr[device];
  }
  out[0] = out[1] = out[2] = out[3] = 0;
  if (ptr == nullptr) return HDIT_OK;  // no kernel of this library has run on that device yet
  int prev = 0;
  HDIT_CUDA_OK(cudaGetDevice(&prev));
  HDIT_CUDA_OK(cudaSetDevice(device));
  cudaError_t e = cudaMemcpy(out, ptr, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && clear) e = cudaMemset(ptr, 0, 16 * sizeof(int32_t));
  cudaSetDevice(prev);
  if (e != cudaSuccess) return set_error(HDIT_ERR_CUDA, "reading the status block: %s", cudaGetErrorString(e));
  return HDIT_OK;
}
