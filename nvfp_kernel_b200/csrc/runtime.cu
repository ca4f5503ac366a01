// Error reporting, device queries and the device status word of libnvfp_b200.so.
#include <cstring>
#include <mutex>

#include "common.h"

namespace nvfp {
namespace {
thread_local char g_error[512] = "";
__device__ uint32_t g_status_word = 0;
constexpr int kMaxDevices = 64;
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { g_error[0] = '\0'; }

// Per-device caches are filled under std::call_once (one flag per device): two host threads making their first
// call on a device at the same time both see a complete entry.
int current_device_info(DeviceInfo* out) {
  static DeviceInfo cache[kMaxDevices];
  static cudaError_t err[kMaxDevices];
  static std::once_flag once[kMaxDevices];
  int dev = 0;
  NVFP_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(NVFP_ERR_CUDA, "device index %d out of range", dev);
  std::call_once(once[dev], [dev] {
    DeviceInfo d;
    cudaError_t e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev);
    err[dev] = e;
    cache[dev] = d;
  });
  if (err[dev] != cudaSuccess)
    return fail(NVFP_ERR_CUDA, "cudaDeviceGetAttribute failed on device %d: %s", dev, cudaGetErrorString(err[dev]));
  *out = cache[dev];
  return NVFP_OK;
}

uint32_t* device_status_word() {
  static uint32_t* cache[kMaxDevices] = {};
  static std::once_flag once[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::call_once(once[dev], [dev] {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) == cudaSuccess) cache[dev] = static_cast<uint32_t*>(p);
  });
  return cache[dev];
}

}  // namespace nvfp

using namespace nvfp;

extern "C" const char* nvfp_last_error(void) { return g_error; }

extern "C" int nvfp_version(void) { return 1000; }

extern "C" int64_t nvfp_sf_rows_padded(int64_t rows) { return round_up(rows, 128); }

extern "C" int64_t nvfp_sf_cols_padded(int64_t k, int block) {
  if (block <= 0) return -1;
  return round_up(k / block, 4);
}

extern "C" int nvfp_device_status(uint32_t* status_out) {
  clear_error();
  NVFP_REQUIRE(status_out != nullptr, "null pointer");
  uint32_t* word = device_status_word();
  if (!word) return fail(NVFP_ERR_CUDA, "cannot locate the device status word");
  NVFP_CUDA(cudaDeviceSynchronize());
  NVFP_CUDA(cudaMemcpy(status_out, word, sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (*status_out != 0) {
    NVFP_CUDA(cudaMemset(word, 0, sizeof(uint32_t)));
    return fail(NVFP_ERR_DEVICE_TIMEOUT, "a kernel gave up on a bounded wait (code 0x%x)", *status_out);
  }
  return NVFP_OK;
}
