// Host-side helpers shared by the translation units of libnvfp_b200.so.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/nvfp_b200.h"

namespace nvfp {

// Stores a printf-style message for nvfp_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

// Properties of the current device, queried once per device (not once per process:
// the reference caches the first device's attribute for all devices,
// kernel/cuda_utils_kernels.cu:18-31).
struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0;
  int cc_minor = 0;
};
int current_device_info(DeviceInfo* out);

inline int64_t round_up(int64_t x, int64_t y) { return (x + y - 1) / y * y; }
inline int64_t ceil_div(int64_t x, int64_t y) { return (x + y - 1) / y; }

// Device status word written by kernels whose bounded waits expire.
uint32_t* device_status_word();

// nvfp_dynamic_fp4_quant without the argument checks.  release_next: the (last) kernel of the call lets a following
// kernel launched with programmatic stream serialization start at once (that kernel must not touch this
// call's outputs before its own griddepcontrol.wait).  *one_pass tells whether the single cooperative launch ran.
int dynamic_fp4_quant_launch(void* out_fp4, void* out_sf, float* gs_out, float* alpha_out, uint32_t* scratch,
                             const void* in, int64_t m, int64_t n, int64_t stride, int in_dtype,
                             const float* gs_weight, bool release_next, bool* one_pass, cudaStream_t stream);
// gs_out = rcp(max|in|) * 2688 and, when gs_other is given, alpha_out = 1 / (gs_out * gs_other[0]), with the
// self-cleaning eight-word scratch of nvfp_activation_scales (no argument checks).
int activation_scales_launch(float* gs_out, float* alpha_out, uint32_t* scratch, const void* in, int64_t m, int64_t n,
                             int64_t stride, int in_dtype, const float* gs_other, cudaStream_t stream);
// nvfp_scaled_fp4_quant without the public wrapper: release_next as above.
int scaled_fp4_quant_launch(void* out_fp4, void* out_sf, const void* in, const float* gs, int64_t m, int64_t n,
                            int64_t stride, int in_dtype, bool release_next, cudaStream_t stream);
// Whether that call would take the one-pass path for an [m, n] tensor on the current device.
bool dynamic_fp4_quant_is_one_pass(int64_t m, int64_t n, int in_dtype);

}  // namespace nvfp

#define NVFP_REQUIRE(cond, ...)                                             \
  do {                                                                      \
    if (!(cond)) return ::nvfp::fail(NVFP_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

#define NVFP_CUDA(call)                                                                   \
  do {                                                                                    \
    cudaError_t e_ = (call);                                                              \
    if (e_ != cudaSuccess)                                                                \
      return ::nvfp::fail(NVFP_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); \
  } while (0)
