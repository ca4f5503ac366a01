// Arithmetic of the NVFP4 quantizer, shared by the quantizer kernels and by the GEMM epilogue that writes its
// result as NVFP4: one definition, so both produce the same bytes.
//
// It follows, step by step, the reference's cvt_warp_fp16_to_fp4 (kernel/nvfp4_utils.cuh:166-242 of
// huweim/nvfp_kernel): block amax in the input type, s = gs * (amax * rcp(6)), ue4m3 round-to-nearest-saturate,
// output scale rcp(s' * rcp(gs)), flush-to-zero fp32 multiplies (the reference is built with --use_fast_math,
// setup.py:45) and cvt.rn.satfinite.e2m1x2.f32.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdint>

namespace nvfp {
namespace {

__device__ __forceinline__ float rcp_approx_ftz(float a) {
  float b;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(b) : "f"(a));
  return b;
}

__device__ __forceinline__ float mul_ftz(float a, float b) {
  float c;
  asm("mul.ftz.f32 %0, %1, %2;" : "=f"(c) : "f"(a), "f"(b));
  return c;
}

// Eight fp32 -> eight e2m1 nibbles in one word; value i lands in bits [4i, 4i+4).
// cvt.rn.satfinite.e2m1x2.f32 d, a, b puts a in the high and b in the low nibble.
__device__ __forceinline__ uint32_t cvt_e2m1x8(float f0, float f1, float f2, float f3, float f4,
                                               float f5, float f6, float f7) {
  uint32_t r;
  asm("{\n"
      ".reg .b8 q0, q1, q2, q3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 q0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 q1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 q2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 q3, %8, %7;\n"
      "mov.b32 %0, {q0, q1, q2, q3};\n"
      "}"
      : "=r"(r)
      : "f"(f0), "f"(f1), "f"(f2), "f"(f3), "f"(f4), "f"(f5), "f"(f6), "f"(f7));
  return r;
}

template <typename T> struct Vec2;
template <> struct Vec2<__half> { using type = __half2; };
template <> struct Vec2<__nv_bfloat16> { using type = __nv_bfloat162; };

template <typename T> __device__ __forceinline__ float2 to_float2(typename Vec2<T>::type v);
template <> __device__ __forceinline__ float2 to_float2<__half>(__half2 v) { return __half22float2(v); }
template <> __device__ __forceinline__ float2 to_float2<__nv_bfloat16>(__nv_bfloat162 v) {
  return __bfloat1622float2(v);
}
template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

// Maximum of two NON-NEGATIVE floats that propagates NaN, as torch.max does (the global scale of a tensor is
// 2688 / torch.abs(x).max() in the reference, speed_test.py:46-47: a NaN anywhere makes it NaN).  Non-negative floats
// order like their bit patterns, and a positive NaN's pattern is above infinity's.  The BLOCK maxima of the quantizers
// are a different matter: they follow the reference kernel's __hmax2, which skips a NaN operand.
__device__ __forceinline__ float max_nan_nonneg(float a, float b) {
  return __uint_as_float(max(__float_as_uint(a), __float_as_uint(b)));
}

template <typename T> __device__ __forceinline__ typename Vec2<T>::type zero2();
template <> __device__ __forceinline__ __half2 zero2<__half>() { return __float2half2_rn(0.0f); }
template <> __device__ __forceinline__ __nv_bfloat162 zero2<__nv_bfloat16>() {
  return __float2bfloat162_rn(0.0f);
}

// One NVFP4 block: 16 values of type T, held as 8 packed pairs, -> its ue4m3 scale byte and 8 bytes of e2m1
// nibbles (value i in bits [4i, 4i+4) of the 64-bit result).  gs: the tensor's global scale, rcp_gs =
// rcp_approx_ftz(gs), rcp6 = rcp_approx_ftz(6.0f).
template <typename T>
__device__ __forceinline__ uint2 nvfp4_quantize_block(const typename Vec2<T>::type (&h2)[8], float gs, float rcp_gs,
                                                      float rcp6, uint8_t& sf_byte) {
  auto mx2 = __habs2(h2[0]);
#pragma unroll
  for (int i = 1; i < 8; ++i) mx2 = __hmax2(mx2, __habs2(h2[i]));
  const float amax = to_float<T>(__hmax(mx2.x, mx2.y));
  const float sf_value = mul_ftz(gs, mul_ftz(amax, rcp6));
  sf_byte = (uint8_t)__nv_cvt_float_to_fp8(sf_value, __NV_SATFINITE, __NV_E4M3);
  const float sf_q = __half2float(__half(__nv_cvt_fp8_to_halfraw(sf_byte, __NV_E4M3)));
  const float out_scale = sf_q != 0.0f ? rcp_approx_ftz(mul_ftz(sf_q, rcp_gs)) : 0.0f;
  float2 f[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    f[i] = to_float2<T>(h2[i]);
    f[i].x = mul_ftz(f[i].x, out_scale);
    f[i].y = mul_ftz(f[i].y, out_scale);
  }
  uint2 packed;
  packed.x = cvt_e2m1x8(f[0].x, f[0].y, f[1].x, f[1].y, f[2].x, f[2].y, f[3].x, f[3].y);
  packed.y = cvt_e2m1x8(f[4].x, f[4].y, f[5].x, f[5].y, f[6].x, f[6].y, f[7].x, f[7].y);
  return packed;
}

}  // namespace
}  // namespace nvfp
