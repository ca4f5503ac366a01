// NVFP4 / MXFP4 quantizers, the approximate-reciprocal op and the global-scale
// reduction for sm_100a.
//
// The arithmetic of the NVFP4 quantizer follows, step by step, the reference's
// cvt_warp_fp16_to_fp4 (kernel/nvfp4_utils.cuh:166-242 of huweim/nvfp_kernel) so
// that packed nibbles and scale bytes are bit-identical: block amax in the input
// type, s = gs*(amax*rcp(6)), ue4m3 round-to-nearest-saturate, output scale
// rcp(s'*rcp(gs)), flush-to-zero fp32 multiplies (the reference is built with
// --use_fast_math, setup.py:45) and cvt.rn.satfinite.e2m1x2.f32.
//
// What is new is the data movement: one CTA owns a 128-row x (4 scale columns) tile,
// which is exactly one 512-byte chunk of the swizzled [mTile][kTile][32][4][4] scale
// layout (kernel/nvfp4_utils.cuh:126-153).  Scale bytes are staged in shared memory
// and leave as 32 coalesced 16-byte stores instead of the reference's scattered
// 1-byte stores; every thread keeps four 16-byte loads in flight; padding bytes of
// the scale tensor are written as zero.
//
// Kernels: quant_fp4_kernel<T, BLOCK, DYNAMIC> (the tiled quantizer; DYNAMIC = the global scale is this tensor's own
// maximum, found in the same cooperative launch), quant_fp4_small_kernel (the same for decode-sized tensors, one
// cluster), amax_kernel (global scale and alpha of a tensor too large for one pass), rcp_kernel.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <mutex>
#include <type_traits>

#include "common.h"
#include "quant_math.cuh"
#include "ptx_sm100.cuh"

namespace nvfp {
namespace {

__device__ __forceinline__ uint64_t global_timer_ns_q() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

template <typename T>
union Pack8 {
  uint4 raw;
  typename Vec2<T>::type h2[4];
};

// |max| of the 8 values held by this thread, in the input type.
template <typename T>
__device__ __forceinline__ typename Vec2<T>::type local_absmax2(const Pack8<T>& v) {
  auto mx = __habs2(v.h2[0]);
#pragma unroll
  for (int i = 1; i < 4; ++i) mx = __hmax2(mx, __habs2(v.h2[i]));
  return mx;
}

// 8 values * scale -> 8 packed nibbles.
template <typename T>
__device__ __forceinline__ uint32_t scale_and_pack(const Pack8<T>& v, float scale) {
  float2 f[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[i] = to_float2<T>(v.h2[i]);
    f[i].x = mul_ftz(f[i].x, scale);
    f[i].y = mul_ftz(f[i].y, scale);
  }
  return cvt_e2m1x8(f[0].x, f[0].y, f[1].x, f[1].y, f[2].x, f[2].y, f[3].x, f[3].y);
}

constexpr int kThreads = 256;
constexpr int kTileRows = 128;
constexpr int kTileCols = 128;   // 8 threads x 16 elements per row segment

// 16 consecutive elements (32 bytes) of one row.
template <typename T>
union Pack16 {
  uint4 raw[2];
  typename Vec2<T>::type h2[8];
};

// One 32-byte load (sm_100 has 256-bit global loads) when the address allows it, else two
// 16-byte loads.
template <typename T>
__device__ __forceinline__ void load16(Pack16<T>& v, const T* src, bool aligned32) {
  if (aligned32) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v.raw[0].x), "=r"(v.raw[0].y), "=r"(v.raw[0].z), "=r"(v.raw[0].w),
                   "=r"(v.raw[1].x), "=r"(v.raw[1].y), "=r"(v.raw[1].z), "=r"(v.raw[1].w)
                 : "l"(src));
  } else {
    v.raw[0] = __ldg(reinterpret_cast<const uint4*>(src));
    v.raw[1] = __ldg(reinterpret_cast<const uint4*>(src) + 1);
  }
}

// BLOCK = elements per scale (16: NVFP4 / ue4m3, 32: MXFP4 / ue8m0).
//
// One CTA owns 128 rows x 128 columns.  A thread owns 16 consecutive elements of a row: for
// NVFP4 that is a whole scale block, so the block maximum needs no shuffle and the scale is
// computed once (the reference computes it twice, in both threads of a pair,
// kernel/nvfp4_utils.cuh:170-216); for MXFP4 two neighbouring threads share a block.  Each thread
// issues its four row segments' loads before touching any of them.  The tile's scale bytes (two
// 512-byte chunks for NVFP4, one for MXFP4) are staged in shared memory and stored with 16-byte
// stores; packed nibbles leave as 8 bytes per thread, 64 contiguous bytes per row.
//
// DYNAMIC (NVFP4 only): the global scale is not an input but 2688 / max|x| of this very tensor.  Every CTA
// holds its whole tile in registers after the loads, so the launch (a cooperative one: all CTAs resident)
// reduces the tile maxima through two words of global memory, waits for the last CTA, and quantizes from
// the registers: the tensor is read once, in one launch, where a global-scale pass plus a quantize pass read
// it twice in two.  The wait is bounded; when it runs out the CTA reports through the device status word and
// goes on with the maximum it sees.
struct DynamicScale {
  uint32_t* scratch;      // [max bits, arrivals] x 2 pairs, [4] = which pair this launch uses (self-cleaning)
  float* gs_out;          // 2688 / max|x|
  const float* gs_other;  // the other operand's global scale, or null
  float* alpha_out;       // 1 / (gs_out * gs_other), written when gs_other is given
  uint32_t* status;       // device status word
  int release_next;       // let a programmatically dependent next kernel start while this one runs
  int wait_prev;          // launched with programmatic stream serialization behind the kernel that writes the
                          // global scale: the tile is loaded first, the scale read after griddepcontrol.wait
};
constexpr uint32_t kErrQuantBarrier = 1u << 8;

template <typename T, int BLOCK, bool DYNAMIC>
__global__ void __launch_bounds__(kThreads)
quant_fp4_kernel(const T* __restrict__ in, int64_t in_stride, const float* __restrict__ gs_ptr,
                 uint8_t* __restrict__ out, uint8_t* __restrict__ sf_out, int m, int n,
                 int num_col_tiles, int num_k_chunks, int mx_rounding, int aligned32, const DynamicScale dyn) {
  static_assert(!DYNAMIC || BLOCK == 16, "only NVFP4 has a global scale");
  if (dyn.release_next) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int kThreadsPerRow = kTileCols / 16;                    // 8
  constexpr int kRowsPerPass = kThreads / kThreadsPerRow;           // 32
  constexpr int kPasses = kTileRows / kRowsPerPass;                 // 4: all in flight at once
  constexpr int kThreadsPerBlock = BLOCK / 16;                      // 1 or 2 threads per scale
  constexpr int kChunksPerTile = kTileCols / (4 * BLOCK);           // 2 or 1 scale chunks per tile

  __shared__ __align__(16) uint8_t sf_stage[kChunksPerTile * 512];

  // Tiles are walked from the END of the tensor backwards: the global-scale pass that normally runs
  // just before this kernel reads the tensor front to back, so its tail is what the L2 still holds.
  const int tile = (int)(gridDim.x - 1 - blockIdx.x);
  const int ct = tile % num_col_tiles;
  const int mt = tile / num_col_tiles;
  const int tid = threadIdx.x;
  const int row_in_pass = tid / kThreadsPerRow;
  const int seg = tid % kThreadsPerRow;
  const int col = ct * kTileCols + seg * 16;
  const int sf_col_in_tile = seg / kThreadsPerBlock;                // 0..7 (NVFP4) or 0..3 (MXFP4)
  const bool col_ok = col < n;

  float gs = 1.0f, rcp_gs = 1.0f;
  if (BLOCK == 16 && !DYNAMIC && !dyn.wait_prev) {
    gs = gs_ptr ? __ldg(gs_ptr) : 1.0f;
    rcp_gs = rcp_approx_ftz(gs);
  }
  // rcp.approx.ftz(6.0f) like the reference, in both formats (kernel/nvfp4_utils.cuh:192 there; its e8m0 branch,
  // :196-202, uses the same product).  On sm_100 the instruction returns 0x3E2AAAAB, the correctly rounded 1/6, so a
  // CPU restatement with that constant is exact (checked on the GPU by the quantizer tests).
  const float rcp6 = rcp_approx_ftz(6.0f);

  Pack16<T> v[kPasses];
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const int row = mt * kTileRows + p * kRowsPerPass + row_in_pass;
    v[p].raw[0] = make_uint4(0u, 0u, 0u, 0u);
    v[p].raw[1] = make_uint4(0u, 0u, 0u, 0u);
    if (col_ok && row < m) load16<T>(v[p], in + (int64_t)row * in_stride + col, aligned32 != 0);
  }
  if (BLOCK == 16 && !DYNAMIC && dyn.wait_prev) {
    asm volatile("griddepcontrol.wait;" ::: "memory");       // the global scale is written by the kernel before
    gs = gs_ptr ? *reinterpret_cast<const volatile float*>(gs_ptr) : 1.0f;
    rcp_gs = rcp_approx_ftz(gs);
  }
  if constexpr (DYNAMIC) {
    __shared__ float warp_max[kThreads / 32];
    __shared__ float gs_shared;
    auto mx2 = __habs2(v[0].h2[0]);
#pragma unroll
    for (int p = 0; p < kPasses; ++p)
#pragma unroll
      for (int i = 0; i < 8; ++i) mx2 = __hmax2_nan(mx2, __habs2(v[p].h2[i]));
    float mx = to_float<T>(__hmax_nan(mx2.x, mx2.y));
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = max_nan_nonneg(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    if ((tid & 31) == 0) warp_max[tid >> 5] = mx;
    __syncthreads();
    if (tid == 0) {
      float r = warp_max[0];
#pragma unroll
      for (int w = 1; w < kThreads / 32; ++w) r = max_nan_nonneg(r, warp_max[w]);
      uint32_t* toggle = dyn.scratch + 4;
      const uint32_t t = *reinterpret_cast<volatile uint32_t*>(toggle) & 1u;
      uint32_t* pair = dyn.scratch + 2u * t;
      atomicMax(&pair[0], __float_as_uint(r));
      __threadfence();
      const bool last = atomicAdd(&pair[1], 1u) == gridDim.x - 1;
      if (!last) {
        const uint64_t t0 = global_timer_ns_q();
        for (uint32_t spin = 0; *reinterpret_cast<volatile uint32_t*>(&pair[1]) < gridDim.x; ++spin) {
          if ((spin & 255u) == 255u && global_timer_ns_q() - t0 > 2000000000ull) {
            atomicOr(dyn.status, kErrQuantBarrier);
            break;
          }
        }
      }
      __threadfence();
      float amax = __uint_as_float(*reinterpret_cast<volatile uint32_t*>(&pair[0]));
      if (amax == 0.0f) amax = 1.0f;
      // same two roundings as amax_kernel: reciprocal(amax) * 2688
      const float g = __fmul_rn(__frcp_rn(amax), 448.0f * 6.0f);
      gs_shared = g;
      if (last) {
        *dyn.gs_out = g;
        if (dyn.gs_other) *dyn.alpha_out = __fdiv_rn(1.0f, __fmul_rn(g, *dyn.gs_other));
        // This pair stays as it is (the others are still reading it); the OTHER pair is made clean for the
        // next launch, which the flipped toggle points at.  Every CTA read the toggle before it arrived.
        uint32_t* other = dyn.scratch + 2u * (t ^ 1u);
        other[0] = 0u;
        other[1] = 0u;
        __threadfence();
        *toggle = t ^ 1u;
      }
    }
    __syncthreads();
    gs = gs_shared;
    rcp_gs = rcp_approx_ftz(gs);
  }
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const int row_in_tile = p * kRowsPerPass + row_in_pass;
    const int row = mt * kTileRows + row_in_tile;
    uint8_t sf_byte;
    uint2 packed;
    if constexpr (BLOCK == 16) {
      packed = nvfp4_quantize_block<T>(v[p].h2, gs, rcp_gs, rcp6, sf_byte);
    } else {
      auto mx2 = __habs2(v[p].h2[0]);
#pragma unroll
      for (int i = 1; i < 8; ++i) mx2 = __hmax2(mx2, __habs2(v[p].h2[i]));
#pragma unroll
      for (int s = 1; s < kThreadsPerBlock; s <<= 1)
        mx2 = __hmax2(__shfl_xor_sync(0xffffffffu, mx2, s), mx2);
      const float amax = to_float<T>(__hmax(mx2.x, mx2.y));
      const float sf_value = mul_ftz(amax, rcp6);
      const uint32_t bits = __float_as_uint(sf_value);
      uint32_t e = (bits >> 23) & 0xffu;
      if (mx_rounding == NVFP_MX_ROUND_CEIL && (bits & 0x7fffffu) != 0 && e < 254) e += 1;
      // An infinite block maximum has exponent bits 255.  The reference's e8m0 branch stores them as they are
      // (kernel/nvfp4_utils.cuh:196-202 there; 255 is the e8m0 NaN code) and `floor` follows it; `ceil` keeps the
      // largest finite scale.  Either way the elements are multiplied by 0.
      if (mx_rounding == NVFP_MX_ROUND_CEIL) e = min(e, 254u);
      if (sf_value != sf_value) e = 255u;
      sf_byte = (uint8_t)e;
      const float out_scale = (e > 0 && e < 254) ? __uint_as_float((254u - e) << 23) : 0.0f;
      float2 f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        f[i] = to_float2<T>(v[p].h2[i]);
        f[i].x = mul_ftz(f[i].x, out_scale);
        f[i].y = mul_ftz(f[i].y, out_scale);
      }
      packed.x = cvt_e2m1x8(f[0].x, f[0].y, f[1].x, f[1].y, f[2].x, f[2].y, f[3].x, f[3].y);
      packed.y = cvt_e2m1x8(f[4].x, f[4].y, f[5].x, f[5].y, f[6].x, f[6].y, f[7].x, f[7].y);
    }
    if (col_ok && row < m)
      *reinterpret_cast<uint2*>(out + (int64_t)row * (n / 2) + col / 2) = packed;
    // padding of the scale tensor (rows past m, columns past n) is zero whatever the global scale is: with a NaN
    // or infinite scale a block of zeros would otherwise get the NaN byte
    if (seg % kThreadsPerBlock == 0)
      sf_stage[(sf_col_in_tile / 4) * 512 + (row_in_tile % 32) * 16 + (row_in_tile / 32) * 4 +
               (sf_col_in_tile % 4)] = (col_ok && row < m) ? sf_byte : (uint8_t)0;
  }
  __syncthreads();
  if (tid < 32 * kChunksPerTile) {
    const int chunk = ct * kChunksPerTile + tid / 32;
    if (chunk < num_k_chunks) {
      uint4* dst = reinterpret_cast<uint4*>(sf_out + ((int64_t)mt * num_k_chunks + chunk) * 512);
      dst[tid % 32] = reinterpret_cast<const uint4*>(sf_stage)[tid];
    }
  }
}

// DYNAMIC quantization of a decode-sized activation (one 128-row scale tile) by ONE CLUSTER of up to eight CTAs,
// launched like any kernel (nothing cooperative): each CTA owns a range of 64-column scale chunks, keeps its part of
// the tensor in registers (up to four 16-element blocks per thread), and the CTAs exchange their maxima through each
// other's shared memory around one cluster barrier (no trip through global memory).  A CTA stages its chunks' scale
// bytes in shared memory (zero where the tensor has no rows) and stores them 16 bytes at a time.  Same bytes as the
// tiled kernel.
constexpr int kSmallThreads = 512;
constexpr int kSmallBlocksPerThread = 4;
constexpr int kSmallMaxCluster = 8;
constexpr int kSmallMaxChunksPerCta = 32;          // 16 KB of staged scale bytes

template <typename T>
__global__ void __launch_bounds__(kSmallThreads)
quant_fp4_small_kernel(const T* __restrict__ in, int64_t in_stride, uint8_t* __restrict__ out,
                       uint8_t* __restrict__ sf_out, int m, int n, int num_k_chunks, int chunks_per_cta, int aligned32,
                       const DynamicScale dyn) {
  if (dyn.release_next) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ __align__(16) uint8_t sf_stage_small[kSmallMaxChunksPerCta * 512];   // [chunk][32][4][4]
  __shared__ float warp_max[kSmallThreads / 32];
  __shared__ float cta_max[kSmallMaxCluster];      // written by the CTAs of the cluster, one slot each
  __shared__ float gs_shared;
  const int tid = threadIdx.x;
  const uint32_t rank = ptx::cluster_ctarank(), csize = gridDim.x;
  // every CTA of the cluster is running once all have arrived here; waited for just before the remote stores
  ptx::cluster_arrive_relaxed();
  // the other operand's scale is needed only at the end: fetched now, beside the tensor's loads
  float gs_other = 1.0f;
  if (tid == 0 && rank == 0 && dyn.gs_other) gs_other = __ldg(dyn.gs_other);
  const int chunk0 = (int)rank * chunks_per_cta;
  const int my_chunks = max(0, min(chunks_per_cta, num_k_chunks - chunk0));
  const int blocks_per_row = n / 16, cols = my_chunks * 4;            // 16-element blocks per row: all, mine
  const int total = m * cols;
  Pack16<T> v[kSmallBlocksPerThread];
#pragma unroll
  for (int i = 0; i < kSmallBlocksPerThread; ++i) {
    const int id = tid + i * kSmallThreads;
    v[i].raw[0] = make_uint4(0u, 0u, 0u, 0u);
    v[i].raw[1] = make_uint4(0u, 0u, 0u, 0u);
    if (id < total) {
      const int row = id / cols, cb = chunk0 * 4 + id % cols;
      if (cb < blocks_per_row) load16<T>(v[i], in + (int64_t)row * in_stride + cb * 16, aligned32 != 0);
    }
  }
  uint4* stage16 = reinterpret_cast<uint4*>(sf_stage_small);
  for (int j = tid; j < my_chunks * 32; j += kSmallThreads) stage16[j] = make_uint4(0u, 0u, 0u, 0u);
  auto mx2 = __habs2(v[0].h2[0]);
#pragma unroll
  for (int i = 0; i < kSmallBlocksPerThread; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) mx2 = __hmax2_nan(mx2, __habs2(v[i].h2[e]));
  float mx = to_float<T>(__hmax_nan(mx2.x, mx2.y));
#pragma unroll
  for (int sh = 16; sh > 0; sh >>= 1) mx = max_nan_nonneg(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
  if ((tid & 31) == 0) warp_max[tid >> 5] = mx;
  __syncthreads();
  ptx::cluster_wait();
  if (tid < 32) {
    float r = tid < kSmallThreads / 32 ? warp_max[tid] : 0.0f;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) r = max_nan_nonneg(r, __shfl_xor_sync(0xffffffffu, r, sh));
    // lane l tells CTA l
    if ((uint32_t)tid < csize)
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ptx::map_to_cta(ptx::smem_u32(&cta_max[rank]), (uint32_t)tid)), "f"(r)
                   : "memory");
  }
  ptx::cluster_arrive();                       // release: the stores above are visible to whoever has waited
  ptx::cluster_wait();
  if (tid == 0) {
    float r = cta_max[0];
    for (uint32_t c = 1; c < csize; ++c) r = max_nan_nonneg(r, cta_max[c]);
    if (r == 0.0f) r = 1.0f;
    // same two roundings as amax_kernel: reciprocal(amax) * 2688
    const float g = __fmul_rn(__frcp_rn(r), 448.0f * 6.0f);
    gs_shared = g;
    if (rank == 0) {
      *dyn.gs_out = g;
      if (dyn.gs_other) *dyn.alpha_out = __fdiv_rn(1.0f, __fmul_rn(g, gs_other));
    }
  }
  __syncthreads();
  const float gs = gs_shared, rcp_gs = rcp_approx_ftz(gs), rcp6 = rcp_approx_ftz(6.0f);
#pragma unroll
  for (int i = 0; i < kSmallBlocksPerThread; ++i) {
    const int id = tid + i * kSmallThreads;
    if (id < total) {
      const int row = id / cols, cbl = id % cols, cb = chunk0 * 4 + cbl;
      if (cb < blocks_per_row) {
        uint8_t sf_byte;
        const uint2 packed = nvfp4_quantize_block<T>(v[i].h2, gs, rcp_gs, rcp6, sf_byte);
        *reinterpret_cast<uint2*>(out + (int64_t)row * (n / 2) + cb * 8) = packed;
        sf_stage_small[(cbl / 4) * 512 + (row % 32) * 16 + (row / 32) * 4 + (cbl % 4)] = sf_byte;
      }
    }
  }
  __syncthreads();
  uint4* dst = reinterpret_cast<uint4*>(sf_out + (int64_t)chunk0 * 512);
  for (int j = tid; j < my_chunks * 32; j += kSmallThreads) dst[j] = stage16[j];
}

__global__ void rcp_kernel(float* __restrict__ out, const float* __restrict__ in, int64_t count) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = rcp_approx_ftz(in[i]);
}

// max |x| over the tensor -> atomicMax on the fp32 bit pattern (non-negative floats
// order like unsigned integers; a NaN, whose pattern is above infinity's, wins every comparison on the way and makes the
// global scale NaN, as torch.abs(x).max() would).  VEC = elements per load: 16 (one 32-byte load, needs 32-byte
// aligned rows) or 8.  Every thread keeps four loads in flight; the grid sweeps the tensor front
// to back.
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
amax_kernel(const T* __restrict__ in, int64_t in_stride, int64_t m, int64_t n, uint32_t* scratch, float* gs_out,
            uint32_t* toggle, const float* gs_other, float* alpha_out, int release_next) {
  if (release_next) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // self-cleaning mode: scratch holds two (maximum, counter) pairs; *toggle says which one this launch uses
  if (toggle) scratch += 2u * (*reinterpret_cast<volatile uint32_t*>(toggle) & 1u);
  const int64_t vec_per_row = n / VEC;
  const int64_t total = m * vec_per_row;
  const bool dense = in_stride == n;            // rows back to back: vector j sits at in + j * VEC, no division
  typename Vec2<T>::type mx2 = zero2<T>();
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += 4 * step) {
    Pack16<T> v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t j = i + u * step;
      v[u].raw[0] = make_uint4(0u, 0u, 0u, 0u);
      v[u].raw[1] = make_uint4(0u, 0u, 0u, 0u);
      if (j < total) {
        const T* src = dense ? in + j * VEC : in + (j / vec_per_row) * in_stride + (j % vec_per_row) * VEC;
        if (VEC == 16) load16<T>(v[u], src, true);
        else v[u].raw[0] = __ldg(reinterpret_cast<const uint4*>(src));
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int e = 0; e < VEC / 2; ++e) mx2 = __hmax2_nan(mx2, __habs2(v[u].h2[e]));
  }
  float mx = to_float<T>(__hmax_nan(mx2.x, mx2.y));
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) mx = max_nan_nonneg(mx, __shfl_xor_sync(0xffffffffu, mx, s));
  __shared__ float warp_max[8];
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = warp_max[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) r = max_nan_nonneg(r, warp_max[w]);
    // scratch[0] = running maximum (fp32 bits), scratch[1] = number of blocks that have contributed
    atomicMax(&scratch[0], __float_as_uint(r));
    __threadfence();
    if (atomicAdd(&scratch[1], 1u) == gridDim.x - 1) {
      // last block: every contribution is visible; finish here instead of in a second launch
      __threadfence();
      float amax = __uint_as_float(*reinterpret_cast<volatile uint32_t*>(&scratch[0]));
      if (amax == 0.0f) amax = 1.0f;
      // torch evaluates `2688 / amax` (scalar / tensor) as reciprocal(amax) * 2688: two roundings.
      // The reference forms its global scales that way (speed_test.py:41,47; nvfp/pseudo_quant.py:94-96).
      const float gs = __fmul_rn(__frcp_rn(amax), 448.0f * 6.0f);
      *gs_out = gs;
      if (alpha_out) *alpha_out = __fdiv_rn(1.0f, __fmul_rn(gs, *gs_other));     // speed_test.py:49 of the reference
      scratch[1] = 0u;
      if (toggle) {
        // leave the OTHER pair clean for the next launch and point the toggle at it: no memset between calls
        const uint32_t t = *toggle & 1u;
        uint32_t* other = scratch + (t ? -2 : 2);
        other[0] = 0u;
        other[1] = 0u;
        __threadfence();
        *toggle = t ^ 1u;
      }
    }
  }
}

template <typename T>
int launch_amax(float* gs_out, uint32_t* scratch, const void* in, int64_t m, int64_t n, int64_t stride,
                cudaStream_t stream, bool self_cleaning = false, const float* gs_other = nullptr,
                float* alpha_out = nullptr, bool release_next = false) {
  DeviceInfo info;
  if (int rc = current_device_info(&info)) return rc;
  uint32_t* toggle = self_cleaning ? scratch + 4 : nullptr;
  if (!self_cleaning) NVFP_CUDA(cudaMemsetAsync(scratch, 0, 2 * sizeof(uint32_t), stream));
  const bool wide = n % 16 == 0 && stride % 16 == 0 && reinterpret_cast<uintptr_t>(in) % 32 == 0;
  const int64_t want = ceil_div(m * (n / (wide ? 16 : 8)), 256 * 4);
  // Three CTAs per SM: every CTA ends with two atomics on the same words, so the grid stays small, and the sweep
  // is bound by DRAM reads either way (measured at 8192 x 8192, back to back: 26.5-28 us with 2 to 5 CTAs per SM and
  // 2, 4 or 8 loads in flight per thread, about 5 TB/s, which is also the rate at which the quantizer reads;
  // 33-47 us with one CTA per SM; 53 us with one iteration per thread and 16 K CTAs).
  // Tensors that one wave of five CTAs per SM covers get one iteration per thread (latency matters there).
  const int64_t ctas = want <= (int64_t)info.sm_count * 5 ? want : (int64_t)info.sm_count * 3;
  const unsigned grid = (unsigned)std::max<int64_t>(1, ctas);
  if (wide)
    amax_kernel<T, 16><<<grid, 256, 0, stream>>>(static_cast<const T*>(in), stride, m, n, scratch, gs_out, toggle,
                                                 gs_other, alpha_out, release_next ? 1 : 0);
  else
    amax_kernel<T, 8><<<grid, 256, 0, stream>>>(static_cast<const T*>(in), stride, m, n, scratch, gs_out, toggle,
                                                gs_other, alpha_out, release_next ? 1 : 0);
  NVFP_CUDA(cudaGetLastError());
  return NVFP_OK;
}

__global__ void alpha_kernel(float* alpha_out, const float* gs_a, const float* gs_b) {
  *alpha_out = __fdiv_rn(1.0f, __fmul_rn(*gs_a, *gs_b));
}

int check_16bit_input(const void* in, int64_t m, int64_t n, int64_t stride, int dtype, int block) {
  NVFP_REQUIRE(m >= 0 && n >= 0, "negative shape (%lld x %lld)", (long long)m, (long long)n);
  NVFP_REQUIRE(in != nullptr || m == 0 || n == 0, "input pointer is null");      // an empty tensor has no storage
  NVFP_REQUIRE(n % block == 0, "The N dimension must be multiple of %d (got %lld).", block, (long long)n);
  NVFP_REQUIRE(dtype == NVFP_DTYPE_F16 || dtype == NVFP_DTYPE_BF16,
               "Unsupported input data type for quantize_to_fp4 (dtype code %d).", dtype);
  NVFP_REQUIRE(stride >= n && stride % 8 == 0,
               "input row stride %lld must be >= n and a multiple of 8 elements", (long long)stride);
  NVFP_REQUIRE((reinterpret_cast<uintptr_t>(in) & 15) == 0, "input must be 16-byte aligned");
  NVFP_REQUIRE(m < (1ll << 31) && n < (1ll << 31), "shape too large");
  return NVFP_OK;
}

template <int BLOCK>
int launch_quant(void* out_fp4, void* out_sf, const void* in, const float* gs, int64_t m, int64_t n,
                 int64_t stride, int dtype, int rounding, cudaStream_t stream, bool wait_prev = false,
                 bool release_next = false) {
  if (int rc = check_16bit_input(in, m, n, stride, dtype, BLOCK)) return rc;
  if (m == 0 || n == 0) return NVFP_OK;
  NVFP_REQUIRE(out_fp4 != nullptr && out_sf != nullptr, "output pointer is null");
  NVFP_REQUIRE((reinterpret_cast<uintptr_t>(out_fp4) & 7) == 0 &&
                   (reinterpret_cast<uintptr_t>(out_sf) & 15) == 0,
               "outputs must be aligned (fp4: 8 bytes, scales: 16 bytes)");
  const int64_t m_tiles = ceil_div(m, kTileRows);
  const int64_t col_tiles = ceil_div(n, kTileCols);
  const int64_t k_chunks = ceil_div(n / BLOCK, 4);
  NVFP_REQUIRE(m_tiles * col_tiles < (1ll << 31), "too many tiles");
  const dim3 grid((unsigned)(m_tiles * col_tiles));
  const int aligned32 = (reinterpret_cast<uintptr_t>(in) % 32 == 0 && stride % 16 == 0) ? 1 : 0;
  DynamicScale chain{};
  chain.release_next = release_next ? 1 : 0;
  chain.wait_prev = wait_prev ? 1 : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = wait_prev ? 1 : 0;
  if (dtype == NVFP_DTYPE_F16) {
    NVFP_CUDA(cudaLaunchKernelEx(&cfg, quant_fp4_kernel<__half, BLOCK, false>, static_cast<const __half*>(in), stride, gs,
                                 static_cast<uint8_t*>(out_fp4), static_cast<uint8_t*>(out_sf), (int)m, (int)n,
                                 (int)col_tiles, (int)k_chunks, rounding, aligned32, chain));
  } else {
    NVFP_CUDA(cudaLaunchKernelEx(&cfg, quant_fp4_kernel<__nv_bfloat16, BLOCK, false>,
                                 static_cast<const __nv_bfloat16*>(in), stride, gs, static_cast<uint8_t*>(out_fp4),
                                 static_cast<uint8_t*>(out_sf), (int)m, (int)n, (int)col_tiles, (int)k_chunks, rounding,
                                 aligned32, chain));
  }
  NVFP_CUDA(cudaGetLastError());
  return NVFP_OK;
}

// CTAs of the one-pass kernel that can be resident at once on the current device (0 on error).
template <typename T>
int dynamic_quant_capacity(int device, int sm_count) {
  static int cached[64] = {};
  static std::once_flag once[64];
  if (device < 0 || device >= 64) return 0;
  std::call_once(once[device], [device, sm_count] {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_fp4_kernel<T, 16, true>, kThreads, 0) != cudaSuccess)
      return;
    // Two tiles per SM at most: measured on B200 inside a layer's forward, 256 tiles (4096 x 1024) take 23.6 us
    // in one pass against 27.6 us in two; at 512 tiles the wait for the slowest CTA costs more than the second
    // read of a tensor that is still in L2 (35.8 against 33.9 us).
    cached[device] = std::max(1, std::min(per_sm, 2) * sm_count);
  });
  return cached[device];
}

template <typename T>
bool dynamic_quant_fits(int64_t m, int64_t n) {
  DeviceInfo info;
  int device = 0;
  if (current_device_info(&info) != NVFP_OK || cudaGetDevice(&device) != cudaSuccess) return false;
  const int64_t tiles = ceil_div(m, kTileRows) * ceil_div(n, kTileCols);
  return tiles > 0 && tiles <= dynamic_quant_capacity<T>(device, info.sm_count);
}

template <typename T>
int launch_dynamic_quant(void* out_fp4, void* out_sf, float* gs_out, float* alpha_out, uint32_t* scratch, const void* in,
                         int64_t m, int64_t n, int64_t stride, const float* gs_other, cudaStream_t stream,
                         bool release_next = false, bool* one_pass = nullptr) {
  const int64_t m_tiles = ceil_div(m, kTileRows), col_tiles = ceil_div(n, kTileCols);
  const int64_t tiles = m_tiles * col_tiles;
  const bool fits = dynamic_quant_fits<T>(m, n);
  if (one_pass) *one_pass = fits;
  // decode-sized (one 128-row scale tile, few enough blocks for one cluster's registers): no grid barrier
  const int64_t k_chunks = ceil_div(n / 16, 4);
  int cluster = 1;
  while (cluster < kSmallMaxCluster && cluster * 2 <= k_chunks) cluster *= 2;
  const int64_t chunks_per_cta = ceil_div(k_chunks, cluster);
  if (m > 0 && n > 0 && m <= kTileRows && chunks_per_cta <= kSmallMaxChunksPerCta &&
      m * chunks_per_cta * 4 <= (int64_t)kSmallThreads * kSmallBlocksPerThread) {
    if (one_pass) *one_pass = true;
    DynamicScale dyn{scratch, gs_out, gs_other, alpha_out, device_status_word(), release_next ? 1 : 0};
    const int aligned32 = (reinterpret_cast<uintptr_t>(in) % 32 == 0 && stride % 16 == 0) ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cluster);
    cfg.blockDim = dim3(kSmallThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NVFP_CUDA(cudaLaunchKernelEx(&cfg, quant_fp4_small_kernel<T>, static_cast<const T*>(in), stride,
                                 static_cast<uint8_t*>(out_fp4), static_cast<uint8_t*>(out_sf), (int)m, (int)n,
                                 (int)k_chunks, (int)chunks_per_cta, aligned32, dyn));
    return NVFP_OK;
  }
  if (!fits) {
    // too large to keep in registers across the grid: global-scale pass, then quantize pass
    // The quantize launch comes up under the global-scale launch, loads its tiles and waits for the scale.
    if (int rc = launch_amax<T>(gs_out, scratch, in, m, n, stride, stream, true, gs_other, gs_other ? alpha_out : nullptr,
                                /*release_next=*/true))
      return rc;
    return launch_quant<16>(out_fp4, out_sf, in, gs_out, m, n, stride,
                            std::is_same<T, __half>::value ? NVFP_DTYPE_F16 : NVFP_DTYPE_BF16, 0, stream,
                            /*wait_prev=*/true, release_next);
  }
  DynamicScale dyn{scratch, gs_out, gs_other, alpha_out, device_status_word(), release_next ? 1 : 0};
  NVFP_REQUIRE(dyn.status != nullptr, "cannot locate the device status word");
  const int aligned32 = (reinterpret_cast<uintptr_t>(in) % 32 == 0 && stride % 16 == 0) ? 1 : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)tiles);
  cfg.blockDim = dim3(kThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  NVFP_CUDA(cudaLaunchKernelEx(&cfg, quant_fp4_kernel<T, 16, true>, static_cast<const T*>(in), stride,
                               static_cast<const float*>(nullptr), static_cast<uint8_t*>(out_fp4),
                               static_cast<uint8_t*>(out_sf), (int)m, (int)n, (int)col_tiles,
                               (int)ceil_div(n / 16, 4), 0, aligned32, dyn));
  return NVFP_OK;
}

}  // namespace

int dynamic_fp4_quant_launch(void* out_fp4, void* out_sf, float* gs_out, float* alpha_out, uint32_t* scratch,
                             const void* in, int64_t m, int64_t n, int64_t stride, int in_dtype,
                             const float* gs_weight, bool release_next, bool* one_pass, cudaStream_t stream) {
  return in_dtype == NVFP_DTYPE_F16
             ? launch_dynamic_quant<__half>(out_fp4, out_sf, gs_out, alpha_out, scratch, in, m, n, stride, gs_weight,
                                            stream, release_next, one_pass)
             : launch_dynamic_quant<__nv_bfloat16>(out_fp4, out_sf, gs_out, alpha_out, scratch, in, m, n, stride,
                                                   gs_weight, stream, release_next, one_pass);
}

int activation_scales_launch(float* gs_out, float* alpha_out, uint32_t* scratch, const void* in, int64_t m, int64_t n,
                             int64_t stride, int in_dtype, const float* gs_other, cudaStream_t stream) {
  return in_dtype == NVFP_DTYPE_F16
             ? launch_amax<__half>(gs_out, scratch, in, m, n, stride, stream, true, gs_other, gs_other ? alpha_out : nullptr)
             : launch_amax<__nv_bfloat16>(gs_out, scratch, in, m, n, stride, stream, true, gs_other,
                                          gs_other ? alpha_out : nullptr);
}

int scaled_fp4_quant_launch(void* out_fp4, void* out_sf, const void* in, const float* gs, int64_t m, int64_t n,
                            int64_t stride, int in_dtype, bool release_next, cudaStream_t stream) {
  return launch_quant<16>(out_fp4, out_sf, in, gs, m, n, stride, in_dtype, 0, stream, /*wait_prev=*/false, release_next);
}

bool dynamic_fp4_quant_is_one_pass(int64_t m, int64_t n, int in_dtype) {
  return in_dtype == NVFP_DTYPE_F16 ? dynamic_quant_fits<__half>(m, n) : dynamic_quant_fits<__nv_bfloat16>(m, n);
}

}  // namespace nvfp

using namespace nvfp;

extern "C" int nvfp_scaled_fp4_quant(void* out_fp4, void* out_sf, const void* in,
                                     const float* global_scale, int64_t m, int64_t n,
                                     int64_t in_row_stride, int in_dtype, void* stream) {
  clear_error();
  return launch_quant<16>(out_fp4, out_sf, in, global_scale, m, n, in_row_stride, in_dtype, 0,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int nvfp_mxfp4_quant(void* out_fp4, void* out_sf, const void* in, int64_t m, int64_t n,
                                int64_t in_row_stride, int in_dtype, int rounding, void* stream) {
  clear_error();
  NVFP_REQUIRE(rounding == NVFP_MX_ROUND_CEIL || rounding == NVFP_MX_ROUND_FLOOR,
               "unknown MXFP4 scale rounding %d", rounding);
  return launch_quant<32>(out_fp4, out_sf, in, nullptr, m, n, in_row_stride, in_dtype, rounding,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int nvfp_reciprocal_approximate_ftz(float* out, const float* in, int64_t count,
                                               void* stream) {
  clear_error();
  NVFP_REQUIRE(count >= 0, "negative element count");
  if (count == 0) return NVFP_OK;
  NVFP_REQUIRE(out != nullptr && in != nullptr, "null pointer");
  const int64_t blocks = ceil_div(count, 256);
  NVFP_REQUIRE(blocks < (1ll << 31), "tensor too large");
  rcp_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(out, in, count);
  NVFP_CUDA(cudaGetLastError());
  return NVFP_OK;
}

extern "C" int nvfp_global_scale(float* gs_out, uint32_t* amax_bits, const void* in, int64_t m,
                                 int64_t n, int64_t in_row_stride, int in_dtype, void* stream_) {
  clear_error();
  if (int rc = check_16bit_input(in, m, n, in_row_stride, in_dtype, 8)) return rc;
  NVFP_REQUIRE(gs_out != nullptr && amax_bits != nullptr, "null pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  return in_dtype == NVFP_DTYPE_F16
             ? launch_amax<__half>(gs_out, amax_bits, in, m, n, in_row_stride, stream)
             : launch_amax<__nv_bfloat16>(gs_out, amax_bits, in, m, n, in_row_stride, stream);
}

extern "C" int nvfp_activation_scales(float* gs_out, float* alpha_out, uint32_t* scratch, const void* in,
                                      int64_t m, int64_t n, int64_t in_row_stride, int in_dtype,
                                      const float* gs_weight, void* stream_) {
  clear_error();
  if (int rc = check_16bit_input(in, m, n, in_row_stride, in_dtype, 8)) return rc;
  NVFP_REQUIRE(gs_out && alpha_out && scratch && gs_weight, "null pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  return in_dtype == NVFP_DTYPE_F16
             ? launch_amax<__half>(gs_out, scratch, in, m, n, in_row_stride, stream, true, gs_weight, alpha_out)
             : launch_amax<__nv_bfloat16>(gs_out, scratch, in, m, n, in_row_stride, stream, true, gs_weight, alpha_out);
}

extern "C" int nvfp_dynamic_fp4_quant(void* out_fp4, void* out_sf, float* gs_out, float* alpha_out, uint32_t* scratch,
                                      const void* in, int64_t m, int64_t n, int64_t in_row_stride, int in_dtype,
                                      const float* gs_weight, void* stream_) {
  clear_error();
  if (int rc = check_16bit_input(in, m, n, in_row_stride, in_dtype, 16)) return rc;
  NVFP_REQUIRE(((out_fp4 != nullptr && out_sf != nullptr) || m == 0 || n == 0) && gs_out != nullptr && scratch != nullptr,
               "null pointer");
  NVFP_REQUIRE(gs_weight == nullptr || alpha_out != nullptr, "alpha output is null although a weight scale is given");
  NVFP_REQUIRE((reinterpret_cast<uintptr_t>(out_fp4) & 7) == 0 && (reinterpret_cast<uintptr_t>(out_sf) & 15) == 0,
               "outputs must be aligned (fp4: 8 bytes, scales: 16 bytes)");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  return in_dtype == NVFP_DTYPE_F16
             ? launch_dynamic_quant<__half>(out_fp4, out_sf, gs_out, alpha_out, scratch, in, m, n, in_row_stride,
                                            gs_weight, stream)
             : launch_dynamic_quant<__nv_bfloat16>(out_fp4, out_sf, gs_out, alpha_out, scratch, in, m, n,
                                                   in_row_stride, gs_weight, stream);
}

extern "C" int nvfp_alpha_from_scales(float* alpha_out, const float* gs_a, const float* gs_b,
                                      void* stream) {
  clear_error();
  NVFP_REQUIRE(alpha_out && gs_a && gs_b, "null pointer");
  alpha_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(alpha_out, gs_a, gs_b);
  NVFP_CUDA(cudaGetLastError());
  return NVFP_OK;
}

// ---------------------------------------------------------------------------------------
// Global scale for callers that may not allocate device memory.
//
// nvfp_global_scale needs one 32-bit scratch word from its caller.  A caller that lives
// inside someone else's memory plan -- an inference engine whose allocator is frozen after
// warm-up, a plugin invoked from a host that forbids cudaMalloc on its threads -- has no word
// to give.  This variant keeps the word in a file-scope device array that every GPU loading
// the library holds until the process exits (kNoAllocScratchWords * 4 bytes).
//
// In host code `g_noalloc_scratch` is only a stand-in for the device symbol, not a device
// address; the address is looked up once per device with cudaGetSymbolAddress (that device
// current) and handed to the kernels.
namespace nvfp {
namespace {
constexpr int kNoAllocScratchWords = 64;              // one 256-byte line; words 0-1: amax bits, block counter
constexpr int64_t kNoAllocMaxElements = 1ll << 32;    // largest tensor this entry point accepts
static __device__ __align__(256) uint32_t g_noalloc_scratch[kNoAllocScratchWords];

int noalloc_scratch_address(uint32_t** out) {
  constexpr int kMaxDevices = 64;
  static uint32_t* cache[kMaxDevices] = {};
  static cudaError_t err[kMaxDevices];
  static std::once_flag once[kMaxDevices];      // two host threads may make the first call on a device together
  int dev = 0;
  NVFP_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(NVFP_ERR_CUDA, "device index %d out of range", dev);
  std::call_once(once[dev], [dev] {
    uint32_t* ptr = nullptr;
    err[dev] = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (err[dev] == cudaSuccess) cache[dev] = ptr;
  });
  if (cache[dev] == nullptr)
    return fail(NVFP_ERR_CUDA, "cudaGetSymbolAddress(g_noalloc_scratch) failed on device %d: %s", dev,
                cudaGetErrorString(err[dev]));
  *out = cache[dev];
  return NVFP_OK;
}
}  // namespace
}  // namespace nvfp

extern "C" int nvfp_global_scale_noalloc(float* gs_out, const void* in, int64_t m, int64_t n,
                                         int64_t in_row_stride, int in_dtype, void* stream_) {
  clear_error();
  if (int rc = check_16bit_input(in, m, n, in_row_stride, in_dtype, 8)) return rc;
  NVFP_REQUIRE(gs_out != nullptr, "null pointer");
  NVFP_REQUIRE(m * n <= kNoAllocMaxElements,
               "nvfp_global_scale_noalloc accepts at most %lld elements, got %lld x %lld; use nvfp_global_scale "
               "with caller-provided scratch for larger tensors",
               (long long)kNoAllocMaxElements, (long long)m, (long long)n);
  uint32_t* scratch = nullptr;
  if (int rc = noalloc_scratch_address(&scratch)) return rc;    // first call on a device: symbol look-up
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // the array keeps the previous call's contents: launch_amax clears the two words it uses, on the stream
  return in_dtype == NVFP_DTYPE_F16
             ? launch_amax<__half>(gs_out, scratch, in, m, n, in_row_stride, stream)
             : launch_amax<__nv_bfloat16>(gs_out, scratch, in, m, n, in_row_stride, stream);
}
