// Block-scaled FP4 GEMM for sm_100a:  D[m,n] = alpha * sum_k (A*sfa)[m,k] * (B*sfb)[n,k].
//
// Replaces the reference's CUTLASS Sm120 instantiation
// (kernel/nvfp4_scaled_mm_sm120_kernels.cu:72-188 of huweim/nvfp_kernel, warp-level
// mma.sync for consumer Blackwell) with a hand-written tcgen05 kernel:
//
//   warp 0   producer: TMA loads of 128 x 256-element A and BN x 256-element B tiles
//            (packed e2m1, 128-byte swizzle) plus bulk copies of the 512-byte scale
//            chunks, into a ring of shared-memory stages guarded by mbarriers
//   warp 1   issuer: copies the scale chunks shared -> tensor memory (tcgen05.cp) and
//            issues one tcgen05.mma (M=128, N=BN, K=64) per 64 elements of K; fp32
//            accumulators live in tensor memory; tcgen05.commit frees stages
//   warps 2-5 epilogue: tcgen05.ld of the accumulator, * alpha, convert, store
//
// The kernel is persistent (one CTA per SM walks the output tiles).  Every wait is
// bounded; on expiry the CTA records a code in the device status word and leaves
// through the common exit, which also frees its tensor memory.
//
// This file holds that kernel (one CTA per 128 x BN tile: mid-size shapes), the shape dispatch and the C entry
// points; gemm_fp4_pair_sm100.cuh holds the kernel for large shapes (CTA pairs, cta_group::2, 256 x 256 tiles),
// gemm_fp4_skinny_sm100.cuh the one for up to 128 activation rows (operands swapped, K split over a cluster).
// The epilogues can, beyond alpha: add a bias, apply silu(gate) * up on interleaved gate/up columns, quantize
// the result to NVFP4 (finish_row_chunk), store to several GPUs or add into the owning GPU's buffer.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "common.h"
#include "quant_math.cuh"
#include "ptx_sm100.cuh"

namespace nvfp {
namespace {

using namespace ptx;

constexpr int kBM = 128;            // rows of A per tile = M of one MMA
constexpr int kStageK = 256;        // elements of K per pipeline stage (= one 128-byte swizzle row)
constexpr int kStageKBytes = 128;
constexpr int kMmaK = 64;           // K of one tcgen05.mma for 4-bit operands
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr uint32_t kSmemLimit = 232448;  // 227 KB

// Status codes (one bit per waiting role) recorded when a bounded wait expires.
constexpr uint32_t kErrProducer = 1u, kErrIssuer = 2u, kErrEpilogue = 4u;

template <int BN, bool MX>
struct Cfg {
  static constexpr int kHalves = BN / 128;                       // 128-row scale tiles of B per tile
  static constexpr int kChunksPerStage = MX ? 2 : 4;              // 512-byte scale chunks per operand tile per stage
  static constexpr int kMmasPerChunk = MX ? 2 : 1;
  static constexpr uint32_t kABytes = kBM * kStageKBytes;         // 16 KB
  static constexpr uint32_t kBBytes = BN * kStageKBytes;
  static constexpr uint32_t kSfaBytes = kChunksPerStage * 512;
  static constexpr uint32_t kSfbBytes = kHalves * kChunksPerStage * 512;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kAccStages = BN == 128 ? 2 : 1;
  static constexpr int kStages = (kSmemLimit - 2048) / kStageBytes > 8 ? 8 : (kSmemLimit - 2048) / kStageBytes;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + 2048;  // + alignment slack and barriers
  // tensor-memory columns: accumulators first, then two slots of scale columns
  static constexpr uint32_t kAccCols = BN;
  static constexpr uint32_t kSfColBase = kAccStages * BN;
  static constexpr uint32_t kSfaCols = 4 * kChunksPerStage;
  static constexpr uint32_t kSfbCols = 4 * kChunksPerStage * kHalves;
  static constexpr uint32_t kSfSlotCols = kSfaCols + kSfbCols;
  static_assert(kSfColBase + 2 * kSfSlotCols <= kTmemCols, "tensor memory budget");
  static_assert(kStages >= 2, "pipeline depth");
};

struct GemmParams {
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* alpha;
  const void* bias;     // n values of the output type added after alpha, or null
  // NVFP4 output: when out_gs is set, the product (rounded to the output type) is quantized in the epilogue with
  // this global scale; d receives [m, n/2] packed bytes and out_sf the swizzled scales of an [m, n] tensor
  const float* out_gs;
  uint8_t* out_sf;
  int act;              // 1: silu(gate) * up on groups of 16 + 16 interleaved columns (output [m, n / 2]), 0: none
  void* d;
  int m, n, k;
  int tiles_m, tiles_n;
  int band;             // CTA-pair kernel: tiles are numbered in bands of this many tile rows (see pair_tile_coords)
  int sf_k_chunks;      // 512-byte chunks per 128-row scale tile along K
  int sfb_row_tiles;    // 128-row scale tiles of B
  uint32_t* status;
  int after_producer;   // launched with programmatic stream serialization behind the kernel that writes A, its
                        // scales and alpha: B and its scales may be fetched before that kernel has finished
  int release_next;     // the next kernel in the stream is launched the same way behind this one and reads nothing
                        // this kernel writes before its own griddepcontrol.wait: let it come up as CTAs retire
  // alpha formed in the epilogue from two global scales, 1 / (alpha[0] * alpha_gs_b[0]) with the roundings of
  // nvfp_alpha_from_scales, when alpha_gs_b is set (alpha then points at the activation's global scale)
  const float* alpha_gs_b;
  // Global scale of the OUTPUT for the next layer's quantizer, from the epilogue: every epilogue warp folds
  // max |value written| into amax_scratch (eight words, zeroed once, self-cleaning: two (max, arrivals) pairs and a
  // toggle, the protocol of nvfp_activation_scales); the last warp of the grid writes amax_gs_out = rcp(max) * 2688
  // and, when amax_gs_other is set, amax_alpha_out = 1 / (amax_gs_out * amax_gs_other[0]).  16-bit outputs only.
  uint32_t* amax_scratch;
  float* amax_gs_out;
  const float* amax_gs_other;
  float* amax_alpha_out;
};

// alpha of the epilogue: read after the kernel that produces it has finished.
__device__ __forceinline__ float load_alpha(const GemmParams& p) {
  if (p.alpha == nullptr) return 1.0f;
  const float a = *reinterpret_cast<const volatile float*>(p.alpha);
  if (p.alpha_gs_b == nullptr) return a;
  return __fdiv_rn(1.0f, __fmul_rn(a, *reinterpret_cast<const volatile float*>(p.alpha_gs_b)));
}

template <typename OutT> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Accumulators of 16 bytes' worth of consecutive output columns (8 values of a 16-bit type, 4 of fp32)
// -> alpha * acc (+ bias) -> packed output.  `bias16` points at the bias of the first of those columns or is null.
template <typename OutT>
__device__ __forceinline__ uint4 scale_bias_pack(const uint32_t* r, float alpha, const void* bias16) {
  uint4 o;
  if constexpr (sizeof(OutT) == 4) {
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias16) b = __ldg(static_cast<const float4*>(bias16));
    o.x = __float_as_uint(fmaf(__uint_as_float(r[0]), alpha, b.x));
    o.y = __float_as_uint(fmaf(__uint_as_float(r[1]), alpha, b.y));
    o.z = __float_as_uint(fmaf(__uint_as_float(r[2]), alpha, b.z));
    o.w = __float_as_uint(fmaf(__uint_as_float(r[3]), alpha, b.w));
  } else {
    float2 b[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
    if (bias16) {
      const uint4 raw = __ldg(static_cast<const uint4*>(bias16));
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if constexpr (std::is_same<OutT, __half>::value) b[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        else b[i] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      }
    }
    o.x = pack2<OutT>(fmaf(__uint_as_float(r[0]), alpha, b[0].x), fmaf(__uint_as_float(r[1]), alpha, b[0].y));
    o.y = pack2<OutT>(fmaf(__uint_as_float(r[2]), alpha, b[1].x), fmaf(__uint_as_float(r[3]), alpha, b[1].y));
    o.z = pack2<OutT>(fmaf(__uint_as_float(r[4]), alpha, b[2].x), fmaf(__uint_as_float(r[5]), alpha, b[2].y));
    o.w = pack2<OutT>(fmaf(__uint_as_float(r[6]), alpha, b[3].x), fmaf(__uint_as_float(r[7]), alpha, b[3].y));
  }
  return o;
}

// Running max |value| over packed 16-bit outputs (eight per uint4), kept as a pair of OutT.
template <typename OutT>
__device__ __forceinline__ void absmax_fold(uint32_t& mx2_bits, const uint4& o) {
  if constexpr (sizeof(OutT) == 2) {
    using V2 = typename Vec2<OutT>::type;
    V2 mx2 = *reinterpret_cast<V2*>(&mx2_bits);
    mx2 = __hmax2_nan(mx2, __habs2(*reinterpret_cast<const V2*>(&o.x)));
    mx2 = __hmax2_nan(mx2, __habs2(*reinterpret_cast<const V2*>(&o.y)));
    mx2 = __hmax2_nan(mx2, __habs2(*reinterpret_cast<const V2*>(&o.z)));
    mx2 = __hmax2_nan(mx2, __habs2(*reinterpret_cast<const V2*>(&o.w)));
    mx2_bits = *reinterpret_cast<uint32_t*>(&mx2);
  }
}

// End of an epilogue warp's work when the output's global scale is wanted (GemmParams::amax_scratch): the warp's
// maximum goes into the scratch pair the toggle points at; the last of `total_warps` warps forms the scale (and alpha),
// cleans the OTHER pair for the next launch and flips the toggle.  Whole warp; mx2_bits: this lane's running maximum.
template <typename OutT>
__device__ __forceinline__ void absmax_finish(const GemmParams& p, uint32_t mx2_bits, uint32_t total_warps) {
  if constexpr (sizeof(OutT) == 2) {
    using V2 = typename Vec2<OutT>::type;
    const V2 mx2 = *reinterpret_cast<V2*>(&mx2_bits);
    float mx = to_float<OutT>(__hmax_nan(mx2.x, mx2.y));
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) mx = max_nan_nonneg(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
    if ((threadIdx.x & 31) == 0) {
      uint32_t* toggle = p.amax_scratch + 4;
      const uint32_t t = *reinterpret_cast<volatile uint32_t*>(toggle) & 1u;   // read before this warp arrives
      uint32_t* pair = p.amax_scratch + 2u * t;
      atomicMax(&pair[0], __float_as_uint(mx));
      __threadfence();
      if (atomicAdd(&pair[1], 1u) == total_warps - 1u) {
        __threadfence();
        float amax = __uint_as_float(*reinterpret_cast<volatile uint32_t*>(&pair[0]));
        if (amax == 0.0f) amax = 1.0f;
        const float g = __fmul_rn(__frcp_rn(amax), 448.0f * 6.0f);      // the roundings of nvfp_global_scale
        *p.amax_gs_out = g;
        if (p.amax_gs_other) *p.amax_alpha_out = __fdiv_rn(1.0f, __fmul_rn(g, *p.amax_gs_other));
        pair[0] = 0u;                 // every warp has contributed: this pair is clean again as well
        pair[1] = 0u;
        uint32_t* other = p.amax_scratch + 2u * (t ^ 1u);
        other[0] = 0u;
        other[1] = 0u;
        __threadfence();
        *toggle = t ^ 1u;
      }
    }
  }
}

// 32 consecutive fp32 accumulators of one row -> 32 outputs, 16-byte stores.  `bias` points at the bias of the
// first column or is null.
template <typename OutT>
__device__ __forceinline__ void store_row_chunk(OutT* dst_elems, const uint32_t (&r)[32], float alpha, const OutT* bias,
                                                uint32_t* mx2_bits = nullptr) {
  uint4* dst = reinterpret_cast<uint4*>(dst_elems);
  constexpr int kPer = 16 / (int)sizeof(OutT);
#pragma unroll
  for (int v = 0; v < 32 / kPer; ++v) {
    const uint4 o = scale_bias_pack<OutT>(&r[kPer * v], alpha, bias ? bias + kPer * v : nullptr);
    dst[v] = o;
    if (mx2_bits) absmax_fold<OutT>(*mx2_bits, o);
  }
}

// silu(g) * u the way a framework evaluates it on 16-bit tensors: silu in fp32, rounded to T, times u in fp32,
// rounded to T.  exp and the division are the hardware approximations (a few fp32 ulps): the result is rounded to
// 8 or 11 bits right away, so it differs from the exact evaluation in about one element in ten thousand, by one
// ulp of T, and the epilogue of a 256 x 256 tile stays shorter than the tile's MMAs.
template <typename T>
__device__ __forceinline__ float silu_mul_16bit(float g, float u) {
  const float s = __fdividef(g, 1.0f + __expf(-g));
  if constexpr (std::is_same<T, __half>::value) return __half2float(__float2half_rn(s)) * u;
  else return __bfloat162float(__float2bfloat16_rn(s)) * u;
}

// NCOLS consecutive accumulators of one row -> alpha * acc (+ bias) rounded to OutT -> NVFP4: NCOLS / 16 blocks of
// 8 bytes and their scale bytes (block b in bits [8b, 8b+8) of sf_word), exactly as the quantizer kernel would
// quantize that OutT tensor.  Rows at or beyond p.m get zero scale bytes (padding of the scale tensor).
template <typename OutT, int NCOLS>
__device__ __forceinline__ void quantize_row_chunk_to_regs(const GemmParams& p, const uint32_t* r, float alpha, const OutT* bias,
                                                           int row, int col0, float gs, float rcp_gs, float rcp6,
                                                           uint2 (&q)[NCOLS / 16], uint32_t& sf_word) {
  static_assert(sizeof(OutT) == 2, "16-bit values only");
  using V2 = typename Vec2<OutT>::type;
  uint32_t w[NCOLS / 2];
#pragma unroll
  for (int piece = 0; piece < NCOLS / 8; ++piece) {
    const int colj = col0 + 8 * piece;
    const uint4 o = scale_bias_pack<OutT>(&r[8 * piece], alpha, (bias && colj < p.n) ? bias + colj : nullptr);
    w[4 * piece + 0] = o.x; w[4 * piece + 1] = o.y; w[4 * piece + 2] = o.z; w[4 * piece + 3] = o.w;
  }
  sf_word = 0;
#pragma unroll
  for (int b = 0; b < NCOLS / 16; ++b) {
    V2 h2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) h2[i] = *reinterpret_cast<const V2*>(&w[8 * b + i]);
    uint8_t sf;
    q[b] = nvfp4_quantize_block<OutT>(h2, gs, rcp_gs, rcp6, sf);
    // a block past the last column is padding of the scale tensor: zero whatever the global scale (a NaN or infinite
    // one would turn a block of zeros into the NaN byte)
    if (col0 + 16 * b < p.n) sf_word |= (uint32_t)sf << (8 * b);
  }
  if (row >= p.m) sf_word = 0;
}

// Everything the epilogue can do to NCOLS (64 or 32) consecutive columns of one row beyond a plain store.
//   values   alpha * acc (+ bias), rounded to OutT (fp16 / bf16)
//   ACT      gated activation: the columns come in groups of 32, 16 "gate" columns followed by their 16 "up" columns
//            (the weight's rows were interleaved that way); each group yields 16 outputs silu(gate) * up, so the
//            output tensor is [m, n / 2]
//   p.out_gs set: the outputs are quantized to NVFP4 exactly as the quantizer kernel would quantize that OutT
//            tensor (8 bytes of nibbles per 16 outputs to p.d, scale bytes, adjacent in the swizzled
//            [rowTile][kTile][32][4][4] layout, to p.out_sf; rows in [m, round_up(m, 128)) get zero scales)
//   else     the outputs are stored to p.d as OutT
template <typename OutT, int NCOLS, bool ACT>
__device__ __forceinline__ void finish_row_chunk(const GemmParams& p, const uint32_t* r, float alpha, const OutT* bias,
                                                 int row, int col0, float gs, float rcp_gs, float rcp6) {
  static_assert(sizeof(OutT) == 2, "16-bit values only");
  using V2 = typename Vec2<OutT>::type;
  constexpr int NOUT = ACT ? NCOLS / 2 : NCOLS;          // outputs of this chunk
  uint32_t w[NCOLS / 2];                                 // the values as packed pairs
#pragma unroll
  for (int piece = 0; piece < NCOLS / 8; ++piece) {
    const int colj = col0 + 8 * piece;
    const uint4 o = scale_bias_pack<OutT>(&r[8 * piece], alpha, (bias && colj < p.n) ? bias + colj : nullptr);
    w[4 * piece + 0] = o.x; w[4 * piece + 1] = o.y; w[4 * piece + 2] = o.z; w[4 * piece + 3] = o.w;
  }
  uint32_t out_pairs[NOUT / 2];
  if constexpr (ACT) {
#pragma unroll
    for (int g = 0; g < NCOLS / 32; ++g)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 gate = to_float2<OutT>(*reinterpret_cast<const V2*>(&w[16 * g + i]));
        const float2 up = to_float2<OutT>(*reinterpret_cast<const V2*>(&w[16 * g + 8 + i]));
        out_pairs[8 * g + i] = pack2<OutT>(silu_mul_16bit<OutT>(gate.x, up.x), silu_mul_16bit<OutT>(gate.y, up.y));
      }
  } else {
#pragma unroll
    for (int i = 0; i < NOUT / 2; ++i) out_pairs[i] = w[i];
  }
  const int out_cols = ACT ? p.n / 2 : p.n, ocol0 = ACT ? col0 / 2 : col0;
  if (p.out_gs == nullptr) {
    if (row < p.m) {
      OutT* dst = static_cast<OutT*>(p.d) + (int64_t)row * out_cols + ocol0;
#pragma unroll
      for (int v = 0; v < NOUT / 8; ++v)
        if (ocol0 + 8 * v < out_cols)
          reinterpret_cast<uint4*>(dst)[v] = make_uint4(out_pairs[4 * v], out_pairs[4 * v + 1], out_pairs[4 * v + 2], out_pairs[4 * v + 3]);
    }
    return;
  }
  constexpr int NBLK = NOUT / 16;
  uint32_t sf_word = 0;
  uint2 q[NBLK];
#pragma unroll
  for (int b = 0; b < NBLK; ++b) {
    V2 h2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) h2[i] = *reinterpret_cast<const V2*>(&out_pairs[8 * b + i]);
    uint8_t sf;
    q[b] = nvfp4_quantize_block<OutT>(h2, gs, rcp_gs, rcp6, sf);
    if (ocol0 + 16 * b < out_cols) sf_word |= (uint32_t)sf << (8 * b);      // padding blocks keep a zero scale byte
  }
  uint8_t* out = static_cast<uint8_t*>(p.d);
  if (row < p.m) {
    uint8_t* dst = out + (int64_t)row * (out_cols / 2) + ocol0 / 2;
#pragma unroll
    for (int b = 0; b < NBLK; ++b)
      if (ocol0 + 16 * b < out_cols) *reinterpret_cast<uint2*>(dst + 8 * b) = q[b];
  } else {
    sf_word = 0;
  }
  const int k_tiles = (out_cols + 63) / 64, k_tile = ocol0 / 64;
  if (row < (p.m + 127) / 128 * 128 && k_tile < k_tiles) {
    uint8_t* dst = p.out_sf + ((int64_t)(row / 128) * k_tiles + k_tile) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 +
                   (ocol0 % 64) / 16;
    if constexpr (NBLK == 4) *reinterpret_cast<uint32_t*>(dst) = sf_word;
    else if constexpr (NBLK == 2) *reinterpret_cast<uint16_t*>(dst) = (uint16_t)sf_word;
    else *dst = (uint8_t)sf_word;
  }
}

// True when the epilogue has more to do than scale, add the bias and store.
__device__ __forceinline__ bool has_fused_output(const GemmParams& p) { return p.out_gs != nullptr || p.act != 0; }

template <int BN, bool MX, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
fp4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const GemmParams p) {
  using C = Cfg<BN, MX>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128-byte swizzle pattern of the operand tiles
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ctrl = smem + C::kStages * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);
  // barrier indices
  constexpr int kFull = 0, kEmpty = C::kStages, kAccFull = 2 * C::kStages,
                kAccEmpty = kAccFull + C::kAccStages, kDrain = kAccEmpty + C::kAccStages,
                kNumBars = kDrain + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* never_set = tmem_slot + 2;   // stays 0: lets the exit-path waits run to their limit

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  auto bar = [&](int i) { return smem_u32(bars + i); };

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(bar(kFull + i), 1);
      mbar_init(bar(kEmpty + i), 1);
    }
    for (int i = 0; i < C::kAccStages; ++i) {
      mbar_init(bar(kAccFull + i), 1);
      mbar_init(bar(kAccEmpty + i), 4);   // one arrival per epilogue warp
    }
    mbar_init(bar(kDrain), 1);
    *abort_flag = 0;
    *never_set = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (p.release_next) griddep_launch_dependents();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_stages = (p.k + kStageK - 1) / kStageK;

  if (warp == 0) {
    // ------------------------------------------------------------ producer ---
    if (elect_one()) {
      // Fill kc of this CTA: K stage kc % k_stages of its (kc / k_stages)-th tile, into ring slot kc % kStages.
      // `what`: the B side (which also arms the barrier with the bytes of both sides), the A side, or both.
      constexpr int kSideB = 1, kSideA = 2;
      auto fill = [&](uint32_t kc, int what) {
        const int tile = (int)blockIdx.x + (int)(kc / (uint32_t)k_stages) * (int)gridDim.x, ks = (int)(kc % (uint32_t)k_stages);
        const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
        const int halves = min(C::kHalves, p.sfb_row_tiles - tn * C::kHalves);
        const uint32_t s = kc % C::kStages;
        const int chunks = min(C::kChunksPerStage, p.sf_k_chunks - ks * C::kChunksPerStage);
        const uint32_t sf_bytes = (uint32_t)chunks * 512u;
        const uint32_t st = smem_base + s * C::kStageBytes;
        const int64_t chunk0 = (int64_t)ks * C::kChunksPerStage;
        if (what & kSideB) {
          mbar_arrive_expect_tx(bar(kFull + s), C::kABytes + C::kBBytes + sf_bytes * (1 + halves));
          tma_load_2d(st + C::kABytes, &tmap_b, bar(kFull + s), ks * kStageKBytes, tn * BN);
          for (int h = 0; h < halves; ++h)
            bulk_load(st + C::kABytes + C::kBBytes + C::kSfaBytes + h * C::kChunksPerStage * 512,
                      p.sfb + ((int64_t)(tn * C::kHalves + h) * p.sf_k_chunks + chunk0) * 512,
                      sf_bytes, bar(kFull + s));
        }
        if (what & kSideA) {
          tma_load_2d(st, &tmap_a, bar(kFull + s), ks * kStageKBytes, tm * kBM);
          bulk_load(st + C::kABytes + C::kBBytes,
                    p.sfa + ((int64_t)tm * p.sf_k_chunks + chunk0) * 512, sf_bytes, bar(kFull + s));
        }
      };
      const int my_tiles = (int)blockIdx.x < num_tiles ? (num_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
      const uint32_t fills = (uint32_t)my_tiles * (uint32_t)k_stages;
      uint32_t kc = 0;   // stage fills issued so far
      if (p.after_producer) {
        // B does not depend on the kernel before this one: fill the ring's B side while that kernel still runs
        const uint32_t early = min(fills, (uint32_t)C::kStages);
        for (uint32_t i = 0; i < early; ++i) fill(i, kSideB);
        griddep_wait();
        for (uint32_t i = 0; i < early; ++i) fill(i, kSideA);
        kc = early;
      }
      for (; kc < fills; ++kc) {
        const uint32_t s = kc % C::kStages, ph = (kc / C::kStages) & 1u;
        if (!mbar_wait_bounded(bar(kEmpty + s), ph ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicOr(p.status, kErrProducer);
          break;
        }
        fill(kc, kSideB | kSideA);
      }
      if (*abort_flag) {
        // give the copies already issued a bounded chance to land before the CTA exits
        for (uint32_t s = 0; s < (uint32_t)C::kStages; ++s) {
          const uint32_t fills = (kc + C::kStages - 1 - s) / C::kStages;
          if (fills) mbar_wait_bounded(bar(kFull + s), (fills - 1) & 1u, never_set, 200000000ull);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- issuer ---
    if (elect_one()) {
      uint32_t kc = 0;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int tn = tile / p.tiles_m;
        const int halves = min(C::kHalves, p.sfb_row_tiles - tn * C::kHalves);
        const int as = it % C::kAccStages;
        const uint32_t acc_ph = (uint32_t)(it / C::kAccStages) & 1u;
        if (!mbar_wait_bounded(bar(kAccEmpty + as), acc_ph ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicOr(p.status, kErrIssuer);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + as * C::kAccCols;
        for (int ks = 0; ks < k_stages; ++ks, ++kc) {
          const uint32_t s = kc % C::kStages, ph = (kc / C::kStages) & 1u;
          if (!mbar_wait_bounded(bar(kFull + s), ph, abort_flag)) {
            *abort_flag = 1;
            atomicOr(p.status, kErrIssuer);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const int chunks = min(C::kChunksPerStage, p.sf_k_chunks - ks * C::kChunksPerStage);
          const int mmas = min(kStageK / kMmaK, (p.k - ks * kStageK + kMmaK - 1) / kMmaK);
          const uint32_t st = smem_base + s * C::kStageBytes;
          const uint32_t sf_slot = tmem_base + C::kSfColBase + (kc & 1u) * C::kSfSlotCols;
          const uint32_t sfa_tmem = sf_slot, sfb_tmem = sf_slot + C::kSfaCols;
          // scales: shared -> tensor memory, one 512-byte chunk (128 rows x 4 scales) per copy, each
          // chunk's copies queued right before the MMAs that consume them so that later copies run
          // under earlier MMAs
          const uint64_t a_desc = make_smem_desc(st, 16, 1024, 2);
          const uint64_t b_desc = make_smem_desc(st + C::kABytes, 16, 1024, 2);
          for (int c = 0; c < chunks; ++c) {
            tc_copy_sf_32x128b_warpx4(
                sfa_tmem + 4 * c,
                make_smem_desc(st + C::kABytes + C::kBBytes + c * 512, 0, 128, 0));
            for (int h = 0; h < halves; ++h)
              tc_copy_sf_32x128b_warpx4(
                  sfb_tmem + 4 * (c * C::kHalves + h),
                  make_smem_desc(st + C::kABytes + C::kBBytes + C::kSfaBytes +
                                     (h * C::kChunksPerStage + c) * 512, 0, 128, 0));
            for (int jj = 0; jj < C::kMmasPerChunk; ++jj) {
              const int j = c * C::kMmasPerChunk + jj;
              if (j >= mmas) break;
              const uint32_t accumulate = (ks | j) != 0 ? 1u : 0u;
              const uint64_t koff = (uint64_t)((j * (kMmaK / 2)) >> 4);   // 32 bytes of K per MMA
              if (MX) {
                const uint32_t sf_id = (uint32_t)jj * 2u;
                tc_mma_mxf4(d_tmem, a_desc + koff, b_desc + koff,
                            make_idesc_fp4_block_scaled(kBM, BN, true, sf_id, sf_id),
                            sfa_tmem + 4 * c, sfb_tmem + 4 * c * C::kHalves, accumulate);
              } else {
                tc_mma_nvf4(d_tmem, a_desc + koff, b_desc + koff,
                            make_idesc_fp4_block_scaled(kBM, BN, false),
                            sfa_tmem + 4 * c, sfb_tmem + 4 * c * C::kHalves, accumulate);
              }
            }
          }
          tc_commit(bar(kEmpty + s));   // stage reusable once these MMAs have read it
        }
        if (ok) tc_commit(bar(kAccFull + as));
      }
      if (*abort_flag) {
        tc_commit(bar(kDrain));
        mbar_wait_bounded(bar(kDrain), 0, never_set, 200000000ull);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue ---
    const int q = warp & 3;                 // TMEM lane quarter this warp may access
    if (p.after_producer) griddep_wait();   // alpha comes from the kernel before this one
    const float alpha = load_alpha(p);
    OutT* d = static_cast<OutT*>(p.d);
    const OutT* bias = static_cast<const OutT*>(p.bias);
    const float out_gs = p.out_gs ? __ldg(p.out_gs) : 1.0f, rcp_out_gs = rcp_approx_ftz(out_gs), rcp6 = rcp_approx_ftz(6.0f);
    uint32_t mx2_bits = 0;                       // running max |value stored| of this lane (pair of OutT)
    const bool track_amax = sizeof(OutT) == 2 && p.amax_scratch != nullptr;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const int as = it % C::kAccStages;
      const uint32_t acc_ph = (uint32_t)(it / C::kAccStages) & 1u;
      // warp-uniform decision: the tensor-memory loads below are .sync.aligned
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(kAccFull + as), acc_ph, abort_flag))) {
        *abort_flag = 1;
        if (lane == 0) atomicOr(p.status, kErrEpilogue);
        break;
      }
      tc_fence_after_sync();
      const int row = tm * kBM + q * 32 + lane;
      const uint32_t t_row = tmem_base + as * C::kAccCols + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col = tn * BN + c * 32;
        if constexpr (sizeof(OutT) == 2) {
          if (has_fused_output(p)) {
            if (p.act) finish_row_chunk<OutT, 32, true>(p, r, alpha, bias, row, col, out_gs, rcp_out_gs, rcp6);
            else finish_row_chunk<OutT, 32, false>(p, r, alpha, bias, row, col, out_gs, rcp_out_gs, rcp6);
            continue;
          }
        }
        if (row < p.m && col < p.n)
          store_row_chunk<OutT>(d + (int64_t)row * p.n + col, r, alpha, bias ? bias + col : nullptr,
                                track_amax ? &mx2_bits : nullptr);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kAccEmpty + as));
    }
    if (track_amax) absmax_finish<OutT>(p, mx2_bits, gridDim.x * 4u);
  }

  // -------------------------------------------------------------- common exit ---
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------ host side ---
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// cuTensorMapEncodeTiled behind a small per-thread cache.  A descriptor is a pure function of its arguments, a layer
// calls with the same weight (and usually the same workspace) addresses every time, and an encode costs about a
// microsecond of host time -- four or five of them per launch are not small beside a 9 us decode kernel.
struct TensorMapKey {
  uintptr_t base;
  uint64_t dims[3], strides[2];
  uint32_t box[3];
  int32_t dtype, rank, swizzle, promotion;
};
CUresult encode_tiled_cached(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base, const cuuint64_t* dims,
                             const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swizzle,
                             CUtensorMapL2promotion promotion) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return CUDA_ERROR_NOT_SUPPORTED;
  constexpr int kSlots = 256;
  struct Slot { TensorMapKey key; CUtensorMap map; bool used; };
  thread_local Slot* table = nullptr;
  if (!table) table = new Slot[kSlots]();
  TensorMapKey key;
  memset(&key, 0, sizeof(key));
  key.base = reinterpret_cast<uintptr_t>(base);
  for (int i = 0; i < rank; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides[i];
  key.dtype = (int32_t)dtype; key.rank = rank; key.swizzle = (int32_t)swizzle; key.promotion = (int32_t)promotion;
  uint64_t h = key.base * 0x9E3779B97F4A7C15ull;
  h ^= (key.dims[0] + 0x632BE59BD9B4E019ull * key.dims[1] + key.box[1] * 1315423911ull + (uint64_t)key.rank) * 0xD6E8FEB86659FD93ull;
  Slot& slot = table[(h >> 40) % kSlots];
  static const bool cache_off = getenv("NVFP_NO_DESCRIPTOR_CACHE") != nullptr;     // for measuring what the cache saves
  if (!cache_off && slot.used && memcmp(&slot.key, &key, sizeof(key)) == 0) {
    *map = slot.map;
    return CUDA_SUCCESS;
  }
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, dtype, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, promotion, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) {
    slot.key = key;
    slot.map = *map;
    slot.used = true;
  }
  return r;
}

// cudaFuncSetAttribute(max dynamic shared memory) once per kernel and device instead of once per launch.
template <typename Kernel>
int ensure_dynamic_smem(Kernel kernel, int bytes) {
  struct Done { const void* fn; int dev; int bytes; };
  thread_local Done done[64];
  thread_local int count = 0;
  int dev = 0;
  NVFP_CUDA(cudaGetDevice(&dev));
  const void* fn = reinterpret_cast<const void*>(kernel);
  for (int i = 0; i < count; ++i)
    if (done[i].fn == fn && done[i].dev == dev && done[i].bytes >= bytes) return NVFP_OK;
  NVFP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (count < 64) done[count++] = Done{fn, dev, bytes};
  return NVFP_OK;
}

// Row-major [rows, k/2] bytes of packed e2m1; box = 128 bytes of K x box_rows rows,
// 128-byte swizzle; out-of-range rows / bytes read as zero.
int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
  const cuuint64_t dims[2] = {(cuuint64_t)(k / 2), (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)(k / 2)};
  const cuuint32_t box[2] = {(cuuint32_t)kStageKBytes, (cuuint32_t)box_rows};
  CUresult r = encode_tiled_cached(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
  if (r != CUDA_SUCCESS) return fail(NVFP_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return NVFP_OK;
}

template <int BN, bool MX, typename OutT>
int launch_config(const GemmParams& base, const void* a, const void* b, int sm_count,
                  cudaStream_t stream) {
  using C = Cfg<BN, MX>;
  GemmParams p = base;
  p.tiles_m = (int)ceil_div(p.m, kBM);
  p.tiles_n = (int)ceil_div(p.n, BN);
  CUtensorMap map_a, map_b;
  if (int rc = make_operand_map(&map_a, a, p.m, p.k, kBM)) return rc;
  if (int rc = make_operand_map(&map_b, b, p.n, p.k, BN)) return rc;
  auto kernel = fp4_gemm_kernel<BN, MX, OutT>;
  if (int rc = ensure_dynamic_smem(kernel, (int)C::kSmemBytes)) return rc;
  const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
  const unsigned grid = (unsigned)std::min<int64_t>(tiles, sm_count);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.after_producer ? 1 : 0;
  NVFP_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, p));
  return NVFP_OK;
}

#include "gemm_fp4_pair_sm100.cuh"
#include "gemm_fp4_skinny_sm100.cuh"

// Scale plumbing between chained layers (see GemmParams): alpha formed in the epilogue from two global scales, and / or
// the output's own global scale (and the next layer's alpha) produced by the epilogue.
struct ChainOpts {
  const float* alpha_gs_b = nullptr;
  uint32_t* amax_scratch = nullptr;
  float* amax_gs_out = nullptr;
  const float* amax_gs_other = nullptr;
  float* amax_alpha_out = nullptr;
};

// `outputs`: n_out destination matrices [m, n] (row-major, out_dtype); more than one only for the
// column-parallel gather, where the extra ones are peer GPUs' buffers.
template <bool MX>
int scaled_mm(void* const* outputs, int n_out, int64_t ld, const void* a, const void* b, const void* sfa, const void* sfb,
              const float* alpha, int64_t m, int64_t n, int64_t k, int out_dtype, cudaStream_t stream,
              const void* bias = nullptr, bool after_producer = false, const float* out_gs = nullptr,
              void* out_sf = nullptr, int act = 0, bool release_next = false, const PeerSync* peer_sync = nullptr,
              const ChainOpts* chain = nullptr) {
  NVFP_REQUIRE(bias == nullptr || (reinterpret_cast<uintptr_t>(bias) & 15) == 0, "bias must be 16-byte aligned");
  const bool fused = out_gs != nullptr || act != 0;
  if (fused) {
    NVFP_REQUIRE(act == 0 || act == 1, "unknown activation code %d", act);
    NVFP_REQUIRE(out_gs == nullptr || (out_sf != nullptr && (reinterpret_cast<uintptr_t>(out_sf) & 15) == 0),
                 "scale output is null or not 16-byte aligned");
    NVFP_REQUIRE(out_dtype == NVFP_DTYPE_F16 || out_dtype == NVFP_DTYPE_BF16,
                 "the epilogue's activation and quantization work on fp16 or bf16 values (dtype code %d)", out_dtype);
    NVFP_REQUIRE(n_out == 1 && ld == n, "a fused epilogue writes one dense destination");
  }
  NVFP_REQUIRE(outputs != nullptr && n_out >= 1 && n_out <= kMaxOutputs,
               "between 1 and %d output matrices are supported, got %d", kMaxOutputs, n_out);
  for (int o = 0; o < n_out; ++o)
    NVFP_REQUIRE((outputs[o] != nullptr || m == 0 || n == 0) && (reinterpret_cast<uintptr_t>(outputs[o]) & 15) == 0,
                 "output %d is null or not 16-byte aligned", o);
  NVFP_REQUIRE(ld >= n && ld % 8 == 0, "leading dimension %lld must be >= n and a multiple of 8", (long long)ld);
  void* d = outputs[0];
  constexpr int kBlock = MX ? 32 : 16;
  constexpr int kAlign = MX ? 64 : 32;
  NVFP_REQUIRE(m >= 0 && n >= 0 && k >= 0, "negative shape");
  NVFP_REQUIRE(k % kAlign == 0, "Expected k to be divisible by %d, but got k: %lld.", kAlign, (long long)k);
  NVFP_REQUIRE(n % 32 == 0, "Expected n to be divisible by 32, but got n: %lld.", (long long)n);
  NVFP_REQUIRE(out_dtype == NVFP_DTYPE_F16 || out_dtype == NVFP_DTYPE_BF16 || out_dtype == NVFP_DTYPE_F32,
               "Unsupported output data type of nvfp4 mm (dtype code %d)", out_dtype);
  NVFP_REQUIRE(MX || alpha != nullptr, "alpha pointer is null");
  NVFP_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31), "shape too large");
  if (m == 0 || n == 0) return NVFP_OK;
  NVFP_REQUIRE(k > 0, "k must be positive");
  NVFP_REQUIRE(d && a && b && sfa && sfb, "null pointer");
  NVFP_REQUIRE(((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                 reinterpret_cast<uintptr_t>(sfa) | reinterpret_cast<uintptr_t>(sfb) |
                 reinterpret_cast<uintptr_t>(d)) & 15) == 0,
               "operands, scales and output must be 16-byte aligned");
  DeviceInfo info;
  if (int rc = current_device_info(&info)) return rc;
  if (info.cc_major != 10)
    return fail(NVFP_ERR_UNSUPPORTED, "No compiled nvfp4 mm kernel for compute capability %d.%d (needs sm_100)",
                info.cc_major, info.cc_minor);
  GemmParams p{};
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.alpha = alpha;
  p.bias = bias;
  p.out_gs = out_gs;
  p.out_sf = static_cast<uint8_t*>(out_sf);
  p.act = act;
  p.release_next = release_next ? 1 : 0;
  p.d = d;
  p.m = (int)m; p.n = (int)n; p.k = (int)k;
  p.sf_k_chunks = (int)ceil_div(k / kBlock, 4);
  p.sfb_row_tiles = (int)ceil_div(n, 128);
  p.status = device_status_word();
  NVFP_REQUIRE(p.status != nullptr, "cannot locate the device status word");
  bool amax_after = false;       // the output's global scale by a pass over the (small) output instead of the epilogue
  if (chain) {
    p.alpha_gs_b = chain->alpha_gs_b;
    if (chain->amax_scratch) {
      NVFP_REQUIRE(!fused && n_out == 1 && ld == n && out_dtype != NVFP_DTYPE_F32 && chain->amax_gs_out != nullptr &&
                       (chain->amax_gs_other == nullptr || chain->amax_alpha_out != nullptr),
                   "the output's global scale is formed for one dense fp16 / bf16 output (and needs its result pointers)");
      p.amax_scratch = chain->amax_scratch;
      p.amax_gs_out = chain->amax_gs_out;
      p.amax_gs_other = chain->amax_gs_other;
      p.amax_alpha_out = chain->amax_alpha_out;
    }
  }
  // Few activation rows (decode): weights are streamed once; swap the operands and split K over a cluster.
  if (n_out == 1 && ld == n && skinny_preferred(m, n, info.sm_count)) {
    // the few-rows kernel does not fold the output's maximum into its epilogue: its output is a few hundred KB, which
    // the global-scale kernel sweeps in a couple of microseconds right after
    amax_after = p.amax_scratch != nullptr;
    p.amax_scratch = nullptr;
    int rc;
    switch (out_dtype) {
      case NVFP_DTYPE_BF16: rc = launch_skinny<MX, __nv_bfloat16>(p, a, b, info.sm_count, stream, after_producer); break;
      case NVFP_DTYPE_F16: rc = launch_skinny<MX, __half>(p, a, b, info.sm_count, stream, after_producer); break;
      default: rc = launch_skinny<MX, float>(p, a, b, info.sm_count, stream, after_producer); break;
    }
    if (rc == NVFP_OK && amax_after)
      rc = activation_scales_launch(chain->amax_gs_out, chain->amax_alpha_out, chain->amax_scratch, d, m, n, n, out_dtype,
                                    chain->amax_gs_other, stream);
    return rc;
  }
  // the kernels below fetch only B before they wait; several destinations only when the ranks are synchronised inside
  // the kernel (a caller that synchronises them around the call does so with launches of its own in between)
  p.after_producer = (after_producer && (n_out == 1 || peer_sync != nullptr)) ? 1 : 0;
  // Large problems: CTA pairs on 256 x 256 tiles (least operand traffic per flop).
  const int64_t pair_tiles = ceil_div(m, kPairBM) * ceil_div(n, kPairBN);
  if (n_out > 1 || ld != n || (m > 128 && n >= 256 && pair_tiles >= info.sm_count / 2)) {
    if (fused)
      return out_dtype == NVFP_DTYPE_BF16
                 ? launch_pair<MX, __nv_bfloat16, kOutFused>(p, a, b, outputs, n_out, ld, info.sm_count, stream)
                 : launch_pair<MX, __half, kOutFused>(p, a, b, outputs, n_out, ld, info.sm_count, stream);
    switch (out_dtype) {
      case NVFP_DTYPE_BF16: return launch_pair<MX, __nv_bfloat16>(p, a, b, outputs, n_out, ld, info.sm_count, stream, peer_sync);
      case NVFP_DTYPE_F16: return launch_pair<MX, __half>(p, a, b, outputs, n_out, ld, info.sm_count, stream, peer_sync);
      default: return launch_pair<MX, float>(p, a, b, outputs, n_out, ld, info.sm_count, stream, peer_sync);
    }
  }
  // Tile-width choice: 256-wide tiles halve the shared-memory traffic per flop but have a single accumulator
  // buffer; use them when there are enough of them to fill the GPU, and also when 128-wide tiles would need more
  // than one wave of CTAs (measured: 512 x 6144 x 4096 21.4 against 24.6 us, 256 x 14336 x 4096 22.5 against 25.5,
  // 128 x 28672 x 4096 25.5 against 26.6; with at most one wave of 128-wide tiles the wide ones lose, 128 x 14336 x
  // 4096 22.0 against 18.4).
  const int64_t tiles256 = ceil_div(m, kBM) * ceil_div(n, 256), tiles128 = ceil_div(m, kBM) * ceil_div(n, 128);
  const bool wide = n >= 256 && (tiles256 >= info.sm_count || (tiles128 > info.sm_count && k >= 2048));
  if (wide) {
    switch (out_dtype) {
      case NVFP_DTYPE_BF16: return launch_config<256, MX, __nv_bfloat16>(p, a, b, info.sm_count, stream);
      case NVFP_DTYPE_F16: return launch_config<256, MX, __half>(p, a, b, info.sm_count, stream);
      default: return launch_config<256, MX, float>(p, a, b, info.sm_count, stream);
    }
  }
  switch (out_dtype) {
    case NVFP_DTYPE_BF16: return launch_config<128, MX, __nv_bfloat16>(p, a, b, info.sm_count, stream);
    case NVFP_DTYPE_F16: return launch_config<128, MX, __half>(p, a, b, info.sm_count, stream);
    default: return launch_config<128, MX, float>(p, a, b, info.sm_count, stream);
  }
}

// One thread waits on an mbarrier that nobody ever arrives at, with the same bounded wait the GEMM roles
// use, and reports the expiry like they do.  Nothing faults and the kernel returns normally.
constexpr uint32_t kErrSelfTest = 1u << 16;
__global__ void selftest_wait_kernel(uint32_t* status, uint64_t limit_ns) {
  __shared__ uint64_t never_completes;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&never_completes), 1);
    fence_mbar_init();
    if (!mbar_wait_bounded(smem_u32(&never_completes), 0, &abort_flag, limit_ns)) atomicOr(status, kErrSelfTest);
  }
}

}  // namespace
}  // namespace nvfp

using namespace nvfp;

extern "C" int nvfp_selftest_wait_timeout(uint64_t limit_ns, void* stream) {
  clear_error();
  NVFP_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ull, "limit must be between 1 ns and 100 ms, got %llu ns",
               (unsigned long long)limit_ns);
  uint32_t* status = device_status_word();
  NVFP_REQUIRE(status != nullptr, "cannot locate the device status word");
  selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_ns);
  NVFP_CUDA(cudaGetLastError());
  return NVFP_OK;
}

extern "C" int nvfp_scaled_fp4_mm(void* d, const void* a, const void* b, const void* sfa,
                                  const void* sfb, const float* alpha, int64_t m, int64_t n,
                                  int64_t k, int out_dtype, void* stream) {
  clear_error();
  return scaled_mm<false>(&d, 1, n, a, b, sfa, sfb, alpha, m, n, k, out_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int nvfp_mxfp4_mm(void* d, const void* a, const void* b, const void* sfa, const void* sfb,
                             const float* alpha, int64_t m, int64_t n, int64_t k, int out_dtype,
                             void* stream) {
  clear_error();
  return scaled_mm<true>(&d, 1, n, a, b, sfa, sfb, alpha, m, n, k, out_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int nvfp_scaled_fp4_mm_bias(void* d, const void* a, const void* b, const void* sfa, const void* sfb,
                                       const float* alpha, const void* bias, int64_t m, int64_t n, int64_t k,
                                       int out_dtype, int mxfp4, void* stream) {
  clear_error();
  return mxfp4 ? scaled_mm<true>(&d, 1, n, a, b, sfa, sfb, alpha, m, n, k, out_dtype, static_cast<cudaStream_t>(stream), bias)
               : scaled_mm<false>(&d, 1, n, a, b, sfa, sfb, alpha, m, n, k, out_dtype, static_cast<cudaStream_t>(stream), bias);
}

extern "C" int nvfp_scaled_fp4_mm_fp4out(void* d_fp4, void* d_sf, const void* a, const void* b, const void* sfa,
                                         const void* sfb, const float* alpha, const void* bias,
                                         const float* out_global_scale, int64_t m, int64_t n, int64_t k,
                                         int value_dtype, int mxfp4, void* stream) {
  clear_error();
  NVFP_REQUIRE(out_global_scale != nullptr, "output global scale is null");
  return mxfp4 ? scaled_mm<true>(&d_fp4, 1, n, a, b, sfa, sfb, alpha, m, n, k, value_dtype, static_cast<cudaStream_t>(stream),
                                 bias, false, out_global_scale, d_sf)
               : scaled_mm<false>(&d_fp4, 1, n, a, b, sfa, sfb, alpha, m, n, k, value_dtype, static_cast<cudaStream_t>(stream),
                                  bias, false, out_global_scale, d_sf);
}

extern "C" int nvfp_scaled_fp4_mm_silu_mul(void* d, void* d_sf, const void* a, const void* b, const void* sfa,
                                           const void* sfb, const float* alpha, const void* bias,
                                           const float* out_global_scale, int64_t m, int64_t n, int64_t k,
                                           int value_dtype, int mxfp4, void* stream) {
  clear_error();
  return mxfp4 ? scaled_mm<true>(&d, 1, n, a, b, sfa, sfb, alpha, m, n, k, value_dtype, static_cast<cudaStream_t>(stream),
                                 bias, false, out_global_scale, d_sf, 1)
               : scaled_mm<false>(&d, 1, n, a, b, sfa, sfb, alpha, m, n, k, value_dtype, static_cast<cudaStream_t>(stream),
                                  bias, false, out_global_scale, d_sf, 1);
}

extern "C" int64_t nvfp_linear_workspace_bytes(int64_t m, int64_t k) {
  if (m < 0 || k < 0) return -1;
  return round_up(m * (k / 2), 256) + round_up(nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(k, 16), 256) + 256;
}

extern "C" int nvfp_linear_forward(void* d, const void* x, int64_t m, int64_t k, int64_t x_row_stride, int x_dtype,
                                   const void* w_fp4, const void* w_sf, const float* w_global_scale, int64_t n,
                                   const void* bias, void* workspace, uint32_t* scratch, int out_dtype, void* stream_) {
  clear_error();
  NVFP_REQUIRE(m >= 0 && n >= 0 && k >= 0, "negative shape");
  NVFP_REQUIRE(k % 32 == 0, "Expected k to be divisible by 32, but got k: %lld.", (long long)k);
  if (m == 0 || n == 0) return NVFP_OK;
  NVFP_REQUIRE(x != nullptr && workspace != nullptr && scratch != nullptr && w_global_scale != nullptr, "null pointer");
  NVFP_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
  NVFP_REQUIRE(x_dtype == NVFP_DTYPE_F16 || x_dtype == NVFP_DTYPE_BF16,
               "Unsupported input data type for quantize_to_fp4 (dtype code %d).", x_dtype);
  NVFP_REQUIRE(x_row_stride >= k && x_row_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0,
               "activation must be 16-byte aligned with a row stride that is >= k and a multiple of 8 elements");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* a_fp4 = ws;
  uint8_t* a_sf = a_fp4 + round_up(m * (k / 2), 256);
  float* gs = reinterpret_cast<float*>(a_sf + round_up(nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(k, 16), 256));
  float* alpha = gs + 1;
  // The launches are chained with programmatic dependent launch: each kernel lets the next one come up while it
  // runs, and the next one touches what its predecessor writes only after griddepcontrol.wait (the quantize launch
  // of the two-launch quantizer loads its tiles first; every GEMM kernel fetches nothing but weights first).
  if (int rc = dynamic_fp4_quant_launch(a_fp4, a_sf, gs, alpha, scratch, x, m, k, x_row_stride, x_dtype, w_global_scale,
                                        /*release_next=*/true, nullptr, stream))
    return rc;
  return scaled_mm<false>(&d, 1, n, a_fp4, w_fp4, a_sf, w_sf, alpha, m, n, k, out_dtype, stream, bias,
                          /*after_producer=*/true);
}

extern "C" int nvfp_scaled_fp4_mm_amax(void* d, const void* a, const void* b, const void* sfa, const void* sfb,
                                       const float* alpha, const void* bias, int64_t m, int64_t n, int64_t k, int out_dtype,
                                       int mxfp4, float* d_global_scale_out, uint32_t* scratch,
                                       const float* next_weight_global_scale, float* next_alpha_out, void* stream) {
  clear_error();
  NVFP_REQUIRE(d_global_scale_out != nullptr && scratch != nullptr, "global-scale output or scratch is null");
  NVFP_REQUIRE(next_weight_global_scale == nullptr || next_alpha_out != nullptr,
               "alpha output is null although the next weight's scale is given");
  if (m == 0 || n == 0) return NVFP_OK;
  ChainOpts chain;
  chain.amax_scratch = scratch;
  chain.amax_gs_out = d_global_scale_out;
  chain.amax_gs_other = next_weight_global_scale;
  chain.amax_alpha_out = next_alpha_out;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return mxfp4 ? scaled_mm<true>(&d, 1, n, a, b, sfa, sfb, alpha, m, n, k, out_dtype, st, bias, false, nullptr, nullptr, 0, false,
                                 nullptr, &chain)
               : scaled_mm<false>(&d, 1, n, a, b, sfa, sfb, alpha, m, n, k, out_dtype, st, bias, false, nullptr, nullptr, 0, false,
                                  nullptr, &chain);
}

extern "C" int nvfp_linear_forward_chained(void* d, const void* x, int64_t m, int64_t k, int64_t x_row_stride, int x_dtype,
                                           const float* x_global_scale, const void* w_fp4, const void* w_sf,
                                           const float* w_global_scale, int64_t n, const void* bias, void* workspace,
                                           uint32_t* scratch, int out_dtype, float* d_global_scale_out,
                                           uint32_t* d_scale_scratch, const float* next_weight_global_scale,
                                           float* next_alpha_out, void* stream_) {
  clear_error();
  NVFP_REQUIRE(m >= 0 && n >= 0 && k >= 0, "negative shape");
  NVFP_REQUIRE(k % 32 == 0, "Expected k to be divisible by 32, but got k: %lld.", (long long)k);
  if (m == 0 || n == 0) return NVFP_OK;
  NVFP_REQUIRE(x != nullptr && workspace != nullptr && w_global_scale != nullptr, "null pointer");
  NVFP_REQUIRE(x_global_scale != nullptr || scratch != nullptr, "scratch is needed when the activation's scale is not given");
  NVFP_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
  NVFP_REQUIRE(x_dtype == NVFP_DTYPE_F16 || x_dtype == NVFP_DTYPE_BF16,
               "Unsupported input data type for quantize_to_fp4 (dtype code %d).", x_dtype);
  NVFP_REQUIRE(x_row_stride >= k && x_row_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0,
               "activation must be 16-byte aligned with a row stride that is >= k and a multiple of 8 elements");
  NVFP_REQUIRE(d_global_scale_out == nullptr || d_scale_scratch != nullptr, "scratch of the output's global scale is null");
  NVFP_REQUIRE(next_weight_global_scale == nullptr || (next_alpha_out != nullptr && d_global_scale_out != nullptr),
               "the next layer's alpha needs the output's global scale and a place to go");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* a_fp4 = ws;
  uint8_t* a_sf = a_fp4 + round_up(m * (k / 2), 256);
  float* gs = reinterpret_cast<float*>(a_sf + round_up(nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(k, 16), 256));
  float* alpha = gs + 1;
  ChainOpts chain;
  const float* alpha_ptr = alpha;
  if (x_global_scale != nullptr) {
    // the scale is known (the layer before formed it in its epilogue): no pass over x for its maximum; alpha is formed
    // by the GEMM's epilogue from the two global scales
    if (int rc = scaled_fp4_quant_launch(a_fp4, a_sf, x, x_global_scale, m, k, x_row_stride, x_dtype, /*release_next=*/true,
                                         stream))
      return rc;
    alpha_ptr = x_global_scale;
    chain.alpha_gs_b = w_global_scale;
  } else {
    if (int rc = dynamic_fp4_quant_launch(a_fp4, a_sf, gs, alpha, scratch, x, m, k, x_row_stride, x_dtype, w_global_scale,
                                          /*release_next=*/true, nullptr, stream))
      return rc;
  }
  if (d_global_scale_out != nullptr) {
    chain.amax_scratch = d_scale_scratch;
    chain.amax_gs_out = d_global_scale_out;
    chain.amax_gs_other = next_weight_global_scale;
    chain.amax_alpha_out = next_alpha_out;
  }
  return scaled_mm<false>(&d, 1, n, a_fp4, w_fp4, a_sf, w_sf, alpha_ptr, m, n, k, out_dtype, stream, bias,
                          /*after_producer=*/true, nullptr, nullptr, 0, false, nullptr, &chain);
}

extern "C" int64_t nvfp_gated_mlp_workspace_bytes(int64_t m, int64_t hidden, int64_t inter) {
  if (m < 0 || hidden < 0 || inter < 0) return -1;
  return nvfp_linear_workspace_bytes(m, hidden) + round_up(m * (inter / 2), 256) +
         round_up(nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(inter, 16), 256);
}

extern "C" int nvfp_gated_mlp_forward(void* y, const void* x, int64_t m, int64_t hidden, int64_t x_row_stride, int x_dtype,
                                      const void* gate_up_fp4, const void* gate_up_sf, const float* gate_up_global_scale,
                                      int64_t inter, const void* down_fp4, const void* down_sf,
                                      const float* act_global_scale, const float* down_alpha, int64_t n_out,
                                      void* workspace, uint32_t* scratch, int out_dtype, void* stream_) {
  clear_error();
  NVFP_REQUIRE(m >= 0 && hidden >= 0 && inter >= 0 && n_out >= 0, "negative shape");
  NVFP_REQUIRE(hidden % 32 == 0 && inter % 32 == 0,
               "Expected hidden and intermediate sizes to be divisible by 32, but got %lld and %lld.", (long long)hidden,
               (long long)inter);
  NVFP_REQUIRE(out_dtype == NVFP_DTYPE_F16 || out_dtype == NVFP_DTYPE_BF16,
               "the gated MLP computes its hidden activation in fp16 or bf16 (dtype code %d)", out_dtype);
  if (m == 0 || n_out == 0) return NVFP_OK;
  NVFP_REQUIRE(inter > 0 && hidden > 0, "empty weight");
  NVFP_REQUIRE(x != nullptr && workspace != nullptr && scratch != nullptr && gate_up_global_scale != nullptr &&
                   act_global_scale != nullptr && down_alpha != nullptr, "null pointer");
  NVFP_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
  NVFP_REQUIRE(x_dtype == NVFP_DTYPE_F16 || x_dtype == NVFP_DTYPE_BF16,
               "Unsupported input data type for quantize_to_fp4 (dtype code %d).", x_dtype);
  NVFP_REQUIRE(x_row_stride >= hidden && x_row_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0,
               "activation must be 16-byte aligned with a row stride that is >= hidden and a multiple of 8 elements");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* x_fp4 = ws;
  uint8_t* x_sf = x_fp4 + round_up(m * (hidden / 2), 256);
  float* gs = reinterpret_cast<float*>(x_sf + round_up(nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(hidden, 16), 256));
  float* alpha = gs + 1;
  void* h_fp4 = ws + nvfp_linear_workspace_bytes(m, hidden);
  void* h_sf = static_cast<uint8_t*>(h_fp4) + round_up(m * (inter / 2), 256);
  if (int rc = dynamic_fp4_quant_launch(x_fp4, x_sf, gs, alpha, scratch, x, m, hidden, x_row_stride, x_dtype,
                                        gate_up_global_scale, /*release_next=*/true, nullptr, stream))
    return rc;
  if (int rc = scaled_mm<false>(&h_fp4, 1, 2 * inter, x_fp4, gate_up_fp4, x_sf, gate_up_sf, alpha, m, 2 * inter, hidden,
                                out_dtype, stream, nullptr, /*after_producer=*/true, act_global_scale, h_sf, /*act=*/1,
                                /*release_next=*/true))
    return rc;
  return scaled_mm<false>(&y, 1, n_out, h_fp4, down_fp4, h_sf, down_sf, down_alpha, m, n_out, inter, out_dtype, stream,
                          nullptr, /*after_producer=*/true);
}

extern "C" int nvfp_scaled_fp4_mm_multi(void* const* dst, int n_dst, const void* a, const void* b,
                                        const void* sfa, const void* sfb, const float* alpha, int64_t m,
                                        int64_t n, int64_t k, int64_t dst_ld, int out_dtype, int mxfp4, void* stream) {
  clear_error();
  return mxfp4 ? scaled_mm<true>(dst, n_dst, dst_ld, a, b, sfa, sfb, alpha, m, n, k, out_dtype, static_cast<cudaStream_t>(stream))
               : scaled_mm<false>(dst, n_dst, dst_ld, a, b, sfa, sfb, alpha, m, n, k, out_dtype, static_cast<cudaStream_t>(stream));
}

namespace nvfp {
namespace {

int scatter_add(void* const* dst, int n_dst, const void* a, const void* b, const void* sfa, const void* sfb,
                const float* alpha, int64_t m, int64_t n, int64_t k, int mxfp4, cudaStream_t st, const PeerSync* peer_sync) {
  NVFP_REQUIRE(dst != nullptr && n_dst >= 1 && n_dst <= kMaxOutputs, "between 1 and %d destinations are supported, got %d",
               kMaxOutputs, n_dst);
  NVFP_REQUIRE(m > 0 && n > 0 && k > 0 && m % (32 * n_dst) == 0,
               "m (%lld) must be a positive multiple of 32 x the number of destinations (%d)", (long long)m, n_dst);
  NVFP_REQUIRE(k % (mxfp4 ? 64 : 32) == 0 && n % 32 == 0, "k must be divisible by %d and n by 32", mxfp4 ? 64 : 32);
  NVFP_REQUIRE(mxfp4 || alpha != nullptr, "alpha pointer is null");
  NVFP_REQUIRE(a && b && sfa && sfb, "null pointer");
  for (int o = 0; o < n_dst; ++o)
    NVFP_REQUIRE(dst[o] != nullptr && (reinterpret_cast<uintptr_t>(dst[o]) & 15) == 0,
                 "destination %d is null or not 16-byte aligned", o);
  DeviceInfo info;
  if (int rc = current_device_info(&info)) return rc;
  if (info.cc_major != 10)
    return fail(NVFP_ERR_UNSUPPORTED, "No compiled nvfp4 mm kernel for compute capability %d.%d (needs sm_100)",
                info.cc_major, info.cc_minor);
  GemmParams p{};
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.alpha = alpha;
  p.d = dst[0];
  p.m = (int)m; p.n = (int)n; p.k = (int)k;
  p.sf_k_chunks = (int)ceil_div(k / (mxfp4 ? 32 : 16), 4);
  p.sfb_row_tiles = (int)ceil_div(n, 128);
  p.status = device_status_word();
  NVFP_REQUIRE(p.status != nullptr, "cannot locate the device status word");
  return mxfp4 ? launch_pair<true, float, kOutScatterAdd>(p, a, b, dst, n_dst, n, info.sm_count, st, peer_sync)
               : launch_pair<false, float, kOutScatterAdd>(p, a, b, dst, n_dst, n, info.sm_count, st, peer_sync);
}

// Checks a peer group and turns it into the kernel's view: `rotated` receives the destinations starting with this
// rank's own (the order in which an epilogue warp walks them, so that at any moment the ranks write to different
// peers), `sync` the flag blocks (world = 0 when the group has none: the caller synchronises).
int unpack_peer_group(const nvfp_peer_group_t* g, void** rotated, PeerSync* sync) {
  NVFP_REQUIRE(g != nullptr, "peer group is null");
  NVFP_REQUIRE(g->world >= 1 && g->world <= kMaxOutputs && g->rank >= 0 && g->rank < g->world,
               "peer group: world %d (1..%d) / rank %d out of range", g->world, kMaxOutputs, g->rank);
  memset(sync, 0, sizeof(*sync));
  bool any = false, all = true;
  for (int r = 0; r < g->world; ++r) {
    NVFP_REQUIRE(g->dst[r] != nullptr, "peer group: destination of rank %d is null", r);
    any = any || g->flags[r] != nullptr;
    all = all && g->flags[r] != nullptr && (reinterpret_cast<uintptr_t>(g->flags[r]) & 127) == 0;
    rotated[r] = g->dst[(g->rank + r) % g->world];
  }
  NVFP_REQUIRE(!any || all, "peer group: flag blocks must be given for every rank (128-byte aligned) or for none");
  if (any && g->world > 1) {
    for (int r = 0; r < g->world; ++r) sync->flags[r] = g->flags[r];
    sync->world = g->world;
    sync->rank = g->rank;
    sync->limit_ns = g->wait_limit_ns ? g->wait_limit_ns : 2000000000ull;
    NVFP_REQUIRE(sync->limit_ns <= 10000000000ull, "peer group: wait limit above 10 s");
  }
  return NVFP_OK;
}

}  // namespace
}  // namespace nvfp

namespace nvfp {
namespace {
// Column-parallel GEMM whose result leaves as NVFP4 into every rank's gathered operand (packed bytes + scales).
int gather_fp4(const nvfp_peer_group_t* g, void* const* dst_sf, int64_t n_total, int64_t n_offset, const void* a,
               const void* b, const void* sfa, const void* sfb, const float* alpha, const void* bias, const float* out_gs,
               int64_t m, int64_t n, int64_t k, int value_dtype, int mxfp4, cudaStream_t stream, bool after_producer) {
  void* rotated[kMaxOutputs];
  PeerSync sync;
  if (int rc = unpack_peer_group(g, rotated, &sync)) return rc;
  NVFP_REQUIRE(dst_sf != nullptr && out_gs != nullptr, "scale destinations or output global scale are null");
  NVFP_REQUIRE(value_dtype == NVFP_DTYPE_F16 || value_dtype == NVFP_DTYPE_BF16,
               "the product is rounded to fp16 or bf16 before it is quantized (dtype code %d)", value_dtype);
  NVFP_REQUIRE(m > 0 && n > 0 && k > 0 && m < (1ll << 31) && n_total < (1ll << 31) && k < (1ll << 31), "bad shape");
  NVFP_REQUIRE(k % (mxfp4 ? 64 : 32) == 0, "Expected k to be divisible by %d, but got k: %lld.", mxfp4 ? 64 : 32, (long long)k);
  NVFP_REQUIRE(n % 64 == 0 && n_offset % 64 == 0 && n_total % 64 == 0 && n_offset >= 0 && n_offset + n <= n_total,
               "slab [%lld, %lld) of %lld columns: offsets and widths must be multiples of 64 (whole scale chunks)",
               (long long)n_offset, (long long)(n_offset + n), (long long)n_total);
  NVFP_REQUIRE(mxfp4 || alpha != nullptr, "alpha pointer is null");
  NVFP_REQUIRE(a && b && sfa && sfb, "null pointer");
  NVFP_REQUIRE(bias == nullptr || (reinterpret_cast<uintptr_t>(bias) & 15) == 0, "bias must be 16-byte aligned");
  GatherFp4 gq;
  memset(&gq, 0, sizeof(gq));
  for (int o = 0; o < g->world; ++o) {
    const int r = (g->rank + o) % g->world;
    NVFP_REQUIRE(dst_sf[r] != nullptr && (reinterpret_cast<uintptr_t>(dst_sf[r]) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(g->dst[r]) & 15) == 0,
                 "destination %d: packed matrix and scale tensor must be non-null and 16-byte aligned", r);
    gq.sf[o] = static_cast<uint8_t*>(dst_sf[r]);
    rotated[o] = static_cast<uint8_t*>(g->dst[r]) + n_offset / 2;
  }
  gq.k_tiles_total = (int)(n_total / 64);
  gq.k_tile0 = (int)(n_offset / 64);
  gq.k_tiles_slab = (int)(n / 64);
  DeviceInfo info;
  if (int rc = current_device_info(&info)) return rc;
  if (info.cc_major != 10)
    return fail(NVFP_ERR_UNSUPPORTED, "No compiled nvfp4 mm kernel for compute capability %d.%d (needs sm_100)",
                info.cc_major, info.cc_minor);
  GemmParams p{};
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.alpha = alpha;
  p.bias = bias;
  p.out_gs = out_gs;
  p.d = rotated[0];
  p.m = (int)m; p.n = (int)n; p.k = (int)k;
  p.sf_k_chunks = (int)ceil_div(k / (mxfp4 ? 32 : 16), 4);
  p.sfb_row_tiles = (int)ceil_div(n, 128);
  p.after_producer = after_producer ? 1 : 0;
  p.status = device_status_word();
  NVFP_REQUIRE(p.status != nullptr, "cannot locate the device status word");
  const PeerSync* ps = sync.world > 1 ? &sync : nullptr;
  if (value_dtype == NVFP_DTYPE_BF16)
    return mxfp4 ? launch_pair<true, __nv_bfloat16, kOutFp4Gather>(p, a, b, rotated, g->world, n_total, info.sm_count, stream, ps, &gq)
                 : launch_pair<false, __nv_bfloat16, kOutFp4Gather>(p, a, b, rotated, g->world, n_total, info.sm_count, stream, ps, &gq);
  return mxfp4 ? launch_pair<true, __half, kOutFp4Gather>(p, a, b, rotated, g->world, n_total, info.sm_count, stream, ps, &gq)
               : launch_pair<false, __half, kOutFp4Gather>(p, a, b, rotated, g->world, n_total, info.sm_count, stream, ps, &gq);
}
}  // namespace
}  // namespace nvfp

extern "C" int nvfp_scaled_fp4_mm_gather_fp4(const nvfp_peer_group_t* group, void* const* dst_sf, int64_t n_total,
                                             int64_t n_offset, const void* a, const void* b, const void* sfa,
                                             const void* sfb, const float* alpha, const void* bias,
                                             const float* out_global_scale, int64_t m, int64_t n, int64_t k,
                                             int value_dtype, int mxfp4, void* stream) {
  clear_error();
  return gather_fp4(group, dst_sf, n_total, n_offset, a, b, sfa, sfb, alpha, bias, out_global_scale, m, n, k, value_dtype,
                    mxfp4, static_cast<cudaStream_t>(stream), false);
}

extern "C" int nvfp_linear_forward_gather_fp4(const nvfp_peer_group_t* group, void* const* dst_sf, int64_t n_total,
                                              int64_t n_offset, const void* x, int64_t m, int64_t k, int64_t x_row_stride,
                                              int x_dtype, const void* w_fp4, const void* w_sf,
                                              const float* w_global_scale, int64_t n, const void* bias,
                                              const float* out_global_scale, void* workspace, uint32_t* scratch,
                                              int value_dtype, void* stream_) {
  clear_error();
  NVFP_REQUIRE(m > 0 && n > 0 && k > 0, "empty shape");
  NVFP_REQUIRE(k % 32 == 0, "Expected k to be divisible by 32, but got k: %lld.", (long long)k);
  NVFP_REQUIRE(x != nullptr && workspace != nullptr && scratch != nullptr && w_global_scale != nullptr, "null pointer");
  NVFP_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
  NVFP_REQUIRE(x_dtype == NVFP_DTYPE_F16 || x_dtype == NVFP_DTYPE_BF16,
               "Unsupported input data type for quantize_to_fp4 (dtype code %d).", x_dtype);
  NVFP_REQUIRE(x_row_stride >= k && x_row_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0,
               "activation must be 16-byte aligned with a row stride that is >= k and a multiple of 8 elements");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* a_fp4 = ws;
  uint8_t* a_sf = a_fp4 + round_up(m * (k / 2), 256);
  float* gs = reinterpret_cast<float*>(a_sf + round_up(nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(k, 16), 256));
  float* alpha = gs + 1;
  if (int rc = dynamic_fp4_quant_launch(a_fp4, a_sf, gs, alpha, scratch, x, m, k, x_row_stride, x_dtype, w_global_scale,
                                        /*release_next=*/true, nullptr, stream))
    return rc;
  return gather_fp4(group, dst_sf, n_total, n_offset, a_fp4, w_fp4, a_sf, w_sf, alpha, bias, out_global_scale, m, n, k,
                    value_dtype, 0, stream, /*after_producer=*/true);
}

extern "C" int nvfp_scaled_fp4_mm_scatter_add(void* const* dst, int n_dst, const void* a, const void* b,
                                              const void* sfa, const void* sfb, const float* alpha, int64_t m,
                                              int64_t n, int64_t k, int mxfp4, void* stream) {
  clear_error();
  return scatter_add(dst, n_dst, a, b, sfa, sfb, alpha, m, n, k, mxfp4, static_cast<cudaStream_t>(stream), nullptr);
}

extern "C" int nvfp_scaled_fp4_mm_gather(const nvfp_peer_group_t* group, int64_t dst_ld, const void* a, const void* b,
                                         const void* sfa, const void* sfb, const float* alpha, int64_t m, int64_t n,
                                         int64_t k, int out_dtype, int mxfp4, void* stream) {
  clear_error();
  void* rotated[kMaxOutputs];
  PeerSync sync;
  if (int rc = unpack_peer_group(group, rotated, &sync)) return rc;
  const PeerSync* ps = sync.world > 1 ? &sync : nullptr;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return mxfp4 ? scaled_mm<true>(rotated, group->world, dst_ld, a, b, sfa, sfb, alpha, m, n, k, out_dtype, st, nullptr, false,
                                 nullptr, nullptr, 0, false, ps)
               : scaled_mm<false>(rotated, group->world, dst_ld, a, b, sfa, sfb, alpha, m, n, k, out_dtype, st, nullptr, false,
                                  nullptr, nullptr, 0, false, ps);
}

extern "C" int nvfp_scaled_fp4_mm_reduce_scatter(const nvfp_peer_group_t* group, const void* a, const void* b,
                                                 const void* sfa, const void* sfb, const float* alpha, int64_t m,
                                                 int64_t n, int64_t k, int mxfp4, void* stream) {
  clear_error();
  void* rotated[kMaxOutputs];
  PeerSync sync;
  if (int rc = unpack_peer_group(group, rotated, &sync)) return rc;
  return scatter_add(group->dst, group->world, a, b, sfa, sfb, alpha, m, n, k, mxfp4, static_cast<cudaStream_t>(stream),
                     sync.world > 1 ? &sync : nullptr);
}

extern "C" int nvfp_linear_forward_gather(const nvfp_peer_group_t* group, int64_t dst_ld, const void* x, int64_t m,
                                          int64_t k, int64_t x_row_stride, int x_dtype, const void* w_fp4,
                                          const void* w_sf, const float* w_global_scale, int64_t n, void* workspace,
                                          uint32_t* scratch, int out_dtype, void* stream_) {
  clear_error();
  void* rotated[kMaxOutputs];
  PeerSync sync;
  if (int rc = unpack_peer_group(group, rotated, &sync)) return rc;
  NVFP_REQUIRE(m >= 0 && n >= 0 && k >= 0, "negative shape");
  NVFP_REQUIRE(k % 32 == 0, "Expected k to be divisible by 32, but got k: %lld.", (long long)k);
  if (m == 0 || n == 0) return NVFP_OK;
  NVFP_REQUIRE(x != nullptr && workspace != nullptr && scratch != nullptr && w_global_scale != nullptr, "null pointer");
  NVFP_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
  NVFP_REQUIRE(x_dtype == NVFP_DTYPE_F16 || x_dtype == NVFP_DTYPE_BF16,
               "Unsupported input data type for quantize_to_fp4 (dtype code %d).", x_dtype);
  NVFP_REQUIRE(x_row_stride >= k && x_row_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0,
               "activation must be 16-byte aligned with a row stride that is >= k and a multiple of 8 elements");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* a_fp4 = ws;
  uint8_t* a_sf = a_fp4 + round_up(m * (k / 2), 256);
  float* gs = reinterpret_cast<float*>(a_sf + round_up(nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(k, 16), 256));
  float* alpha = gs + 1;
  // same chain as nvfp_linear_forward: the GEMM comes up under the quantizer, fetches weights, announces ready to the
  // peers, and touches the activation operand only after the quantizer has finished
  if (int rc = dynamic_fp4_quant_launch(a_fp4, a_sf, gs, alpha, scratch, x, m, k, x_row_stride, x_dtype, w_global_scale,
                                        /*release_next=*/true, nullptr, stream))
    return rc;
  return scaled_mm<false>(rotated, group->world, dst_ld, a_fp4, w_fp4, a_sf, w_sf, alpha, m, n, k, out_dtype, stream, nullptr,
                          /*after_producer=*/true, nullptr, nullptr, 0, false, sync.world > 1 ? &sync : nullptr);
}

#ifdef NVFP_PAIR_TRACE
// Instrumented build only: copies the per-cluster clock counters of the last fp4_gemm_pair_kernel launches to the host
// (out: clusters x kTraceSlots uint64; see g_pair_trace) and clears them.
extern "C" int nvfp_debug_pair_trace(unsigned long long* out, int clusters) {
  clear_error();
  NVFP_REQUIRE(out != nullptr && clusters > 0 && clusters <= kTraceClusters, "bad trace request");
  NVFP_CUDA(cudaDeviceSynchronize());
  NVFP_CUDA(cudaMemcpyFromSymbol(out, g_pair_trace, sizeof(unsigned long long) * kTraceSlots * clusters));
  static unsigned long long zeros[kTraceClusters][kTraceSlots];
  NVFP_CUDA(cudaMemcpyToSymbol(g_pair_trace, zeros, sizeof(zeros)));
  return NVFP_OK;
}
#endif
