/*
 * nvfp_b200.h -- C ABI of libnvfp_b200.so: NVFP4 / MXFP4 quantize and block-scaled
 * FP4 GEMM for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes, enqueues its work on the
 * given CUDA stream (a cudaStream_t passed as void*; NULL = the legacy default
 * stream) of the CURRENT device and returns without synchronising.  The return value
 * is an nvfp_status_t; on failure nvfp_last_error() holds a message for the calling
 * thread.  Nothing here allocates device memory unless the comment on the function
 * says so.  The caller owns every buffer.
 *
 * Each declaration cites the interface of the reference implementation
 * (huweim/nvfp_kernel, paths relative to that project) that it replaces.
 */
#ifndef NVFP_B200_H_
#define NVFP_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  NVFP_OK = 0,
  NVFP_ERR_INVALID_ARGUMENT = 1, /* shape / dtype / alignment rejected on the host      */
  NVFP_ERR_CUDA = 2,             /* a CUDA runtime or driver call failed                 */
  NVFP_ERR_DEVICE_TIMEOUT = 3,   /* a bounded wait inside a kernel expired (see below)   */
  NVFP_ERR_UNSUPPORTED = 4       /* the current device is not sm_100                     */
} nvfp_status_t;

/* element types of 16-bit inputs / outputs */
#define NVFP_DTYPE_F16 0
#define NVFP_DTYPE_BF16 1
#define NVFP_DTYPE_F32 2 /* GEMM output only: unrounded partial sums for K-split layers */

/* MXFP4 scale rounding: exponent of amax/6 rounded up (no element saturates), or
 * truncated (the reference's disabled e8m0 branch, kernel/nvfp4_utils.cuh:196-202).
 * A block whose maximum is infinite gets the largest finite scale byte (254) when rounding
 * up and, like that branch, the raw exponent bits (255, the e8m0 NaN code) when truncating;
 * its elements become zeros (finite ones) and the largest e2m1 code (infinite ones) either way.
 * NaN elements do not take part in a block's maximum; a block of nothing but NaNs gets 255. */
#define NVFP_MX_ROUND_CEIL 0
#define NVFP_MX_ROUND_FLOOR 1

/* Message describing the last failure on the calling thread ("" if none). */
const char* nvfp_last_error(void);

/* Library / ABI version (major*1000 + minor). */
int nvfp_version(void);

/* Number of padded scale rows / columns for a [rows, k] operand:
 *   rows_padded = round_up(rows, 128), cols_padded = round_up(k / block, 4)
 * (nvfp/_ops_real.py:48-54 and kernel/nvfp4_scaled_mm_sm120_kernels.cu:254-259). */
int64_t nvfp_sf_rows_padded(int64_t rows);
int64_t nvfp_sf_cols_padded(int64_t k, int block);

/*
 * NVFP4 quantizer.  Replaces scaled_fp4_quant_sm1xxa (kernel/nvfp4_quant.h:4-7,
 * kernel/nvfp4_quant_kernels.cu:69-99) and its kernel cvt_fp16_to_fp4
 * (kernel/nvfp4_utils.cuh:245-280); results are bit-identical to it.
 *
 *   in            [m, n] fp16 / bf16, row stride in_row_stride elements (>= n, multiple of 8),
 *                 base 16-byte aligned, n % 16 == 0
 *   global_scale  device pointer to one fp32 (NULL = 1.0f, kernel/nvfp4_utils.cuh:258)
 *   out_fp4       [m, n/2] bytes, element 2j in the low nibble of byte j
 *   out_sf        round_up(m,128) x round_up(n/16,4) ue4m3 bytes in the swizzled
 *                 [mTile][kTile][32][4][4] layout (kernel/nvfp4_utils.cuh:126-153).
 *                 Unlike the reference, padding bytes are written (as 0).
 */
int nvfp_scaled_fp4_quant(void* out_fp4, void* out_sf, const void* in, const float* global_scale,
                          int64_t m, int64_t n, int64_t in_row_stride, int in_dtype, void* stream);

/*
 * MXFP4 quantizer: 32-element blocks, ue8m0 scales in the same swizzled layout
 * (round_up(m,128) x round_up(n/32,4) bytes), no global scale.  n % 32 == 0.
 * The reference has no reachable counterpart; the closest code is the UE8M0_SF
 * template branch at kernel/nvfp4_utils.cuh:196-202 (16-element blocks, disabled at
 * kernel/nvfp4_quant_kernels.cu:90-91).
 */
int nvfp_mxfp4_quant(void* out_fp4, void* out_sf, const void* in, int64_t m, int64_t n,
                     int64_t in_row_stride, int in_dtype, int rounding, void* stream);

/*
 * Block-scaled FP4 GEMM  D[m,n] = alpha * sum_k (A*sfa)[m,k] * (B*sfb)[n,k], fp32
 * accumulation, fp16 / bf16 output.  Replaces cutlass_scaled_fp4_mm
 * (kernel/nvfp4_scaled_mm_entry.h:4-7, kernel/nvfp4_scaled_mm_entry.cu:23-36) and the
 * CUTLASS instantiation behind it (kernel/nvfp4_scaled_mm_sm120_kernels.cu:72-294),
 * with the same argument checks: k % 32 == 0, n % 32 == 0, contiguous operands.
 *
 *   a    [m, k/2] packed e2m1, b [n, k/2] packed e2m1 (weights are [N, K], K-major)
 *   sfa  round_up(m,128) x round_up(k/16,4) ue4m3, swizzled; sfb likewise for n.
 *        When k is not a multiple of 64 the last MMA covers scale columns past k/16: their operand bytes read as
 *        zero, so those scale bytes must be zero or at least finite (0x7F / 0xFF would turn 0 * scale into NaN).
 *        The quantizers here write every padding byte as 0; for scale tensors produced elsewhere use
 *        nvfp_kernel_b200.sharding.zero_scale_padding once, at load time.
 *   alpha device pointer to one fp32, read by the kernel's epilogue
 *   d    [m, n] out_dtype (fp16 / bf16 as in the reference, or fp32), row-major,
 *        16-byte aligned
 */
int nvfp_scaled_fp4_mm(void* d, const void* a, const void* b, const void* sfa, const void* sfb,
                       const float* alpha, int64_t m, int64_t n, int64_t k, int out_dtype,
                       void* stream);

/* Same for MXFP4 operands: 32-element blocks, ue8m0 scales
 * (round_up(rows,128) x round_up(k/32,4)), k % 64 == 0.  alpha may be NULL (= 1).
 * No counterpart in the reference (see nvfp_mxfp4_quant). */
int nvfp_mxfp4_mm(void* d, const void* a, const void* b, const void* sfa, const void* sfb,
                  const float* alpha, int64_t m, int64_t n, int64_t k, int out_dtype, void* stream);

/*
 * The same product with a bias added in the epilogue: D = alpha * acc + bias[n], rounded once to the output type
 * (the reference adds a bias, when a layer has one, in a separate pass over D; no counterpart there).
 *   bias   device, n values of the OUTPUT type (fp16 / bf16 / fp32), 16-byte aligned; NULL = no bias
 *   mxfp4  0: NVFP4 operands (as nvfp_scaled_fp4_mm), 1: MXFP4 operands (as nvfp_mxfp4_mm; alpha may be NULL)
 */
int nvfp_scaled_fp4_mm_bias(void* d, const void* a, const void* b, const void* sfa, const void* sfb,
                            const float* alpha, const void* bias, int64_t m, int64_t n, int64_t k,
                            int out_dtype, int mxfp4, void* stream);

/*
 * The product written as NVFP4: alpha * acc (+ bias) is rounded to value_dtype (fp16 or bf16) and quantized in the
 * GEMM epilogue with the global scale out_global_scale[0], bit for bit what nvfp_scaled_fp4_mm(_bias) followed by
 * nvfp_scaled_fp4_quant(out, out_global_scale) would produce, without the [m, n] tensor ever reaching memory.  For a
 * next layer whose activation scale is known beforehand (calibrated); no counterpart in the reference.
 *   d_fp4  device, [m, n/2] bytes, 16-byte aligned
 *   d_sf   device, nvfp_sf_rows_padded(m) x nvfp_sf_cols_padded(n, 16) bytes in the swizzled layout; padding zero
 *   bias   n values of value_dtype or NULL;  mxfp4 selects the INPUT operand format as in nvfp_scaled_fp4_mm_bias
 */
int nvfp_scaled_fp4_mm_fp4out(void* d_fp4, void* d_sf, const void* a, const void* b, const void* sfa, const void* sfb,
                              const float* alpha, const void* bias, const float* out_global_scale, int64_t m,
                              int64_t n, int64_t k, int value_dtype, int mxfp4, void* stream);

/*
 * Gate/up projection of a gated MLP with the activation in the epilogue.  b holds the two projections' rows
 * interleaved in groups of 16: rows [32g, 32g+16) are gate rows 16g.., rows [32g+16, 32g+32) the matching up rows
 * (quantized as ONE tensor, after interleaving).  Per row and group the epilogue forms v = alpha * acc (+ bias)
 * rounded to value_dtype, then out[16g + i] = value_dtype(value_dtype(silu(v_gate[i])) * v_up[i]), silu in fp32:
 * what a framework computes with silu(gate) * up on fp16 / bf16 tensors.  The [m, n] product never reaches memory.
 *   out_global_scale NULL: d receives [m, n/2] values of value_dtype; d_sf is ignored
 *   out_global_scale set:  the [m, n/2] result is quantized to NVFP4 as by nvfp_scaled_fp4_quant(result,
 *                          out_global_scale): d receives [m, n/4] packed bytes, d_sf the swizzled scales of an
 *                          [m, n/2] tensor -- the down projection's activation operand
 *   bias  n values of value_dtype in the interleaved order, or NULL.  No counterpart in the reference.
 */
int nvfp_scaled_fp4_mm_silu_mul(void* d, void* d_sf, const void* a, const void* b, const void* sfa, const void* sfb,
                                const float* alpha, const void* bias, const float* out_global_scale, int64_t m,
                                int64_t n, int64_t k, int value_dtype, int mxfp4, void* stream);

/*
 * One call for the forward of an NVFP4 linear layer with online activation quantization, the reference's
 * FP4GemmWithOnlineActivation.forward (speed_test.py:43-50): d = (1 / (gs_x * gs_w)) * quant(x) @ w^T (+ bias) with
 * gs_x = rcp(max|x|) * 2688.  Same bytes as nvfp_dynamic_fp4_quant followed by nvfp_scaled_fp4_mm_bias.  For few
 * rows (the shapes that take the one-pass quantizer and the few-rows GEMM) the GEMM is launched with programmatic
 * stream serialization: it streams its weights while the quantizer still runs and touches the activation operand
 * only after the quantizer has finished.
 *   x          device, [m, k] fp16 / bf16, row stride x_row_stride elements, 16-byte aligned
 *   w_fp4/w_sf the weight as nvfp_scaled_fp4_quant produced it ([n, k/2] and its swizzled scales); must be complete
 *              before this call's stream position is reached (it is read before the quantizer finishes)
 *   w_global_scale  device fp32, the weight's global scale
 *   bias       n values of the output type or NULL
 *   workspace  device, nvfp_linear_workspace_bytes(m, k) bytes, 256-byte aligned: quantized activation, its scales,
 *              gs_x and alpha; contents are dead after the call's kernels have run
 *   scratch    eight uint32 zeroed once, as for nvfp_activation_scales
 */
int64_t nvfp_linear_workspace_bytes(int64_t m, int64_t k);
int nvfp_linear_forward(void* d, const void* x, int64_t m, int64_t k, int64_t x_row_stride, int x_dtype,
                        const void* w_fp4, const void* w_sf, const float* w_global_scale, int64_t n,
                        const void* bias, void* workspace, uint32_t* scratch, int out_dtype, void* stream);

/*
 * Chains of layers: the global scale a layer's quantizer needs (2688 / max|x|) is the global scale of the tensor the
 * layer BEFORE it wrote, so that layer's GEMM can form it in its epilogue and the consumer skips its pass over x
 * (the reference spends abs().max() and a division per layer on it, speed_test.py:46-47).
 *
 * nvfp_scaled_fp4_mm_amax: nvfp_scaled_fp4_mm_bias that also writes
 *   d_global_scale_out[0] = rcp(max|d|) * 2688 over the [m, n] fp16 / bf16 values it stored (the value
 *                           nvfp_global_scale(d) would give; NaNs are ignored by the maximum), and, when
 *   next_weight_global_scale is given, next_alpha_out[0] = 1 / (d_global_scale_out[0] * next_weight_global_scale[0]).
 *   scratch  eight uint32 zeroed once, self-cleaning, as for nvfp_activation_scales; NOT the buffer a quantizer
 *            launched before this GEMM in the same call chain uses
 *
 * nvfp_linear_forward_chained: nvfp_linear_forward with both ends of the chain open:
 *   x_global_scale  device fp32 or NULL.  Given: x is quantized with it (no pass for the maximum) and the GEMM forms
 *                   alpha = 1 / (x_global_scale * w_global_scale) itself.  NULL: dynamic, as nvfp_linear_forward
 *                   (scratch needed).
 *   d_global_scale_out / d_scale_scratch / next_weight_global_scale / next_alpha_out  as above, or NULL: not wanted.
 * Same bytes as the separate calls nvfp_global_scale -> nvfp_scaled_fp4_quant -> nvfp_scaled_fp4_mm_bias.
 */
int nvfp_scaled_fp4_mm_amax(void* d, const void* a, const void* b, const void* sfa, const void* sfb, const float* alpha,
                            const void* bias, int64_t m, int64_t n, int64_t k, int out_dtype, int mxfp4,
                            float* d_global_scale_out, uint32_t* scratch, const float* next_weight_global_scale,
                            float* next_alpha_out, void* stream);
int nvfp_linear_forward_chained(void* d, const void* x, int64_t m, int64_t k, int64_t x_row_stride, int x_dtype,
                                const float* x_global_scale, const void* w_fp4, const void* w_sf,
                                const float* w_global_scale, int64_t n, const void* bias, void* workspace,
                                uint32_t* scratch, int out_dtype, float* d_global_scale_out, uint32_t* d_scale_scratch,
                                const float* next_weight_global_scale, float* next_alpha_out, void* stream);

/*
 * One call for a gated MLP with NVFP4 weights, y = down(silu(gate(x)) * up(x)): the quantizer of x, the gate/up GEMM
 * with the activation and the NVFP4 quantization of its result in the epilogue (nvfp_scaled_fp4_mm_silu_mul), and
 * the down GEMM, chained with programmatic dependent launch: each GEMM comes up while the kernel before it still
 * runs, streams its WEIGHTS meanwhile and touches what that kernel writes only after it has finished.  Same bytes as
 * the three separate calls.  No counterpart in the reference (its FP4GemmWithOnlineActivation, speed_test.py:36-50,
 * is one layer).
 *   x             device, [m, hidden] fp16 / bf16, row stride x_row_stride elements, 16-byte aligned
 *   gate_up_fp4/sf  [2 * inter, hidden / 2] and swizzled scales: gate and up rows interleaved in groups of 16,
 *                 quantized as one tensor with global scale gate_up_global_scale
 *   down_fp4/sf   [n_out, inter / 2] and swizzled scales
 *   act_global_scale  device fp32, the (calibrated) global scale of silu(gate) * up
 *   down_alpha    device fp32, 1 / (act_global_scale * global scale of the down weight)
 *   y             device, [m, n_out] of out_dtype (fp16 or bf16, also the type the hidden activation is rounded to)
 *   workspace     device, nvfp_gated_mlp_workspace_bytes(m, hidden, inter) bytes, 256-byte aligned; dead afterwards
 *   scratch       eight uint32 zeroed once, as for nvfp_activation_scales
 * All weights and scales must be complete before this call's stream position is reached.
 */
int64_t nvfp_gated_mlp_workspace_bytes(int64_t m, int64_t hidden, int64_t inter);
int nvfp_gated_mlp_forward(void* y, const void* x, int64_t m, int64_t hidden, int64_t x_row_stride, int x_dtype,
                           const void* gate_up_fp4, const void* gate_up_sf, const float* gate_up_global_scale,
                           int64_t inter, const void* down_fp4, const void* down_sf, const float* act_global_scale,
                           const float* down_alpha, int64_t n_out, void* workspace, uint32_t* scratch,
                           int out_dtype, void* stream);

/*
 * The same GEMM with the [m, n] result written to n_dst (1..8) destinations instead of one, each a
 * row-major matrix with leading dimension dst_ld elements (>= n, multiple of 8), so that a slab can land
 * directly in its columns of a wider gathered matrix: dst[0] is
 * normally local memory, the others point into PEER GPUs' memory (peer-mapped addresses, e.g. of a
 * symmetric buffer).  This is the column-parallel layer's all-gather fused into the GEMM epilogue:
 * every output tile leaves shared memory once per destination as a TMA store, over NVLink for peers,
 * while the next tile is being computed.  The caller synchronises the ranks around the call (nobody
 * may still read a destination when the call starts; readers wait until every writer's stream has
 * passed the call).  mxfp4 != 0 selects 32-element blocks with ue8m0 scales.  The reference has no
 * distributed code; there is no counterpart.
 */
int nvfp_scaled_fp4_mm_multi(void* const* dst, int n_dst, const void* a, const void* b, const void* sfa,
                             const void* sfb, const float* alpha, int64_t m, int64_t n, int64_t k,
                             int64_t dst_ld, int out_dtype, int mxfp4, void* stream);

/*
 * Row-parallel (K-split) layers: this rank's GEMM yields a PARTIAL [m, n] product; destination r
 * (r = 0..n_dst-1, a [m / n_dst, n] fp32 matrix in rank r's memory, peer-mapped for r != own rank)
 * owns rows [r*m/n_dst, (r+1)*m/n_dst) of the sum.  The epilogue adds every 32-row block of the
 * partial product into its owner's matrix with a TMA reduction (fp32 add at the destination's memory,
 * over NVLink for peers): the reduce-scatter fused into the GEMM.  The caller zeroes the destinations
 * and synchronises the ranks before the call, and again before reading.  m % (32 * n_dst) == 0.
 * No counterpart in the reference.
 */
int nvfp_scaled_fp4_mm_scatter_add(void* const* dst, int n_dst, const void* a, const void* b, const void* sfa,
                                   const void* sfb, const float* alpha, int64_t m, int64_t n, int64_t k,
                                   int mxfp4, void* stream);

/*
 * Tensor-parallel layers with the ranks synchronised INSIDE the GEMM kernel.  The two entry points above leave it to
 * the caller to synchronise the ranks before and after the call (two collectives or barrier kernels per layer); the
 * ones below need nothing around them.  The reference has no distributed code; there is no counterpart.
 *
 * A peer group describes the ranks (one process per GPU, 2..8 GPUs of one node) as THIS rank sees them:
 *   dst[r]    rank r's destination matrix, mapped into this process (peer-mapped for r != rank)
 *   flags[r]  rank r's flag block: NVFP_PEER_FLAG_WORDS uint32, 128-byte aligned, peer-mapped like dst, zeroed ONCE
 *             (with all ranks synchronised on the host afterwards) and then owned by the library: ready / done
 *             announcements and a call counter.  Each destination buffer has its own flag block.  All NULL: no
 *             in-kernel synchronisation, the caller synchronises as for the entry points above.
 *   wait_limit_ns  bound of every in-kernel wait on a peer's flag; 0 = two seconds.
 * Protocol: the kernel announces "ready" to every peer when it starts (nothing on this rank reads this rank's
 * destination any more: every earlier reader precedes the call in stream order); it writes into a peer's destination
 * only after that peer's ready; when its last store has been performed it announces "done" and waits for every
 * peer's done, so that when the kernel has finished, this rank's destination holds every rank's contribution.  All
 * ranks must make the same sequence of calls on a flag block.  A wait that exceeds the limit (a peer that is late
 * or gone) sets bit 5 (0x20) of the device status word; the kernel then skips its stores to peers (if it was a
 * ready wait) and returns: the call's result is incomplete, nothing hangs, and the next call works again once
 * the peer is back.
 */
#define NVFP_MAX_RANKS 8
#define NVFP_PEER_FLAG_WORDS 32
typedef struct {
  int world;
  int rank;
  void* dst[NVFP_MAX_RANKS];
  uint32_t* flags[NVFP_MAX_RANKS];
  uint64_t wait_limit_ns;
} nvfp_peer_group_t;

/*
 * Column-parallel layer, all-gather fused into the GEMM: this rank's [m, n] product is stored into every rank's
 * gathered matrix.  group->dst[r]: where this rank's slab starts in rank r's [m, dst_ld] row-major matrix (that is,
 * base + rank * n elements), 16-byte aligned; dst_ld >= n, a multiple of 8.  Otherwise as nvfp_scaled_fp4_mm_multi.
 */
int nvfp_scaled_fp4_mm_gather(const nvfp_peer_group_t* group, int64_t dst_ld, const void* a, const void* b,
                              const void* sfa, const void* sfb, const float* alpha, int64_t m, int64_t n, int64_t k,
                              int out_dtype, int mxfp4, void* stream);

/*
 * Row-parallel (K-split) layer, reduce-scatter fused into the GEMM: group->dst[r] is rank r's [m / world, n] fp32
 * matrix, which owns rows [r*m/world, (r+1)*m/world) of the sum and must be zero when rank r's call starts (zero it
 * on the same stream before the call: the kernel announces ready after that).  Otherwise as
 * nvfp_scaled_fp4_mm_scatter_add.
 */
int nvfp_scaled_fp4_mm_reduce_scatter(const nvfp_peer_group_t* group, const void* a, const void* b, const void* sfa,
                                      const void* sfb, const float* alpha, int64_t m, int64_t n, int64_t k, int mxfp4,
                                      void* stream);

/*
 * nvfp_linear_forward for a column-parallel layer with the fused gather: quantizer and GEMM chained in one call, the
 * GEMM's tiles stored into every rank's gathered matrix (group->dst as for nvfp_scaled_fp4_mm_gather).  workspace and
 * scratch as for nvfp_linear_forward.
 */
int nvfp_linear_forward_gather(const nvfp_peer_group_t* group, int64_t dst_ld, const void* x, int64_t m, int64_t k,
                               int64_t x_row_stride, int x_dtype, const void* w_fp4, const void* w_sf,
                               const float* w_global_scale, int64_t n, void* workspace, uint32_t* scratch,
                               int out_dtype, void* stream);

/*
 * Column-parallel layer whose gathered output is the NEXT layer's NVFP4 activation operand: every tile is quantized in
 * the epilogue (as nvfp_scaled_fp4_mm_fp4out does, same bytes) and its packed nibbles and scale bytes are stored into
 * every rank's gathered operand: 0.5625 bytes per element cross NVLink instead of 2.
 *   group->dst[r]  BASE of rank r's packed matrix, [m, n_total / 2] bytes, 16-byte aligned
 *   dst_sf[r]      base of rank r's scale tensor, nvfp_sf_rows_padded(m) x (n_total / 16) bytes in the swizzled layout
 *                  of an [m, n_total] tensor; rows between m and the padded row count receive zeros
 *   n_offset       first column of this rank's [m, n] slab in the gathered matrix; n, n_offset and n_total are
 *                  multiples of 64 (whole 512-byte scale chunks per rank)
 *   out_global_scale  device fp32: the (calibrated) global scale of the gathered tensor, the same on every rank
 *   bias           n values of value_dtype (fp16 / bf16) or NULL
 * Synchronisation of the ranks as for nvfp_scaled_fp4_mm_gather.  No counterpart in the reference.
 */
int nvfp_scaled_fp4_mm_gather_fp4(const nvfp_peer_group_t* group, void* const* dst_sf, int64_t n_total, int64_t n_offset,
                                  const void* a, const void* b, const void* sfa, const void* sfb, const float* alpha,
                                  const void* bias, const float* out_global_scale, int64_t m, int64_t n, int64_t k,
                                  int value_dtype, int mxfp4, void* stream);

/* The same behind the online activation quantizer, chained in one call (cf. nvfp_linear_forward_gather). */
int nvfp_linear_forward_gather_fp4(const nvfp_peer_group_t* group, void* const* dst_sf, int64_t n_total, int64_t n_offset,
                                   const void* x, int64_t m, int64_t k, int64_t x_row_stride, int x_dtype,
                                   const void* w_fp4, const void* w_sf, const float* w_global_scale, int64_t n,
                                   const void* bias, const float* out_global_scale, void* workspace, uint32_t* scratch,
                                   int value_dtype, void* stream);

/*
 * y[i] = rcp.approx.ftz.f32(x[i]).  Replaces reciprocal_approximate_ftz_tensor
 * (kernel/reciprocal_kernels.h:4-5, kernel/reciprocal_kernels.cu:91-121); fp32 only,
 * the one dtype reachable through the reference's Python wrapper (nvfp/ops.py:87-92).
 */
int nvfp_reciprocal_approximate_ftz(float* out, const float* in, int64_t count, void* stream);

/*
 * Per-tensor global scale  gs = rcp(max|x|) * (448 * 6)  (both steps correctly rounded fp32,
 * which is how torch evaluates `2688 / amax`) as one fp32 on the device.
 * Replaces the torch sequence abs().max() -> 2688/amax of speed_test.py:40-41,46-47
 * and nvfp/pseudo_quant.py:94-96 with one kernel (the last block to finish forms the scale) and no temporary.
 *   amax_bits  device scratch, TWO uint32 (8 bytes, 8-byte aligned); the call resets them on the stream
 *              first; afterwards word 0 holds the bit pattern of max|x| as fp32.
 *   gs_out     device, one fp32; amax == 0 gives gs = 2688 (amax treated as 1,
 *              as in test_refactor.py:21-25).  Like torch.abs(x).max(), the maximum is NaN when any
 *              element is NaN (gs = NaN) and infinite when one is infinite (gs = 0); so are the scales of
 *              nvfp_activation_scales, nvfp_dynamic_fp4_quant and nvfp_scaled_fp4_mm_amax.
 */
int nvfp_global_scale(float* gs_out, uint32_t* amax_bits, const void* in, int64_t m, int64_t n,
                      int64_t in_row_stride, int in_dtype, void* stream);

/*
 * One launch for everything the activation side of a layer needs before quantizing (the reference
 * spends 4-5 launches on it, speed_test.py:46-49): gs_out = rcp(max|x|) * 2688 and
 * alpha_out = 1 / (gs_out * gs_weight[0]).
 *   scratch  EIGHT uint32 (32 bytes), zeroed ONCE by the caller before the first use and then left
 *            alone: the kernel keeps two (maximum, counter) pairs and a toggle in it and cleans up
 *            after itself, so no memset runs between calls.  Calls sharing a scratch must be ordered
 *            on one stream.
 */
int nvfp_activation_scales(float* gs_out, float* alpha_out, uint32_t* scratch, const void* in, int64_t m,
                           int64_t n, int64_t in_row_stride, int in_dtype, const float* gs_weight, void* stream);

/*
 * Dynamic per-tensor NVFP4 quantization in one pass: gs_out = rcp(max|x|) * 2688 of THIS tensor, the tensor
 * quantized with it exactly as nvfp_scaled_fp4_quant would (same bytes), and, when gs_weight is given,
 * alpha_out = 1 / (gs_out * gs_weight[0]).  Replaces the reference's abs().max() -> division -> quantize chain
 * (speed_test.py:46-48) and reads the tensor once: decode-sized tensors (up to 128 rows, a few thousand 16-element
 * blocks) are handled by one cluster of CTAs that exchange their maxima through shared memory; while the tensor has
 * no more 128 x 128 tiles than two per SM (296 on a B200: 4.8 M elements), one cooperative launch keeps every tile in
 * registers across the reduction of the maximum; larger tensors take the global-scale launch followed by the
 * quantize launch.
 *   scratch   as for nvfp_activation_scales (eight uint32 zeroed once; may be the same buffer)
 *   gs_weight device fp32 or NULL; alpha_out may be NULL when gs_weight is
 * A CTA that waits more than two seconds for the others gives up, sets bit 8 of the device status word
 * (nvfp_device_status) and quantizes with the maximum it has seen.
 */
int nvfp_dynamic_fp4_quant(void* out_fp4, void* out_sf, float* gs_out, float* alpha_out, uint32_t* scratch,
                           const void* in, int64_t m, int64_t n, int64_t in_row_stride, int in_dtype,
                           const float* gs_weight, void* stream);

/*
 * Same result as nvfp_global_scale, for callers that cannot hand over scratch memory because
 * they may not allocate any: code running under an engine whose device allocator is closed
 * after warm-up, or on host threads where cudaMalloc is forbidden.  No counterpart in the
 * reference.  The amax word lives in a 256-byte array inside the library (held by every GPU
 * that loads it, until exit); the call allocates nothing and calls no allocating routine.
 *   - tensors of more than 2^32 elements are rejected (NVFP_ERR_INVALID_ARGUMENT);
 *   - the first call on each device looks the array's address up (cudaGetSymbolAddress) and, under lazy module
 *     loading, that look-up or the first launch may load the module and allocate its globals: make the first
 *     call during warm-up, before the allocator is closed and before any stream capture.  Later calls
 *     allocate nothing;
 *   - all calls on a device share the array: the call clears the word it uses on its stream,
 *     but two calls that overlap on the GPU (different streams) race.  Serialise them.
 */
int nvfp_global_scale_noalloc(float* gs_out, const void* in, int64_t m, int64_t n,
                              int64_t in_row_stride, int in_dtype, void* stream);

/* alpha_out[0] = 1 / (gs_a[0] * gs_b[0]) in fp32 on the device (speed_test.py:49). */
int nvfp_alpha_from_scales(float* alpha_out, const float* gs_a, const float* gs_b, void* stream);

/*
 * Kernels here never spin without a limit: a wait on an mbarrier that does not
 * complete within about two seconds makes the kernel record a code in a per-device
 * status word and return.  This call synchronises the current device, reads and
 * clears that word: *status_out == 0 means no kernel gave up since the last call.
 * Returns NVFP_ERR_DEVICE_TIMEOUT when the word was non-zero.
 */
int nvfp_device_status(uint32_t* status_out);

/*
 * Exercises that path without any failure: one thread of a one-CTA kernel waits on an mbarrier nobody arrives
 * at, gives up after limit_ns (1 ns .. 100 ms), records bit 16 in the status word and the kernel returns
 * normally.  nvfp_device_status then reports NVFP_ERR_DEVICE_TIMEOUT with that bit and clears the word.  For tests of
 * the error plumbing; the context stays usable.
 */
int nvfp_selftest_wait_timeout(uint64_t limit_ns, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NVFP_B200_H_ */
