// Torch extension module `scaled_fp4_ops`: the three entry points the reference's
// binding.cpp:10-17 exports (same names, argument order and checks), plus the MXFP4 and
// helper entry points, each a thin wrapper over the C ABI of libnvfp_b200.so.  No device
// code lives here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "../../include/nvfp_b200.h"

namespace {

void* current_stream(const torch::Tensor& t) {
  return static_cast<void*>(at::cuda::getCurrentCUDAStream(t.get_device()).stream());
}

void check_status(int rc) {
  if (rc == NVFP_OK) return;
  if (rc == NVFP_ERR_UNSUPPORTED) TORCH_CHECK_NOT_IMPLEMENTED(false, nvfp_last_error());
  TORCH_CHECK(false, nvfp_last_error());
}

int dtype_code(const torch::Tensor& t, const char* what) {
  if (t.scalar_type() == at::ScalarType::Half) return NVFP_DTYPE_F16;
  if (t.scalar_type() == at::ScalarType::BFloat16) return NVFP_DTYPE_BF16;
  TORCH_CHECK(false, what);
  return -1;
}

#define CHECK_OPERAND(x, st, name)                                      \
  TORCH_CHECK((x).is_cuda(), name, " must be a CUDA tensor");           \
  TORCH_CHECK((x).is_contiguous(), name, " must be contiguous");        \
  TORCH_CHECK((x).scalar_type() == (st), "Inconsistency of Tensor type: ", name)

int64_t round_up(int64_t x, int64_t y) { return (x + y - 1) / y * y; }

// kernel/nvfp4_quant_kernels.cu:69-99 of the reference.
void scaled_fp4_quant_sm1xxa(torch::Tensor const& output, torch::Tensor const& input,
                             torch::Tensor const& output_sf, torch::Tensor const& input_sf) {
  TORCH_CHECK(input.dim() == 2, "input must be a matrix");
  const int64_t m = input.size(0), n = input.size(1);
  TORCH_CHECK(n % 16 == 0, "The N dimension must be multiple of 16.");
  const int dt = dtype_code(input, "Unsupported input data type for quantize_to_fp4.");
  TORCH_CHECK(input.is_cuda() && output.is_cuda() && output_sf.is_cuda() && input_sf.is_cuda(),
              "all tensors must be CUDA tensors");
  TORCH_CHECK(input.stride(1) == 1, "input rows must be dense");
  TORCH_CHECK(output.is_contiguous() && output_sf.is_contiguous(), "outputs must be contiguous");
  TORCH_CHECK(output.numel() * output.element_size() >= m * n / 2, "output too small");
  TORCH_CHECK(output_sf.numel() * output_sf.element_size() >= round_up(m, 128) * round_up(n / 16, 4),
              "output_sf too small");
  TORCH_CHECK(input_sf.scalar_type() == at::ScalarType::Float, "input_sf must be fp32");
  const at::cuda::OptionalCUDAGuard guard(device_of(input));
  check_status(nvfp_scaled_fp4_quant(output.data_ptr(), output_sf.data_ptr(), input.data_ptr(),
                                     static_cast<const float*>(input_sf.data_ptr()), m, n,
                                     m > 1 ? input.stride(0) : n, dt, current_stream(input)));
}

void scaled_mxfp4_quant(torch::Tensor const& output, torch::Tensor const& input,
                        torch::Tensor const& output_sf, int64_t rounding) {
  TORCH_CHECK(input.dim() == 2, "input must be a matrix");
  const int64_t m = input.size(0), n = input.size(1);
  TORCH_CHECK(n % 32 == 0, "The N dimension must be multiple of 32.");
  const int dt = dtype_code(input, "Unsupported input data type for quantize_to_fp4.");
  TORCH_CHECK(input.is_cuda() && output.is_cuda() && output_sf.is_cuda(), "all tensors must be CUDA tensors");
  TORCH_CHECK(input.stride(1) == 1, "input rows must be dense");
  TORCH_CHECK(output.is_contiguous() && output_sf.is_contiguous(), "outputs must be contiguous");
  TORCH_CHECK(output.numel() * output.element_size() >= m * n / 2, "output too small");
  TORCH_CHECK(output_sf.numel() * output_sf.element_size() >= round_up(m, 128) * round_up(n / 32, 4),
              "output_sf too small");
  const at::cuda::OptionalCUDAGuard guard(device_of(input));
  check_status(nvfp_mxfp4_quant(output.data_ptr(), output_sf.data_ptr(), input.data_ptr(), m, n,
                                m > 1 ? input.stride(0) : n, dt, (int)rounding, current_stream(input)));
}

// Argument checks of kernel/nvfp4_scaled_mm_sm120_kernels.cu:222-273 of the reference.
void scaled_mm_impl(torch::Tensor& D, torch::Tensor const& A, torch::Tensor const& B,
                    torch::Tensor const& A_sf, torch::Tensor const& B_sf,
                    c10::optional<torch::Tensor> const& alpha, bool mx,
                    c10::optional<torch::Tensor> const& bias = c10::nullopt) {
  const auto sf_dtype = mx ? at::ScalarType::Float8_e8m0fnu : at::ScalarType::Float8_e4m3fn;
  CHECK_OPERAND(A, at::ScalarType::Byte, "a");
  CHECK_OPERAND(B, at::ScalarType::Byte, "b");
  CHECK_OPERAND(A_sf, sf_dtype, "scale_a");
  CHECK_OPERAND(B_sf, sf_dtype, "scale_b");
  if (alpha.has_value()) { CHECK_OPERAND(*alpha, at::ScalarType::Float, "alpha"); }
  TORCH_CHECK(mx || alpha.has_value(), "alpha is required");
  TORCH_CHECK(D.is_cuda() && D.is_contiguous(), "out must be a contiguous CUDA tensor");
  TORCH_CHECK(A.dim() == 2, "a must be a matrix");
  TORCH_CHECK(B.dim() == 2, "b must be a matrix");
  TORCH_CHECK(A.sizes()[1] == B.sizes()[1], "a and b shapes cannot be multiplied (", A.sizes()[0], "x",
              A.sizes()[1], " and ", B.sizes()[0], "x", B.sizes()[1], ")");
  const int64_t m = A.sizes()[0], n = B.sizes()[0], k = A.sizes()[1] * 2;
  const int64_t alignment = mx ? 64 : 32, block = mx ? 32 : 16;
  TORCH_CHECK(k % alignment == 0, "Expected k to be divisible by ", alignment, ", but got a shape: (",
              A.sizes()[0], "x", A.sizes()[1], "), k: ", k, ".");
  TORCH_CHECK(n % 32 == 0, "Expected n to be divisible by 32, but got b shape: (", B.sizes()[0], "x",
              B.sizes()[1], ").");
  const int64_t rounded_m = round_up(m, 128), rounded_n = round_up(n, 128), rounded_k = round_up(k / block, 4);
  TORCH_CHECK(A_sf.dim() == 2, "scale_a must be a matrix");
  TORCH_CHECK(B_sf.dim() == 2, "scale_b must be a matrix");
  TORCH_CHECK(A_sf.sizes()[1] == B_sf.sizes()[1], "scale_a and scale_b shapes cannot be multiplied (",
              A_sf.sizes()[0], "x", A_sf.sizes()[1], " and ", B_sf.sizes()[0], "x", B_sf.sizes()[1], ")");
  TORCH_CHECK(A_sf.sizes()[0] == rounded_m && A_sf.sizes()[1] == rounded_k,
              "scale_a must be padded and swizzled to a shape (", rounded_m, "x", rounded_k,
              "), but got a shape (", A_sf.sizes()[0], "x", A_sf.sizes()[1], ")");
  TORCH_CHECK(B_sf.sizes()[0] == rounded_n && B_sf.sizes()[1] == rounded_k,
              "scale_b must be padded and swizzled to a shape (", rounded_n, "x", rounded_k,
              "), but got a shape (", B_sf.sizes()[0], "x", B_sf.sizes()[1], ")");
  TORCH_CHECK(D.dim() == 2 && D.sizes()[0] == m && D.sizes()[1] == n, "out must have shape (", m, "x", n, ")");
  int dt;
  if (D.scalar_type() == at::ScalarType::BFloat16) dt = NVFP_DTYPE_BF16;
  else if (D.scalar_type() == at::ScalarType::Half) dt = NVFP_DTYPE_F16;
  else if (D.scalar_type() == at::ScalarType::Float) dt = NVFP_DTYPE_F32;
  else TORCH_CHECK(false, "Unsupported output data type of nvfp4 mm (", D.scalar_type(), ")");
  const at::cuda::OptionalCUDAGuard guard(device_of(A));
  const float* alpha_ptr = alpha.has_value() ? static_cast<const float*>(alpha->data_ptr()) : nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->is_contiguous() && bias->dim() == 1 && bias->sizes()[0] == n,
                "bias must be a contiguous CUDA vector of ", n, " elements");
    TORCH_CHECK(bias->scalar_type() == D.scalar_type(), "bias must have the output's dtype");
    check_status(nvfp_scaled_fp4_mm_bias(D.data_ptr(), A.data_ptr(), B.data_ptr(), A_sf.data_ptr(), B_sf.data_ptr(),
                                         alpha_ptr, bias->data_ptr(), m, n, k, dt, mx ? 1 : 0, current_stream(A)));
    return;
  }
  auto fn = mx ? nvfp_mxfp4_mm : nvfp_scaled_fp4_mm;
  check_status(fn(D.data_ptr(), A.data_ptr(), B.data_ptr(), A_sf.data_ptr(), B_sf.data_ptr(), alpha_ptr,
                  m, n, k, dt, current_stream(A)));
}

// D = alpha * (A*A_sf) @ (B*B_sf)^T + bias, one rounding; bias: [n] of D's dtype.
void scaled_fp4_mm_bias(torch::Tensor& D, torch::Tensor const& A, torch::Tensor const& B, torch::Tensor const& A_sf,
                        torch::Tensor const& B_sf, c10::optional<torch::Tensor> const& alpha,
                        torch::Tensor const& bias, bool mx) {
  scaled_mm_impl(D, A, B, A_sf, B_sf, alpha, mx, bias);
}

void cutlass_scaled_fp4_mm(torch::Tensor& D, torch::Tensor const& A, torch::Tensor const& B,
                           torch::Tensor const& A_sf, torch::Tensor const& B_sf,
                           torch::Tensor const& alpha) {
  scaled_mm_impl(D, A, B, A_sf, B_sf, alpha, false);
}

void mxfp4_scaled_mm(torch::Tensor& D, torch::Tensor const& A, torch::Tensor const& B,
                     torch::Tensor const& A_sf, torch::Tensor const& B_sf,
                     c10::optional<torch::Tensor> const& alpha) {
  scaled_mm_impl(D, A, B, A_sf, B_sf, alpha, true);
}

// D_fp4 / D_sf = NVFP4 quantization (global scale out_gs) of value_dtype(alpha * (A*A_sf) @ (B*B_sf)^T + bias), done in
// the GEMM epilogue.  value_dtype_code: NVFP_DTYPE_F16 or NVFP_DTYPE_BF16.
void scaled_fp4_mm_fp4out(torch::Tensor& D_fp4, torch::Tensor& D_sf, torch::Tensor const& A, torch::Tensor const& B,
                          torch::Tensor const& A_sf, torch::Tensor const& B_sf, c10::optional<torch::Tensor> const& alpha,
                          c10::optional<torch::Tensor> const& bias, torch::Tensor const& out_gs, int64_t value_dtype_code,
                          bool mx) {
  CHECK_OPERAND(A, at::ScalarType::Byte, "a");
  CHECK_OPERAND(B, at::ScalarType::Byte, "b");
  TORCH_CHECK(A_sf.is_cuda() && A_sf.is_contiguous() && B_sf.is_cuda() && B_sf.is_contiguous(),
              "scales must be contiguous CUDA tensors");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.sizes()[1] == B.sizes()[1], "a and b shapes cannot be multiplied");
  TORCH_CHECK(mx || alpha.has_value(), "alpha is required");
  const int64_t m = A.sizes()[0], n = B.sizes()[0], k = A.sizes()[1] * 2;
  TORCH_CHECK(A_sf.element_size() * A_sf.numel() == nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(k, mx ? 32 : 16) &&
                  B_sf.element_size() * B_sf.numel() == nvfp_sf_rows_padded(n) * nvfp_sf_cols_padded(k, mx ? 32 : 16),
              "operand scales must be padded and swizzled");
  TORCH_CHECK(D_fp4.is_cuda() && D_fp4.is_contiguous() && D_fp4.scalar_type() == at::ScalarType::Byte &&
                  D_fp4.numel() == m * (n / 2), "output must be contiguous uint8 [m, n/2]");
  TORCH_CHECK(D_sf.is_cuda() && D_sf.is_contiguous() &&
                  D_sf.element_size() * D_sf.numel() >= nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(n, 16),
              "output scales too small for the padded layout");
  TORCH_CHECK(out_gs.is_cuda() && out_gs.scalar_type() == at::ScalarType::Float, "output global scale must be CUDA fp32");
  const void* bias_ptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->is_contiguous() && bias->dim() == 1 && bias->sizes()[0] == n,
                "bias must be a contiguous CUDA vector of ", n, " elements");
    TORCH_CHECK((value_dtype_code == NVFP_DTYPE_BF16 && bias->scalar_type() == at::ScalarType::BFloat16) ||
                    (value_dtype_code == NVFP_DTYPE_F16 && bias->scalar_type() == at::ScalarType::Half),
                "bias must have the dtype the product is rounded to");
    bias_ptr = bias->data_ptr();
  }
  const at::cuda::OptionalCUDAGuard guard(device_of(A));
  const float* alpha_ptr = alpha.has_value() ? static_cast<const float*>(alpha->data_ptr()) : nullptr;
  check_status(nvfp_scaled_fp4_mm_fp4out(D_fp4.data_ptr(), D_sf.data_ptr(), A.data_ptr(), B.data_ptr(), A_sf.data_ptr(),
                                         B_sf.data_ptr(), alpha_ptr, bias_ptr, static_cast<const float*>(out_gs.data_ptr()),
                                         m, n, k, (int)value_dtype_code, mx ? 1 : 0, current_stream(A)));
}

// Gate/up projection with silu(gate) * up in the epilogue (B's rows interleaved in groups of 16).  D: [m, n/2] of the
// value dtype when out_gs is absent; uint8 [m, n/4] plus D_sf (swizzled scales of an [m, n/2] tensor) when it is given.
void scaled_fp4_mm_silu_mul(torch::Tensor& D, c10::optional<torch::Tensor> D_sf, torch::Tensor const& A,
                            torch::Tensor const& B, torch::Tensor const& A_sf, torch::Tensor const& B_sf,
                            c10::optional<torch::Tensor> const& alpha, c10::optional<torch::Tensor> const& bias,
                            c10::optional<torch::Tensor> const& out_gs, int64_t value_dtype_code, bool mx) {
  CHECK_OPERAND(A, at::ScalarType::Byte, "a");
  CHECK_OPERAND(B, at::ScalarType::Byte, "b");
  TORCH_CHECK(A_sf.is_cuda() && A_sf.is_contiguous() && B_sf.is_cuda() && B_sf.is_contiguous(),
              "scales must be contiguous CUDA tensors");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.sizes()[1] == B.sizes()[1], "a and b shapes cannot be multiplied");
  TORCH_CHECK(mx || alpha.has_value(), "alpha is required");
  const int64_t m = A.sizes()[0], n = B.sizes()[0], k = A.sizes()[1] * 2;
  TORCH_CHECK(n % 32 == 0, "Expected n to be divisible by 32, but got b shape: (", B.sizes()[0], "x", B.sizes()[1], ").");
  TORCH_CHECK(A_sf.element_size() * A_sf.numel() == nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(k, mx ? 32 : 16) &&
                  B_sf.element_size() * B_sf.numel() == nvfp_sf_rows_padded(n) * nvfp_sf_cols_padded(k, mx ? 32 : 16),
              "operand scales must be padded and swizzled");
  TORCH_CHECK(D.is_cuda() && D.is_contiguous(), "output must be a contiguous CUDA tensor");
  const bool quantized = out_gs.has_value() && out_gs->defined();
  void* sf_ptr = nullptr;
  if (quantized) {
    TORCH_CHECK(out_gs->is_cuda() && out_gs->scalar_type() == at::ScalarType::Float, "output global scale must be CUDA fp32");
    TORCH_CHECK(D.scalar_type() == at::ScalarType::Byte && D.numel() == m * (n / 4), "output must be uint8 [m, n/4]");
    TORCH_CHECK(D_sf.has_value() && D_sf->is_cuda() && D_sf->is_contiguous() &&
                    D_sf->element_size() * D_sf->numel() >= nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(n / 2, 16),
                "output scales missing or too small for the padded layout");
    sf_ptr = D_sf->data_ptr();
  } else {
    TORCH_CHECK(D.numel() == m * (n / 2) &&
                    ((value_dtype_code == NVFP_DTYPE_BF16 && D.scalar_type() == at::ScalarType::BFloat16) ||
                     (value_dtype_code == NVFP_DTYPE_F16 && D.scalar_type() == at::ScalarType::Half)),
                "output must be [m, n/2] of the value dtype");
  }
  const void* bias_ptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->is_contiguous() && bias->dim() == 1 && bias->sizes()[0] == n,
                "bias must be a contiguous CUDA vector of ", n, " elements");
    TORCH_CHECK((value_dtype_code == NVFP_DTYPE_BF16 && bias->scalar_type() == at::ScalarType::BFloat16) ||
                    (value_dtype_code == NVFP_DTYPE_F16 && bias->scalar_type() == at::ScalarType::Half),
                "bias must have the value dtype");
    bias_ptr = bias->data_ptr();
  }
  const at::cuda::OptionalCUDAGuard guard(device_of(A));
  const float* alpha_ptr = alpha.has_value() ? static_cast<const float*>(alpha->data_ptr()) : nullptr;
  check_status(nvfp_scaled_fp4_mm_silu_mul(D.data_ptr(), sf_ptr, A.data_ptr(), B.data_ptr(), A_sf.data_ptr(), B_sf.data_ptr(),
                                           alpha_ptr, bias_ptr,
                                           quantized ? static_cast<const float*>(out_gs->data_ptr()) : nullptr, m, n, k,
                                           (int)value_dtype_code, mx ? 1 : 0, current_stream(A)));
}

// Checks shared by the two entry points that take raw destination addresses (peer GPUs' buffers): a wrong size
// there is a fault on another GPU, not a Python error, so everything that can be checked on the host is.
void check_peer_call_operands(torch::Tensor const& A_sf, torch::Tensor const& B_sf, int64_t m, int64_t n, int64_t k, bool mx,
                              std::vector<int64_t> const& dst_ptrs) {
  const int block = mx ? 32 : 16;
  TORCH_CHECK(k % (mx ? 64 : 32) == 0 && n % 32 == 0, "Expected k to be divisible by ", mx ? 64 : 32,
              " and n by 32, but got k: ", k, ", n: ", n, ".");
  TORCH_CHECK(A_sf.element_size() * A_sf.numel() == nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(k, block),
              "scale_a must be padded and swizzled to ", nvfp_sf_rows_padded(m), "x", nvfp_sf_cols_padded(k, block), " bytes");
  TORCH_CHECK(B_sf.element_size() * B_sf.numel() == nvfp_sf_rows_padded(n) * nvfp_sf_cols_padded(k, block),
              "scale_b must be padded and swizzled to ", nvfp_sf_rows_padded(n), "x", nvfp_sf_cols_padded(k, block), " bytes");
  TORCH_CHECK(!dst_ptrs.empty() && dst_ptrs.size() <= 8, "between 1 and 8 destinations are supported, got ", dst_ptrs.size());
  for (int64_t p : dst_ptrs) TORCH_CHECK(p != 0 && p % 16 == 0, "destination addresses must be non-null and 16-byte aligned");
}

// GEMM whose [m, n] result goes to several destinations given as raw device addresses (the local
// output first, then peer GPUs' buffers): the column-parallel gather fused into the epilogue.
void scaled_fp4_mm_multi(std::vector<int64_t> const& dst_ptrs, int64_t dst_ld, int64_t out_dtype_code, torch::Tensor const& A,
                         torch::Tensor const& B, torch::Tensor const& A_sf, torch::Tensor const& B_sf,
                         c10::optional<torch::Tensor> const& alpha, bool mx) {
  CHECK_OPERAND(A, at::ScalarType::Byte, "a");
  CHECK_OPERAND(B, at::ScalarType::Byte, "b");
  TORCH_CHECK(A_sf.is_cuda() && A_sf.is_contiguous() && B_sf.is_cuda() && B_sf.is_contiguous(),
              "scales must be contiguous CUDA tensors");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.sizes()[1] == B.sizes()[1], "a and b shapes cannot be multiplied");
  TORCH_CHECK(mx || alpha.has_value(), "alpha is required");
  const int64_t m = A.sizes()[0], n = B.sizes()[0], k = A.sizes()[1] * 2;
  check_peer_call_operands(A_sf, B_sf, m, n, k, mx, dst_ptrs);
  TORCH_CHECK(out_dtype_code == NVFP_DTYPE_F16 || out_dtype_code == NVFP_DTYPE_BF16 || out_dtype_code == NVFP_DTYPE_F32,
              "unknown output dtype code ", out_dtype_code);
  TORCH_CHECK(dst_ld >= n, "destination leading dimension ", dst_ld, " is smaller than n = ", n);
  std::vector<void*> dst;
  for (int64_t p : dst_ptrs) dst.push_back(reinterpret_cast<void*>(p));
  const at::cuda::OptionalCUDAGuard guard(device_of(A));
  const float* alpha_ptr = alpha.has_value() ? static_cast<const float*>(alpha->data_ptr()) : nullptr;
  check_status(nvfp_scaled_fp4_mm_multi(dst.data(), (int)dst.size(), A.data_ptr(), B.data_ptr(), A_sf.data_ptr(),
                                        B_sf.data_ptr(), alpha_ptr, m, n, k, dst_ld, (int)out_dtype_code, mx ? 1 : 0,
                                        current_stream(A)));
}

// K-split partial product added into per-rank fp32 destinations (raw device addresses, one per rank):
// the row-parallel reduce-scatter fused into the epilogue.
void scaled_fp4_mm_scatter_add(std::vector<int64_t> const& dst_ptrs, torch::Tensor const& A, torch::Tensor const& B,
                               torch::Tensor const& A_sf, torch::Tensor const& B_sf,
                               c10::optional<torch::Tensor> const& alpha, bool mx) {
  CHECK_OPERAND(A, at::ScalarType::Byte, "a");
  CHECK_OPERAND(B, at::ScalarType::Byte, "b");
  TORCH_CHECK(A_sf.is_cuda() && A_sf.is_contiguous() && B_sf.is_cuda() && B_sf.is_contiguous(),
              "scales must be contiguous CUDA tensors");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.sizes()[1] == B.sizes()[1], "a and b shapes cannot be multiplied");
  TORCH_CHECK(mx || alpha.has_value(), "alpha is required");
  const int64_t m = A.sizes()[0], n = B.sizes()[0], k = A.sizes()[1] * 2;
  check_peer_call_operands(A_sf, B_sf, m, n, k, mx, dst_ptrs);
  TORCH_CHECK(m % (32 * (int64_t)dst_ptrs.size()) == 0, "m = ", m, " must be a multiple of 32 x the number of destinations (",
              dst_ptrs.size(), ")");
  std::vector<void*> dst;
  for (int64_t p : dst_ptrs) dst.push_back(reinterpret_cast<void*>(p));
  const at::cuda::OptionalCUDAGuard guard(device_of(A));
  const float* alpha_ptr = alpha.has_value() ? static_cast<const float*>(alpha->data_ptr()) : nullptr;
  check_status(nvfp_scaled_fp4_mm_scatter_add(dst.data(), (int)dst.size(), A.data_ptr(), B.data_ptr(), A_sf.data_ptr(),
                                              B_sf.data_ptr(), alpha_ptr, m, n, k, mx ? 1 : 0, current_stream(A)));
}

// nvfp_peer_group_t from Python: destination and flag-block addresses per rank (raw device addresses, rank order).
nvfp_peer_group_t make_peer_group(std::vector<int64_t> const& dst_ptrs, std::vector<int64_t> const& flag_ptrs, int64_t rank,
                                  int64_t wait_limit_ns) {
  TORCH_CHECK(!dst_ptrs.empty() && dst_ptrs.size() <= NVFP_MAX_RANKS, "between 1 and 8 ranks are supported, got ", dst_ptrs.size());
  TORCH_CHECK(flag_ptrs.empty() || flag_ptrs.size() == dst_ptrs.size(), "one flag block per rank, or none");
  TORCH_CHECK(rank >= 0 && rank < (int64_t)dst_ptrs.size(), "rank ", rank, " out of range");
  TORCH_CHECK(wait_limit_ns >= 0, "negative wait limit");
  nvfp_peer_group_t g = {};
  g.world = (int)dst_ptrs.size();
  g.rank = (int)rank;
  g.wait_limit_ns = (uint64_t)wait_limit_ns;
  for (size_t r = 0; r < dst_ptrs.size(); ++r) {
    TORCH_CHECK(dst_ptrs[r] != 0 && dst_ptrs[r] % 16 == 0, "destination addresses must be non-null and 16-byte aligned");
    g.dst[r] = reinterpret_cast<void*>(dst_ptrs[r]);
    if (!flag_ptrs.empty()) {
      TORCH_CHECK(flag_ptrs[r] != 0 && flag_ptrs[r] % 128 == 0, "flag blocks must be non-null and 128-byte aligned");
      g.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
    }
  }
  return g;
}

// Column-parallel GEMM with the gather fused in and the ranks synchronised inside the kernel (nvfp_scaled_fp4_mm_gather).
void scaled_fp4_mm_gather(std::vector<int64_t> const& dst_ptrs, std::vector<int64_t> const& flag_ptrs, int64_t rank,
                          int64_t wait_limit_ns, int64_t dst_ld, int64_t out_dtype_code, torch::Tensor const& A,
                          torch::Tensor const& B, torch::Tensor const& A_sf, torch::Tensor const& B_sf,
                          c10::optional<torch::Tensor> const& alpha, bool mx) {
  CHECK_OPERAND(A, at::ScalarType::Byte, "a");
  CHECK_OPERAND(B, at::ScalarType::Byte, "b");
  TORCH_CHECK(A_sf.is_cuda() && A_sf.is_contiguous() && B_sf.is_cuda() && B_sf.is_contiguous(),
              "scales must be contiguous CUDA tensors");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.sizes()[1] == B.sizes()[1], "a and b shapes cannot be multiplied");
  TORCH_CHECK(mx || alpha.has_value(), "alpha is required");
  const int64_t m = A.sizes()[0], n = B.sizes()[0], k = A.sizes()[1] * 2;
  check_peer_call_operands(A_sf, B_sf, m, n, k, mx, dst_ptrs);
  TORCH_CHECK(out_dtype_code == NVFP_DTYPE_F16 || out_dtype_code == NVFP_DTYPE_BF16 || out_dtype_code == NVFP_DTYPE_F32,
              "unknown output dtype code ", out_dtype_code);
  TORCH_CHECK(dst_ld >= n, "destination leading dimension ", dst_ld, " is smaller than n = ", n);
  const nvfp_peer_group_t g = make_peer_group(dst_ptrs, flag_ptrs, rank, wait_limit_ns);
  const at::cuda::OptionalCUDAGuard guard(device_of(A));
  const float* alpha_ptr = alpha.has_value() ? static_cast<const float*>(alpha->data_ptr()) : nullptr;
  check_status(nvfp_scaled_fp4_mm_gather(&g, dst_ld, A.data_ptr(), B.data_ptr(), A_sf.data_ptr(), B_sf.data_ptr(), alpha_ptr,
                                         m, n, k, (int)out_dtype_code, mx ? 1 : 0, current_stream(A)));
}

// Row-parallel GEMM with the reduce-scatter fused in, ranks synchronised inside the kernel.
void scaled_fp4_mm_reduce_scatter(std::vector<int64_t> const& dst_ptrs, std::vector<int64_t> const& flag_ptrs, int64_t rank,
                                  int64_t wait_limit_ns, torch::Tensor const& A, torch::Tensor const& B,
                                  torch::Tensor const& A_sf, torch::Tensor const& B_sf,
                                  c10::optional<torch::Tensor> const& alpha, bool mx) {
  CHECK_OPERAND(A, at::ScalarType::Byte, "a");
  CHECK_OPERAND(B, at::ScalarType::Byte, "b");
  TORCH_CHECK(A_sf.is_cuda() && A_sf.is_contiguous() && B_sf.is_cuda() && B_sf.is_contiguous(),
              "scales must be contiguous CUDA tensors");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.sizes()[1] == B.sizes()[1], "a and b shapes cannot be multiplied");
  TORCH_CHECK(mx || alpha.has_value(), "alpha is required");
  const int64_t m = A.sizes()[0], n = B.sizes()[0], k = A.sizes()[1] * 2;
  check_peer_call_operands(A_sf, B_sf, m, n, k, mx, dst_ptrs);
  TORCH_CHECK(m % (32 * (int64_t)dst_ptrs.size()) == 0, "m = ", m, " must be a multiple of 32 x the number of ranks (",
              dst_ptrs.size(), ")");
  const nvfp_peer_group_t g = make_peer_group(dst_ptrs, flag_ptrs, rank, wait_limit_ns);
  const at::cuda::OptionalCUDAGuard guard(device_of(A));
  const float* alpha_ptr = alpha.has_value() ? static_cast<const float*>(alpha->data_ptr()) : nullptr;
  check_status(nvfp_scaled_fp4_mm_reduce_scatter(&g, A.data_ptr(), B.data_ptr(), A_sf.data_ptr(), B_sf.data_ptr(), alpha_ptr,
                                                 m, n, k, mx ? 1 : 0, current_stream(A)));
}

// Whole forward of a column-parallel NVFP4 layer with the fused gather in one call (nvfp_linear_forward_gather).
void linear_forward_gather(std::vector<int64_t> const& dst_ptrs, std::vector<int64_t> const& flag_ptrs, int64_t rank,
                           int64_t wait_limit_ns, int64_t dst_ld, int64_t out_dtype_code, torch::Tensor const& X,
                           torch::Tensor const& W, torch::Tensor const& W_sf, torch::Tensor const& gs_w,
                           torch::Tensor& workspace, torch::Tensor& scratch) {
  TORCH_CHECK(X.dim() == 2 && X.stride(1) == 1, "input must be a matrix with dense rows");
  CHECK_OPERAND(W, at::ScalarType::Byte, "weight");
  TORCH_CHECK(W_sf.is_cuda() && W_sf.is_contiguous(), "weight scales must be a contiguous CUDA tensor");
  TORCH_CHECK(X.is_cuda() && gs_w.is_cuda() && workspace.is_cuda() && scratch.is_cuda(), "all tensors must be CUDA tensors");
  TORCH_CHECK(gs_w.scalar_type() == at::ScalarType::Float, "weight global scale must be fp32");
  const int64_t m = X.size(0), k = X.size(1), n = W.size(0);
  TORCH_CHECK(W.dim() == 2 && W.size(1) * 2 == k, "a and b shapes cannot be multiplied (", m, "x", k, " and ", n, "x",
              W.size(1) * 2, ")");
  TORCH_CHECK(k % 32 == 0 && n % 32 == 0, "Expected k and n to be divisible by 32, but got k: ", k, ", n: ", n, ".");
  TORCH_CHECK(W_sf.element_size() * W_sf.numel() == nvfp_sf_rows_padded(n) * nvfp_sf_cols_padded(k, 16),
              "scale_b must be padded and swizzled to a shape (", nvfp_sf_rows_padded(n), "x", nvfp_sf_cols_padded(k, 16), ")");
  TORCH_CHECK(out_dtype_code == NVFP_DTYPE_F16 || out_dtype_code == NVFP_DTYPE_BF16 || out_dtype_code == NVFP_DTYPE_F32,
              "unknown output dtype code ", out_dtype_code);
  TORCH_CHECK(dst_ld >= n, "destination leading dimension ", dst_ld, " is smaller than n = ", n);
  TORCH_CHECK(workspace.element_size() * workspace.numel() >= nvfp_linear_workspace_bytes(m, k), "workspace too small");
  TORCH_CHECK(scratch.element_size() * scratch.numel() >= 32, "scratch must hold 32 bytes");
  const nvfp_peer_group_t g = make_peer_group(dst_ptrs, flag_ptrs, rank, wait_limit_ns);
  const int xdt = dtype_code(X, "Unsupported input data type for quantize_to_fp4.");
  const at::cuda::OptionalCUDAGuard guard(device_of(X));
  check_status(nvfp_linear_forward_gather(&g, dst_ld, X.data_ptr(), m, k, m > 1 ? X.stride(0) : k, xdt, W.data_ptr(),
                                          W_sf.data_ptr(), static_cast<const float*>(gs_w.data_ptr()), n, workspace.data_ptr(),
                                          static_cast<uint32_t*>(scratch.data_ptr()), (int)out_dtype_code, current_stream(X)));
}

// Whole forward of a column-parallel NVFP4 layer whose gathered output is NVFP4 (nvfp_linear_forward_gather_fp4).
// packed_ptrs / sf_ptrs: BASE addresses of every rank's gathered packed matrix and scale tensor, rank order.
void linear_forward_gather_fp4(std::vector<int64_t> const& packed_ptrs, std::vector<int64_t> const& sf_ptrs,
                               std::vector<int64_t> const& flag_ptrs, int64_t rank, int64_t wait_limit_ns, int64_t n_total,
                               int64_t n_offset, int64_t value_dtype_code, torch::Tensor const& X, torch::Tensor const& W,
                               torch::Tensor const& W_sf, torch::Tensor const& gs_w, c10::optional<torch::Tensor> const& bias,
                               torch::Tensor const& out_gs, torch::Tensor& workspace, torch::Tensor& scratch) {
  TORCH_CHECK(X.dim() == 2 && X.stride(1) == 1, "input must be a matrix with dense rows");
  CHECK_OPERAND(W, at::ScalarType::Byte, "weight");
  TORCH_CHECK(W_sf.is_cuda() && W_sf.is_contiguous(), "weight scales must be a contiguous CUDA tensor");
  TORCH_CHECK(X.is_cuda() && gs_w.is_cuda() && out_gs.is_cuda() && workspace.is_cuda() && scratch.is_cuda(),
              "all tensors must be CUDA tensors");
  TORCH_CHECK(gs_w.scalar_type() == at::ScalarType::Float && out_gs.scalar_type() == at::ScalarType::Float, "scales must be fp32");
  const int64_t m = X.size(0), k = X.size(1), n = W.size(0);
  TORCH_CHECK(W.dim() == 2 && W.size(1) * 2 == k, "a and b shapes cannot be multiplied (", m, "x", k, " and ", n, "x",
              W.size(1) * 2, ")");
  TORCH_CHECK(W_sf.element_size() * W_sf.numel() == nvfp_sf_rows_padded(n) * nvfp_sf_cols_padded(k, 16),
              "scale_b must be padded and swizzled to a shape (", nvfp_sf_rows_padded(n), "x", nvfp_sf_cols_padded(k, 16), ")");
  TORCH_CHECK(sf_ptrs.size() == packed_ptrs.size(), "one scale tensor per rank");
  TORCH_CHECK(workspace.element_size() * workspace.numel() >= nvfp_linear_workspace_bytes(m, k), "workspace too small");
  TORCH_CHECK(scratch.element_size() * scratch.numel() >= 32, "scratch must hold 32 bytes");
  const void* bias_ptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->is_contiguous() && bias->dim() == 1 && bias->size(0) == n, "bias must be a contiguous CUDA vector of ", n, " elements");
    TORCH_CHECK((value_dtype_code == NVFP_DTYPE_BF16 && bias->scalar_type() == at::ScalarType::BFloat16) ||
                    (value_dtype_code == NVFP_DTYPE_F16 && bias->scalar_type() == at::ScalarType::Half), "bias must have the value dtype");
    bias_ptr = bias->data_ptr();
  }
  const nvfp_peer_group_t g = make_peer_group(packed_ptrs, flag_ptrs, rank, wait_limit_ns);
  void* sf[NVFP_MAX_RANKS] = {};
  for (size_t r = 0; r < sf_ptrs.size(); ++r) sf[r] = reinterpret_cast<void*>(sf_ptrs[r]);
  const int xdt = dtype_code(X, "Unsupported input data type for quantize_to_fp4.");
  const at::cuda::OptionalCUDAGuard guard(device_of(X));
  check_status(nvfp_linear_forward_gather_fp4(&g, sf, n_total, n_offset, X.data_ptr(), m, k, m > 1 ? X.stride(0) : k, xdt,
                                              W.data_ptr(), W_sf.data_ptr(), static_cast<const float*>(gs_w.data_ptr()), n,
                                              bias_ptr, static_cast<const float*>(out_gs.data_ptr()), workspace.data_ptr(),
                                              static_cast<uint32_t*>(scratch.data_ptr()), (int)value_dtype_code, current_stream(X)));
}

// kernel/reciprocal_kernels.cu:91-121 of the reference (fp32, the only reachable dtype).
void reciprocal_approximate_ftz_tensor(torch::Tensor const& input, torch::Tensor& output) {
  TORCH_CHECK(input.scalar_type() == at::ScalarType::Float, "Input tensor must be float");
  TORCH_CHECK(output.scalar_type() == input.scalar_type(),
              "Output tensor must have the same dtype as input tensor");
  TORCH_CHECK(input.sizes() == output.sizes(), "Input and output tensors must have the same shape");
  TORCH_CHECK(input.is_cuda() && output.is_cuda(), "Input and output tensors must be on CUDA device");
  TORCH_CHECK(input.is_contiguous() && output.is_contiguous(), "tensors must be contiguous");
  const at::cuda::OptionalCUDAGuard guard(device_of(input));
  check_status(nvfp_reciprocal_approximate_ftz(static_cast<float*>(output.data_ptr()),
                                               static_cast<const float*>(input.data_ptr()),
                                               input.numel(), current_stream(input)));
}

void global_scale(torch::Tensor& gs_out, torch::Tensor& scratch, torch::Tensor const& input) {
  TORCH_CHECK(input.dim() == 2 && input.stride(1) == 1, "input must be a matrix with dense rows");
  TORCH_CHECK(gs_out.is_cuda() && scratch.is_cuda() && input.is_cuda(), "all tensors must be CUDA tensors");
  TORCH_CHECK(gs_out.scalar_type() == at::ScalarType::Float && gs_out.numel() >= 1, "gs_out must be fp32");
  TORCH_CHECK(scratch.element_size() * scratch.numel() >= 8, "scratch must hold 8 bytes");
  const int dt = dtype_code(input, "Unsupported input data type for global_scale.");
  const at::cuda::OptionalCUDAGuard guard(device_of(input));
  check_status(nvfp_global_scale(static_cast<float*>(gs_out.data_ptr()),
                                 static_cast<uint32_t*>(scratch.data_ptr()), input.data_ptr(),
                                 input.size(0), input.size(1),
                                 input.size(0) > 1 ? input.stride(0) : input.size(1), dt,
                                 current_stream(input)));
}

void activation_scales(torch::Tensor& gs_out, torch::Tensor& alpha_out, torch::Tensor& scratch,
                       torch::Tensor const& input, torch::Tensor const& gs_weight) {
  TORCH_CHECK(input.dim() == 2 && input.stride(1) == 1, "input must be a matrix with dense rows");
  TORCH_CHECK(gs_out.is_cuda() && alpha_out.is_cuda() && scratch.is_cuda() && input.is_cuda() && gs_weight.is_cuda(),
              "all tensors must be CUDA tensors");
  TORCH_CHECK(gs_out.scalar_type() == at::ScalarType::Float && alpha_out.scalar_type() == at::ScalarType::Float &&
                  gs_weight.scalar_type() == at::ScalarType::Float, "scales must be fp32");
  TORCH_CHECK(scratch.element_size() * scratch.numel() >= 32, "scratch must hold 32 bytes");
  const int dt = dtype_code(input, "Unsupported input data type for activation_scales.");
  const at::cuda::OptionalCUDAGuard guard(device_of(input));
  check_status(nvfp_activation_scales(static_cast<float*>(gs_out.data_ptr()), static_cast<float*>(alpha_out.data_ptr()),
                                      static_cast<uint32_t*>(scratch.data_ptr()), input.data_ptr(), input.size(0),
                                      input.size(1), input.size(0) > 1 ? input.stride(0) : input.size(1), dt,
                                      static_cast<const float*>(gs_weight.data_ptr()), current_stream(input)));
}

// output / output_sf as for scaled_fp4_quant_sm1xxa; gs_out and alpha_out: fp32 [1]; gs_weight: fp32 [1] or
// an undefined tensor (then alpha_out is not written).
void dynamic_scaled_fp4_quant(torch::Tensor& output, torch::Tensor& output_sf, torch::Tensor& gs_out,
                              torch::Tensor& alpha_out, torch::Tensor& scratch, torch::Tensor const& input,
                              std::optional<torch::Tensor> const& gs_weight) {
  TORCH_CHECK(input.dim() == 2 && input.stride(1) == 1, "input must be a matrix with dense rows");
  TORCH_CHECK(output.is_cuda() && output_sf.is_cuda() && gs_out.is_cuda() && alpha_out.is_cuda() && scratch.is_cuda() &&
                  input.is_cuda(), "all tensors must be CUDA tensors");
  TORCH_CHECK(output.is_contiguous() && output_sf.is_contiguous(), "outputs must be contiguous");
  TORCH_CHECK(gs_out.scalar_type() == at::ScalarType::Float && alpha_out.scalar_type() == at::ScalarType::Float,
              "scales must be fp32");
  TORCH_CHECK(scratch.element_size() * scratch.numel() >= 32, "scratch must hold 32 bytes");
  const int64_t m = input.size(0), n = input.size(1);
  TORCH_CHECK(output.scalar_type() == at::ScalarType::Byte && output.numel() == m * (n / 2), "output must be uint8 [m, n/2]");
  TORCH_CHECK(output_sf.element_size() * output_sf.numel() >= nvfp_sf_rows_padded(m) * nvfp_sf_cols_padded(n, 16),
              "output_sf is too small for the padded scale layout");
  const float* gsw = nullptr;
  if (gs_weight.has_value() && gs_weight->defined()) {
    TORCH_CHECK(gs_weight->is_cuda() && gs_weight->scalar_type() == at::ScalarType::Float, "gs_weight must be CUDA fp32");
    gsw = static_cast<const float*>(gs_weight->data_ptr());
  }
  const int dt = dtype_code(input, "Unsupported input data type for quantize_to_fp4.");
  const at::cuda::OptionalCUDAGuard guard(device_of(input));
  check_status(nvfp_dynamic_fp4_quant(output.data_ptr(), output_sf.data_ptr(), static_cast<float*>(gs_out.data_ptr()),
                                      static_cast<float*>(alpha_out.data_ptr()), static_cast<uint32_t*>(scratch.data_ptr()),
                                      input.data_ptr(), m, n, m > 1 ? input.stride(0) : n, dt, gsw, current_stream(input)));
}

// Whole forward of an NVFP4 layer in one call: D = quant(X) @ W^T / (gs_x * gs_w) (+ bias).  `workspace`: uint8,
// at least linear_workspace_bytes(m, k) bytes, 256-byte aligned.
int64_t linear_workspace_bytes(int64_t m, int64_t k) { return nvfp_linear_workspace_bytes(m, k); }

void linear_forward(torch::Tensor& D, torch::Tensor const& X, torch::Tensor const& W, torch::Tensor const& W_sf,
                    torch::Tensor const& gs_w, std::optional<torch::Tensor> const& bias, torch::Tensor& workspace,
                    torch::Tensor& scratch) {
  TORCH_CHECK(X.dim() == 2 && X.stride(1) == 1, "input must be a matrix with dense rows");
  CHECK_OPERAND(W, at::ScalarType::Byte, "weight");
  TORCH_CHECK(W_sf.is_cuda() && W_sf.is_contiguous(), "weight scales must be a contiguous CUDA tensor");
  TORCH_CHECK(D.is_cuda() && D.is_contiguous() && X.is_cuda() && gs_w.is_cuda() && workspace.is_cuda() && scratch.is_cuda(),
              "all tensors must be CUDA tensors");
  TORCH_CHECK(gs_w.scalar_type() == at::ScalarType::Float, "weight global scale must be fp32");
  const int64_t m = X.size(0), k = X.size(1), n = W.size(0);
  TORCH_CHECK(W.dim() == 2 && W.size(1) * 2 == k, "a and b shapes cannot be multiplied (", m, "x", k, " and ", n, "x",
              W.size(1) * 2, ")");
  TORCH_CHECK(n % 32 == 0, "Expected n to be divisible by 32, but got b shape: (", W.sizes()[0], "x", W.sizes()[1], ").");
  TORCH_CHECK(W_sf.element_size() * W_sf.numel() == nvfp_sf_rows_padded(n) * nvfp_sf_cols_padded(k, 16),
              "scale_b must be padded and swizzled to a shape (", nvfp_sf_rows_padded(n), "x", nvfp_sf_cols_padded(k, 16), ")");
  TORCH_CHECK(D.dim() == 2 && D.size(0) == m && D.size(1) == n, "out must have shape (", m, "x", n, ")");
  TORCH_CHECK(workspace.element_size() * workspace.numel() >= nvfp_linear_workspace_bytes(m, k), "workspace too small");
  TORCH_CHECK(scratch.element_size() * scratch.numel() >= 32, "scratch must hold 32 bytes");
  int dt;
  if (D.scalar_type() == at::ScalarType::BFloat16) dt = NVFP_DTYPE_BF16;
  else if (D.scalar_type() == at::ScalarType::Half) dt = NVFP_DTYPE_F16;
  else if (D.scalar_type() == at::ScalarType::Float) dt = NVFP_DTYPE_F32;
  else TORCH_CHECK(false, "Unsupported output data type of nvfp4 mm (", D.scalar_type(), ")");
  const void* bias_ptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->is_contiguous() && bias->dim() == 1 && bias->size(0) == n &&
                    bias->scalar_type() == D.scalar_type(), "bias must be a contiguous CUDA vector of ", n, " elements of the output's dtype");
    bias_ptr = bias->data_ptr();
  }
  const int xdt = dtype_code(X, "Unsupported input data type for quantize_to_fp4.");
  const at::cuda::OptionalCUDAGuard guard(device_of(X));
  check_status(nvfp_linear_forward(D.data_ptr(), X.data_ptr(), m, k, m > 1 ? X.stride(0) : k, xdt, W.data_ptr(),
                                   W_sf.data_ptr(), static_cast<const float*>(gs_w.data_ptr()), n, bias_ptr,
                                   workspace.data_ptr(), static_cast<uint32_t*>(scratch.data_ptr()), dt, current_stream(X)));
}

// linear_forward with the chain open at both ends (nvfp_linear_forward_chained): x_gs = known global scale of X or
// nullopt (dynamic); out_gs = where the OUTPUT's global scale goes (with out_scratch) or nullopt; next_gs_w / next_alpha:
// the next layer's weight scale and where its alpha goes, or nullopt.
void linear_forward_chained(torch::Tensor& D, torch::Tensor const& X, std::optional<torch::Tensor> const& x_gs,
                            torch::Tensor const& W, torch::Tensor const& W_sf, torch::Tensor const& gs_w,
                            std::optional<torch::Tensor> const& bias, torch::Tensor& workspace, torch::Tensor& scratch,
                            std::optional<torch::Tensor> const& out_gs, std::optional<torch::Tensor> const& out_scratch,
                            std::optional<torch::Tensor> const& next_gs_w, std::optional<torch::Tensor> const& next_alpha) {
  TORCH_CHECK(X.dim() == 2 && X.stride(1) == 1, "input must be a matrix with dense rows");
  CHECK_OPERAND(W, at::ScalarType::Byte, "weight");
  TORCH_CHECK(W_sf.is_cuda() && W_sf.is_contiguous(), "weight scales must be a contiguous CUDA tensor");
  TORCH_CHECK(D.is_cuda() && D.is_contiguous() && X.is_cuda() && gs_w.is_cuda() && workspace.is_cuda() && scratch.is_cuda(),
              "all tensors must be CUDA tensors");
  TORCH_CHECK(gs_w.scalar_type() == at::ScalarType::Float, "weight global scale must be fp32");
  const int64_t m = X.size(0), k = X.size(1), n = W.size(0);
  TORCH_CHECK(W.dim() == 2 && W.size(1) * 2 == k, "a and b shapes cannot be multiplied (", m, "x", k, " and ", n, "x",
              W.size(1) * 2, ")");
  TORCH_CHECK(n % 32 == 0, "Expected n to be divisible by 32, but got b shape: (", W.sizes()[0], "x", W.sizes()[1], ").");
  TORCH_CHECK(W_sf.element_size() * W_sf.numel() == nvfp_sf_rows_padded(n) * nvfp_sf_cols_padded(k, 16),
              "scale_b must be padded and swizzled to a shape (", nvfp_sf_rows_padded(n), "x", nvfp_sf_cols_padded(k, 16), ")");
  TORCH_CHECK(D.dim() == 2 && D.size(0) == m && D.size(1) == n, "out must have shape (", m, "x", n, ")");
  TORCH_CHECK(workspace.element_size() * workspace.numel() >= nvfp_linear_workspace_bytes(m, k), "workspace too small");
  TORCH_CHECK(scratch.element_size() * scratch.numel() >= 32, "scratch must hold 32 bytes");
  int dt;
  if (D.scalar_type() == at::ScalarType::BFloat16) dt = NVFP_DTYPE_BF16;
  else if (D.scalar_type() == at::ScalarType::Half) dt = NVFP_DTYPE_F16;
  else TORCH_CHECK(false, "chained layers write fp16 or bf16 (", D.scalar_type(), ")");
  auto f32 = [](std::optional<torch::Tensor> const& t, const char* what) -> float* {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::ScalarType::Float && t->numel() >= 1, what, " must be a CUDA fp32 tensor");
    return static_cast<float*>(t->data_ptr());
  };
  uint32_t* out_scratch_ptr = nullptr;
  if (out_scratch.has_value() && out_scratch->defined()) {
    TORCH_CHECK(out_scratch->is_cuda() && out_scratch->element_size() * out_scratch->numel() >= 32, "output scratch must hold 32 bytes");
    out_scratch_ptr = static_cast<uint32_t*>(out_scratch->data_ptr());
  }
  const void* bias_ptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->is_contiguous() && bias->dim() == 1 && bias->size(0) == n &&
                    bias->scalar_type() == D.scalar_type(), "bias must be a contiguous CUDA vector of ", n, " elements of the output's dtype");
    bias_ptr = bias->data_ptr();
  }
  const int xdt = dtype_code(X, "Unsupported input data type for quantize_to_fp4.");
  const at::cuda::OptionalCUDAGuard guard(device_of(X));
  check_status(nvfp_linear_forward_chained(D.data_ptr(), X.data_ptr(), m, k, m > 1 ? X.stride(0) : k, xdt, f32(x_gs, "x_gs"),
                                           W.data_ptr(), W_sf.data_ptr(), static_cast<const float*>(gs_w.data_ptr()), n, bias_ptr,
                                           workspace.data_ptr(), static_cast<uint32_t*>(scratch.data_ptr()), dt,
                                           f32(out_gs, "out_gs"), out_scratch_ptr, f32(next_gs_w, "next_gs_w"),
                                           f32(next_alpha, "next_alpha"), current_stream(X)));
}

// Gated MLP in one call: Y = down(silu(gate(X)) * up(X)); see nvfp_gated_mlp_forward.
int64_t gated_mlp_workspace_bytes(int64_t m, int64_t hidden, int64_t inter) {
  return nvfp_gated_mlp_workspace_bytes(m, hidden, inter);
}

void gated_mlp_forward(torch::Tensor& Y, torch::Tensor const& X, torch::Tensor const& GU, torch::Tensor const& GU_sf,
                       torch::Tensor const& gs_gu, torch::Tensor const& DW, torch::Tensor const& DW_sf,
                       torch::Tensor const& gs_act, torch::Tensor const& alpha_down, torch::Tensor& workspace,
                       torch::Tensor& scratch) {
  TORCH_CHECK(X.dim() == 2 && X.stride(1) == 1, "input must be a matrix with dense rows");
  CHECK_OPERAND(GU, at::ScalarType::Byte, "gate/up weight");
  CHECK_OPERAND(DW, at::ScalarType::Byte, "down weight");
  TORCH_CHECK(GU_sf.is_cuda() && GU_sf.is_contiguous() && DW_sf.is_cuda() && DW_sf.is_contiguous(),
              "weight scales must be contiguous CUDA tensors");
  TORCH_CHECK(Y.is_cuda() && Y.is_contiguous() && X.is_cuda() && gs_gu.is_cuda() && gs_act.is_cuda() &&
                  alpha_down.is_cuda() && workspace.is_cuda() && scratch.is_cuda(), "all tensors must be CUDA tensors");
  TORCH_CHECK(gs_gu.scalar_type() == at::ScalarType::Float && gs_act.scalar_type() == at::ScalarType::Float &&
                  alpha_down.scalar_type() == at::ScalarType::Float, "scales must be fp32");
  const int64_t m = X.size(0), hidden = X.size(1), inter = GU.size(0) / 2, n_out = DW.size(0);
  TORCH_CHECK(GU.dim() == 2 && GU.size(0) % 32 == 0 && GU.size(1) * 2 == hidden,
              "gate/up weight must be (2 * inter) x (hidden / 2) bytes with 2 * inter divisible by 32");
  TORCH_CHECK(DW.dim() == 2 && DW.size(1) * 2 == inter && n_out % 32 == 0,
              "down weight must be n x (inter / 2) bytes with n divisible by 32");
  TORCH_CHECK(GU_sf.element_size() * GU_sf.numel() == nvfp_sf_rows_padded(2 * inter) * nvfp_sf_cols_padded(hidden, 16) &&
                  DW_sf.element_size() * DW_sf.numel() == nvfp_sf_rows_padded(n_out) * nvfp_sf_cols_padded(inter, 16),
              "weight scales must be padded and swizzled");
  TORCH_CHECK(Y.dim() == 2 && Y.size(0) == m && Y.size(1) == n_out, "out must have shape (", m, "x", n_out, ")");
  TORCH_CHECK(workspace.element_size() * workspace.numel() >= nvfp_gated_mlp_workspace_bytes(m, hidden, inter),
              "workspace too small");
  TORCH_CHECK(scratch.element_size() * scratch.numel() >= 32, "scratch must hold 32 bytes");
  int dt;
  if (Y.scalar_type() == at::ScalarType::BFloat16) dt = NVFP_DTYPE_BF16;
  else if (Y.scalar_type() == at::ScalarType::Half) dt = NVFP_DTYPE_F16;
  else TORCH_CHECK(false, "the gated MLP writes fp16 or bf16 (", Y.scalar_type(), ")");
  const int xdt = dtype_code(X, "Unsupported input data type for quantize_to_fp4.");
  const at::cuda::OptionalCUDAGuard guard(device_of(X));
  check_status(nvfp_gated_mlp_forward(Y.data_ptr(), X.data_ptr(), m, hidden, m > 1 ? X.stride(0) : hidden, xdt,
                                      GU.data_ptr(), GU_sf.data_ptr(), static_cast<const float*>(gs_gu.data_ptr()), inter,
                                      DW.data_ptr(), DW_sf.data_ptr(), static_cast<const float*>(gs_act.data_ptr()),
                                      static_cast<const float*>(alpha_down.data_ptr()), n_out, workspace.data_ptr(),
                                      static_cast<uint32_t*>(scratch.data_ptr()), dt, current_stream(X)));
}

void alpha_from_scales(torch::Tensor& alpha_out, torch::Tensor const& gs_a, torch::Tensor const& gs_b) {
  TORCH_CHECK(alpha_out.is_cuda() && gs_a.is_cuda() && gs_b.is_cuda(), "all tensors must be CUDA tensors");
  TORCH_CHECK(alpha_out.scalar_type() == at::ScalarType::Float && gs_a.scalar_type() == at::ScalarType::Float &&
                  gs_b.scalar_type() == at::ScalarType::Float, "all tensors must be fp32");
  const at::cuda::OptionalCUDAGuard guard(device_of(alpha_out));
  check_status(nvfp_alpha_from_scales(static_cast<float*>(alpha_out.data_ptr()),
                                      static_cast<const float*>(gs_a.data_ptr()),
                                      static_cast<const float*>(gs_b.data_ptr()), current_stream(alpha_out)));
}

int64_t device_status() {
  uint32_t word = 0;
  int rc = nvfp_device_status(&word);
  if (rc != NVFP_OK && rc != NVFP_ERR_DEVICE_TIMEOUT) check_status(rc);
  return word;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("scaled_fp4_quant_sm1xxa", &scaled_fp4_quant_sm1xxa);
  m.def("cutlass_scaled_fp4_mm", &cutlass_scaled_fp4_mm);
  m.def("reciprocal_approximate_ftz_tensor", &reciprocal_approximate_ftz_tensor);
  m.def("scaled_mxfp4_quant", &scaled_mxfp4_quant);
  m.def("mxfp4_scaled_mm", &mxfp4_scaled_mm);
  m.def("scaled_fp4_mm_bias", &scaled_fp4_mm_bias);
  m.def("scaled_fp4_mm_fp4out", &scaled_fp4_mm_fp4out);
  m.def("scaled_fp4_mm_silu_mul", &scaled_fp4_mm_silu_mul);
  m.def("scaled_fp4_mm_multi", &scaled_fp4_mm_multi);
  m.def("scaled_fp4_mm_scatter_add", &scaled_fp4_mm_scatter_add);
  m.def("scaled_fp4_mm_gather", &scaled_fp4_mm_gather);
  m.def("scaled_fp4_mm_reduce_scatter", &scaled_fp4_mm_reduce_scatter);
  m.def("linear_forward_gather", &linear_forward_gather);
  m.def("linear_forward_gather_fp4", &linear_forward_gather_fp4);
  m.def("global_scale", &global_scale);
  m.def("activation_scales", &activation_scales);
  m.def("dynamic_scaled_fp4_quant", &dynamic_scaled_fp4_quant);
  m.def("linear_workspace_bytes", &linear_workspace_bytes);
  m.def("linear_forward", &linear_forward);
  m.def("linear_forward_chained", &linear_forward_chained);
  m.def("gated_mlp_workspace_bytes", &gated_mlp_workspace_bytes);
  m.def("gated_mlp_forward", &gated_mlp_forward);
  m.def("alpha_from_scales", &alpha_from_scales);
  m.def("device_status", &device_status);
}
