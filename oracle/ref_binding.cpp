// Python binding for the REFERENCE's own CUDA quantizer and reciprocal op, compiled from
// the reference checkout where it lies (never copied into this repository) for sm_100a.
// TEST INFRASTRUCTURE ONLY: this is the bit-exactness authority for the NVFP4 quantizer
// and the kernel to beat; the product never loads it.
//
// Declarations repeat kernel/nvfp4_quant.h:4-7 and kernel/reciprocal_kernels.h:4-5 of
// the reference (its binding.cpp also pulls in the CUTLASS GEMM, which cannot be built:
// third_party/cutlass is empty and the kernel targets sm_120a).
#include <torch/extension.h>

void scaled_fp4_quant_sm1xxa(torch::Tensor const& output, torch::Tensor const& input,
                             torch::Tensor const& output_sf, torch::Tensor const& input_sf);
void reciprocal_approximate_ftz_tensor(torch::Tensor const& input, torch::Tensor& output);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("scaled_fp4_quant_sm1xxa", &scaled_fp4_quant_sm1xxa);
  m.def("reciprocal_approximate_ftz_tensor", &reciprocal_approximate_ftz_tensor);
}
