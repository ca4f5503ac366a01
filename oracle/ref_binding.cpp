// Python binding for the REFERENCE's own CUDA quantizer and reciprocal op, compiled from
// the reference checkout where it lies (never copied into this repository) for sm_100a.
// TEST INFRASTRUCTURE ONLY: this is the bit-exactness authority for the NVFP4 quantizer
// and the kernel to beat; the product never loads it.
//
// Declarations repeat kernel/nvfp4_quant.h:4-7 and kernel/reciprocal_kernels.h:4-5 of
// the reference (its binding.cpp also pulls in the CUTLASS GEMM, which cannot be built:
// third_party/cutlass is empty and the kernel targets sm_120a).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <torch/extension.h>

void scaled_fp4_quant_sm1xxa(torch::Tensor const& output, torch::Tensor const& input,
                             torch::Tensor const& output_sf, torch::Tensor const& input_sf);
void reciprocal_approximate_ftz_tensor(torch::Tensor const& input, torch::Tensor& output);

// The reference's launcher template (kernel/nvfp4_quant_kernels.cu:31-53), explicitly instantiated there for half
// and __nv_bfloat16 (:56-67).  Its `useUE8M0` argument selects the e8m0 branch of the quantizer
// (cvt_warp_fp16_to_fp4<Type, true>, kernel/nvfp4_utils.cuh:196-202), which the reference's own entry point forces
// off (kernel/nvfp4_quant_kernels.cu:90-91).  Calling the instantiation directly runs that branch as compiled from
// the reference's sources: 16-element blocks, scale byte = exponent bits of amax * rcp(6) (global scale null = 1).
namespace vllm {
template <typename T>
void invokeFP4Quantization(int m, int n, T const* input, float const* SFScale, int64_t* output, int32_t* SFOuput,
                           bool useUE8M0, int multiProcessorCount, cudaStream_t stream);
}

// output: uint8 [m, n/2]; output_sf: int32 [round_up(m,128), round_up(n/16,4)/4] (swizzled ue8m0 bytes).
void scaled_fp4_quant_ue8m0(torch::Tensor const& output, torch::Tensor const& input, torch::Tensor const& output_sf) {
  TORCH_CHECK(input.is_cuda() && input.is_contiguous() && input.dim() == 2 && input.size(1) % 16 == 0);
  const int m = (int)input.size(0), n = (int)input.size(1);
  const at::cuda::OptionalCUDAGuard guard(device_of(input));
  auto stream = at::cuda::getCurrentCUDAStream(input.get_device());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  auto out = static_cast<int64_t*>(output.data_ptr());
  auto sf = static_cast<int32_t*>(output_sf.data_ptr());
  if (input.scalar_type() == at::ScalarType::Half)
    vllm::invokeFP4Quantization<half>(m, n, static_cast<half const*>(input.data_ptr()), nullptr, out, sf, true, sms, stream);
  else if (input.scalar_type() == at::ScalarType::BFloat16)
    vllm::invokeFP4Quantization<__nv_bfloat16>(m, n, static_cast<__nv_bfloat16 const*>(input.data_ptr()), nullptr, out,
                                               sf, true, sms, stream);
  else
    TORCH_CHECK(false, "fp16 or bf16 input expected");
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("scaled_fp4_quant_sm1xxa", &scaled_fp4_quant_sm1xxa);
  m.def("reciprocal_approximate_ftz_tensor", &reciprocal_approximate_ftz_tensor);
  m.def("scaled_fp4_quant_ue8m0", &scaled_fp4_quant_ue8m0);
}
