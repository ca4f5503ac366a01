"""B200-native NVFP4 / MXFP4 quantize-and-GEMM: drop-in for the `nvfp` package of
huweim/nvfp_kernel on its real-kernel path (nvfp/__init__.py:1-27 there)."""
from .ops import (
    activation_scales,
    alpha_from_scales,
    cutlass_scaled_fp4_mm,
    device_status,
    dynamic_scaled_fp4_quant,
    get_active_backend,
    global_scale,
    linear_forward,
    linear_forward_chained,
    gated_mlp_forward,
    mxfp4_scaled_mm,
    reciprocal_approximate_ftz_tensor,
    interleave_gate_up,
    scaled_fp4_mm_fp4out,
    scaled_fp4_mm_silu_mul,
    scaled_fp4_quant,
    scaled_mxfp4_quant,
)
from .linear import QuantLinear
from .host_pipeline import HostPipeline
from .mlp import QuantGatedMLP

__all__ = [
    "scaled_fp4_quant",
    "cutlass_scaled_fp4_mm",
    "get_active_backend",
    "reciprocal_approximate_ftz_tensor",
    "scaled_mxfp4_quant",
    "mxfp4_scaled_mm",
    "global_scale",
    "alpha_from_scales",
    "activation_scales",
    "device_status",
    "dynamic_scaled_fp4_quant",
    "linear_forward",
    "linear_forward_chained",
    "gated_mlp_forward",
    "scaled_fp4_mm_fp4out",
    "scaled_fp4_mm_silu_mul",
    "interleave_gate_up",
    "QuantLinear",
    "HostPipeline",
    "QuantGatedMLP",
]
