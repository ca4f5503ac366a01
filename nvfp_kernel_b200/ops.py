"""Public op API: same names, signatures and results as the reference's nvfp/ops.py:68-92.

There is one backend, the hand-written sm_100a kernels; the reference's
NVFP_GEMM_BACKEND switch and its Triton emulation backend (nvfp/ops.py:28-65) do not
exist here, and nothing falls back to PyTorch when the extension is missing.
"""
from __future__ import annotations

import torch

from . import _ops_real as _impl
from ._ops_real import _load_scaled_fp4_ops


def get_active_backend() -> str:
    """Always "real"; raises if the compiled extension cannot be loaded."""
    _load_scaled_fp4_ops(("scaled_fp4_quant_sm1xxa", "cutlass_scaled_fp4_mm"))
    return "real"


def scaled_fp4_quant(input: torch.Tensor, input_global_scale: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return _impl.scaled_fp4_quant(input, input_global_scale)


def cutlass_scaled_fp4_mm(a, b, block_scale_a, block_scale_b, alpha, out_dtype, bias=None) -> torch.Tensor:
    """The reference's signature plus an optional `bias` ([n], out_dtype) added in the GEMM epilogue."""
    return _impl.cutlass_scaled_fp4_mm(a, b, block_scale_a, block_scale_b, alpha, out_dtype, bias)


def reciprocal_approximate_ftz_tensor(x: torch.Tensor):
    y = torch.zeros_like(x)
    assert x.dtype == torch.float
    ext = _load_scaled_fp4_ops(("reciprocal_approximate_ftz_tensor",))
    ext.reciprocal_approximate_ftz_tensor(x.contiguous(), y)
    return y


# --- additions with no counterpart in the reference ---------------------------------
scaled_mxfp4_quant = _impl.scaled_mxfp4_quant
mxfp4_scaled_mm = _impl.mxfp4_scaled_mm
global_scale = _impl.global_scale
alpha_from_scales = _impl.alpha_from_scales
activation_scales = _impl.activation_scales
dynamic_scaled_fp4_quant = _impl.dynamic_scaled_fp4_quant
linear_forward = _impl.linear_forward
linear_forward_chained = _impl.linear_forward_chained
gated_mlp_forward = _impl.gated_mlp_forward
scaled_fp4_mm_fp4out = _impl.scaled_fp4_mm_fp4out
scaled_fp4_mm_silu_mul = _impl.scaled_fp4_mm_silu_mul
interleave_gate_up = _impl.interleave_gate_up


def device_status() -> int:
    """Synchronises and returns the device status word (0 = no kernel gave up a wait)."""
    return int(_load_scaled_fp4_ops(("device_status",)).device_status())
