"""Port of the reference's torch pseudo-quant path, used as the timed CPU baseline.

TEST INFRASTRUCTURE ONLY.  Same sequence of torch operations as the reference
(quantize_linear_weight_to_nvfp4 + dequantize_to_dtype for both operands, then a float64
matmul: nvfp/pseudo_quant.py:38-63,70-99,138-180 and example.py:42-44 there), on CPU, with
the correctly rounded reciprocal standing in for the CUDA-only approximate one and the
e2m1 rounding written out instead of torch's private test helper.  Its quantizer output is
checked against oracle/nvfp_oracle.py (and so against the reference fixtures) by the tests.
"""
from __future__ import annotations

import torch

E2M1_MAX = 6.0
E4M3_MAX = 448.0
E4M3_TINY = 2.0 ** -6
_LUT = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=torch.float32)


def _e2m1_codes(y: torch.Tensor) -> torch.Tensor:
    a = y.abs()
    code = (a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8) + (a > 1.25).to(torch.uint8) \
        + (a >= 1.75).to(torch.uint8) + (a > 2.5).to(torch.uint8) + (a >= 3.5).to(torch.uint8) \
        + (a > 5.0).to(torch.uint8)
    return code | (torch.signbit(y).to(torch.uint8) << 3)


def _swizzle(sf: torch.Tensor) -> torch.Tensor:
    mn, sf_k = sf.shape
    mt, kt = (mn + 127) // 128, (sf_k + 3) // 4
    padded = torch.zeros((mt * 128, kt * 4), dtype=sf.dtype)
    padded[:mn, :sf_k] = sf
    return padded.reshape(mt, 4, 32, kt, 4).transpose(1, 3).reshape(mt * 128, kt * 4)


def _unswizzle(sf: torch.Tensor, mn: int, sf_k: int) -> torch.Tensor:
    rp, cp = sf.shape
    return sf.reshape(rp // 128, cp // 4, 32, 4, 4).transpose(1, 3).reshape(rp, cp)[:mn, :sf_k]


def quantize(x: torch.Tensor):
    """-> (packed uint8 [m, k/2], swizzled e4m3 scales as uint8, fp32 global scale)."""
    gs = ((E4M3_MAX * E2M1_MAX) / x.float().abs().amax()).to(torch.float32)
    m, k = x.shape
    xb = x.float().reshape(m, k // 16, 16)
    block_scale = (xb.abs().amax(dim=-1) / E2M1_MAX).float()
    sf8 = torch.clamp(block_scale * gs, min=E4M3_TINY, max=E4M3_MAX).to(torch.float8_e4m3fn)
    total = sf8.float() * (1.0 / gs.double()).float()
    y = torch.clamp(xb * (1.0 / total.double()).float().unsqueeze(-1), -E2M1_MAX, E2M1_MAX).reshape(m, k)
    codes = _e2m1_codes(y)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return packed, _swizzle(sf8.view(torch.uint8)), gs


def dequantize(packed: torch.Tensor, sf_swz: torch.Tensor, gs: torch.Tensor) -> torch.Tensor:
    m, kh = packed.shape
    k = kh * 2
    lo, hi = packed & 0xF, packed >> 4
    nib = torch.stack((lo, hi), dim=-1).reshape(m, k)
    vals = _LUT[(nib & 7).long()]
    vals = torch.where((nib & 8) != 0, -vals, vals).reshape(m, k // 16, 16)
    sf = _unswizzle(sf_swz, m, k // 16).view(torch.float8_e4m3fn).to(torch.double) / gs
    return (vals * sf.unsqueeze(-1)).reshape(m, k)


def pseudo_quant_linear(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """float64 [M, N]: what the reference computes as
    nvfp4_pseudo_quantize(a) @ nvfp4_pseudo_quantize(w).T (example.py:42-44)."""
    return dequantize(*quantize(a)) @ dequantize(*quantize(w)).T
