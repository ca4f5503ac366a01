"""Pins to code compiled from the reference's own sources (oracle/_ref), for the paths whose other tests compare one
kernel of this package with another:

  * MXFP4 `floor` scale rounding against the reference's disabled UE8M0_SF branch
    (cvt_warp_fp16_to_fp4<Type, true>, kernel/nvfp4_utils.cuh:196-202 there);
  * the fused producers -- one-pass dynamic quantization, GEMM with NVFP4 output, gate/up GEMM with activation and
    NVFP4 output -- against the bytes of the reference quantizer kernel.
"""
import numpy as np
import pytest
import torch

from helpers import (capi_dynamic_quant, capi_mm, capi_mm_fp4out, capi_mx_quant, capi_quant, capi_rcp, load_ref_quantizer,
                     ref_quant, ref_quant_ue8m0, unswizzle_gpu)
from inputs import DISTRIBUTIONS, gemm_inputs, make_input

pytestmark = pytest.mark.gpu
REF = load_ref_quantizer()
needs_ref = pytest.mark.skipif(REF is None, reason="oracle/_ref (reference quantizer for sm_100a) not built")
needs_ue8m0 = pytest.mark.skipif(REF is None or not hasattr(REF, "scaled_fp4_quant_ue8m0"),
                                 reason="oracle/_ref was built without the e8m0 entry point: rerun oracle/build_oracle.py")
TORCH_DT = {"bf16": torch.bfloat16, "fp16": torch.float16}


def test_hardware_reciprocal_of_six_is_the_correctly_rounded_constant():
    """The reference forms block scales with rcp.approx.ftz(6.0f) (kernel/nvfp4_utils.cuh:192); the CPU restatements
    use fl(1/6) = 0x3E2AAAAB.  On sm_100 the two are the same number, so neither format has a constant to argue about."""
    r = capi_rcp(torch.tensor([6.0], dtype=torch.float32, device="cuda"))
    assert r.view(torch.int32).item() == 0x3E2AAAAB


@needs_ue8m0
@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_mxfp4_floor_mode_equals_the_reference_ue8m0_branch(dt):
    """The reference's e8m0 branch works on 16-element blocks, this package's MXFP4 on 32.  On an input whose every
    32-block is two copies of one 16-element half, both must pick the same scale (the block maximum is the same) and
    therefore the same nibbles: `floor` mode's packed bytes equal the reference's, and each 32-block scale byte
    equals both of the reference's 16-block bytes."""
    for dist in DISTRIBUTIONS + ("zeros_mixed", "specials", "student_t3"):
        for m, n in ((128, 128), (129, 96), (1, 4096), (300, 2048)):
            half = make_input(dist, (m, n // 2), TORCH_DT[dt], seed=17).reshape(m, n // 32, 1, 16)
            x = half.expand(m, n // 32, 2, 16).reshape(m, n).contiguous().cuda()
            r_fp4, r_sf = ref_quant_ue8m0(x)
            fp4, sf = capi_mx_quant(x, "floor")
            assert torch.equal(fp4, r_fp4), f"{dist} {m}x{n}: {(fp4 != r_fp4).sum().item()} packed bytes differ"
            r_lin = unswizzle_gpu(r_sf, m, n // 16)
            lin = unswizzle_gpu(sf, m, n // 32)
            assert torch.equal(r_lin[:, 0::2], r_lin[:, 1::2]), "reference halves disagree: the input is not what it should be"
            assert torch.equal(lin, r_lin[:, 0::2]), f"{dist} {m}x{n}: scale bytes differ"


@needs_ue8m0
def test_mxfp4_rceil_differs_from_floor_only_by_the_documented_rule():
    """`rceil` (the default) is a build decision, not the reference's branch: its scale byte is the floor byte plus one
    exactly where amax/6 is not a power of two, never otherwise."""
    x = make_input("student_t3", (256, 1024), torch.bfloat16, seed=19).cuda()
    _, sf_floor = capi_mx_quant(x, "floor")
    _, sf_ceil = capi_mx_quant(x, "rceil")
    lin_f = unswizzle_gpu(sf_floor, 256, 32).int()
    lin_c = unswizzle_gpu(sf_ceil, 256, 32).int()
    amax = x.float().reshape(256, 32, 32).abs().amax(-1)
    scaled = (amax * torch.tensor(0x3E2AAAAB, dtype=torch.int32).view(torch.float32).item()).to(torch.float32)
    pow2 = (scaled.view(torch.int32) & 0x7FFFFF) == 0
    assert torch.equal(lin_c - lin_f, (~pow2).int() * (lin_f < 254).int())


@needs_ref
@pytest.mark.parametrize("shape", [(16, 4096), (1, 4096), (128, 1024), (300, 2048), (4096, 1024), (2048, 8192)])
@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_one_pass_dynamic_quantization_vs_reference_kernel(shape, dt):
    """nvfp_dynamic_fp4_quant (one cluster / one cooperative launch / two launches, by size) against the reference
    kernel given the same global scale: identical packed bytes and identical valid scale bytes."""
    scratch = torch.zeros(8, dtype=torch.int32, device="cuda")
    for dist in ("normal", "outliers", "zeros_mixed"):
        x = make_input(dist, shape, TORCH_DT[dt], seed=23).cuda()
        fp4, sf, gs, _ = capi_dynamic_quant(x, scratch)
        amax = x.float().abs().max()
        assert gs.item() == (2688.0 / (amax if amax > 0 else torch.ones_like(amax))).item()
        r_fp4, r_sf = ref_quant(x, gs)
        assert torch.equal(fp4, r_fp4), (dist, shape)
        assert torch.equal(unswizzle_gpu(sf, shape[0], shape[1] // 16), unswizzle_gpu(r_sf, shape[0], shape[1] // 16))


def _quantized_operands(m, n, k, dt, seed):
    a, w = gemm_inputs(m, n, k, seed=seed, w_std=0.05)
    a, w = a.to(dt).cuda(), w.to(dt).cuda()
    ga = (2688.0 / a.float().abs().max()).reshape(1)
    gw = (2688.0 / w.float().abs().max()).reshape(1)
    a_fp4, a_sf = capi_quant(a, ga)
    w_fp4, w_sf = capi_quant(w, gw)
    return a_fp4, a_sf, w_fp4, w_sf, (1.0 / (ga * gw)).to(torch.float32)


@needs_ref
# shapes that take the few-rows kernel, the one-CTA tile kernel and the CTA-pair kernel
@pytest.mark.parametrize("m,n,k", [(16, 4096, 1024), (100, 512, 512), (300, 1024, 2048), (2048, 4096, 1024)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_gemm_with_nvfp4_output_vs_reference_kernel(m, n, k, dt):
    """nvfp_scaled_fp4_mm_fp4out against the REFERENCE quantizer applied to the GEMM's own 16-bit output."""
    a_fp4, a_sf, w_fp4, w_sf, alpha = _quantized_operands(m, n, k, dt, seed=m + n)
    plain = capi_mm(a_fp4, w_fp4, a_sf, w_sf, alpha, dt).contiguous()
    out_gs = (2688.0 / plain.float().abs().max()).reshape(1)
    r_fp4, r_sf = ref_quant(plain, out_gs)
    fp4, sf = capi_mm_fp4out(a_fp4, w_fp4, a_sf, w_sf, alpha, out_gs, dt)
    assert torch.equal(fp4, r_fp4), f"{(fp4 != r_fp4).sum().item()} packed bytes differ"
    assert torch.equal(unswizzle_gpu(sf, m, n // 16), unswizzle_gpu(r_sf, m, n // 16))


@needs_ref
@pytest.mark.parametrize("m,inter,k", [(16, 2048, 1024), (100, 512, 512), (300, 1440, 1024), (2048, 2048, 1024)])
def test_gate_up_gemm_with_activation_and_nvfp4_output_vs_reference_kernel(m, inter, k):
    """nvfp_scaled_fp4_mm_silu_mul with an output global scale against the REFERENCE quantizer applied to the same
    entry point's bf16 result."""
    import nvfp_kernel_b200 as nv
    torch.manual_seed(m + inter)
    x = torch.randn(m, k).to(torch.bfloat16).cuda()
    w_gu = nv.interleave_gate_up((torch.randn(inter, k) * 0.05).to(torch.bfloat16).cuda(),
                                 (torch.randn(inter, k) * 0.05).to(torch.bfloat16).cuda())
    gx, ggu = nv.global_scale(x), nv.global_scale(w_gu)
    x_fp4, x_sf = nv.scaled_fp4_quant(x, gx)
    gu_fp4, gu_sf = nv.scaled_fp4_quant(w_gu, ggu)
    alpha = nv.alpha_from_scales(gx, ggu)
    h = nv.scaled_fp4_mm_silu_mul(x_fp4, gu_fp4, x_sf, gu_sf, alpha, torch.bfloat16)
    gh = nv.global_scale(h)
    r_fp4, r_sf = ref_quant(h, gh)
    fp4, sf = nv.scaled_fp4_mm_silu_mul(x_fp4, gu_fp4, x_sf, gu_sf, alpha, torch.bfloat16, out_global_scale=gh)
    assert torch.equal(fp4, r_fp4)
    assert torch.equal(unswizzle_gpu(sf.view(torch.uint8), m, inter // 16), unswizzle_gpu(r_sf, m, inter // 16))
    assert nv.device_status() == 0
