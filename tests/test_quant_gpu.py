"""NVFP4 / MXFP4 quantizer parity on the GPU, through the C ABI.

Bit-exactness authorities, in order: (1) the reference's own CUDA quantizer built for
sm_100a (oracle/_ref, run live here), (2) its committed outputs (tests/golden/
ref_kernel_sm100.npz), (3) the CPU oracle replaying the hardware reciprocal.
"""
import os

import numpy as np
import pytest
import torch

from helpers import capi_dynamic_quant, capi_global_scale, capi_mx_quant, capi_quant, capi_rcp, gpu_rcp_table, load_ref_quantizer
from inputs import DISTRIBUTIONS, make_input
from oracle import c_oracle, nvfp_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TORCH_DT = {"bf16": torch.bfloat16, "fp16": torch.float16}
ALL_DISTS = DISTRIBUTIONS + ("zeros_mixed",)
# with a given global scale the quantizers are also compared on infinities, NaNs, -0 and denormals
QUANT_DISTS = ALL_DISTS + ("specials",)


REF = load_ref_quantizer()
needs_ref = pytest.mark.skipif(REF is None, reason="oracle/_ref (reference quantizer for sm_100a) not built")


def _gs_for(x):
    amax = x.float().abs().max()
    return (torch.tensor(448.0 * 6.0) / (amax if amax > 0 else torch.tensor(1.0))).to(torch.float32).reshape(1)


def _ref_quant(x, gs):
    m, n = x.shape
    out = torch.empty((m, n // 2), dtype=torch.uint8, device="cuda")
    rm, rn = (m + 127) // 128 * 128, (n // 16 + 3) // 4 * 4
    sf = torch.full((rm, rn // 4), 0x55555555, dtype=torch.int32, device="cuda")
    REF.scaled_fp4_quant_sm1xxa(out, x, sf, gs)
    return out, sf.view(torch.uint8).reshape(rm, rn)


def _valid_sf(sf, m, n, block=16):
    return O.unswizzle_128x4(sf.cpu().numpy(), m, n // block)


def _padding_is_zero(sf, m, n, block=16):
    sfn = sf.cpu().numpy().copy()
    rp, cp = sfn.shape
    lin = O.unswizzle_128x4(sfn, rp, cp).copy()
    lin[:m, :n // block] = 0
    return not lin.any()


@needs_ref
@pytest.mark.parametrize("shape", [(128, 128), (129, 80), (1, 4096), (17, 14336), (16, 16), (300, 2048), (1024, 1024)])
@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_bit_exact_vs_reference_kernel(shape, dt):
    for dist in QUANT_DISTS:
        x = make_input(dist, shape, TORCH_DT[dt], seed=11).cuda()
        gs = _gs_for(x).cuda()
        r_fp4, r_sf = _ref_quant(x, gs)
        fp4, sf = capi_quant(x, gs)
        assert torch.equal(fp4, r_fp4), f"{dist}: packed nibbles differ in {(fp4 != r_fp4).sum().item()} bytes"
        assert np.array_equal(_valid_sf(sf, *shape), _valid_sf(r_sf, *shape)), f"{dist}: scale bytes differ"
        assert _padding_is_zero(sf, *shape), f"{dist}: scale padding not zero"


@needs_ref
@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_special_values_vs_reference_kernel(dt):
    """Infinities, NaNs, negative zero, denormals and the largest finite value inside otherwise ordinary blocks, and
    blocks made of nothing else: the bytes must be the reference kernel's, whatever it does with them."""
    tdt = TORCH_DT[dt]
    x = make_input("normal", (256, 512), tdt, seed=23)
    big = torch.finfo(tdt).max
    tiny = torch.finfo(tdt).smallest_normal
    specials = [float("inf"), -float("inf"), float("nan"), -0.0, tiny / 4, -tiny / 8, big, -big, 0.0]
    for i, v in enumerate(specials):
        x[3 + 7 * i, 5 + 16 * i] = v              # one special value in an ordinary block
        x[200 + i, 64:80] = v                     # a block of nothing else
        x[100 + i, 16 * i: 16 * i + 16:2] = v     # every other element of a block
    x = x.cuda()
    # ordinary global scales, then degenerate ones (zero, denormal, huge, infinite, NaN, negative)
    for gs_value in (1.0, 2688.0 / 4.0, 37.5, 0.0, 1e-39, 3e38, float("inf"), float("nan"), -2.0):
        gs = torch.tensor([gs_value], dtype=torch.float32, device="cuda")
        r_fp4, r_sf = _ref_quant(x, gs)
        fp4, sf = capi_quant(x, gs)
        assert torch.equal(fp4, r_fp4), f"gs {gs_value}: packed nibbles differ in {(fp4 != r_fp4).sum().item()} bytes"
        assert np.array_equal(_valid_sf(sf, 256, 512), _valid_sf(r_sf, 256, 512)), f"gs {gs_value}: scale bytes differ"


@needs_ref
def test_bit_exact_vs_reference_kernel_full_size():
    """BASELINE size 8192 x 8192 (bf16, N(0,1)) and the outlier-channel activations."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((8192, 8192), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    for variant in range(2):
        if variant == 1:
            x[:, ::97] *= 50
        gs = (2688.0 / x.float().abs().max()).reshape(1)
        r_fp4, r_sf = _ref_quant(x, gs)
        fp4, sf = capi_quant(x, gs)
        assert torch.equal(fp4, r_fp4)
        assert torch.equal(sf, r_sf)   # no padding at this shape: whole tensors must agree


def test_matches_committed_reference_kernel_outputs():
    path = os.path.join(ROOT, "tests", "golden", "ref_kernel_sm100.npz")
    if not os.path.exists(path):
        pytest.skip("tests/golden/ref_kernel_sm100.npz not generated yet")
    gold = np.load(path)
    for dist in QUANT_DISTS:
        for shape in ((128, 128), (129, 80)):
            for dt in ("bf16", "fp16"):
                key = f"{dist}_{shape[0]}x{shape[1]}_{dt}"
                x = make_input(dist, shape, TORCH_DT[dt], seed=11)
                gs = torch.from_numpy(gold[key + "_gs"])
                fp4, sf = capi_quant(x.cuda(), gs.cuda())
                assert np.array_equal(fp4.cpu().numpy(), gold[key + "_fp4"]), key
                assert np.array_equal(_valid_sf(sf, *shape), gold[key + "_sf"]), key


@pytest.mark.parametrize("dist", QUANT_DISTS)
@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_bit_exact_vs_cpu_oracle_with_hardware_reciprocal(dist, dt):
    for shape in ((129, 80), (256, 192)):
        x = make_input(dist, shape, TORCH_DT[dt], seed=11)
        gs = _gs_for(x)
        rin, rout = gpu_rcp_table(gs.item())
        fp4, sf = capi_quant(x.cuda(), gs.cuda())
        o_fp4, o_sf, _ = O.nvfp4_quantize_kernel(x, gs.item(), rcp=O.RcpTable(rin, rout))
        assert np.array_equal(fp4.cpu().numpy(), o_fp4), f"{dist} {shape}"
        assert np.array_equal(sf.cpu().numpy(), o_sf), f"{dist} {shape}"
        c_fp4, c_sf = c_oracle.quantize_nvfp4(x, gs.item(), rin, rout)
        assert np.array_equal(o_fp4, c_fp4) and np.array_equal(o_sf, c_sf)


def test_null_global_scale_means_one_and_strided_rows():
    x = make_input("normal", (64, 256), torch.bfloat16, 4).cuda()
    one = torch.ones(1, device="cuda")
    a = capi_quant(x, None)
    b = capi_quant(x, one)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    wide = make_input("normal", (64, 512), torch.bfloat16, 4).cuda()
    view = wide[:, 128:384]                 # row stride 512, 16-byte aligned start
    c = capi_quant(view, one)
    d = capi_quant(view.contiguous(), one)
    assert torch.equal(c[0], d[0]) and torch.equal(c[1], d[1])


def test_more_than_two_to_the_31_elements():
    """A tensor of 2.4e9 elements (49152 x 49152, 4.8 GB of bf16): element offsets no longer fit 32 bits.  The global
    scale equals torch's, and row bands from the start, the middle and the end quantize to the bytes the same rows give
    as a small tensor of their own (dynamic one-launch call included)."""
    m = n = 49152
    x = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    for r0 in range(0, m, 4096):                       # filled in bands to keep the temporaries small
        x[r0:r0 + 4096] = torch.randn((4096, n), generator=g, device="cuda").to(torch.bfloat16)
    x[m - 3, n - 5] = 40.0
    gs = capi_global_scale(x)
    assert gs.item() == ((448.0 * 6.0) / torch.tensor(40.0)).item()
    fp4, sf = capi_quant(x, gs)
    scratch = torch.zeros(8, dtype=torch.int32, device="cuda")
    d_fp4, d_sf, d_gs, _ = capi_dynamic_quant(x, scratch, None)
    assert torch.equal(d_gs, gs) and torch.equal(d_fp4, fp4) and torch.equal(d_sf, sf)
    del d_fp4, d_sf
    k_cols = n // 16
    for r0 in (0, 24576 - 128, m - 256):
        band = x[r0:r0 + 256].contiguous()
        b_fp4, b_sf = capi_quant(band, gs)
        assert torch.equal(fp4[r0:r0 + 256], b_fp4), r0
        assert torch.equal(sf[r0:r0 + 256], b_sf), r0          # 128-row scale tiles: whole tiles of the swizzled tensor


def test_rows_and_tiles_are_independent_full_size():
    """Size-independent properties at the BASELINE size: permuting rows permutes the
    output, and any aligned sub-block quantizes to the same bytes as the full tensor."""
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn((8192, 8192), generator=g, device="cuda").to(torch.bfloat16)
    gs = (2688.0 / x.float().abs().max()).reshape(1)
    fp4, sf = capi_quant(x, gs)
    perm = torch.randperm(8192, generator=g, device="cuda")
    p_fp4, p_sf = capi_quant(x[perm].contiguous(), gs)
    assert torch.equal(p_fp4, fp4[perm])
    lin = sf.reshape(64, 128, 32, 4, 4).transpose(1, 3).reshape(8192, 512)
    p_lin = p_sf.reshape(64, 128, 32, 4, 4).transpose(1, 3).reshape(8192, 512)
    assert torch.equal(p_lin, lin[perm])
    s_fp4, s_sf = capi_quant(x[1024:1536, 2048:3072].contiguous(), gs)
    assert torch.equal(s_fp4, fp4[1024:1536, 1024:1536])
    s_lin = s_sf.reshape(4, 16, 32, 4, 4).transpose(1, 3).reshape(512, 64)
    assert torch.equal(s_lin, lin[1024:1536, 128:192])
    # quantization error bound: |x - dequant| <= half a quantization step of the block
    vals = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], device="cuda")
    nib = torch.stack((fp4 & 0xF, fp4 >> 4), -1).reshape(8192, 8192).long()
    scale = lin.contiguous().view(torch.float8_e4m3fn).float() / gs
    deq = (vals[nib].reshape(8192, 512, 16) * scale.unsqueeze(-1)).reshape(8192, 8192)
    err = (deq - x.float()).abs().reshape(8192, 512, 16)
    assert (err <= scale.unsqueeze(-1) * 1.0 + 1e-6).all()   # coarsest step of e2m1 is 2 -> half step 1


@needs_ref
def test_reciprocal_op_bit_exact_vs_reference_op():
    g = torch.Generator().manual_seed(3)
    x = torch.cat([torch.randn(100000, generator=g) * 10, torch.tensor([0.0, -0.0, 1e-40, -1e-40, 6.0, 1e38, 3e38,
                   float("inf"), -float("inf"), 2.0 ** -126, 2.0 ** 126, 2.0 ** 127])]).cuda()
    mine = capi_rcp(x)
    theirs = torch.zeros_like(x)
    REF.reciprocal_approximate_ftz_tensor(x, theirs)
    assert torch.equal(mine.view(torch.int32), theirs.view(torch.int32))


def test_reciprocal_op_close_to_true_reciprocal():
    x = torch.linspace(0.001, 1000, 200001, device="cuda")
    y = capi_rcp(x)
    rel = ((y.double() - 1.0 / x.double()).abs() * x.double()).max().item()
    assert rel < 2.0 ** -22
    assert capi_rcp(torch.zeros(1, device="cuda")).item() == float("inf")


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_global_scale_of_a_tensor_with_nan_or_infinity_follows_torch(dt):
    """2688 / torch.abs(x).max() (speed_test.py:46-47 of the reference) is NaN as soon as one element is, and 0 when the
    maximum is infinite.  Every way to the global scale says the same: the sweep, the sweep that also forms alpha, and
    the dynamic quantizers (one cluster, one cooperative launch, two launches), whose bytes are those of the quantizer
    called with that scale."""
    tdt = TORCH_DT[dt]
    gs_w = torch.tensor([3.0], dtype=torch.float32, device="cuda")
    scratch = torch.zeros(8, dtype=torch.int32, device="cuda")
    for shape in ((16, 4096), (129, 80), (1024, 1024), (4096, 4096)):
        for special, check in ((float("nan"), lambda g: bool(torch.isnan(g).all())),
                               (-float("inf"), lambda g: g.item() == 0.0)):
            x = make_input("normal", shape, tdt, seed=31).cuda()
            x[shape[0] // 2, shape[1] // 3] = special
            want = (448.0 * 6.0) / torch.abs(x).max().to(torch.float32)
            assert check(want.reshape(1)), "the torch formula itself"
            gs = capi_global_scale(x)
            assert check(gs), (shape, special, gs.item())
            fp4, sf, gs_d, alpha = capi_dynamic_quant(x, scratch, gs_w)
            assert check(gs_d), (shape, special, gs_d.item())
            assert torch.isnan(alpha).all() if special != special else torch.isinf(alpha).all()
            q, qsf = capi_quant(x, gs_d)
            assert torch.equal(fp4, q) and torch.equal(sf, qsf), (shape, special)
    # and a clean tensor right after, with the same scratch words
    x = make_input("normal", (1024, 1024), tdt, seed=32).cuda()
    assert capi_dynamic_quant(x, scratch, gs_w)[2].item() == ((448.0 * 6.0) / torch.abs(x).max().to(torch.float32)).item()


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_global_scale_matches_torch_formula(dt):
    for dist in ALL_DISTS:
        for shape in ((1, 4096), (129, 80), (1024, 1024)):
            x = make_input(dist, shape, TORCH_DT[dt], seed=7).cuda()
            gs = capi_global_scale(x)
            amax = torch.abs(x).max().to(torch.float32)           # speed_test.py:46-47 of the reference
            want = (448.0 * 6.0) / amax
            assert gs.item() == want.item(), (dist, shape)
    z = torch.zeros((4, 64), dtype=TORCH_DT[dt], device="cuda")
    assert capi_global_scale(z).item() == 2688.0


def test_fused_activation_scales_repeated_calls():
    """One launch for gs and alpha with a scratch that is zeroed once and cleans itself: many calls in a
    row on tensors with rising and falling maxima must each equal the torch formulas of the reference
    (speed_test.py:46-49)."""
    import nvfp_kernel_b200 as nv
    scratch = torch.zeros(8, dtype=torch.int32, device="cuda")
    gs_w = torch.tensor([37.25], device="cuda")
    for i, (dist, shape) in enumerate([("large", (300, 2048)), ("small", (129, 80)), ("normal", (1, 4096)),
                                       ("abs_large", (1024, 1024)), ("small", (16, 16)), ("outliers", (4096, 512))] * 2):
        x = make_input(dist, shape, torch.bfloat16 if i % 2 else torch.float16, seed=i).cuda()
        gs, alpha = nv.activation_scales(x, gs_w, scratch)
        a_scale = (448.0 * 6.0) / torch.abs(x).max().to(torch.float32)
        assert gs.item() == a_scale.item(), (i, dist, shape)
        assert alpha.item() == (1.0 / (a_scale * gs_w)).item(), (i, dist, shape)
    z = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    assert nv.activation_scales(z, gs_w, scratch)[0].item() == 2688.0


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_one_pass_dynamic_quant_equals_global_scale_then_quantize(dt):
    """nvfp_dynamic_fp4_quant (maximum, global scale, alpha and quantization by one CTA for decode-sized tensors, in one
    cooperative launch while the tensor's tiles fit the GPU at once, two launches beyond) must give the bytes of the two-step flow of the
    reference (speed_test.py:46-49): gs = 2688/max|x|, then scaled_fp4_quant(x, gs).  One scratch, zeroed once,
    serves all calls, large and small shapes interleaved."""
    from helpers import capi_dynamic_quant
    scratch = torch.zeros(8, dtype=torch.int32, device="cuda")
    gs_w = torch.tensor([37.25], device="cuda")
    shapes = [(1, 4096), (16, 4096), (128, 14336), (129, 80), (300, 2064), (2368, 4096), (1, 16), (2432, 4096),
              (4096, 4096), (17, 8192), (8192, 1024), (4, 16384), (3, 16400), (128, 512), (100, 640), (5, 8192),
              (7, 9360)]
    for i, shape in enumerate(shapes):
        dist = ALL_DISTS[i % len(ALL_DISTS)]
        x = make_input(dist, shape, TORCH_DT[dt], seed=100 + i).cuda()
        fp4, sf, gs, alpha = capi_dynamic_quant(x, scratch, gs_w)
        want_gs = (448.0 * 6.0) / torch.abs(x).max().to(torch.float32)
        assert gs.item() == want_gs.item(), (dist, shape)
        assert alpha.item() == (1.0 / (want_gs * gs_w)).item(), (dist, shape)
        ref_fp4, ref_sf = capi_quant(x, gs)
        assert torch.equal(fp4, ref_fp4), (dist, shape)
        assert torch.equal(sf, ref_sf), (dist, shape)
    # strided rows, no weight scale (alpha untouched), all-zero input
    big = make_input("normal", (64, 512), TORCH_DT[dt], seed=5).cuda()
    view = big[:, 128:384]
    fp4, sf, gs, alpha = capi_dynamic_quant(view, scratch, None)
    assert torch.isnan(alpha).all()
    ref_fp4, ref_sf = capi_quant(view, gs)
    assert torch.equal(fp4, ref_fp4) and torch.equal(sf, ref_sf)
    assert gs.item() == ((448.0 * 6.0) / torch.abs(view).max().to(torch.float32)).item()
    z = torch.zeros((4, 64), dtype=TORCH_DT[dt], device="cuda")
    fp4, sf, gs, _ = capi_dynamic_quant(z, scratch, gs_w)
    assert gs.item() == 2688.0 and not fp4.any()


@pytest.mark.parametrize("rounding", ["rceil", "floor"])
@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_mxfp4_bit_exact_vs_cpu_restatement(rounding, dt):
    """CUDA against the CPU restatement, both roundings.  The restatement's `floor` mode is pinned to the reference's
    e8m0 branch (test_oracle_cpu.py, test_reference_pins_gpu.py); `rceil` is this package's own rule."""
    for dist in QUANT_DISTS + ("student_t3",):
        for shape in ((128, 128), (129, 96), (1, 4096), (300, 2048)):
            x = make_input(dist, shape, TORCH_DT[dt], seed=13)
            fp4, sf = capi_mx_quant(x.cuda(), rounding)
            o_fp4, o_sf, _ = O.mxfp4_quantize(x, rounding)
            assert np.array_equal(fp4.cpu().numpy(), o_fp4), (dist, shape)
            assert np.array_equal(sf.cpu().numpy(), o_sf), (dist, shape)


def test_python_api_matches_capi_and_reference_shapes():
    import nvfp_kernel_b200 as nv
    x = make_input("normal", (2, 65, 256), torch.bfloat16, 21).cuda()     # leading dims are flattened
    gs = nv.global_scale(x)
    fp4, sf = nv.scaled_fp4_quant(x, gs)
    assert fp4.shape == (130, 128) and fp4.dtype == torch.uint8
    assert sf.shape == (256, 16) and sf.dtype == torch.float8_e4m3fn
    c_fp4, c_sf = capi_quant(x.reshape(130, 256), gs)
    assert torch.equal(fp4, c_fp4) and torch.equal(sf.view(torch.uint8), c_sf)
    y = nv.reciprocal_approximate_ftz_tensor(torch.tensor([2.0, 4.0], device="cuda"))
    assert y.tolist() == [0.5, 0.25]
    m_fp4, m_sf = nv.scaled_mxfp4_quant(x)
    assert m_sf.dtype == torch.float8_e8m0fnu and m_sf.shape == (256, 8)
    with pytest.raises(AssertionError, match="multiple of 16"):
        nv.scaled_fp4_quant(torch.zeros(4, 24, dtype=torch.bfloat16, device="cuda"), gs)
    with pytest.raises(AssertionError, match="fp16 or bf16"):
        nv.scaled_fp4_quant(torch.zeros(4, 32, dtype=torch.float32, device="cuda"), gs)
    with pytest.raises(AssertionError, match="fp32"):
        nv.scaled_fp4_quant(torch.zeros(4, 32, dtype=torch.bfloat16, device="cuda"), gs.half())
    assert nv.device_status() == 0
