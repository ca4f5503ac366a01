"""The oracle against the reference's own outputs (tests/golden/ref_torch_path.npz, made by
running the reference's torch path), and the three restatements against each other."""
import hashlib
import os

import numpy as np
import pytest
import torch

from inputs import DISTRIBUTIONS, c1_inputs, make_input, mx_duplicated_halves
from oracle import c_oracle, nvfp_oracle as O, pseudo_path

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_torch_path.npz"))
CASES = [(d, s, t) for d in DISTRIBUTIONS for s in ((128, 128), (129, 80)) for t in ("bf16", "fp16")]
TORCH_DT = {"bf16": torch.bfloat16, "fp16": torch.float16}


def _case(dist, shape, dt):
    key = f"{dist}_{shape[0]}x{shape[1]}_{dt}"
    x = torch.from_numpy(GOLD[key + "_x"]).view(TORCH_DT[dt])
    return key, x, GOLD[key + "_gs"][0]


def test_fixture_inputs_reproducible():
    """The committed inputs are what the seeded generators produce on this machine."""
    for dist, shape, dt in CASES:
        key, x, _ = _case(dist, shape, dt)
        assert torch.equal(make_input(dist, shape, TORCH_DT[dt], seed=11).view(torch.int16), x.view(torch.int16)), key


def test_e2m1_codec_matches_reference():
    packed = O.pack_nibbles(O.e2m1_encode(GOLD["e2m1_probe_in"]).reshape(1, -1))
    assert np.array_equal(packed, GOLD["e2m1_probe_packed"])
    for code in range(16):
        v = O.e2m1_decode(np.uint8(code))
        assert O.e2m1_encode(v) == code or (code == 8 and O.e2m1_encode(v) == 8)


def test_e4m3_codec_matches_torch():
    vals = np.concatenate([np.linspace(0, 500, 20001), np.exp2(np.linspace(-12, 9, 4001)),
                           O.e4m3_decode(np.arange(0, 127, dtype=np.uint8)).astype(np.float64)]).astype(np.float32)
    ours = O.e4m3_encode_satfinite(vals)
    theirs = torch.from_numpy(np.minimum(vals, 448.0)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(ours, theirs)
    all_bytes = np.arange(0, 127, dtype=np.uint8)
    assert np.array_equal(O.e4m3_encode_satfinite(O.e4m3_decode(all_bytes)), all_bytes)
    assert np.array_equal(O.e4m3_decode(all_bytes),
                          torch.from_numpy(all_bytes).view(torch.float8_e4m3fn).float().numpy())


def test_swizzle_matches_reference():
    ramp = np.arange(256 * 8, dtype=np.int32).reshape(256, 8)
    assert np.array_equal(O.swizzle_128x4(ramp), GOLD["swizzle_ramp"])
    assert np.array_equal(O.unswizzle_128x4(O.swizzle_128x4(ramp), 256, 8), ramp)
    m, kb = np.meshgrid(np.arange(256), np.arange(8), indexing="ij")
    off = O.sf_swizzled_offset(m, kb, 2)
    assert np.array_equal(O.swizzle_128x4(ramp).reshape(-1)[off], ramp)
    ragged = np.arange(129 * 5, dtype=np.uint8).reshape(129, 5)
    sw = O.swizzle_128x4(ragged, pad_value=0)
    assert sw.shape == (256, 8)
    assert np.array_equal(O.unswizzle_128x4(sw, 129, 5), ragged)


@pytest.mark.parametrize("dist,shape,dt", CASES)
def test_torch_path_quantizer_matches_reference(dist, shape, dt):
    key, x, gs = _case(dist, shape, dt)
    fp4, swz, lin = O.nvfp4_quantize_torch_path(x, gs)
    assert np.array_equal(fp4, GOLD[key + "_fp4"])
    assert np.array_equal(lin, GOLD[key + "_sf_lin"])
    assert np.array_equal(O.unswizzle_128x4(swz, shape[0], shape[1] // 16), GOLD[key + "_sf_unswz"])
    if key + "_deq" in GOLD:
        assert np.array_equal(O.dequantize(fp4, swz, gs), GOLD[key + "_deq"])


@pytest.mark.parametrize("dist,shape,dt", CASES)
def test_kernel_semantics_agree_with_reference_outside_tiny_blocks(dist, shape, dt):
    """The kernel restatement differs from the torch path only where the scaled block
    amax is below 2^-6 (the torch path clamps the scale there)."""
    key, x, gs = _case(dist, shape, dt)
    fp4, _, lin = O.nvfp4_quantize_kernel(x, gs)
    xb = x.float().numpy().reshape(shape[0], -1, 16)
    scaled = np.abs(xb).max(-1) / 6.0 * gs
    normal = scaled >= 2.0 ** -6
    assert np.array_equal(lin[normal], GOLD[key + "_sf_lin"][normal])
    same = np.repeat(normal, 8, axis=1)
    assert np.array_equal(fp4[same], GOLD[key + "_fp4"][same])


@pytest.mark.parametrize("dist", DISTRIBUTIONS + ("zeros_mixed",))
@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_c_oracle_equals_numpy_oracle(dist, dt):
    x = make_input(dist, (131, 208), TORCH_DT[dt], seed=5)
    gs = O.global_scale_from_amax(x.float().abs().max().item() or 1.0)
    fp4, swz, _ = O.nvfp4_quantize_kernel(x, gs)
    cfp4, cswz = c_oracle.quantize_nvfp4(x, gs)
    assert np.array_equal(fp4, cfp4) and np.array_equal(swz, cswz)
    for rounding in ("rceil", "floor"):
        x32 = x[:, :192]
        mfp4, mswz, _ = O.mxfp4_quantize(x32, rounding)
        cm, cs = c_oracle.quantize_mxfp4(x32, rounding)
        assert np.array_equal(mfp4, cm) and np.array_equal(mswz, cs)
    assert c_oracle.amax(x) == x.float().abs().max().item()


def test_c_gemm_equals_numpy_gemm():
    a = make_input("normal", (70, 192), torch.bfloat16, 1)
    w = make_input("normal", (96, 192), torch.bfloat16, 2)
    ga = O.global_scale_from_amax(a.float().abs().max().item())
    gw = O.global_scale_from_amax(w.float().abs().max().item())
    af, asf, _ = O.nvfp4_quantize_kernel(a, ga)
    wf, wsf, _ = O.nvfp4_quantize_kernel(w, gw)
    alpha = np.float32(1.0) / (ga * gw)
    ref = O.scaled_mm_reference(af, wf, asf, wsf, alpha)
    got = c_oracle.scaled_mm(af, wf, asf, wsf, alpha)
    np.testing.assert_allclose(got, ref, rtol=1e-12, atol=0)
    # and it approximates the unquantized product
    exact = a.double().numpy() @ w.double().numpy().T
    assert np.abs(ref - exact).max() < 0.2 * np.abs(exact).max()
    mf, msf, _ = O.mxfp4_quantize(a)
    nf, nsf, _ = O.mxfp4_quantize(w)
    ref = O.scaled_mm_reference(mf, nf, msf, nsf, 1.0, block=32, scale_format="e8m0")
    got = c_oracle.scaled_mm(mf, nf, msf, nsf, 1.0, block=32, ue8m0=True)
    np.testing.assert_allclose(got, ref, rtol=1e-12, atol=0)


def test_mxfp4_properties():
    x = make_input("student_t3", (64, 256), torch.bfloat16, 3)
    for rounding in ("rceil", "floor"):
        fp4, swz, lin = O.mxfp4_quantize(x, rounding)
        deq = O.dequantize(fp4, swz, 1.0, block=32, scale_format="e8m0")
        amax = np.abs(x.float().numpy().reshape(64, -1, 32)).max(-1)
        scale = O.e8m0_decode(lin)
        if rounding == "rceil":
            assert (amax <= 6.0 * scale * (1 + 1e-6)).all()           # nothing saturates
            assert (amax > 3.0 * scale * (1 - 1e-6))[amax > 0].all()  # and the scale is tight
            assert np.abs(deq - x.double().numpy()).max() <= 0.5 * scale.max() * 2.0
        else:
            assert (amax >= 6.0 * scale * (1 - 1e-6))[amax > 0].all()
    # powers of two times 6 are represented exactly with either rounding
    y = torch.full((1, 32), 6.0 * 2.0 ** -3, dtype=torch.bfloat16)
    for rounding in ("rceil", "floor"):
        fp4, swz, lin = O.mxfp4_quantize(y, rounding)
        assert lin[0, 0] == 127 - 3 and (fp4 == 0x77).all()


@pytest.mark.parametrize("dist", DISTRIBUTIONS + ("zeros_mixed", "specials", "student_t3"))
def test_mxfp4_floor_restatement_matches_the_reference_ue8m0_branch(dist):
    """tests/golden/ref_kernel_ue8m0_sm100.npz holds what the reference's own e8m0 branch (16-element blocks,
    kernel/nvfp4_utils.cuh:196-202, compiled from its sources and run on a B200 by make_ref_kernel_golden.py)
    produced for inputs whose 32-blocks are two copies of one 16-element half.  The oracle's 32-block `floor`
    quantizer must give the same packed bytes, and its scale byte must equal both of the reference's."""
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_kernel_ue8m0_sm100.npz"))
    for shape in ((128, 128), (129, 96)):
        for dt in ("bf16", "fp16"):
            key = f"{dist}_{shape[0]}x{shape[1]}_{dt}"
            x = mx_duplicated_halves(dist, shape, TORCH_DT[dt], seed=17)
            fp4, _, lin = O.mxfp4_quantize(x, "floor")
            sf16 = gold[key + "_sf16"]
            assert np.array_equal(sf16[:, 0::2], sf16[:, 1::2]), key
            assert np.array_equal(lin, sf16[:, 0::2]), key
            assert np.array_equal(fp4, gold[key + "_fp4"]), (key, int((fp4 != gold[key + "_fp4"]).sum()))


def test_pseudo_path_port_matches_oracle_and_reference_c1():
    """BASELINE config 1 through the CPU-baseline port; hashes and output samples were
    produced by the reference's own torch path."""
    a, w = c1_inputs()
    sha = lambda arr: np.frombuffer(hashlib.sha256(np.ascontiguousarray(arr).tobytes()).digest(), dtype=np.uint8)
    assert np.array_equal(sha(a.view(torch.int16).numpy()), GOLD["c1_a_sha"]), "seeded input differs on this machine"
    assert np.array_equal(sha(w.view(torch.int16).numpy()), GOLD["c1_w_sha"])
    a_fp4, a_sf, a_gs = pseudo_path.quantize(a)
    w_fp4, w_sf, w_gs = pseudo_path.quantize(w)
    assert a_gs.item() == GOLD["c1_a_gs"][0] and w_gs.item() == GOLD["c1_w_gs"][0]
    assert np.array_equal(sha(a_fp4.numpy()), GOLD["c1_a_fp4_sha"])
    assert np.array_equal(sha(w_fp4.numpy()), GOLD["c1_w_fp4_sha"])
    assert np.array_equal(sha(a_sf.numpy()), GOLD["c1_a_sf_sha"])
    assert np.array_equal(sha(w_sf.numpy()), GOLD["c1_w_sf_sha"])
    o_fp4, o_sf, _ = O.nvfp4_quantize_torch_path(a, a_gs.item())
    assert np.array_equal(o_fp4, a_fp4.numpy()) and np.array_equal(o_sf, a_sf.numpy())
    y = pseudo_path.dequantize(a_fp4, a_sf, a_gs) @ pseudo_path.dequantize(w_fp4, w_sf, w_gs).T
    np.testing.assert_allclose(y[:64, :64].numpy(), GOLD["c1_y_corner"], rtol=1e-9, atol=1e-12)
    np.testing.assert_allclose(y[::97].numpy(), GOLD["c1_y_rows"], rtol=1e-9, atol=1e-12)
    # the oracle's GEMM reference reproduces the reference's float64 result
    alpha = np.float32(1.0) / (np.float32(a_gs.item()) * np.float32(w_gs.item()))
    ref = O.scaled_mm_reference(a_fp4.numpy()[:64], w_fp4.numpy()[:64], a_sf.numpy(), w_sf.numpy()[:128], alpha)
    np.testing.assert_allclose(ref, GOLD["c1_y_corner"], rtol=2e-6)


def test_rcp_table_replay():
    gs = np.float32(123.456)
    inp = np.concatenate([O.rcp_probe_inputs(gs), O.rcp_second_pass_inputs(O.rcp_true(np.array([gs]))[0])])
    table = O.RcpTable(inp, O.rcp_true(inp))
    x = make_input("normal", (16, 64), torch.bfloat16, 9)
    a = O.nvfp4_quantize_kernel(x, gs, rcp=table)
    b = O.nvfp4_quantize_kernel(x, gs)
    assert all(np.array_equal(u, v) for u, v in zip(a, b))


KERNEL_GOLD_PATH = os.path.join(os.path.dirname(__file__), "golden", "ref_kernel_sm100.npz")


@pytest.mark.skipif(not os.path.exists(KERNEL_GOLD_PATH), reason="reference-kernel fixture not generated")
@pytest.mark.parametrize("dist", DISTRIBUTIONS + ("zeros_mixed", "specials"))
def test_kernel_restatement_matches_reference_cuda_kernel_outputs(dist):
    """tests/golden/ref_kernel_sm100.npz holds outputs of the reference's own CUDA quantizer
    run on a B200, with the hardware reciprocals it used; the numpy and C restatements must
    reproduce its bytes exactly (tiny, zero and denormal blocks included)."""
    gold = np.load(KERNEL_GOLD_PATH)
    for shape in ((128, 128), (129, 80)):
        for dt in ("bf16", "fp16"):
            key = f"{dist}_{shape[0]}x{shape[1]}_{dt}"
            x = make_input(dist, shape, TORCH_DT[dt], seed=11)
            if key + "_x" in gold:
                assert np.array_equal(x.view(torch.int16).numpy(), gold[key + "_x"])
            gs, rin, rout = gold[key + "_gs"][0], gold[key + "_rcp_in"], gold[key + "_rcp_out"]
            fp4, _, lin = O.nvfp4_quantize_kernel(x, gs, rcp=O.RcpTable(rin, rout))
            assert np.array_equal(fp4, gold[key + "_fp4"]), key
            assert np.array_equal(lin, gold[key + "_sf"]), key
            c_fp4, c_sf = c_oracle.quantize_nvfp4(x, gs, rin, rout)
            assert np.array_equal(c_fp4, fp4) and np.array_equal(O.unswizzle_128x4(c_sf, shape[0], shape[1] // 16), lin)
