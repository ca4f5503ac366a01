"""Helpers for the GPU parity tests: calls through the C ABI (ctypes) with torch tensors
as device buffers, and comparison utilities."""
from __future__ import annotations

import importlib.util
import os

import torch

from nvfp_kernel_b200 import _capi

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_REF = []


def load_ref_quantizer():
    """The reference's own CUDA quantizer built for sm_100a (oracle/_ref, recipe oracle/build_oracle.py), or None
    when it has not been built.  Test infrastructure only."""
    if not _REF:
        mod = None
        d = os.path.join(_ROOT, "oracle", "_ref")
        names = [f for f in os.listdir(d) if f.startswith("ref_scaled_fp4_ops") and f.endswith(".so")] if os.path.isdir(d) else []
        if names and torch.cuda.is_available():
            spec = importlib.util.spec_from_file_location("ref_scaled_fp4_ops", os.path.join(d, names[0]))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
        _REF.append(mod)
    return _REF[0]


def ref_quant(x: torch.Tensor, gs: torch.Tensor):
    """NVFP4 bytes of the reference kernel: (packed [m, n/2], swizzled scale bytes with 0x55 where it writes nothing)."""
    ref = load_ref_quantizer()
    m, n = x.shape
    out = torch.empty((m, n // 2), dtype=torch.uint8, device="cuda")
    rm, rn = sf_shape(m, n, 16)
    sf = torch.full((rm, rn // 4), 0x55555555, dtype=torch.int32, device="cuda")
    ref.scaled_fp4_quant_sm1xxa(out, x.contiguous(), sf, gs)
    return out, sf.view(torch.uint8).reshape(rm, rn)


def ref_quant_ue8m0(x: torch.Tensor):
    """The reference's e8m0 branch (16-element blocks, no global scale): (packed, swizzled ue8m0 scale bytes)."""
    ref = load_ref_quantizer()
    m, n = x.shape
    out = torch.empty((m, n // 2), dtype=torch.uint8, device="cuda")
    rm, rn = sf_shape(m, n, 16)
    sf = torch.full((rm, rn // 4), 0x55555555, dtype=torch.int32, device="cuda")
    ref.scaled_fp4_quant_ue8m0(out, x.contiguous(), sf)
    return out, sf.view(torch.uint8).reshape(rm, rn)


def unswizzle_gpu(sf_swz: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """[rowTile][kTile][32][4][4] bytes -> the valid [rows, cols] scale bytes."""
    rp, cp = sf_swz.shape
    return sf_swz.reshape(rp // 128, cp // 4, 32, 4, 4).transpose(1, 3).reshape(rp, cp)[:rows, :cols]


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.dtype) -> int:
    return {torch.float16: _capi.NVFP_DTYPE_F16, torch.bfloat16: _capi.NVFP_DTYPE_BF16,
            torch.float32: _capi.NVFP_DTYPE_F32}[t]


def sf_shape(m: int, n: int, block: int):
    return ((m + 127) // 128 * 128, (n // block + 3) // 4 * 4)


def capi_quant(x: torch.Tensor, gs: torch.Tensor | None, fill: int = 0xAA):
    """NVFP4 quantize through nvfp_scaled_fp4_quant.  Outputs are pre-filled with `fill`
    so that bytes the kernel does not write are visible."""
    lib = _capi.load()
    m, n = x.shape
    out = torch.full((m, n // 2), fill, dtype=torch.uint8, device=x.device)
    sf = torch.full(sf_shape(m, n, 16), fill, dtype=torch.uint8, device=x.device)
    _capi.check(lib.nvfp_scaled_fp4_quant(out.data_ptr(), sf.data_ptr(), x.data_ptr(),
                                          gs.data_ptr() if gs is not None else None, m, n,
                                          x.stride(0) if m > 1 else n, _dt(x.dtype), _stream()))
    return out, sf


def capi_mx_quant(x: torch.Tensor, rounding: str = "rceil", fill: int = 0xAA):
    lib = _capi.load()
    m, n = x.shape
    out = torch.full((m, n // 2), fill, dtype=torch.uint8, device=x.device)
    sf = torch.full(sf_shape(m, n, 32), fill, dtype=torch.uint8, device=x.device)
    _capi.check(lib.nvfp_mxfp4_quant(out.data_ptr(), sf.data_ptr(), x.data_ptr(), m, n,
                                     x.stride(0) if m > 1 else n, _dt(x.dtype),
                                     0 if rounding == "rceil" else 1, _stream()))
    return out, sf


def capi_mm(a, b, sfa, sfb, alpha, out_dtype=torch.bfloat16, mx: bool = False, bias=None):
    lib = _capi.load()
    m, n, k = a.shape[0], b.shape[0], a.shape[1] * 2
    # canary-padded output: the kernel must not write outside [m, n]
    buf = torch.full((m * n + 256,), float("nan"), dtype=out_dtype, device=a.device)
    d = buf[128:128 + m * n].view(m, n)
    alpha_ptr = alpha.data_ptr() if alpha is not None else None
    if bias is not None:
        assert bias.dtype == out_dtype and bias.numel() == n
        _capi.check(lib.nvfp_scaled_fp4_mm_bias(d.data_ptr(), a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                                                alpha_ptr, bias.data_ptr(), m, n, k, _dt(out_dtype), 1 if mx else 0,
                                                _stream()))
    else:
        fn = lib.nvfp_mxfp4_mm if mx else lib.nvfp_scaled_fp4_mm
        _capi.check(fn(d.data_ptr(), a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), alpha_ptr, m, n, k,
                       _dt(out_dtype), _stream()))
    assert _capi.device_status() == 0, "a kernel gave up on a bounded wait"
    assert torch.isnan(buf[:128]).all() and torch.isnan(buf[128 + m * n:]).all(), "out-of-bounds write"
    return d


def capi_global_scale(x: torch.Tensor) -> torch.Tensor:
    lib = _capi.load()
    gs = torch.empty(1, dtype=torch.float32, device=x.device)
    scratch = torch.empty(2, dtype=torch.int32, device=x.device)
    m, n = x.shape
    _capi.check(lib.nvfp_global_scale(gs.data_ptr(), scratch.data_ptr(), x.data_ptr(), m, n,
                                      x.stride(0) if m > 1 else n, _dt(x.dtype), _stream()))
    return gs


def capi_dynamic_quant(x: torch.Tensor, scratch: torch.Tensor, gs_weight: torch.Tensor | None = None, fill: int = 0xAA):
    """One-pass dynamic NVFP4 quantization through nvfp_dynamic_fp4_quant: (fp4, scales, gs, alpha)."""
    lib = _capi.load()
    m, n = x.shape
    out = torch.full((m, n // 2), fill, dtype=torch.uint8, device=x.device)
    sf = torch.full(sf_shape(m, n, 16), fill, dtype=torch.uint8, device=x.device)
    scal = torch.full((2,), float("nan"), dtype=torch.float32, device=x.device)
    _capi.check(lib.nvfp_dynamic_fp4_quant(out.data_ptr(), sf.data_ptr(), scal[:1].data_ptr(), scal[1:].data_ptr(),
                                           scratch.data_ptr(), x.data_ptr(), m, n, x.stride(0) if m > 1 else n,
                                           _dt(x.dtype), gs_weight.data_ptr() if gs_weight is not None else None,
                                           _stream()))
    assert _capi.device_status() == 0, "a kernel gave up on a bounded wait"
    return out, sf, scal[:1], scal[1:]


def capi_mm_fp4out(a, b, sfa, sfb, alpha, out_gs, value_dtype=torch.bfloat16, mx: bool = False, bias=None, fill: int = 0xAA):
    """GEMM whose result leaves as NVFP4 (nvfp_scaled_fp4_mm_fp4out): (packed [m, n/2], swizzled scales)."""
    lib = _capi.load()
    m, n, k = a.shape[0], b.shape[0], a.shape[1] * 2
    out = torch.full((m, n // 2), fill, dtype=torch.uint8, device=a.device)
    sf = torch.full(sf_shape(m, n, 16), fill, dtype=torch.uint8, device=a.device)
    _capi.check(lib.nvfp_scaled_fp4_mm_fp4out(out.data_ptr(), sf.data_ptr(), a.data_ptr(), b.data_ptr(), sfa.data_ptr(),
                                              sfb.data_ptr(), alpha.data_ptr() if alpha is not None else None,
                                              bias.data_ptr() if bias is not None else None, out_gs.data_ptr(), m, n, k,
                                              _dt(value_dtype), 1 if mx else 0, _stream()))
    assert _capi.device_status() == 0, "a kernel gave up on a bounded wait"
    return out, sf


def capi_linear_forward(x, w_fp4, w_sf, w_gs, scratch, out_dtype=torch.bfloat16, bias=None):
    """Whole layer forward through nvfp_linear_forward."""
    lib = _capi.load()
    m, k = x.shape
    n = w_fp4.shape[0]
    buf = torch.full((m * n + 256,), float("nan"), dtype=out_dtype, device=x.device)
    d = buf[128:128 + m * n].view(m, n)
    ws = torch.empty(lib.nvfp_linear_workspace_bytes(m, k), dtype=torch.uint8, device=x.device)
    _capi.check(lib.nvfp_linear_forward(d.data_ptr(), x.data_ptr(), m, k, x.stride(0) if m > 1 else k, _dt(x.dtype),
                                        w_fp4.data_ptr(), w_sf.data_ptr(), w_gs.data_ptr(), n,
                                        bias.data_ptr() if bias is not None else None, ws.data_ptr(),
                                        scratch.data_ptr(), _dt(out_dtype), _stream()))
    assert _capi.device_status() == 0, "a kernel gave up on a bounded wait"
    assert torch.isnan(buf[:128]).all() and torch.isnan(buf[128 + m * n:]).all(), "out-of-bounds write"
    return d


def capi_gated_mlp_forward(x, gu_fp4, gu_sf, gu_gs, d_fp4, d_sf, act_gs, down_alpha, scratch, out_dtype=torch.bfloat16):
    """Whole gated MLP through nvfp_gated_mlp_forward."""
    lib = _capi.load()
    m, hidden = x.shape
    inter, n = gu_fp4.shape[0] // 2, d_fp4.shape[0]
    buf = torch.full((m * n + 256,), float("nan"), dtype=out_dtype, device=x.device)
    y = buf[128:128 + m * n].view(m, n)
    ws = torch.empty(lib.nvfp_gated_mlp_workspace_bytes(m, hidden, inter), dtype=torch.uint8, device=x.device)
    _capi.check(lib.nvfp_gated_mlp_forward(y.data_ptr(), x.data_ptr(), m, hidden, x.stride(0) if m > 1 else hidden,
                                           _dt(x.dtype), gu_fp4.data_ptr(), gu_sf.data_ptr(), gu_gs.data_ptr(), inter,
                                           d_fp4.data_ptr(), d_sf.data_ptr(), act_gs.data_ptr(), down_alpha.data_ptr(), n,
                                           ws.data_ptr(), scratch.data_ptr(), _dt(out_dtype), _stream()))
    assert _capi.device_status() == 0, "a kernel gave up on a bounded wait"
    assert torch.isnan(buf[:128]).all() and torch.isnan(buf[128 + m * n:]).all(), "out-of-bounds write"
    return y


def capi_rcp(x: torch.Tensor) -> torch.Tensor:
    lib = _capi.load()
    y = torch.empty_like(x)
    _capi.check(lib.nvfp_reciprocal_approximate_ftz(y.data_ptr(), x.data_ptr(), x.numel(), _stream()))
    return y


def gpu_rcp_table(gs: float, device="cuda"):
    """(inputs, outputs) of the hardware reciprocal for every value the NVFP4 quantizer
    can feed it for global scale `gs`: lets the CPU oracle replay rcp.approx.ftz exactly."""
    from oracle import nvfp_oracle as O
    first = torch.tensor([6.0, gs], dtype=torch.float32, device=device)
    r1 = capi_rcp(first)
    second = torch.from_numpy(O.rcp_second_pass_inputs(r1[1].item())).to(device)
    r2 = capi_rcp(second)
    return (torch.cat([first, second]).cpu().numpy(), torch.cat([r1, r2]).cpu().numpy())


def dequant_gpu(packed: torch.Tensor, sf_swz: torch.Tensor, block: int, ue8m0: bool, dtype=torch.float32):
    """value * block scale on the GPU (exact in bf16 and fp32), [rows, k]."""
    rows, kh = packed.shape
    k = kh * 2
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6],
                       dtype=torch.float32, device=packed.device)
    nib = torch.stack((packed & 0xF, packed >> 4), dim=-1).reshape(rows, k).long()
    vals = lut[nib]
    rp, cp = sf_swz.shape
    sf = sf_swz.reshape(rp // 128, cp // 4, 32, 4, 4).transpose(1, 3).reshape(rp, cp)[:rows, :k // block]
    sf = sf.contiguous().view(torch.float8_e8m0fnu if ue8m0 else torch.float8_e4m3fn).float()
    return (vals.reshape(rows, k // block, block) * sf.unsqueeze(-1)).reshape(rows, k).to(dtype)


def check_gemm(out: torch.Tensor, ref: torch.Tensor, rel: float = 1e-2):
    """Tolerance of the GEMM contract: max|out-ref| <= rel*max|ref| and per element
    |out-ref| <= rel*|ref| + 2^-8 * rms(ref)."""
    out, ref = out.double(), ref.double()
    assert torch.isfinite(out).all(), "non-finite output"
    err = (out - ref).abs()
    rms = ref.pow(2).mean().sqrt()
    mx = ref.abs().max()
    assert err.max() <= rel * mx + 1e-30, f"max err {err.max().item():.4g} vs max|ref| {mx.item():.4g}"
    bad = err > rel * ref.abs() + rms * 2.0 ** -8 + 1e-30
    assert not bad.any(), f"{int(bad.sum())} elements outside tolerance; worst {err.max().item():.4g}"
    return float(err.max()), float(mx)


def capi_mm_gather_fp4(a, b, sfa, sfb, alpha, out_gs, packed_bases, sf_bases, n_total, n_offset, rank=0, flags=None,
                       value_dtype=torch.bfloat16, bias=None, wait_limit_ns=0):
    """nvfp_scaled_fp4_mm_gather_fp4: this rank's [m, n] product quantized in the epilogue and stored at columns
    [n_offset, n_offset + n) of every destination (device tensors: packed [m, n_total / 2], scales swizzled)."""
    import ctypes
    lib = _capi.load()
    m, n, k = a.shape[0], b.shape[0], a.shape[1] * 2
    g = _capi.PeerGroup()
    g.world, g.rank, g.wait_limit_ns = len(packed_bases), rank, wait_limit_ns
    sf_arr = (ctypes.c_void_p * _capi.NVFP_MAX_RANKS)()
    for r, (pk, sf) in enumerate(zip(packed_bases, sf_bases)):
        g.dst[r] = pk.data_ptr() if hasattr(pk, "data_ptr") else pk
        sf_arr[r] = sf.data_ptr() if hasattr(sf, "data_ptr") else sf
        if flags is not None:
            g.flags[r] = flags[r].data_ptr() if hasattr(flags[r], "data_ptr") else flags[r]
    _capi.check(lib.nvfp_scaled_fp4_mm_gather_fp4(ctypes.byref(g), sf_arr, n_total, n_offset, a.data_ptr(), b.data_ptr(),
                                                  sfa.data_ptr(), sfb.data_ptr(), alpha.data_ptr() if alpha is not None else None,
                                                  bias.data_ptr() if bias is not None else None, out_gs.data_ptr(), m, n, k,
                                                  _dt(value_dtype), 0, _stream()))
