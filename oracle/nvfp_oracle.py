"""CPU oracle for the NVFP4 / MXFP4 quantize -> block-scaled GEMM path (numpy).

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module; it
is the checker used by the test-suite, by the smoke test and by the CPU-baseline
leg of the benchmark.  The product path is the CUDA library and fails loudly when
that library is missing.

Every function restates, in plain numpy, what the reference computes:

* quantizer arithmetic ........ kernel/nvfp4_utils.cuh:166-242 (authoritative,
  compiled with --use_fast_math, i.e. flush-to-zero fp32 multiplies) and the torch
  restatement nvfp/pseudo_quant.py:38-63
* nibble packing .............. kernel/nvfp4_utils.cuh:70-109, nvfp/pseudo_quant.py:15-28
* swizzled 128x4 scale layout . kernel/nvfp4_utils.cuh:111-156, nvfp/pseudo_quant.py:70-86,157-162
* dequantize .................. nvfp/pseudo_quant.py:138-180
* GEMM contract ............... kernel/nvfp4_scaled_mm_sm120_kernels.cu:74-90,151-164

Parity status: the NVFP4 quantizer is pinned by fixtures under tests/golden/
(outputs of the reference's own torch path, and of the reference's CUDA quantizer
built for sm_100a).  The MXFP4 functions have no counterpart that can be executed
in the reference (its e8m0 branch, kernel/nvfp4_utils.cuh:196-202, is unreachable):
MXFP4 parity is unpinned and is a self-consistency check only.

The reciprocal is injectable because the kernel uses the hardware approximation
``rcp.approx.ftz.f32`` (kernel/nvfp4_utils.cuh:159-163), which is not the correctly
rounded 1/x for every input.  ``rcp_true`` is the default; ``RcpTable`` replays
values captured from a GPU.
"""
from __future__ import annotations

import numpy as np

E2M1_MAX = 6.0
E4M3_MAX = 448.0
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
_F32_MIN_NORMAL = np.float32(2.0 ** -126)


# --------------------------------------------------------------------------- #
# fp32 helpers with the kernel's flush-to-zero semantics
# --------------------------------------------------------------------------- #
def _ftz(x: np.ndarray) -> np.ndarray:
    """Flush fp32 denormals to zero, keeping the sign."""
    x = np.asarray(x, dtype=np.float32)
    den = (np.abs(x) < _F32_MIN_NORMAL) & (x != 0)
    if den.any():
        x = np.where(den, np.copysign(np.float32(0), x), x)
    return x


def mul_ftz(a, b) -> np.ndarray:
    """``mul.ftz.f32``: denormal inputs and outputs are flushed (fast-math build,
    setup.py:45 of the reference)."""
    with np.errstate(all="ignore"):
        return _ftz(_ftz(a) * _ftz(b))


def rcp_true(x) -> np.ndarray:
    """Stand-in for ``rcp.approx.ftz.f32``: correctly rounded 1/x with ftz.  The
    hardware instruction may differ from this by one unit in the last place."""
    x = _ftz(x)
    with np.errstate(all="ignore"):
        r = (1.0 / x.astype(np.float64)).astype(np.float32)
    return _ftz(r)


class RcpTable:
    """Replays ``rcp.approx.ftz.f32`` results captured on a GPU (bit patterns)."""

    def __init__(self, inputs: np.ndarray, outputs: np.ndarray):
        ib = np.asarray(inputs, dtype=np.float32).view(np.uint32)
        ob = np.asarray(outputs, dtype=np.float32).view(np.uint32)
        self._map = dict(zip(ib.tolist(), ob.tolist()))

    def __call__(self, x) -> np.ndarray:
        x = np.asarray(x, dtype=np.float32)
        bits = np.ascontiguousarray(x).view(np.uint32)
        uniq, inv = np.unique(bits, return_inverse=True)

        def one(u: int) -> int:
            if u in self._map:
                return self._map[u]
            # not captured because no finite scale leads there: the instruction's results for NaN and infinity
            if (u & 0x7FFFFFFF) > 0x7F800000:
                return 0x7FFFFFFF                       # NaN in, NaN out
            if (u & 0x7FFFFFFF) == 0x7F800000:
                return u & 0x80000000                   # 1 / +-inf = +-0
            raise KeyError(f"reciprocal of bit pattern {u} was not captured")

        out = np.array([one(int(u)) for u in uniq], dtype=np.uint32)
        return out[inv].reshape(x.shape).view(np.float32)


def rcp_probe_inputs(gs: float) -> np.ndarray:
    """Every value the NVFP4 quantizer can feed to the reciprocal for one tensor:
    6.0, gs, and s'*rcp(gs) for the 126 positive finite e4m3 values s'.  The last
    group depends on rcp(gs) itself, so capture in two passes (see
    ``rcp_second_pass_inputs``)."""
    return np.array([6.0, gs], dtype=np.float32)


def rcp_second_pass_inputs(rcp_gs: float) -> np.ndarray:
    sf = e4m3_decode(np.arange(1, 127, dtype=np.uint8))
    return mul_ftz(sf, np.float32(rcp_gs))


# --------------------------------------------------------------------------- #
# element formats
# --------------------------------------------------------------------------- #
def e4m3_encode_satfinite(s) -> np.ndarray:
    """``cvt.rn.satfinite.e4m3x2.f32`` for non-negative inputs, as used by the
    ``__nv_fp8_e4m3(float)`` constructor at kernel/nvfp4_utils.cuh:205.
    Round to nearest even, saturate to 448, NaN -> 0x7f."""
    s = np.asarray(s, dtype=np.float32)
    nan = np.isnan(s)
    v = np.where(nan, 0, s).astype(np.float64)
    v = np.minimum(v, E4M3_MAX)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(v > 0, v, 1.0)))
    e = np.maximum(e, -6.0)
    step = np.exp2(e - 3.0)
    q = np.rint(v / step) * step  # rint is round-half-even
    q = np.minimum(q, E4M3_MAX)
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(q > 0, q, 1.0)))
    normal = q >= 2.0 ** -6
    mant = np.where(normal, q / np.exp2(e2) * 8.0 - 8.0, q * 512.0)
    expf = np.where(normal, e2 + 7.0, 0.0)
    byte = (expf.astype(np.int64) << 3) | mant.astype(np.int64)
    byte = np.where(nan, 0x7F, byte)
    return byte.astype(np.uint8)


def e4m3_decode(b) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8).astype(np.int64)
    e = (b >> 3) & 0xF
    m = b & 0x7
    val = np.where(e == 0, m * 2.0 ** -9, (8 + m) * np.exp2(e - 10.0))
    val = np.where((b & 0x7F) == 0x7F, np.nan, val)
    val = np.where(b & 0x80, -val, val)
    return val.astype(np.float32)


def e8m0_decode(b) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8).astype(np.float64)
    return np.where(b == 255, np.nan, np.exp2(b - 127.0))


def e2m1_encode(y) -> np.ndarray:
    """``cvt.rn.satfinite.e2m1x2.f32`` per element (kernel/nvfp4_utils.cuh:70-109):
    round to nearest, ties to the even code, |y| > 6 -> 6, sign in bit 3 (so -0 and
    tiny negatives give 0x8), NaN -> 0x7."""
    y = np.asarray(y, dtype=np.float32)
    a = np.abs(y).astype(np.float64)
    code = np.zeros(a.shape, dtype=np.uint8)
    # thresholds between consecutive codes; strict/inclusive chosen for ties-to-even
    code = np.where(a > 0.25, 1, code)
    code = np.where(a >= 0.75, 2, code)
    code = np.where(a > 1.25, 3, code)
    code = np.where(a >= 1.75, 4, code)
    code = np.where(a > 2.5, 5, code)
    code = np.where(a >= 3.5, 6, code)
    code = np.where(a > 5.0, 7, code)
    code = code.astype(np.uint8)
    sign = (np.signbit(y).astype(np.uint8) << 3)
    out = code | sign
    return np.where(np.isnan(y), np.uint8(0x7), out).astype(np.uint8)


def _block_absmax(xb) -> np.ndarray:
    """max |x| over the last axis the way __hmax2 / __hmax form it (kernel/nvfp4_utils.cuh:170-187): a NaN operand is
    skipped, the result is NaN only if every element is."""
    return np.fmax.reduce(np.abs(xb), axis=-1).astype(np.float32)


def e2m1_decode(nib) -> np.ndarray:
    nib = np.asarray(nib, dtype=np.uint8)
    v = E2M1_VALUES[nib & 0x7]
    return np.where(nib & 0x8, -v, v).astype(np.float32)


def pack_nibbles(nib: np.ndarray) -> np.ndarray:
    """Element 2j in bits 0-3 and element 2j+1 in bits 4-7 of byte j
    (kernel/nvfp4_utils.cuh:78-82; nvfp/pseudo_quant.py:15-20)."""
    nib = np.asarray(nib, dtype=np.uint8)
    assert nib.shape[-1] % 2 == 0
    return (nib[..., 0::2] | (nib[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


# --------------------------------------------------------------------------- #
# swizzled 128x4 scale-factor layout
# --------------------------------------------------------------------------- #
def round_up(x: int, y: int) -> int:
    return (x + y - 1) // y * y


def sf_swizzled_offset(m, kb, num_k_tiles):
    """Byte offset of the scale of (row m, K-block kb) in the
    [mTile][kTile][32][4][4] layout (kernel/nvfp4_utils.cuh:126-153)."""
    m = np.asarray(m, dtype=np.int64)
    kb = np.asarray(kb, dtype=np.int64)
    return ((m // 128) * (num_k_tiles * 512) + (kb // 4) * 512 + (m % 32) * 16
            + ((m % 128) // 32) * 4 + (kb % 4))


def swizzle_128x4(sf_linear: np.ndarray, pad_value: int = 0) -> np.ndarray:
    """[rows, sf_cols] -> padded, swizzled [round_up(rows,128), round_up(sf_cols,4)]
    (nvfp/pseudo_quant.py:70-86).  Padding is filled with ``pad_value``; the
    reference leaves it uninitialised."""
    rows, cols = sf_linear.shape
    mt, kt = (rows + 127) // 128, (cols + 3) // 4
    padded = np.full((mt * 128, kt * 4), pad_value, dtype=sf_linear.dtype)
    padded[:rows, :cols] = sf_linear
    t = padded.reshape(mt, 4, 32, kt, 4).transpose(0, 3, 2, 1, 4)
    return np.ascontiguousarray(t).reshape(mt * 128, kt * 4)


def unswizzle_128x4(sf_swz: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """Inverse of ``swizzle_128x4`` followed by slicing (nvfp/pseudo_quant.py:157-162)."""
    rp, cp = sf_swz.shape
    mt, kt = rp // 128, cp // 4
    t = sf_swz.reshape(mt, kt, 32, 4, 4).transpose(0, 3, 2, 1, 4)
    return np.ascontiguousarray(t).reshape(rp, cp)[:rows, :cols]


# --------------------------------------------------------------------------- #
# NVFP4 quantizer
# --------------------------------------------------------------------------- #
def _as_f32_matrix(x) -> np.ndarray:
    """Accepts a numpy float array or a torch fp16/bf16/fp32 tensor; returns the
    exact values as float32 [m, n]."""
    if hasattr(x, "detach"):
        x = x.detach().cpu().float().numpy()
    x = np.asarray(x, dtype=np.float32)
    return x.reshape(-1, x.shape[-1])


def nvfp4_quantize_kernel(x, global_scale, rcp=rcp_true, pad_value: int = 0):
    """Bit-level restatement of ``cvt_warp_fp16_to_fp4`` (kernel/nvfp4_utils.cuh:166-242).

    x: [m, n] values exactly representable in the kernel's input type (fp16/bf16),
    n % 16 == 0.  Returns (packed uint8 [m, n/2], swizzled scale bytes uint8
    [round_up(m,128), round_up(n/16,4)], linear scale bytes [m, n/16]).
    """
    x = _as_f32_matrix(x)
    m, n = x.shape
    assert n % 16 == 0
    gs = np.float32(global_scale)
    xb = x.reshape(m, n // 16, 16)
    amax = _block_absmax(xb)                                   # :170-187 (exact in input type)
    r6 = rcp(np.array([6.0], dtype=np.float32))[0]
    sf_value = mul_ftz(gs, mul_ftz(amax, r6))                   # :192
    sf_byte = e4m3_encode_satfinite(sf_value)                    # :205
    sf_q = e4m3_decode(sf_byte)                                  # :208
    rg = rcp(np.array([gs], dtype=np.float32))[0]
    denom = mul_ftz(sf_q, rg)
    out_scale = np.zeros_like(sf_q)                              # :213-216
    nz = sf_q != 0
    if nz.any():
        out_scale[nz] = rcp(denom[nz])
    y = mul_ftz(xb, out_scale[..., None].astype(np.float32))     # :224-235
    nib = e2m1_encode(y).reshape(m, n)                            # :238
    packed = pack_nibbles(nib)
    return packed, swizzle_128x4(sf_byte, pad_value), sf_byte


def nvfp4_quantize_torch_path(x, global_scale, rcp=rcp_true):
    """Restatement of the reference's torch quantizer ``pytorch_nvfp4_quantize``
    (nvfp/pseudo_quant.py:38-63): true division by 6, block scale clamped to
    [2^-6, 448] before the e4m3 cast, plain (non-flushing) fp32 multiplies, values
    clamped to [-6, 6].  Differs from the kernel only for blocks whose scaled amax is
    below 2^-6 (or which are all zero)."""
    x = _as_f32_matrix(x)
    m, n = x.shape
    assert n % 16 == 0
    gs = np.float32(global_scale)
    xb = x.reshape(m, n // 16, 16)
    amax = _block_absmax(xb)
    block_scale = (amax / np.float32(6.0)).astype(np.float32)
    scaled = (block_scale * gs).astype(np.float32)
    clamped = np.clip(scaled, np.float32(2.0 ** -6), np.float32(E4M3_MAX))
    sf_byte = e4m3_encode_satfinite(clamped)
    sf_q = e4m3_decode(sf_byte)
    rg = rcp(np.array([gs], dtype=np.float32))[0]
    with np.errstate(all="ignore"):
        total = (sf_q * rg).astype(np.float32)
        y = (xb * rcp(total)[..., None]).astype(np.float32)
    y = np.clip(y, -E2M1_MAX, E2M1_MAX)
    nib = e2m1_encode(y).reshape(m, n)
    return pack_nibbles(nib), swizzle_128x4(sf_byte, 0), sf_byte


def global_scale_from_amax(amax) -> np.float32:
    """gs = (448*6)/amax as torch evaluates `scalar / tensor`: fp32 reciprocal, then times
    2688 (speed_test.py:40-41, nvfp/pseudo_quant.py:94-96)."""
    return np.float32(np.float32(np.float32(1.0) / np.float32(amax)) * np.float32(E4M3_MAX * E2M1_MAX))


# --------------------------------------------------------------------------- #
# MXFP4 quantizer (32-element blocks, e8m0 scales, no global scale)
# --------------------------------------------------------------------------- #
def mxfp4_quantize(x, rounding: str = "rceil", pad_value: int = 0):
    """32-element MXFP4 quantizer.  The reference holds no reachable MXFP4 path; what it holds is a
    disabled e8m0 branch of its quantizer (kernel/nvfp4_utils.cuh:196-202: exponent bits of
    amax*rcp(6), 16-element blocks).  ``rounding="floor"`` is that branch widened to 32-element
    blocks, and is PINNED to it: tests/golden/ref_kernel_ue8m0_sm100.npz holds the branch's own
    output (compiled from the reference's sources, run on a B200) on inputs whose 32-blocks are two
    equal halves, and this function reproduces it byte for byte (tests/test_oracle_cpu.py).
    ``rounding="rceil"`` rounds the exponent up (the behaviour of ``cvt.rp.satfinite.ue8m0x2.f32``) so
    no element saturates: a build decision without a counterpart in the reference.  The element scale is
    the exact reciprocal power of two, applied with a flush-to-zero multiply.
    Returns (packed [m, n/2], swizzled e8m0 bytes, linear e8m0 bytes [m, n/32]).
    """
    x = _as_f32_matrix(x)
    m, n = x.shape
    assert n % 32 == 0
    xb = x.reshape(m, n // 32, 32)
    amax = _block_absmax(xb)
    r6 = rcp_true(np.array([6.0], dtype=np.float32))[0]
    sf_value = mul_ftz(amax, r6)
    bits = sf_value.view(np.uint32)
    exp = ((bits >> 23) & 0xFF).astype(np.int64)
    if rounding == "rceil":
        exp = np.where(((bits & 0x7FFFFF) != 0) & (exp < 254), exp + 1, exp)
    elif rounding != "floor":
        raise ValueError(rounding)
    nanblk = np.isnan(sf_value)
    # an infinite block maximum: the reference's branch stores the raw exponent bits, 255 (the e8m0 NaN code), and
    # `floor` follows it; `rceil` keeps the largest finite scale, 254
    exp = np.where(nanblk, 255, exp if rounding == "floor" else np.minimum(exp, 254))
    sf_byte = exp.astype(np.uint8)
    # 1 / 2^(exp-127) as an fp32 bit pattern; exp 0 (zero / flushed block) -> scale 0
    inv_bits = np.where((exp > 0) & (exp < 254), (254 - exp) << 23, 0).astype(np.uint32)
    inv = inv_bits.view(np.float32)
    y = mul_ftz(xb, inv[..., None])
    nib = e2m1_encode(y).reshape(m, n)
    return pack_nibbles(nib), swizzle_128x4(sf_byte, pad_value), sf_byte


# --------------------------------------------------------------------------- #
# dequantize and GEMM reference
# --------------------------------------------------------------------------- #
def dequantize(packed, sf_swizzled, global_scale=1.0, block: int = 16,
               scale_format: str = "e4m3") -> np.ndarray:
    """float64 [m, k] = e2m1 value * block scale / global scale
    (nvfp/pseudo_quant.py:166-180)."""
    packed = np.asarray(packed, dtype=np.uint8)
    m, kh = packed.shape
    k = kh * 2
    vals = e2m1_decode(unpack_nibbles(packed)).astype(np.float64).reshape(m, k // block, block)
    sf = unswizzle_128x4(np.asarray(sf_swizzled, dtype=np.uint8), m, k // block)
    sfv = e4m3_decode(sf).astype(np.float64) if scale_format == "e4m3" else e8m0_decode(sf)
    return (vals * (sfv / np.float64(global_scale))[..., None]).reshape(m, k)


def scaled_mm_reference(a_packed, b_packed, sfa, sfb, alpha, block: int = 16,
                        scale_format: str = "e4m3") -> np.ndarray:
    """float64 D = alpha * dequant(A) @ dequant(B)^T on the bytes the kernel consumes,
    not rounded to the output type (contract of
    kernel/nvfp4_scaled_mm_sm120_kernels.cu:151-164 with beta = 0)."""
    a = dequantize(a_packed, sfa, 1.0, block, scale_format)
    b = dequantize(b_packed, sfb, 1.0, block, scale_format)
    return np.float64(alpha) * (a @ b.T)


def gemm_tolerance_ok(out, ref, rel: float = 1e-2):
    """Stated tolerance: max|out-ref| <= rel*max|ref| and per element
    |out-ref| <= rel*|ref| + 2^-8*rms(ref).  Returns (ok, max_abs_err, max|ref|)."""
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    err = np.abs(out - ref)
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    mx = float(np.max(np.abs(ref))) if ref.size else 0.0
    ok = bool(np.all(np.isfinite(out))) and float(err.max(initial=0.0)) <= rel * mx + 1e-30 \
        and bool(np.all(err <= rel * np.abs(ref) + rms * 2.0 ** -8 + 1e-30))
    return ok, float(err.max(initial=0.0)), mx
