"""ctypes wrapper of oracle/libnvfp_oracle.so (the C restatement, nvfp_oracle.c).

TEST INFRASTRUCTURE ONLY.  Inputs are torch CPU tensors or numpy arrays.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def load():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libnvfp_oracle.so")
        if not os.path.exists(path):
            from . import build_oracle
            build_oracle.build_c()
        lib = ctypes.CDLL(path)
        vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        lib.nvfp_oracle_quantize_nvfp4.argtypes = [vp, i32, i64, i64, i64, f32, vp, vp, i32, vp, vp]
        lib.nvfp_oracle_quantize_nvfp4.restype = None
        lib.nvfp_oracle_quantize_mxfp4.argtypes = [vp, i32, i64, i64, i64, i32, vp, vp]
        lib.nvfp_oracle_quantize_mxfp4.restype = None
        lib.nvfp_oracle_scaled_mm.argtypes = [vp, vp, vp, vp, f32, i64, i64, i64, i32, i32, vp]
        lib.nvfp_oracle_scaled_mm.restype = i32
        lib.nvfp_oracle_amax.argtypes = [vp, i32, i64, i64, i64]
        lib.nvfp_oracle_amax.restype = f32
        _LIB = lib
    return _LIB


def _raw16(x):
    """torch fp16/bf16 CPU tensor -> (uint16 numpy view [m, n], is_bf16)."""
    import torch
    x = x.detach().cpu().contiguous()
    x = x.reshape(-1, x.shape[-1])
    assert x.dtype in (torch.float16, torch.bfloat16)
    return x.view(torch.int16).numpy().view(np.uint16), int(x.dtype == torch.bfloat16)


def _sf_shape(m, n, block):
    return ((m + 127) // 128 * 128, (n // block + 3) // 4 * 4)


def quantize_nvfp4(x, gs: float, rcp_in=None, rcp_out=None):
    raw, is_bf16 = _raw16(x)
    m, n = raw.shape
    out = np.empty((m, n // 2), dtype=np.uint8)
    sf = np.empty(_sf_shape(m, n, 16), dtype=np.uint8)
    if rcp_in is not None:
        ri = np.ascontiguousarray(np.asarray(rcp_in, dtype=np.float32)).view(np.uint32)
        ro = np.ascontiguousarray(np.asarray(rcp_out, dtype=np.float32)).view(np.uint32)
        args = (ri.ctypes.data, ro.ctypes.data, len(ri))
    else:
        args = (None, None, 0)
    load().nvfp_oracle_quantize_nvfp4(raw.ctypes.data, is_bf16, m, n, n, float(np.float32(gs)), *args,
                                      out.ctypes.data, sf.ctypes.data)
    return out, sf


def quantize_mxfp4(x, rounding: str = "rceil"):
    raw, is_bf16 = _raw16(x)
    m, n = raw.shape
    out = np.empty((m, n // 2), dtype=np.uint8)
    sf = np.empty(_sf_shape(m, n, 32), dtype=np.uint8)
    load().nvfp_oracle_quantize_mxfp4(raw.ctypes.data, is_bf16, m, n, n, 0 if rounding == "rceil" else 1,
                                      out.ctypes.data, sf.ctypes.data)
    return out, sf


def scaled_mm(a, b, sfa, sfb, alpha: float, block: int = 16, ue8m0: bool = False) -> np.ndarray:
    a, b = np.ascontiguousarray(a, dtype=np.uint8), np.ascontiguousarray(b, dtype=np.uint8)
    sfa, sfb = np.ascontiguousarray(sfa, dtype=np.uint8), np.ascontiguousarray(sfb, dtype=np.uint8)
    m, k, n = a.shape[0], a.shape[1] * 2, b.shape[0]
    d = np.empty((m, n), dtype=np.float64)
    rc = load().nvfp_oracle_scaled_mm(a.ctypes.data, b.ctypes.data, sfa.ctypes.data, sfb.ctypes.data,
                                      float(np.float32(alpha)), m, n, k, block, int(ue8m0), d.ctypes.data)
    if rc:
        raise MemoryError("nvfp_oracle_scaled_mm")
    return d


def amax(x) -> float:
    raw, is_bf16 = _raw16(x)
    return float(load().nvfp_oracle_amax(raw.ctypes.data, is_bf16, raw.shape[0], raw.shape[1], raw.shape[1]))
