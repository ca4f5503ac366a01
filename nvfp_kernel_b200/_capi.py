"""ctypes view of libnvfp_b200.so (declarations: include/nvfp_b200.h).

Used by code that wants the C ABI without torch types in the way (tests, the smoke
test, the benchmark).  There is no fallback: a missing library raises.
"""
from __future__ import annotations

import ctypes
import os

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libnvfp_b200.so")

NVFP_OK = 0
NVFP_ERR_INVALID_ARGUMENT = 1
NVFP_ERR_CUDA = 2
NVFP_ERR_DEVICE_TIMEOUT = 3
NVFP_ERR_UNSUPPORTED = 4
NVFP_DTYPE_F16 = 0
NVFP_DTYPE_BF16 = 1
NVFP_DTYPE_F32 = 2
NVFP_MX_ROUND_CEIL = 0
NVFP_MX_ROUND_FLOOR = 1

_vp, _i64, _int = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int

# name -> (restype, argtypes); every symbol declared in include/nvfp_b200.h
PROTOTYPES = {
    "nvfp_last_error": (ctypes.c_char_p, []),
    "nvfp_version": (_int, []),
    "nvfp_sf_rows_padded": (_i64, [_i64]),
    "nvfp_sf_cols_padded": (_i64, [_i64, _int]),
    "nvfp_scaled_fp4_quant": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "nvfp_mxfp4_quant": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "nvfp_scaled_fp4_mm": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "nvfp_mxfp4_mm": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "nvfp_scaled_fp4_mm_multi": (_int, [ctypes.POINTER(ctypes.c_void_p), _int, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _int, _vp]),
    "nvfp_scaled_fp4_mm_scatter_add": (_int, [ctypes.POINTER(ctypes.c_void_p), _int, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "nvfp_scaled_fp4_mm_gather": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "nvfp_scaled_fp4_mm_reduce_scatter": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "nvfp_linear_forward_gather": (_int, [_vp, _i64, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _i64, _vp, _vp, _int, _vp]),
    "nvfp_scaled_fp4_mm_gather_fp4": (_int, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "nvfp_linear_forward_gather_fp4": (_int, [_vp, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _i64, _vp, _vp,
                                              _vp, _vp, _int, _vp]),
    "nvfp_reciprocal_approximate_ftz": (_int, [_vp, _vp, _i64, _vp]),
    "nvfp_global_scale": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "nvfp_activation_scales": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp]),
    "nvfp_scaled_fp4_mm_bias": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "nvfp_scaled_fp4_mm_fp4out": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "nvfp_scaled_fp4_mm_silu_mul": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "nvfp_linear_workspace_bytes": (_i64, [_i64, _i64]),
    "nvfp_linear_forward": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _int, _vp]),
    "nvfp_scaled_fp4_mm_amax": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp, _vp, _vp, _vp, _vp]),
    "nvfp_linear_forward_chained": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _int,
                                           _vp, _vp, _vp, _vp, _vp]),
    "nvfp_gated_mlp_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "nvfp_gated_mlp_forward": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64,
                                      _vp, _vp, _int, _vp]),
    "nvfp_dynamic_fp4_quant": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp]),
    "nvfp_global_scale_noalloc": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "nvfp_alpha_from_scales": (_int, [_vp, _vp, _vp, _vp]),
    "nvfp_device_status": (_int, [ctypes.POINTER(ctypes.c_uint32)]),
    "nvfp_selftest_wait_timeout": (_int, [ctypes.c_uint64, _vp]),
}

NVFP_MAX_RANKS = 8
NVFP_PEER_FLAG_WORDS = 32


class PeerGroup(ctypes.Structure):
    """nvfp_peer_group_t of include/nvfp_b200.h."""
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("dst", ctypes.c_void_p * NVFP_MAX_RANKS),
                ("flags", ctypes.c_void_p * NVFP_MAX_RANKS), ("wait_limit_ns", ctypes.c_uint64)]


_lib = None


class NvfpError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libnvfp_b200 status {code}: {message}")
        self.code = code


def lib_path() -> str:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Loads the shared library and attaches prototypes; raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m nvfp_kernel_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        lib = ctypes.CDLL(_LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != NVFP_OK:
        raise NvfpError(rc, load().nvfp_last_error().decode())


def device_status() -> int:
    """Synchronises the current device and returns (and clears) its status word."""
    word = ctypes.c_uint32(0)
    rc = load().nvfp_device_status(ctypes.byref(word))
    if rc not in (NVFP_OK, NVFP_ERR_DEVICE_TIMEOUT):
        check(rc)
    return word.value
