"""The C-ABI library without a GPU: it loads, exports every symbol the header declares
(and nothing is declared that is not exported), and its pure-host entry points work."""
import ctypes
import os
import re

import pytest
import torch

from nvfp_kernel_b200 import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "nvfp_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nvfp_[a-z0-9_]+)\s*\(", text)))


def test_header_and_library_agree():
    lib = _capi.load()
    declared = _declared_symbols()
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/nvfp_b200.h but not exported"
    assert sorted(_capi.PROTOTYPES) == declared, "ctypes prototypes and header differ"


def test_host_only_entry_points():
    lib = _capi.load()
    assert lib.nvfp_version() >= 1000
    assert lib.nvfp_sf_rows_padded(1) == 128 and lib.nvfp_sf_rows_padded(129) == 256
    assert lib.nvfp_sf_cols_padded(80, 16) == 8 and lib.nvfp_sf_cols_padded(8192, 16) == 512
    assert lib.nvfp_sf_cols_padded(8192, 32) == 256
    assert lib.nvfp_last_error() is not None
    # workspaces: quantized activation + scales + two scalars; the MLP adds the quantized hidden activation
    lin = lib.nvfp_linear_workspace_bytes(300, 1024)
    assert lin == 300 * 512 + 384 * 64 + 256 and lin % 256 == 0
    assert lib.nvfp_gated_mlp_workspace_bytes(300, 1024, 2048) == lin + 300 * 1024 + 384 * 128
    assert lib.nvfp_linear_workspace_bytes(-1, 64) == -1 and lib.nvfp_gated_mlp_workspace_bytes(1, 64, -64) == -1


def test_argument_validation_needs_no_gpu():
    """Bad arguments are rejected on the host, before any CUDA call."""
    lib = _capi.load()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf) // 16 * 16 + 16
    rc = lib.nvfp_scaled_fp4_quant(p, p, p, None, 4, 24, 24, _capi.NVFP_DTYPE_BF16, None)
    assert rc == _capi.NVFP_ERR_INVALID_ARGUMENT and b"multiple of 16" in lib.nvfp_last_error()
    rc = lib.nvfp_scaled_fp4_quant(p, p, p, None, 4, 32, 32, 7, None)
    assert rc == _capi.NVFP_ERR_INVALID_ARGUMENT and b"data type" in lib.nvfp_last_error()
    rc = lib.nvfp_scaled_fp4_mm(p, p, p, p, p, p, 4, 32, 48, _capi.NVFP_DTYPE_BF16, None)
    assert rc == _capi.NVFP_ERR_INVALID_ARGUMENT and b"divisible by 32" in lib.nvfp_last_error()
    rc = lib.nvfp_scaled_fp4_mm(p, p, p, p, p, p, 4, 40, 64, _capi.NVFP_DTYPE_BF16, None)
    assert rc == _capi.NVFP_ERR_INVALID_ARGUMENT and b"n to be divisible" in lib.nvfp_last_error()
    rc = lib.nvfp_gated_mlp_forward(p, p, 4, 64, 64, _capi.NVFP_DTYPE_BF16, p, p, p, 48, p, p, p, p, 64, p, p,
                                    _capi.NVFP_DTYPE_BF16, None)
    assert rc == _capi.NVFP_ERR_INVALID_ARGUMENT and b"divisible by 32" in lib.nvfp_last_error()
    rc = lib.nvfp_gated_mlp_forward(p, p, 4, 64, 64, _capi.NVFP_DTYPE_BF16, p, p, p, 64, p, p, p, p, 64, p, p,
                                    _capi.NVFP_DTYPE_F32, None)
    assert rc == _capi.NVFP_ERR_INVALID_ARGUMENT and b"fp16 or bf16" in lib.nvfp_last_error()
    rc = lib.nvfp_mxfp4_quant(p, p, p, 4, 64, 64, _capi.NVFP_DTYPE_BF16, 9, None)
    assert rc == _capi.NVFP_ERR_INVALID_ARGUMENT
    with pytest.raises(_capi.NvfpError):
        _capi.check(rc)


def test_python_wrappers_assert_like_the_reference():
    import nvfp_kernel_b200 as nv
    import nvfp.ops as compat
    assert compat.scaled_fp4_quant is not None and nv.get_active_backend() == "real"
    x = torch.zeros(4, 32, dtype=torch.bfloat16)
    gs = torch.ones(1)
    with pytest.raises(AssertionError, match="CUDA tensor"):
        nv.scaled_fp4_quant(x, gs)
    u8 = torch.zeros(4, 16, dtype=torch.uint8)
    with pytest.raises(AssertionError, match="CUDA tensor"):
        nv.cutlass_scaled_fp4_mm(u8, u8, u8, u8, gs, torch.bfloat16)
    with pytest.raises(ValueError, match="real"):
        nv.QuantLinear(64, 128, mode="emulation")
    with pytest.raises(ValueError):
        nv.QuantLinear(64, 128, format="int4")


def test_extension_exports_reference_symbols():
    from nvfp_kernel_b200._ops_real import _load_scaled_fp4_ops
    ext = _load_scaled_fp4_ops(("scaled_fp4_quant_sm1xxa", "cutlass_scaled_fp4_mm",
                                "reciprocal_approximate_ftz_tensor"))
    with pytest.raises(RuntimeError, match="missing required"):
        _load_scaled_fp4_ops(("no_such_symbol",))
    assert ext.__name__ == "scaled_fp4_ops"


def test_root_ops_shim_and_build_profile():
    """`import ops` from the repository root resolves the four names the reference's scripts use (ops.py:2-7 and
    speed_test.py:5 there); setup.py takes NVFP_BUILD_PROFILE like the reference's (setup.py:7-15 there)."""
    import subprocess
    import sys
    import ops
    import nvfp_kernel_b200.ops as real
    for name in ("scaled_fp4_quant", "cutlass_scaled_fp4_mm", "get_active_backend", "reciprocal_approximate_ftz_tensor"):
        assert getattr(ops, name) is getattr(real, name)
    assert ops.get_active_backend() == "real"

    def run(profile):
        env = dict(os.environ, NVFP_BUILD_PROFILE=profile)
        return subprocess.run([sys.executable, "setup.py", "--name"], cwd=ROOT, env=env, capture_output=True, text=True)
    ok = run("real")
    assert ok.returncode == 0 and ok.stdout.strip().splitlines()[-1] == "nvfp_kernel_b200", ok.stderr
    assert run("emulation").returncode == 0                     # accepted, builds the real kernels
    bad = run("bogus")
    assert bad.returncode != 0 and "Invalid NVFP_BUILD_PROFILE" in bad.stderr


def test_peer_group_struct_and_its_validation():
    """nvfp_peer_group_t as ctypes sees it matches the header (two ints, eight destinations, eight flag blocks, the wait
    limit), and a malformed group is rejected on the host before anything is launched."""
    assert ctypes.sizeof(_capi.PeerGroup) == 2 * 4 + 8 * 8 + 8 * 8 + 8
    lib = _capi.load()
    buf = ctypes.create_string_buffer(8192)
    p = ctypes.addressof(buf) // 256 * 256 + 256
    g = _capi.PeerGroup()
    g.world, g.rank = 0, 0
    args = (4096, p, p, p, p, p, 256, 4096, 256, _capi.NVFP_DTYPE_BF16, 0, None)
    assert lib.nvfp_scaled_fp4_mm_gather(ctypes.byref(g), *args) == _capi.NVFP_ERR_INVALID_ARGUMENT
    assert b"world" in lib.nvfp_last_error()
    g.world, g.rank = 2, 2
    assert lib.nvfp_scaled_fp4_mm_gather(ctypes.byref(g), *args) == _capi.NVFP_ERR_INVALID_ARGUMENT
    g.rank = 1
    g.dst[0], g.dst[1] = p, None
    assert lib.nvfp_scaled_fp4_mm_gather(ctypes.byref(g), *args) == _capi.NVFP_ERR_INVALID_ARGUMENT
    assert b"destination of rank 1" in lib.nvfp_last_error()
    g.dst[1] = p + 1024
    g.flags[0] = p + 2048                       # flag blocks for every rank or for none
    assert lib.nvfp_scaled_fp4_mm_gather(ctypes.byref(g), *args) == _capi.NVFP_ERR_INVALID_ARGUMENT
    assert b"flag blocks" in lib.nvfp_last_error()
    # NVFP4 gather: slabs are whole 64-column scale chunks
    g.flags[0] = None
    sf = (ctypes.c_void_p * _capi.NVFP_MAX_RANKS)(p, p)
    rc = lib.nvfp_scaled_fp4_mm_gather_fp4(ctypes.byref(g), sf, 4096, 96, p, p, p, p, p, None, p, 256, 2048, 256,
                                           _capi.NVFP_DTYPE_BF16, 0, None)
    assert rc == _capi.NVFP_ERR_INVALID_ARGUMENT and b"multiples of 64" in lib.nvfp_last_error()
    # chained layers: the output's scale needs its scratch
    rc = lib.nvfp_scaled_fp4_mm_amax(p, p, p, p, p, p, None, 256, 256, 256, _capi.NVFP_DTYPE_BF16, 0, p, None, None, None, None)
    assert rc == _capi.NVFP_ERR_INVALID_ARGUMENT
