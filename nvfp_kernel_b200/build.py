"""In-tree build of the native parts (no GPU needed: nvcc cross-compiles sm_100a).

    python -m nvfp_kernel_b200.build            # library + torch extension
    python -m nvfp_kernel_b200.build --lib      # only libnvfp_b200.so
    python -m nvfp_kernel_b200.build --trace    # libnvfp_b200_trace.so, the instrumented build for pair_trace.py

Outputs, both inside this package directory:
  libnvfp_b200.so                 CUDA kernels + C ABI (include/nvfp_b200.h); no torch dependency
  scaled_fp4_ops.<abi>.so         thin torch extension with the reference's three entry points
                                  (binding.cpp of the reference) on top of the C ABI
The reference builds for sm_120a only (setup.py:43-47 there); this builds for sm_100a only.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
ROOT = os.path.dirname(PKG_DIR)
LIB_PATH = os.path.join(PKG_DIR, "libnvfp_b200.so")
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
EXT_PATH = os.path.join(PKG_DIR, "scaled_fp4_ops" + EXT_SUFFIX)

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]
CU_SOURCES = ["runtime.cu", "quant_sm100.cu", "gemm_fp4_sm100.cu"]


def _digest(paths, extra=()) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(os.path.basename(p).encode() + b"\0" + f.read())
    for e in extra:
        h.update(str(e).encode())
    return h.hexdigest()


def _up_to_date(target: str, digest: str) -> bool:
    stamp = target + ".stamp"
    if not (os.path.exists(target) and os.path.exists(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == digest


def _write_stamp(target: str, digest: str) -> None:
    with open(target + ".stamp", "w") as f:
        f.write(digest)


def _run(cmd, **kw):
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd, **kw)


def build_lib(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in CU_SOURCES]
    deps = srcs + [os.path.join(CSRC, "common.h"), os.path.join(CSRC, "ptx_sm100.cuh"),
                   os.path.join(CSRC, "gemm_fp4_pair_sm100.cuh"),
                   os.path.join(CSRC, "gemm_fp4_skinny_sm100.cuh"), os.path.join(CSRC, "quant_math.cuh"),
                   os.path.join(ROOT, "include", "nvfp_b200.h")]
    digest = _digest(deps, NVCC_FLAGS)
    if not force and _up_to_date(LIB_PATH, digest):
        return LIB_PATH
    objs = []
    for s in srcs:
        o = os.path.join(PKG_DIR, "build", os.path.basename(s) + ".o")
        os.makedirs(os.path.dirname(o), exist_ok=True)
        _run([NVCC, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", s, "-o", o])
        objs.append(o)
    _run([NVCC, "-shared", "-o", LIB_PATH, *objs, "-cudart", "shared"])
    _write_stamp(LIB_PATH, digest)
    return LIB_PATH


TRACE_LIB_PATH = os.path.join(PKG_DIR, "libnvfp_b200_trace.so")


def build_trace_lib(force: bool = False) -> str:
    """libnvfp_b200_trace.so: the same library compiled with -DNVFP_PAIR_TRACE (the CTA-pair GEMM counts where its
    roles wait; read with nvfp_debug_pair_trace).  Used by nvfp_kernel_b200.pair_trace only; never the product path."""
    srcs = [os.path.join(CSRC, s) for s in CU_SOURCES]
    digest = _digest(srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))], NVCC_FLAGS + ["trace"])
    if not force and _up_to_date(TRACE_LIB_PATH, digest):
        return TRACE_LIB_PATH
    objs = []
    for s in srcs:
        o = os.path.join(PKG_DIR, "build", "trace_" + os.path.basename(s) + ".o")
        os.makedirs(os.path.dirname(o), exist_ok=True)
        _run([NVCC, *NVCC_FLAGS, "-DNVFP_PAIR_TRACE", "-c", s, "-o", o])
        objs.append(o)
    _run([NVCC, "-shared", "-o", TRACE_LIB_PATH, *objs, "-cudart", "shared"])
    _write_stamp(TRACE_LIB_PATH, digest)
    return TRACE_LIB_PATH


def build_torch_ext(force: bool = False) -> str:
    """g++ only: the extension holds no device code, it forwards to libnvfp_b200.so."""
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths

    src = os.path.join(CSRC, "binding.cpp")
    digest = _digest([src, os.path.join(ROOT, "include", "nvfp_b200.h")], [torch.__version__])
    if not force and _up_to_date(EXT_PATH, digest) and os.path.exists(LIB_PATH):
        return EXT_PATH
    build_lib()
    incs = []
    for p in include_paths("cuda") if "device_type" in include_paths.__code__.co_varnames else include_paths(True):
        incs += ["-isystem", p]
    incs += ["-isystem", sysconfig.get_paths()["include"], "-isystem", "/usr/local/cuda/include"]
    libs = []
    for p in library_paths("cuda") if "device_type" in library_paths.__code__.co_varnames else library_paths(True):
        libs += ["-L" + p, "-Wl,-rpath," + p]
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=scaled_fp4_ops",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *incs, src, "-o", EXT_PATH, *libs, "-L" + PKG_DIR, "-l:libnvfp_b200.so", "-Wl,-rpath,$ORIGIN",
           "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    _run(cmd)
    _write_stamp(EXT_PATH, digest)
    return EXT_PATH


def build_all(force: bool = False) -> None:
    build_lib(force)
    build_torch_ext(force)


if __name__ == "__main__":
    force = "--force" in sys.argv
    if "--trace" in sys.argv:
        print(build_trace_lib(force))
    elif "--lib" in sys.argv:
        print(build_lib(force, verbose="-v" in sys.argv))
    else:
        build_all(force)
        print(LIB_PATH)
        print(EXT_PATH)
