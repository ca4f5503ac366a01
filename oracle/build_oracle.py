"""Builds the checkers under oracle/ (test infrastructure; the product never loads them).

  python oracle/build_oracle.py            # C restatement + (if a reference checkout is found) oracle/_ref
  python oracle/build_oracle.py --ref /path/to/reference

The reference checkout (huweim/nvfp_kernel) is taken from --ref, else from the environment variable
NVFP_REFERENCE_ROOT, else from a directory named `reference` beside this repository.

  oracle/libnvfp_oracle.so   gcc build of nvfp_oracle.c (CPU restatement, OpenMP)
  oracle/_ref/ref_scaled_fp4_ops.<abi>.so
        the reference's own quantizer kernel (kernel/nvfp4_quant_kernels.cu,
        kernel/cuda_utils_kernels.cu, kernel/reciprocal_kernels.cu of the reference
        checkout, compiled in place with the reference's flags -O3 --use_fast_math but
        for compute_100a instead of compute_120a) behind oracle/ref_binding.cpp.
        Needs a GPU to run; built here, carried to the GPU box as a binary.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
REF_OUT = os.path.join(HERE, "_ref")
C_LIB = os.path.join(HERE, "libnvfp_oracle.so")
REF_EXT = os.path.join(REF_OUT, "ref_scaled_fp4_ops" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
REF_SOURCES = ["kernel/nvfp4_quant_kernels.cu", "kernel/cuda_utils_kernels.cu", "kernel/reciprocal_kernels.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def reference_root() -> str | None:
    """Where the reference checkout lies: $NVFP_REFERENCE_ROOT, else `reference` beside this repository."""
    cand = os.environ.get("NVFP_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isfile(os.path.join(cand, "kernel", "nvfp4_utils.cuh")) else None


def _digest(paths, extra=()):
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as f:
            h.update(os.path.basename(p).encode() + b"\0" + f.read())
    for e in extra:
        h.update(str(e).encode())
    return h.hexdigest()


def _fresh(target, digest):
    try:
        return os.path.exists(target) and open(target + ".stamp").read().strip() == digest
    except OSError:
        return False


def _run(cmd):
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build_c(force: bool = False) -> str:
    src = os.path.join(HERE, "nvfp_oracle.c")
    digest = _digest([src])
    if not force and _fresh(C_LIB, digest):
        return C_LIB
    _run(["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-fno-fast-math", "-o", C_LIB, src, "-lm"])
    open(C_LIB + ".stamp", "w").write(digest)
    return C_LIB


def build_ref(ref_root: str | None = None, force: bool = False) -> str | None:
    """Returns the path of the built extension, or None when the checkout is absent
    (the GPU box only has the prebuilt file)."""
    ref_root = ref_root or reference_root()
    if ref_root is None or not os.path.isdir(os.path.join(ref_root, "kernel")):
        return REF_EXT if os.path.exists(REF_EXT) else None
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths
    srcs = [os.path.join(ref_root, s) for s in REF_SOURCES]
    binding = os.path.join(HERE, "ref_binding.cpp")
    digest = _digest(srcs + [binding], [torch.__version__])
    if not force and _fresh(REF_EXT, digest):
        return REF_EXT
    os.makedirs(REF_OUT, exist_ok=True)
    incs = ["-I" + os.path.join(ref_root, "kernel")]
    for p in include_paths("cuda"):
        incs += ["-isystem", p]
    incs += ["-isystem", sysconfig.get_paths()["include"]]
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    common = ["-DTORCH_EXTENSION_NAME=ref_scaled_fp4_ops", "-DTORCH_API_INCLUDE_EXTENSION_H", abi, "-std=c++17"]
    objs = []
    for s in srcs:
        o = os.path.join(REF_OUT, os.path.basename(s) + ".o")
        _run([NVCC, "-O3", "--use_fast_math", "-gencode=arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", *common, *incs, "-c", s, "-o", o])
        objs.append(o)
    o = os.path.join(REF_OUT, "ref_binding.o")
    _run(["g++", "-O2", "-fPIC", *common, *incs, "-c", binding, "-o", o])
    objs.append(o)
    libs = []
    for p in library_paths("cuda"):
        libs += ["-L" + p, "-Wl,-rpath," + p]
    _run(["g++", "-shared", "-o", REF_EXT, *objs, *libs, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
          "-ltorch", "-ltorch_python", "-lcudart"])
    open(REF_EXT + ".stamp", "w").write(digest)
    return REF_EXT


if __name__ == "__main__":
    ref = sys.argv[sys.argv.index("--ref") + 1] if "--ref" in sys.argv else None
    if "--no-c" not in sys.argv:
        print(build_c("--force" in sys.argv))
    print(build_ref(ref, "--force" in sys.argv))
