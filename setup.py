"""pip install --no-build-isolation -e .   (or: python setup.py build_ext --inplace)

Builds the two native parts IN-TREE for sm_100a -- nvfp_kernel_b200/libnvfp_b200.so (nvcc) and the torch extension
nvfp_kernel_b200/scaled_fp4_ops.<abi>.so (g++) -- by running nvfp_kernel_b200/build.py, and installs the packages
`nvfp_kernel_b200` and the import-name shim `nvfp`.  Counterpart of the reference's setup.py:7-15,43-47, which builds
one CUDAExtension for sm_120a.  NVFP_BUILD_PROFILE is accepted for compatibility with the reference's build scripts:
"real" (default) is what is built; "emulation" / "emulation_only" have nothing to select here (there is no emulation
backend) and build the same thing with a note.
"""
import importlib.util
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_ext import build_ext as _build_ext
from setuptools.command.build_py import build_py as _build_py
from setuptools.command.develop import develop as _develop

HERE = os.path.dirname(os.path.abspath(__file__))
profile = os.getenv("NVFP_BUILD_PROFILE", "real").strip().lower()
if profile == "emulation":
    profile = "emulation_only"
if profile not in {"emulation_only", "real"}:
    raise ValueError(f"Invalid NVFP_BUILD_PROFILE={profile!r}; expected 'emulation_only' or 'real'.")
if profile != "real":
    print("NVFP_BUILD_PROFILE=emulation_only: this package has no emulation backend; building the real kernels",
          file=sys.stderr)


def _native_build():
    spec = importlib.util.spec_from_file_location("_nvfp_native_build", os.path.join(HERE, "nvfp_kernel_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build_all(force="--force" in sys.argv)


class build_ext(_build_ext):
    def run(self):
        _native_build()


class build_py(_build_py):
    def run(self):
        _native_build()
        super().run()


class develop(_develop):
    def run(self):
        _native_build()
        super().run()


class build_native(Command):
    description = "build libnvfp_b200.so and the scaled_fp4_ops extension in-tree (sm_100a)"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        _native_build()


setup(
    name="nvfp_kernel_b200",
    version="1.1.0",
    description="B200-native NVFP4 / MXFP4 quantize-and-GEMM (drop-in for the nvfp package of huweim/nvfp_kernel)",
    packages=find_packages(include=["nvfp_kernel_b200", "nvfp_kernel_b200.*", "nvfp"]),
    py_modules=["ops"],
    package_data={"nvfp_kernel_b200": ["*.so", "csrc/*"]},
    include_package_data=True,
    cmdclass={"build_ext": build_ext, "build_py": build_py, "develop": develop, "build_native": build_native},
    python_requires=">=3.9",
    zip_safe=False,
)
