"""Builds the in-tree CUDA extension `megalodon_b200/_C*.so` for sm_100a:

    python setup.py build_ext --inplace
"""
import os

from setuptools import find_packages, setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join("megalodon_b200", "csrc")


def sources():
    out = [os.path.join(CSRC, "bindings.cpp"), os.path.join(CSRC, "cpu_ops.cpp"), os.path.join(CSRC, "cpu_ops_bwd.cpp")]
    for name in sorted(os.listdir(os.path.join(ROOT, CSRC))):
        if name.endswith(".cu"):
            out.append(os.path.join(CSRC, name))
    return out


NVCC_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "--expt-relaxed-constexpr",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
]

setup(
    name="megalodon_b200",
    version="0.1.0",
    packages=find_packages(include=["megalodon_b200", "megalodon_b200.*", "megalodon"]),
    ext_modules=[
        CUDAExtension(
            "megalodon_b200._C",
            sources(),
            include_dirs=[os.path.join(ROOT, CSRC)],
            extra_compile_args={"cxx": ["-O3", "-std=c++17"], "nvcc": NVCC_FLAGS},
        )
    ],
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=True)},
)
