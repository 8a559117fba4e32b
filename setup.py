"""In-tree build of the native extension ``rl_engine._C`` for sm_100a only.

    python setup.py build_ext --inplace

Kernel sources do not include torch headers, so they compile in seconds; only ``csrc/ops.cpp`` and
the runtime see torch/pybind11.  The arch is passed as an explicit ``-gencode`` flag, which makes
torch's extension builder skip its own architecture list.
"""

import glob
import os

from setuptools import find_packages, setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))

CXX_FLAGS = ["-O3", "-std=c++17"]
NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xfatbin",
    "-compress-all",
]
# ``rl_engine._C_dbg`` is the same sources with -DRLK_DEBUG_BOUNDS=1 (checked index accesses that report to the
# error word); it is loaded instead of ``_C`` when RLK_DEBUG_BOUNDS=1 is set at import time.  RLK_SKIP_DEBUG_EXT=1
# skips building it.
DEBUG_FLAG = "-DRLK_DEBUG_BOUNDS=1"
if os.environ.get("RLK_ATTN_PROFILE") == "1":  # per-phase cycle counters in the attention forward kernel
    NVCC_FLAGS.append("-DRLK_ATTN_PROFILE=1")
    CXX_FLAGS.append("-DRLK_ATTN_PROFILE=1")
if os.environ.get("RLK_PTXAS_VERBOSE") == "1":
    NVCC_FLAGS += ["-Xptxas", "-v"]


def sources():
    rel = lambda paths: sorted(os.path.relpath(p, ROOT) for p in paths)
    return (
        ["csrc/ops.cpp"]
        + rel(glob.glob(os.path.join(ROOT, "csrc", "runtime", "*.cpp")))
        + rel(glob.glob(os.path.join(ROOT, "csrc", "kernels", "*.cu")))
    )


setup(
    name="rl_engine",
    version="0.1.0",
    packages=find_packages(include=["rl_engine", "rl_engine.*", "rl_kernel_b200", "rl_kernel_b200.*"]),
    ext_modules=[
        CUDAExtension(
            name="rl_engine._C",
            sources=sources(),
            include_dirs=[os.path.join(ROOT, "csrc")],
            extra_compile_args={"cxx": CXX_FLAGS, "nvcc": NVCC_FLAGS},
        )
    ] + ([] if os.environ.get("RLK_SKIP_DEBUG_EXT") == "1" else [
        CUDAExtension(
            name="rl_engine._C_dbg",
            sources=sources(),
            include_dirs=[os.path.join(ROOT, "csrc")],
            extra_compile_args={"cxx": CXX_FLAGS + [DEBUG_FLAG], "nvcc": NVCC_FLAGS + [DEBUG_FLAG]},
        )
    ]),
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=True)},
)
