"""In-tree build of the native extension: ``python setup.py build_ext --inplace``.

Every CUDA source is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``); passing the arch flags
explicitly keeps torch's own architecture list out of the command line. The result lands beside the Python package as
``scalingcontrasts_b200/_C*.so`` so that it travels with the source tree.
"""
import os

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join("scalingcontrasts_b200", "csrc")
SOURCES = [os.path.join(CSRC, name) for name in (
    "bindings.cpp", "domain.cpp", "oracle_cpu.cpp", "rail.cpp",
    "collectives.cu", "loss_small.cu", "loss_fwd.cu", "loss_bwd.cu", "no_alloc.cu", "tower.cu", "optim.cu",
)]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr"]
# Tuning knob of the forward kernel (16 or 8 epilogue warps); the default is the measured best.
if os.environ.get("SC_FWD_EPILOGUE_WARPS"):
    NVCC_FLAGS.append("-DSC_FWD_EPILOGUE_WARPS=" + os.environ["SC_FWD_EPILOGUE_WARPS"])
# Diagnostic build of the forward kernel with in-kernel phase timers (the `trace` argument of `forward`).
if os.environ.get("SC_FWD_TRACE"):
    NVCC_FLAGS.append("-DSC_FWD_TRACE=" + os.environ["SC_FWD_TRACE"])

# A/B switch for the helper warps' sleeping waits in the forward kernel (1: sleep between polls, 0: poll back to back).
if os.environ.get("SC_FWD_HELPER_SLEEP"):
    NVCC_FLAGS.append("-DSC_FWD_HELPER_SLEEP=" + os.environ["SC_FWD_HELPER_SLEEP"])

EXTENSIONS = [CUDAExtension(
    name="scalingcontrasts_b200._C",
    sources=SOURCES,
    include_dirs=[os.path.join(ROOT, CSRC)],
    extra_compile_args={"cxx": ["-O2", "-std=c++17"], "nvcc": NVCC_FLAGS},
)]
# The bounds-checked debug build of the same sources (every computed global index is compared with its limit; a miss is
# recorded and skipped, never trapped): `SC_NATIVE_VARIANT=bounds` makes the package load it instead of `_C`.
# SC_BUILD_BOUNDS=0 leaves it out.
if os.environ.get("SC_BUILD_BOUNDS", "1") != "0":
    EXTENSIONS.append(CUDAExtension(
        name="scalingcontrasts_b200._C_bounds",
        sources=SOURCES,
        include_dirs=[os.path.join(ROOT, CSRC)],
        extra_compile_args={"cxx": ["-O2", "-std=c++17", "-DSC_BOUNDS=1"], "nvcc": NVCC_FLAGS + ["-DSC_BOUNDS=1"]},
    ))

setup(
    name="scalingcontrasts_b200",
    version="0.1.0",
    packages=[],
    ext_modules=EXTENSIONS,
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=True)},
)
