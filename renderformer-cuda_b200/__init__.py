"""B200-native (sm_100a) layer kernels for RenderFormer inference.

The directory name carries a hyphen, so it is imported through the `renderformer_cuda_b200`
module at the repository root:

    import renderformer_cuda_b200 as rfk
    rfk.ops.rmsnorm(...)

Contents: `csrc/` (CUDA kernels and the C ABI of include/rfk.h), `build.py` (in-tree nvcc
build), `_abi.py` (ctypes binding generated from the headers), `ops.py` (Python mirror of the
reference's kernel operators). Importing the package does not load the shared library; the
first operator call does, and raises if it has not been built.
"""
from . import _abi, ops  # noqa: F401
from .ops import RfkError, version  # noqa: F401

__all__ = ["ops", "RfkError", "version"]
