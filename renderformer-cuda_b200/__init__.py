"""B200-native (sm_100a) layer kernels for RenderFormer inference.

The directory name carries a hyphen, so it is imported through the `renderformer_cuda_b200`
module at the repository root:

    import renderformer_cuda_b200 as rfk
    rfk.ops.rmsnorm(...)

Contents: `csrc/` (CUDA kernels and the C ABI of include/rfk.h), `build.py` (in-tree nvcc
build), `_abi.py` (ctypes binding generated from the headers), `ops.py` (Python mirror of the
reference's kernel operators), `session.py` (layer records, session, view scheduler), `assets.py`
(safetensors weights and scenes in, EXR / PNG out; include/rfk_io.h). Importing the package does not
load the shared libraries; the first call does, and raises if they have not been built.
"""
from . import _abi, assets, ops  # noqa: F401
from .ops import RfkError, version  # noqa: F401

__all__ = ["ops", "assets", "RfkError", "version"]
