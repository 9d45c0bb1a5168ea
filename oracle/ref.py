"""ctypes door onto the reference engine's own CUDA code, built unchanged by oracle/Makefile
into oracle/_ref/libref_kernels.so (src/kernels) and oracle/_ref/libref_layers.so
(src/kernels + src/layers, needs cuBLAS and cuDNN).

TEST INFRASTRUCTURE ONLY: used by the GPU parity tests, by the script that generates the
golden fixtures, and by the reference arm of the benchmark. The product never loads it.

    ref.available()                       -> bool
    ref.call("ref_rmsnorm", x, g, y, rows, dim, eps)    # torch CUDA tensors, ints, floats;
                                                        # the current stream is appended
"""
from __future__ import annotations

import ctypes
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
_libs: dict[str, ctypes.CDLL | None] = {}


def _load(name: str):
    if name not in _libs:
        p = REF_DIR / name
        try:
            _libs[name] = ctypes.CDLL(str(p)) if p.exists() else None
        except OSError:
            _libs[name] = None
    return _libs[name]


def kernels():
    return _load("libref_kernels.so")


def layers():
    return _load("libref_layers.so")


def available() -> bool:
    return kernels() is not None


def layers_available() -> bool:
    return layers() is not None


class Raw:
    """Pass a raw integer as a pointer (e.g. a cuBLAS handle or a host struct address)."""

    def __init__(self, v):
        self.v = v


def _conv(a):
    import torch

    if a is None:
        return ctypes.c_void_p(0)
    if isinstance(a, Raw):
        return ctypes.c_void_p(a.v)
    if isinstance(a, torch.Tensor):
        assert a.is_cuda and a.is_contiguous()
        return ctypes.c_void_p(a.data_ptr())
    if isinstance(a, bool):
        return ctypes.c_int(int(a))
    if isinstance(a, int):
        return ctypes.c_int(a)
    if isinstance(a, float):
        return ctypes.c_float(a)
    if isinstance(a, (ctypes.Structure, ctypes._Pointer, ctypes.c_void_p)) or type(a).__name__ == "CArgObject":
        return a  # ctypes.byref(struct) arrives as a CArgObject
    raise TypeError(type(a))


def call(name: str, *args, lib=None, stream=None):
    """Call a `ref_*` wrapper; the CUDA stream (torch's current one by default) goes last."""
    import torch

    lib = lib or (kernels() if hasattr(kernels(), name) else layers())
    fn = getattr(lib, name)
    fn.restype = None
    s = torch.cuda.current_stream().cuda_stream if stream is None else stream
    fn(*[_conv(a) for a in args], ctypes.c_void_p(s))


class DecoderLayerW(ctypes.Structure):
    """Mirror of RefDecoderLayerW in oracle/ref_shim_layers.cu (device pointers)."""

    _fields_ = [(n, ctypes.c_void_p) for n in (
        "query_norm_gamma", "kv_norm_gamma", "q_proj_w", "k_proj_w", "v_proj_w", "cross_out_w",
        "cross_q_norm", "cross_k_norm", "self_attn_norm_gamma", "swin_in_w", "swin_out_w",
        "swin_q_norm", "swin_k_norm", "ffn_norm_gamma", "w1", "w2", "w3")]


def cublas_create() -> int:
    fn = layers().ref_cublas_create
    fn.restype = ctypes.c_void_p
    h = fn()
    if not h:
        raise RuntimeError("cublasCreate failed in the reference library")
    return h


def cublas_destroy(h: int) -> None:
    layers().ref_cublas_destroy(ctypes.c_void_p(h))
