"""CPU tests of the drop-in boundary: the shared library loads, exports every symbol that
include/*.h declares, and rejects bad arguments before touching the device."""
import ctypes

import pytest

import renderformer_cuda_b200 as pkg
from renderformer_cuda_b200 import _abi


def test_headers_declare_symbols():
    syms = _abi.declared_symbols()
    assert "rfk.h" in syms and len(syms["rfk.h"]) >= 40
    for required in ("rfk_rmsnorm", "rfk_rmsnorm_f32", "rfk_triangle_rope_freqs", "rfk_apply_rope",
                     "rfk_apply_rope_one", "rfk_nerf_pe", "rfk_nerf_pe_f32", "rfk_softmax_inplace",
                     "rfk_softmax_cast_fp16", "rfk_softmax_cast_fp16_masked", "rfk_fused_silu_mul",
                     "rfk_elu", "rfk_pow10_minus1", "rfk_ray_gen", "rfk_world_to_cam",
                     "rfk_rmsnorm_residual_f32_cast16"):
        assert required in syms["rfk.h"], required


@pytest.mark.parametrize("header", sorted(_abi.declared_symbols()))
def test_library_exports_every_declared_symbol(header):
    path = _abi.library_path(header)
    assert path.exists(), f"{path} not built (python renderformer-cuda_b200/build.py)"
    lib = _abi.load(header)  # raises if a declared symbol is missing
    for name in _abi.declared_symbols()[header]:
        assert hasattr(lib, name)


def test_version_and_status_strings():
    assert pkg.version().startswith("rfk ")
    lib = _abi.load("rfk.h")
    assert lib.rfk_status_string(0) == b"ok"
    assert b"invalid" in lib.rfk_status_string(-1)


def test_null_and_bad_shapes_are_rejected_without_a_device():
    lib = _abi.load("rfk.h")
    null = ctypes.c_void_p(0)
    fake = ctypes.c_void_p(256)  # never dereferenced: argument checks come first
    assert lib.rfk_rmsnorm(null, null, null, 4, 64, 1e-6, null) == -1
    assert lib.rfk_rmsnorm(fake, fake, fake, -1, 64, 1e-6, null) == -1
    assert lib.rfk_rmsnorm(fake, fake, fake, 0, 64, 1e-6, null) == 0          # empty input: no launch
    assert lib.rfk_softmax_cast_fp16(fake, fake, 4, 100, 96, 104, null) == -1  # stride < cols
    assert lib.rfk_softmax_cast_fp16(fake, fake, 0, 100, 104, 104, null) == 0
    assert lib.rfk_apply_rope_one(fake, fake, fake, 1, 4, 8, 63, null) == -1   # odd head_dim
    assert lib.rfk_nerf_pe_f32(fake, fake, 1, 8, 3, 33, 0.0, 5.0, 1, null) == -3  # > 32 frequencies
    assert lib.rfk_ray_gen(fake, fake, fake, fake, 1, 0, null) == -1
    assert lib.rfk_window_gather(fake, fake, 1, 10, 10, 8, 4, 0, null) == -1   # 10 % 4 != 0
    assert lib.rfk_rmsnorm_residual_f16(fake, fake, fake, fake, 2, 64, 1e-3, null) == -1  # y aliases x
    assert lib.rfk_launch_count() == 0


def test_python_mirror_refuses_cpu_tensors():
    import torch
    x = torch.zeros(2, 64, dtype=torch.float16)
    g = torch.ones(64)
    with pytest.raises(ValueError, match="CUDA tensor"):
        pkg.ops.rmsnorm(x, g, x, 2, 64)
