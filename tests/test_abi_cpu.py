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
    assert b"bounded" in lib.rfk_status_string(-4)


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
    # the fused attention entries: argument checks before any device work
    assert lib.rfk_flash_attention(fake, fake, fake, fake, 1, 2, 16, 8, 9, 64, 0, 0.125, null) == -1   # n_keys > Sk
    assert lib.rfk_flash_attention(fake, fake, fake, fake, 1, 2, 16, 8, 8, 48, 0, 0.125, null) == -2   # head size
    assert lib.rfk_flash_attention(fake, fake, fake, fake, 0, 2, 16, 8, 8, 64, 0, 0.125, null) == 0    # empty batch
    assert lib.rfk_flash_attention_set_path(7) == -1
    # the extended attention, the head-split projection and the normed window attention: checks before any device work
    ws_bytes = lib.rfk_flash_attention_workspace_bytes()
    assert ws_bytes > 20 << 20
    assert lib.rfk_flash_attention_ex(fake, fake, fake, fake, null, 0, 0, 0.0, fake, ws_bytes - 1, 0, 1, 2, 16, 8, 8, 64, 0, 0.125, null) == -1   # workspace too small
    assert lib.rfk_flash_attention_ex(fake, fake, fake, fake, fake, 0, 128, 1e-3, null, 0, 0, 1, 2, 16, 8, 8, 64, 0, 0.125, null) == -1     # statistics without tiles
    assert lib.rfk_flash_attention_ex(fake, fake, fake, fake, null, 0, 0, 0.0, null, 0, 0, 1, 2, 16, 8, 8, 128, 0, 0.125, null) == -2       # tcgen05 kernel: head size 64 only
    assert lib.rfk_flash_attention_ex(fake, fake, fake, fake, null, 0, 0, 0.0, null, 0, 0, 1, 2, 0, 8, 8, 64, 0, 0.125, null) == 0          # no queries
    assert lib.rfk_gemm_f16_heads(fake, 64, fake, 64, fake, 0, null, 1, 64, 256, 64, 32, 4, null) == -1     # statistics asked for, no buffer
    assert lib.rfk_gemm_f16_heads(fake, 64, fake, 64, fake, 0, null, 0, 64, 200, 64, 32, 4, null) == -1     # N not parts * heads * 64
    assert lib.rfk_gemm_f16_heads(fake, 64, fake, 64, fake, 0, null, 0, 0, 256, 64, 32, 4, null) == 0       # no rows
    assert lib.rfk_window_attention_normed(fake, fake, fake, fake, null, fake, fake, 4, fake, null, 1024, 1e-3, 4, 16, 64, 64, 4, 0.125, null) == -1  # no k weights
    assert lib.rfk_window_attention_normed(fake, fake, fake, fake, null, fake, fake, 4, fake, fake, 1024, 1e-3, 4, 16, 49, 64, 4, 0.125, null) == -2  # 7x7 windows
    assert lib.rfk_rope_one_oop_strided(fake, fake, fake, fake, 1, 0, 0, 0, 4, 8, 64, 8, 8, null, -1, null) == -1   # negative stride
    assert lib.rfk_window_attention(fake, fake, fake, fake, null, 4, 2, 49, 64, 4, 0.125, null) == -2  # 7x7 windows
    assert lib.rfk_rmsnorm_residual_f16_windows(fake, fake, fake, fake, 1, 10, 10, 64, 4, 0, 1, 1e-3, null) == -1
    assert lib.rfk_rmsnorm_residual_f16_windows(fake, fake, fake, ctypes.c_void_p(512), 1, 8, 8, 60, 4, 0, 3, 1e-3, null) == -1
    # DPT head glue: null pointers, non-positive extents; empty problems are successes
    assert lib.rfk_bilinear_upsample(null, fake, 1, 1, 4, 4, 8, 8, null) == -1
    assert lib.rfk_bilinear_upsample(fake, fake, 1, 1, 4, 0, 8, 8, null) == -1
    assert lib.rfk_bilinear_upsample(fake, fake, 0, 3, 4, 4, 8, 8, null) == 0
    assert lib.rfk_silu_inplace(null, 8, null) == -1
    assert lib.rfk_silu_inplace(fake, 0, null) == 0
    assert lib.rfk_add_bias_nchw(fake, null, 1, 2, 16, null) == -1
    assert lib.rfk_add_bias_nchw(fake, fake, 1, 0, 16, null) == -1
    assert lib.rfk_permute_bsd_to_nchw(fake, null, 1, 4, 4, null) == -1
    assert lib.rfk_permute_bsd_to_nchw(fake, fake, 1, 0, 4, null) == 0
    assert lib.rfk_launch_count() == 0


def test_python_mirror_refuses_cpu_tensors():
    import torch
    x = torch.zeros(2, 64, dtype=torch.float16)
    g = torch.ones(64)
    with pytest.raises(ValueError, match="CUDA tensor"):
        pkg.ops.rmsnorm(x, g, x, 2, 64)


def test_compat_header_compiles_and_links_reference_style_code(tmp_path):
    """Host code written against the reference's rf:: kernel interface builds against
    include/rfk_compat.h and links librfk.so (compile + link only, nothing runs)."""
    import shutil
    import subprocess
    from pathlib import Path
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    root = Path(__file__).resolve().parent.parent
    src = tmp_path / "caller.cu"
    src.write_text(r'''
#include <rfk_compat.h>
// call sites in the style of src/layers/attention.cu:193-194,210 and src/pipeline/render_session.cu:194-208,249-253
void reference_style_caller(half* q, half* k, const float* g, const half* c, const half* s, float* scores, half* p,
                            const bool* mask, float* c2w, float* fov, float* ro, half* rd, half* tri, half* vn,
                            float* out32, float* x32, const half* r16, cudaStream_t st) {
    rf::rmsnorm(q, g, q, 4096, 1024, rf::kEpsFp16, st);
    rf::rmsnorm_f32(x32, g, x32, 16, 1024);
    rf::apply_rope(q, k, c, s, 1, 16, 4096, 64, st);
    rf::apply_rope_one(q, c, s, 1, 16, 4096, 64, st);
    rf::triangle_rope_freqs(q, g, q, k, 1, 5672, 3, 64, st);
    rf::softmax_cast_fp16(scores, p, 65536, 5633, 5640, 5640, st);
    rf::softmax_cast_fp16_masked(scores, p, mask, 16, 64, 64, 64, 1, st);
    rf::swin_masked_softmax_inplace(scores, mask, 64, 16, 64, 64, st);
    rf::softmax_inplace(scores, 16, 64);
    rf::fused_silu_mul(q, k, q, 4096 * 4096, st);
    rf::nerf_pe_f32(x32, p, 1, 5633, 9, 6, 0, 5, true, st);
    rf::ray_gen(c2w, fov, ro, rd, 1, 512, st);
    rf::world_to_cam(c2w, tri, vn, 1, 5633, st);
    rf::elu(p, p, 786432, 1e-3f, st);
    rf::pow10_minus1(out32, out32, 786432, st);
    rf::residual_add(q, k, 4096 * 1024, st);
    rf::residual_add_mixed(x32, r16, 1024, st);
    rf::cast_fp32_to_fp16(x32, q, 1024, st);
}
''')
    pkg_dir = root / "renderformer-cuda_b200"
    out = tmp_path / "libcaller.so"
    cmd = [nvcc, "-std=c++17", "-DRFK_COMPAT_CHECK", "-gencode", "arch=compute_100a,code=sm_100a", "-shared",
           "-Xcompiler", "-fPIC", f"-I{root / 'include'}", str(src), "-o", str(out), f"-L{pkg_dir}", "-lrfk"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    assert out.exists()
