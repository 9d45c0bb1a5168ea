"""Python mirror of the reference engine's kernel operators, bound to librfk.so.

Each function keeps the name, argument order and meaning of the reference operator it stands
for (BANANASJIM/renderformer-cuda `src/kernels/*.h`, plus the helper kernels of
`src/layers/transformer.cu`, `src/layers/attention.cu` and
`src/pipeline/render_session.cu`), takes CUDA `torch.Tensor`s in place of raw device
pointers, launches on torch's current stream and raises `RfkError` for a non-zero status.
torch is used for device memory and streams only: all arithmetic happens in the CUDA kernels
behind the C ABI (include/rfk.h). There is no CPU path.
"""
from __future__ import annotations

import ctypes

import torch

from . import _abi

K_EPS_FP16 = 0.0009765625      # rf::kEpsFp16, src/kernels/rmsnorm.h:9
K_EPS_FP32 = 1.1920929e-07     # rf::kEpsFp32, src/kernels/rmsnorm.h:10


class RfkError(RuntimeError):
    def __init__(self, fn: str, status: int):
        self.status = status
        text = _lib().rfk_status_string(status).decode()
        super().__init__(f"{fn} failed with status {status}: {text}")


def _lib():
    return _abi.load("rfk.h")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None, dtype=None, name="tensor"):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _call(name: str, *args):
    rc = getattr(_lib(), name)(*args)
    if rc != 0:
        raise RfkError(name, rc)


H, F, U8 = torch.float16, torch.float32, torch.uint8


def _mask_ptr(mask):
    if mask is None:
        return None
    if mask.dtype == torch.bool:
        mask = mask.view(torch.uint8)
    return _p(mask, U8, "mask")


def version() -> str:
    return _lib().rfk_version().decode()


def launch_count() -> int:
    return int(_lib().rfk_launch_count())


# ------------------------------------------------------------------ RMSNorm

def rmsnorm(x, gamma, y, rows, dim, eps=K_EPS_FP16):
    _call("rfk_rmsnorm", _p(x, H, "x"), _p(gamma, F, "gamma"), _p(y, H, "y"), rows, dim, eps, _stream())


def rmsnorm_f32(x, gamma, y, rows, dim, eps=K_EPS_FP32):
    _call("rfk_rmsnorm_f32", _p(x, F, "x"), _p(gamma, F, "gamma"), _p(y, F, "y"), rows, dim, eps, _stream())


def rmsnorm_residual_f32_cast16(h, r, gamma, y16, rows, dim, eps):
    _call("rfk_rmsnorm_residual_f32_cast16", _p(h, F, "h"), _p(r, F, "r"), _p(gamma, F, "gamma"),
          _p(y16, H, "y16"), rows, dim, eps, _stream())


def rmsnorm_residual_mixed_cast16(h, r, gamma, y16, rows, dim, eps):
    _call("rfk_rmsnorm_residual_mixed_cast16", _p(h, F, "h"), _p(r, H, "r"), _p(gamma, F, "gamma"),
          _p(y16, H, "y16"), rows, dim, eps, _stream())


def rmsnorm_residual_f16_windows(x, r, gamma, y, B, Hh, W, dim, ws, shift, windowed_operand, eps=K_EPS_FP16):
    """windowed_operand 1: y written in swin window order; 2: r read in window order."""
    _call("rfk_rmsnorm_residual_f16_windows", _p(x, H, "x"), _p(r, H, "r"), _p(gamma, F, "gamma"), _p(y, H, "y"),
          B, Hh, W, dim, ws, shift, windowed_operand, eps, _stream())


def rmsnorm_residual_f16(x, r, gamma, y, rows, dim, eps=K_EPS_FP16):
    _call("rfk_rmsnorm_residual_f16", _p(x, H, "x"), _p(r, H, "r"), _p(gamma, F, "gamma"),
          _p(y, H, "y"), rows, dim, eps, _stream())


# ------------------------------------------------- residual / cast plumbing

def residual_add(y, residual, n):
    _call("rfk_residual_add", _p(y, H, "y"), _p(residual, H, "residual"), n, _stream())


def residual_add_f32(y, residual, n):
    _call("rfk_residual_add_f32", _p(y, F, "y"), _p(residual, F, "residual"), n, _stream())


def residual_add_mixed(y, residual, n):
    _call("rfk_residual_add_mixed", _p(y, F, "y"), _p(residual, H, "residual"), n, _stream())


def cast_fp32_to_fp16(inp, out, n):
    _call("rfk_cast_fp32_to_fp16", _p(inp, F, "in"), _p(out, H, "out"), n, _stream())


def cast_fp16_to_fp32(inp, out, n):
    _call("rfk_cast_fp16_to_fp32", _p(inp, H, "in"), _p(out, F, "out"), n, _stream())


def broadcast_add(out, bc, n, dim):
    _call("rfk_broadcast_add", _p(out, H, "out"), _p(bc, H, "bc"), n, dim, _stream())


# --------------------------------------------------------------------- RoPE

def triangle_rope_freqs(pos, learned_freqs, out_cos, out_sin, batch, seq_len, num_freqs, head_dim):
    _call("rfk_triangle_rope_freqs", _p(pos, H, "pos"), _p(learned_freqs, F, "learned_freqs"),
          _p(out_cos, H, "out_cos"), _p(out_sin, H, "out_sin"), batch, seq_len, num_freqs, head_dim,
          _stream())


def apply_rope(q, k, cos_vals, sin_vals, batch, num_heads, seq_len, head_dim):
    _call("rfk_apply_rope", _p(q, H, "q"), _p(k, H, "k"), _p(cos_vals, H, "cos"), _p(sin_vals, H, "sin"),
          batch, num_heads, seq_len, head_dim, _stream())


def apply_rope_one(x, cos_vals, sin_vals, batch, num_heads, seq_len, head_dim):
    _call("rfk_apply_rope_one", _p(x, H, "x"), _p(cos_vals, H, "cos"), _p(sin_vals, H, "sin"),
          batch, num_heads, seq_len, head_dim, _stream())


def apply_rope_f32(q, k, cos_vals, sin_vals, batch, num_heads, seq_len, head_dim):
    _call("rfk_apply_rope_f32", _p(q, F, "q"), _p(k, F, "k"), _p(cos_vals, H, "cos"),
          _p(sin_vals, H, "sin"), batch, num_heads, seq_len, head_dim, _stream())


def apply_rope_one_f32(x, cos_vals, sin_vals, batch, num_heads, seq_len, head_dim):
    _call("rfk_apply_rope_one_f32", _p(x, F, "x"), _p(cos_vals, H, "cos"), _p(sin_vals, H, "sin"),
          batch, num_heads, seq_len, head_dim, _stream())


def rope_one_oop(src, dst, cos_vals, sin_vals, batch, num_heads, seq_len, head_dim,
                 src_seq_stride=None, dst_seq_stride=None, copy_tail=False):
    _call("rfk_rope_one_oop", _p(src, H, "src"), _p(dst, H, "dst"), _p(cos_vals, H, "cos"),
          _p(sin_vals, H, "sin"), batch, num_heads, seq_len, head_dim,
          seq_len if src_seq_stride is None else src_seq_stride,
          seq_len if dst_seq_stride is None else dst_seq_stride, int(copy_tail), _stream())


def rope_one_oop_strided(src, dst, cos_vals, sin_vals, batch, src_batch_stride, dst_batch_stride, table_batch_stride,
                         num_heads, seq_len, head_dim, src_seq_stride=None, dst_seq_stride=None, col_scale=None,
                         col_scale_batch_stride=0):
    """rope_one_oop with explicit batch strides (elements) and an optional per-(head, element) factor
    col_scale [batch][num_heads * head_dim] applied before the one rounding."""
    _call("rfk_rope_one_oop_strided", _p(src, H, "src"), _p(dst, H, "dst"), _p(cos_vals, H, "cos"), _p(sin_vals, H, "sin"),
          batch, src_batch_stride, dst_batch_stride, table_batch_stride, num_heads, seq_len, head_dim,
          seq_len if src_seq_stride is None else src_seq_stride, seq_len if dst_seq_stride is None else dst_seq_stride,
          _p(col_scale, F, "col_scale"), col_scale_batch_stride, _stream())


def qkv_norm_rope_transpose(x, row_stride, gammas, outs, use_rope, cos_vals, sin_vals,
                            batch, seq_len, num_heads, head_dim, eps=K_EPS_FP16, out_seq_stride=0):
    n = len(outs)
    g_arr = (ctypes.c_void_p * n)(*[_p(g, F, "gamma") for g in gammas])
    o_arr = (ctypes.c_void_p * n)(*[_p(o, H, "out") for o in outs])
    r_arr = (ctypes.c_int * n)(*[int(bool(r)) for r in use_rope])
    _call("rfk_qkv_norm_rope_transpose", _p(x, H, "x"), row_stride, n, g_arr, o_arr, r_arr,
          _p(cos_vals, H, "cos"), _p(sin_vals, H, "sin"), batch, seq_len, num_heads, head_dim, eps,
          out_seq_stride, _stream())


def transpose_bshd_to_bhsd(inp, out, batch, seq_len, num_heads, head_dim):
    _call("rfk_transpose_bshd_to_bhsd", _p(inp, H, "in"), _p(out, H, "out"), batch, seq_len, num_heads,
          head_dim, _stream())


def transpose_bhsd_to_bsd(inp, out, batch, num_heads, seq_len, head_dim):
    _call("rfk_transpose_bhsd_to_bsd", _p(inp, H, "in"), _p(out, H, "out"), batch, num_heads, seq_len,
          head_dim, _stream())


# ------------------------------------------------------------------ NeRF PE

def nerf_pe(inp, out, batch, seq_len, in_dim, num_freqs, min_freq_exp, max_freq_exp, include_input):
    _call("rfk_nerf_pe", _p(inp, H, "input"), _p(out, H, "output"), batch, seq_len, in_dim, num_freqs,
          min_freq_exp, max_freq_exp, int(include_input), _stream())


def nerf_pe_f32(inp, out, batch, seq_len, in_dim, num_freqs, min_freq_exp, max_freq_exp, include_input):
    _call("rfk_nerf_pe_f32", _p(inp, F, "input"), _p(out, H, "output"), batch, seq_len, in_dim,
          num_freqs, min_freq_exp, max_freq_exp, int(include_input), _stream())


# ------------------------------------------------------------------ softmax

def softmax_inplace(data, rows, cols):
    _call("rfk_softmax_inplace", _p(data, F, "data"), rows, cols, _stream())


def masked_softmax_inplace(data, mask, rows, cols, mask_rows):
    _call("rfk_masked_softmax_inplace", _p(data, F, "data"), _mask_ptr(mask), rows, cols, mask_rows,
          _stream())


def swin_masked_softmax_inplace(data, mask, BnW, num_heads, ws2, nW):
    _call("rfk_swin_masked_softmax_inplace", _p(data, F, "data"), _mask_ptr(mask), BnW, num_heads, ws2,
          nW, _stream())


def softmax_cast_fp16(inp, out, rows, cols, in_stride, out_stride):
    _call("rfk_softmax_cast_fp16", _p(inp, F, "in"), _p(out, H, "out"), rows, cols, in_stride,
          out_stride, _stream())


def softmax_cast_fp16_masked(inp, out, mask, rows, cols, in_stride, out_stride, mask_rows):
    _call("rfk_softmax_cast_fp16_masked", _p(inp, F, "in"), _p(out, H, "out"), _mask_ptr(mask), rows,
          cols, in_stride, out_stride, mask_rows, _stream())


def softmax_cast_fp16_scaled(inp, out, rows, cols, in_stride, out_stride, scale):
    _call("rfk_softmax_cast_fp16_scaled", _p(inp, F, "in"), _p(out, H, "out"), rows, cols, in_stride,
          out_stride, scale, _stream())


def softmax_probs_inplace(scores, rows, n_valid, stride, scale=1.0):
    _call("rfk_softmax_probs_inplace", _p(scores, F, "scores"), rows, n_valid, stride, scale, _stream())


def swin_softmax_probs_inplace(scores, mask, BnW, num_heads, ws2, nW):
    _call("rfk_swin_softmax_probs_inplace", _p(scores, F, "scores"), _mask_ptr(mask), BnW, num_heads,
          ws2, nW, _stream())


def swin_softmax_cast_fp16(inp, out, mask, BnW, num_heads, ws2, nW):
    _call("rfk_swin_softmax_cast_fp16", _p(inp, F, "in"), _p(out, H, "out"), _mask_ptr(mask), BnW,
          num_heads, ws2, nW, _stream())


# ---------------------------------------------------------------- attention

def flash_attention(q, k, v, o, B, Hh, Sq, Sk, n_keys, D, o_bshd=False, scale=None):
    _call("rfk_flash_attention", _p(q, H, "q"), _p(k, H, "k"), _p(v, H, "v"), _p(o, H, "o"), B, Hh, Sq, Sk, n_keys, D,
          int(o_bshd), float(scale if scale is not None else D ** -0.5), _stream())


def window_attention(q, k, v, o, mask, BnW, Hh, nW, window_tokens=64, head_dim=64, scale=None):
    _call("rfk_window_attention", _p(q, H, "q"), _p(k, H, "k"), _p(v, H, "v"), _p(o, H, "o"), _mask_ptr(mask), BnW, Hh,
          window_tokens, head_dim, nW, float(scale if scale is not None else head_dim ** -0.5), _stream())


def flash_attention_ex(q, k, v, o, B, Hh, Sq, Sk, n_keys, D, q_row_ss=None, ss_tiles=0, norm_dim=0, workspace=None,
                       o_bshd=False, scale=None, eps=K_EPS_FP16, v_shared=False):
    """flash_attention (tcgen05 kernel) with optional row statistics - rows scaled by rsqrt(sum(q_row_ss[row]) / norm_dim +
    eps), the query's RMSNorm applied to the scores while its weight rides on the keys - and an optional workspace
    (flash_attention_workspace()) for the key split; v_shared: v is [Hh, Sk, D], the same values for every batch element."""
    _call("rfk_flash_attention_ex", _p(q, H, "q"), _p(k, H, "k"), _p(v, H, "v"), _p(o, H, "o"), _p(q_row_ss, F, "q_row_ss"),
          ss_tiles, norm_dim, eps, _p(workspace, U8, "workspace"), 0 if workspace is None else workspace.numel(), int(v_shared),
          B, Hh, Sq, Sk, n_keys, D, int(o_bshd), float(scale if scale is not None else D ** -0.5), _stream())


def flash_attention_workspace():
    """A zeroed workspace for flash_attention_ex's key split (one per stream of overlapping launches)."""
    return torch.zeros(int(_lib().rfk_flash_attention_workspace_bytes()), dtype=U8, device="cuda")


def flash_attention_set_split(on):
    _call("rfk_flash_attention_set_split", int(bool(on)))


def window_attention_normed(q, k, v, o, mask, q_row_ss, k_row_ss, ss_tiles, gamma_q, gamma_k, norm_dim, BnW, Hh, nW,
                            window_tokens=64, head_dim=64, scale=None, eps=K_EPS_FP16):
    """window_attention over un-normalised Q, K with the RMSNorm (row statistics + weights) applied while staging."""
    _call("rfk_window_attention_normed", _p(q, H, "q"), _p(k, H, "k"), _p(v, H, "v"), _p(o, H, "o"), _mask_ptr(mask),
          _p(q_row_ss, F, "q_row_ss"), _p(k_row_ss, F, "k_row_ss"), ss_tiles, _p(gamma_q, F, "gamma_q"),
          _p(gamma_k, F, "gamma_k"), norm_dim, eps, BnW, Hh, window_tokens, head_dim, nW,
          float(scale if scale is not None else head_dim ** -0.5), _stream())


def flash_attention_set_path(path):
    """0 automatic, 1 mma.sync kernel, 2 tcgen05 kernel (head_dim 64)."""
    _call("rfk_flash_attention_set_path", int(path))


def flash_attention_error(clear=True):
    """Error word of the tcgen05 attention kernel on the current device (0 = none)."""
    import ctypes
    code = ctypes.c_int(-1)
    _call("rfk_flash_attention_error", ctypes.byref(code), int(clear))
    return code.value


# ------------------------------------------------------- dense projections

GEMM_EPI_NONE, GEMM_EPI_RESIDUAL, GEMM_EPI_SWIGLU = 0, 1, 2


def gemm_f16(a, w, c, M, N, K, w_up=None, bias=None, residual=None, lda=None, ldw=None, ldc=None, ldr=None):
    """c[M,N] = epilogue(a[M,K] w[N,K]^T) on the tcgen05 tensor cores (rfk_gemm_f16): plain (+ bias), with
    `residual` added, or - with `w_up` - silu(a w^T) * (a w_up^T). Mirrors rf::linear (src/layers/linear.h:9)
    and the fused steps of rf::ffn_swiglu (src/layers/transformer.cu:63-76)."""
    epi = GEMM_EPI_SWIGLU if w_up is not None else GEMM_EPI_RESIDUAL if residual is not None else GEMM_EPI_NONE
    _call("rfk_gemm_f16", _p(a, H, "a"), lda or K, _p(w, H, "w"), ldw or K, _p(w_up, H, "w_up"), _p(bias, H, "bias"),
          _p(residual, H, "residual"), (ldr or N) if residual is not None else 0, _p(c, H, "c"), ldc or N, M, N, K, epi,
          _stream())


def gemm_f16_heads(a, w, out, row_ss, ss_parts_mask, M, N, K, seq_len, num_heads, part_stride=0, lda=None, ldw=None):
    """Projection stored head-split ([groups][heads][seq_len][64] per part) with the rows' partial sums of squares
    (rfk_gemm_f16_heads): the producer side of the deferred QK-RMSNorm."""
    _call("rfk_gemm_f16_heads", _p(a, H, "a"), lda or K, _p(w, H, "w"), ldw or K, _p(out, H, "out"), part_stride,
          _p(row_ss, F, "row_ss"), ss_parts_mask, M, N, K, seq_len, num_heads, _stream())


def gemm_set_path(path):
    """0 automatic (tcgen05 kernel on CTA pairs), 1 library GEMM only (rfk_gemm_f16 refuses), 2 as 0, 3 single-CTA kernel."""
    _call("rfk_gemm_set_path", int(path))


def gemm_error(clear=True):
    """Error word of the tcgen05 GEMM kernel on the current device (0 = none)."""
    import ctypes
    code = ctypes.c_int(-1)
    _call("rfk_gemm_error", ctypes.byref(code), int(clear))
    return code.value


# -------------------------------------------------------------- activations

def fused_silu_mul(a, b, out, n):
    _call("rfk_fused_silu_mul", _p(a, H, "a"), _p(b, H, "b"), _p(out, H, "out"), n, _stream())


def fused_silu_mul_f32(a, b, out, n):
    _call("rfk_fused_silu_mul_f32", _p(a, F, "a"), _p(b, F, "b"), _p(out, F, "out"), n, _stream())


def swiglu(gate_up, out, rows, hidden):
    _call("rfk_swiglu", _p(gate_up, H, "gate_up"), _p(out, H, "out"), rows, hidden, _stream())


def swiglu_inplace(gate_up, rows, hidden):
    _call("rfk_swiglu_inplace", _p(gate_up, H, "gate_up"), rows, hidden, _stream())


def elu(x, y, n, alpha=1e-3):
    _call("rfk_elu", _p(x, H, "x"), _p(y, H, "y"), n, alpha, _stream())


def pow10_minus1(x, y, n):
    _call("rfk_pow10_minus1", _p(x, F, "x"), _p(y, F, "y"), n, _stream())


def bilinear_upsample(inp, out, N, C, H_in, W_in, H_out, W_out):
    _call("rfk_bilinear_upsample", _p(inp, H, "in"), _p(out, H, "out"), N, C, H_in, W_in, H_out, W_out, _stream())


def silu_inplace(x, n):
    _call("rfk_silu_inplace", _p(x, H, "x"), n, _stream())


def add_bias_nchw(x, bias, N, C, HW):
    _call("rfk_add_bias_nchw", _p(x, H, "x"), _p(bias, H, "bias"), N, C, HW, _stream())


def permute_bsd_to_nchw(inp, out, B, S, D):
    _call("rfk_permute_bsd_to_nchw", _p(inp, H, "in"), _p(out, H, "out"), B, S, D, _stream())


# channels-last ([N, H, W, C]) companions: the layout the DPT head runs on

def bias_act_residual_nhwc(x, bias, residual, rows, C, silu=False):
    """x[r, c] = act(half(x + bias[c])) (+ residual) in place; bias / residual may be None."""
    _call("rfk_bias_act_residual_nhwc", _p(x, H, "x"), _p(bias, H, "bias"), _p(residual, H, "residual"), rows, C, int(silu), _stream())


def silu(x, y, n):
    _call("rfk_silu", _p(x, H, "x"), _p(y, H, "y"), n, _stream())


def bilinear_upsample_nhwc(inp, out, N, H_in, W_in, H_out, W_out, C):
    _call("rfk_bilinear_upsample_nhwc", _p(inp, H, "in"), _p(out, H, "out"), N, H_in, W_in, H_out, W_out, C, _stream())


def depth_to_space_bias_nhwc(inp, bias, out, N, H_, W_, C, f):
    _call("rfk_depth_to_space_bias_nhwc", _p(inp, H, "in"), _p(bias, H, "bias"), _p(out, H, "out"), N, H_, W_, C, f, _stream())


def permute_nhwc_to_nchw(inp, out, N, HW, C):
    _call("rfk_permute_nhwc_to_nchw", _p(inp, H, "in"), _p(out, H, "out"), N, HW, C, _stream())


def pointwise_conv_to_planar(inp, weight, bias, out, N, HW, C_in, C_out):
    """1x1 convolution from channels-last C_in to C_out <= 4 planes + bias: in [N*HW, C_in] -> out [N, C_out, HW]."""
    _call("rfk_pointwise_conv_to_planar", _p(inp, H, "in"), _p(weight, H, "weight"), _p(bias, H, "bias"), _p(out, H, "out"),
          N, HW, C_in, C_out, _stream())


def permute_filter(w, out, K, C, RS, mode):
    """mode 0: [K, C, RS] -> [K, RS, C]; mode 1: transposed-convolution filter [Cin, Cout, f*f] -> [(p, co), ci]."""
    _call("rfk_permute_filter", _p(w, H, "w"), _p(out, H, "out"), K, C, RS, mode, _stream())


def post_elu_pow10(x, y, n, alpha=1e-3):
    _call("rfk_post_elu_pow10", _p(x, H, "x"), _p(y, F, "y"), n, alpha, _stream())


# ------------------------------------------------- per-view ray front end

def ray_gen(c2w, fov, rays_o, rays_d, batch, img_res):
    _call("rfk_ray_gen", _p(c2w, F, "c2w"), _p(fov, F, "fov"), _p(rays_o, F, "rays_o"),
          _p(rays_d, H, "rays_d"), batch, img_res, _stream())


def ray_gen_patchify(c2w, fov, rays_o, ray_pat, batch, img_res, patch_size):
    _call("rfk_ray_gen_patchify", _p(c2w, F, "c2w"), _p(fov, F, "fov"), _p(rays_o, F, "rays_o"),
          _p(ray_pat, H, "ray_pat"), batch, img_res, patch_size, _stream())


def patchify(inp, out, Hh, W, C, ps):
    _call("rfk_patchify", _p(inp, H, "in"), _p(out, H, "out"), Hh, W, C, ps, _stream())


def world_to_cam(c2w, tri, vn, batch, n_tris):
    _call("rfk_world_to_cam", _p(c2w, F, "c2w"), _p(tri, H, "tri"), _p(vn, H, "vn"), batch, n_tris,
          _stream())


def world_to_cam_f32(c2w, verts, normals, batch, n_verts):
    _call("rfk_world_to_cam_f32", _p(c2w, F, "c2w"), _p(verts, F, "verts"), _p(normals, F, "normals"),
          batch, n_verts, _stream())


def view_geometry(c2w, tri_world, vn_world, world_center, learned_freqs, vtri, vvn, vpos, k_cos,
                  k_sin, n_tris, n_register, seq_pad, num_freqs, head_dim):
    _call("rfk_view_geometry", _p(c2w, F, "c2w"), _p(tri_world, H, "tri_world"),
          _p(vn_world, H, "vn_world"), _p(world_center, F, "world_center"),
          _p(learned_freqs, F, "learned_freqs"), _p(vtri, H, "vtri"), _p(vvn, H, "vvn"),
          _p(vpos, H, "vpos"), _p(k_cos, H, "k_cos"), _p(k_sin, H, "k_sin"), n_tris, n_register,
          seq_pad, num_freqs, head_dim, _stream())


# ----------------------------------------------------- swin window layout

def window_gather(x, windows, B, Hh, W, C, ws, shift):
    _call("rfk_window_gather", _p(x, H, "x"), _p(windows, H, "windows"), B, Hh, W, C, ws, shift,
          _stream())


def window_scatter(windows, x, B, Hh, W, C, ws, shift, residual_into=False):
    _call("rfk_window_scatter", _p(windows, H, "windows"), _p(x, H, "x"), B, Hh, W, C, ws, shift,
          int(residual_into), _stream())
