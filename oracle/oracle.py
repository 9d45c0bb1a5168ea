"""numpy front end of the CPU oracle (oracle/rfk_oracle.c -> oracle/liboracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the host-core
baseline leg of the benchmark. The product path never imports this module.

Every function takes and returns numpy arrays (float16 arrays stand for the engine's `half`),
never modifies its inputs unless the name says `_` in place, and follows the semantics of the
reference kernel named in the C source.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_lib = None


def build(force: bool = False) -> Path:
    """Compile liboracle.so with gcc (a few seconds)."""
    so = HERE / "liboracle.so"
    src = HERE / "rfk_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "oracle"], check=True, capture_output=True)
    return so


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.oracle_max_threads.restype = ctypes.c_int
        _lib.oracle_get_threads.restype = ctypes.c_int
    return _lib


def set_threads(n: int) -> None:
    lib().oracle_set_threads(ctypes.c_int(n))


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


L, I, Fl = ctypes.c_long, ctypes.c_int, ctypes.c_float
f16, f32 = np.float16, np.float32

# ------------------------------------------------------------------ RMSNorm


def rmsnorm(x, gamma, eps):
    x = _c(x, f16); rows, dim = x.shape
    y = np.empty_like(x)
    lib().oracle_rmsnorm_f16(_ptr(x), _ptr(_c(gamma, f32)), _ptr(y), L(rows), I(dim), Fl(eps))
    return y


def rmsnorm_f32(x, gamma, eps):
    x = _c(x, f32); rows, dim = x.shape
    y = np.empty_like(x)
    lib().oracle_rmsnorm_f32(_ptr(x), _ptr(_c(gamma, f32)), _ptr(y), L(rows), I(dim), Fl(eps))
    return y


def rmsnorm_residual_f32_cast16(h, r, gamma, eps):
    """Returns (h_updated fp32, y16). r may be fp32, fp16 (mixed form) or None."""
    h = _c(h, f32).copy(); rows, dim = h.shape
    y = np.empty(h.shape, f16)
    r_is_half = 0
    if r is not None:
        r_is_half = int(r.dtype == np.float16)
        r = _c(r, f16 if r_is_half else f32)
    lib().oracle_rmsnorm_residual_f32_cast16(_ptr(h), _ptr(r), I(r_is_half), _ptr(_c(gamma, f32)),
                                             _ptr(y), L(rows), I(dim), Fl(eps))
    return h, y


def rmsnorm_residual_f16(x, r, gamma, eps):
    """Returns (x_updated fp16, y fp16)."""
    x = _c(x, f16).copy(); rows, dim = x.shape
    y = np.empty_like(x)
    lib().oracle_rmsnorm_residual_f16(_ptr(x), _ptr(None if r is None else _c(r, f16)),
                                      _ptr(_c(gamma, f32)), _ptr(y), L(rows), I(dim), Fl(eps))
    return x, y


# ---------------------------------------------- residual / cast plumbing


def residual_add(y, r):
    y = _c(y, f16).copy(); lib().oracle_residual_add_f16(_ptr(y), _ptr(_c(r, f16)), L(y.size)); return y


def residual_add_f32(y, r):
    y = _c(y, f32).copy(); lib().oracle_residual_add_f32(_ptr(y), _ptr(_c(r, f32)), L(y.size)); return y


def residual_add_mixed(y, r):
    y = _c(y, f32).copy(); lib().oracle_residual_add_mixed(_ptr(y), _ptr(_c(r, f16)), L(y.size)); return y


def cast_fp32_to_fp16(a):
    a = _c(a, f32); o = np.empty(a.shape, f16); lib().oracle_cast_f32_to_f16(_ptr(a), _ptr(o), L(a.size)); return o


def cast_fp16_to_fp32(a):
    a = _c(a, f16); o = np.empty(a.shape, f32); lib().oracle_cast_f16_to_f32(_ptr(a), _ptr(o), L(a.size)); return o


def broadcast_add(out, bc):
    out = _c(out, f16).copy(); bc = _c(bc, f16)
    lib().oracle_broadcast_add(_ptr(out), _ptr(bc), L(out.size), I(bc.size)); return out


# --------------------------------------------------------------------- RoPE


def triangle_rope_freqs(pos, freqs, head_dim):
    """pos [..., 9] fp16 -> (cos, sin) [..., head_dim] fp16."""
    pos = _c(pos, f16); freqs = _c(freqs, f32)
    tokens = pos.size // 9
    shape = pos.shape[:-1] + (head_dim,)
    c = np.empty(shape, f16); s = np.empty(shape, f16)
    lib().oracle_triangle_rope_freqs(_ptr(pos), _ptr(freqs), _ptr(c), _ptr(s), L(tokens),
                                     I(freqs.size), I(head_dim))
    return c, s


def apply_rope(x, cos_vals, sin_vals):
    """x [B,H,S,D] fp16 or fp32, tables [B,1,S,D] / [B,S,D] fp16; returns the rotated copy."""
    B, Hh, S, D = x.shape
    c = _c(cos_vals, f16).reshape(B, S, D); s = _c(sin_vals, f16).reshape(B, S, D)
    if x.dtype == np.float16:
        x = _c(x, f16).copy()
        lib().oracle_apply_rope_f16(_ptr(x), _ptr(c), _ptr(s), I(B), I(Hh), I(S), I(D))
    else:
        x = _c(x, f32).copy()
        lib().oracle_apply_rope_f32(_ptr(x), _ptr(c), _ptr(s), I(B), I(Hh), I(S), I(D))
    return x


# ------------------------------------------------------------------ NeRF PE


def nerf_pe(x, num_freqs, min_exp, max_exp, include_input):
    """x [..., in_dim] fp16 or fp32 -> [..., out_dim] fp16."""
    is_half = x.dtype == np.float16
    x = _c(x, f16 if is_half else f32)
    in_dim = x.shape[-1]; rows = x.size // in_dim
    out_dim = in_dim * num_freqs * 2 + (in_dim if include_input else 0)
    out = np.empty(x.shape[:-1] + (out_dim,), f16)
    lib().oracle_nerf_pe(_ptr(x), I(int(is_half)), _ptr(out), L(rows), I(in_dim), I(num_freqs),
                         Fl(min_exp), Fl(max_exp), I(int(include_input)))
    return out


# ------------------------------------------------------------------ softmax


def softmax_cast_fp16(scores, cols, out_stride, mask=None, scale=1.0):
    """scores [rows, in_stride] fp32 -> probabilities [rows, out_stride] fp16."""
    scores = _c(scores, f32); rows, in_stride = scores.shape
    out = np.empty((rows, out_stride), f16)
    mr = 1
    if mask is not None:
        mask = _c(mask, np.uint8).reshape(-1, cols); mr = mask.shape[0]
    lib().oracle_softmax_cast_fp16(_ptr(scores), _ptr(out), _ptr(mask), I(mr), L(rows), I(cols),
                                   L(in_stride), L(out_stride), Fl(scale))
    return out


def softmax_inplace(data, mask=None, swin=None):
    """data [rows, cols] fp32. mask [mask_rows, cols]; swin = (heads, nW) selects window mapping."""
    data = _c(data, f32).copy(); rows, cols = data.shape
    mr, ws2, heads, nW, sw = 1, 0, 0, 0, 0
    if mask is not None:
        mask = _c(mask, np.uint8).reshape(-1, cols); mr = mask.shape[0]
        if swin is not None:
            heads, nW = swin; ws2 = cols; sw = 1
    lib().oracle_softmax_inplace(_ptr(data), _ptr(mask), I(sw), I(mr), I(ws2), I(heads), I(nW),
                                 L(rows), I(cols))
    return data


# ------------------------------------------------------------------- linear


def linear(x, w, bias=None):
    """x [M,K] fp16 (any row pitch), w [N,K] fp16 -> half(x w^T) (+ bias), fp32 accumulation (rf::linear)."""
    x = np.asarray(x)
    assert x.dtype == f16 and x.ndim == 2 and x.strides[1] == 2 and x.strides[0] % 2 == 0
    w = _c(w, f16)
    M, K = x.shape; N = w.shape[0]
    out = np.empty((M, N), f16)
    lib().oracle_linear_f16(_ptr(x), L(x.strides[0] // 2), _ptr(w), _ptr(None if bias is None else _c(bias, f16)), _ptr(out),
                            L(M), I(N), I(K))
    return out


# ---------------------------------------------------------------- attention


def sdpa(Q, K, V, n_keys=None, mask=None, o_bshd=False, scale=None):
    """Q [B,H,Sq,D], K,V [B,H,Sk,D] fp16 -> O fp16 ([B,H,Sq,D] or [B,Sq,H*D]); mask [nW,Sq,Sk] bytes (0 = masked out)."""
    Q, K, V = _c(Q, f16), _c(K, f16), _c(V, f16)
    B, Hh, Sq, D = Q.shape; Sk = K.shape[2]
    n_keys = Sk if n_keys is None else n_keys
    nW = 1
    if mask is not None:
        mask = _c(mask, np.uint8); nW = mask.shape[0]
        assert mask.shape == (nW, Sq, Sk) and n_keys == Sk
    out = np.empty((B, Sq, Hh * D) if o_bshd else (B, Hh, Sq, D), f16)
    lib().oracle_sdpa(_ptr(Q), _ptr(K), _ptr(V), _ptr(out), I(B), I(Hh), I(Sq), I(Sk), I(n_keys), I(D),
                      Fl(scale if scale is not None else D ** -0.5), _ptr(mask), I(nW), I(int(o_bshd)))
    return out


def sdpa_f32acc(Q, K, V, n_keys=None, scale=None):
    """The unmasked attention with fp32 accumulation (the timed host-core port); O [B,Sq,H*D] fp16."""
    Q, K, V = _c(Q, f16), _c(K, f16), _c(V, f16)
    B, Hh, Sq, D = Q.shape; Sk = K.shape[2]
    out = np.empty((B, Sq, Hh * D), f16)
    lib().oracle_sdpa_f32acc(_ptr(Q), _ptr(K), _ptr(V), _ptr(out), I(B), I(Hh), I(Sq), I(Sk), I(Sk if n_keys is None else n_keys),
                             I(D), Fl(scale if scale is not None else D ** -0.5))
    return out


# -------------------------------------------------------------- activations


def fused_silu_mul(a, b):
    if a.dtype == np.float16:
        a = _c(a, f16); o = np.empty_like(a)
        lib().oracle_silu_mul_f16(_ptr(a), _ptr(_c(b, f16)), _ptr(o), L(a.size))
    else:
        a = _c(a, f32); o = np.empty_like(a)
        lib().oracle_silu_mul_f32(_ptr(a), _ptr(_c(b, f32)), _ptr(o), L(a.size))
    return o


def swiglu(gate_up):
    gate_up = _c(gate_up, f16); rows, two_h = gate_up.shape
    o = np.empty((rows, two_h // 2), f16)
    lib().oracle_swiglu(_ptr(gate_up), _ptr(o), L(rows), I(two_h // 2)); return o


def elu(x, alpha=1e-3):
    x = _c(x, f16); o = np.empty_like(x); lib().oracle_elu(_ptr(x), _ptr(o), L(x.size), Fl(alpha)); return o


def pow10_minus1(x):
    x = _c(x, f32); o = np.empty_like(x); lib().oracle_pow10_minus1(_ptr(x), _ptr(o), L(x.size)); return o


def post_elu_pow10(x, alpha=1e-3):
    x = _c(x, f16); o = np.empty(x.shape, f32)
    lib().oracle_post_elu_pow10(_ptr(x), _ptr(o), L(x.size), Fl(alpha)); return o


# ------------------------------------------------- DPT head glue


def bilinear_upsample(x, H_out, W_out):
    x = _c(x, f16); N, C, Hi, Wi = x.shape
    o = np.empty((N, C, H_out, W_out), f16)
    lib().oracle_bilinear_upsample(_ptr(x), _ptr(o), L(N * C), I(Hi), I(Wi), I(H_out), I(W_out)); return o


def silu(x):
    x = _c(x, f16); o = np.empty_like(x); lib().oracle_silu(_ptr(x), _ptr(o), L(x.size)); return o


def add_bias_nchw(x, bias):
    x = _c(x, f16).copy(); bias = _c(bias, f16); N, C = x.shape[:2]
    lib().oracle_add_bias_nchw(_ptr(x), _ptr(bias), L(N), I(C), L(x.size // (N * C))); return x


def permute_bsd_to_nchw(x):
    x = _c(x, f16); B, S, D = x.shape
    o = np.empty((B, D, S), f16)
    lib().oracle_permute_bsd_to_nchw(_ptr(x), _ptr(o), L(B), L(S), L(D)); return o


# ------------------------------------------------- per-view ray front end


def ray_gen(c2w, fov, res, patch_size=0):
    """Returns (rays_o [B,3] fp32, rays_d [B,res,res,3] fp16 or tokens [B,nP,3*ps*ps])."""
    c2w = _c(c2w, f32).reshape(-1, 16); fov = _c(fov, f32).reshape(-1); B = fov.size
    ro = np.empty((B, 3), f32)
    if patch_size:
        out = np.empty((B, (res // patch_size) ** 2, 3 * patch_size * patch_size), f16)
    else:
        out = np.empty((B, res, res, 3), f16)
    lib().oracle_ray_gen(_ptr(c2w), _ptr(fov), _ptr(ro), _ptr(out), I(B), I(res), I(patch_size))
    return ro, out


def world_to_cam(c2w, tri, vn=None):
    """tri/vn [B, n_verts, 3] (any shape with B leading) fp16 or fp32; returns transformed copies."""
    c2w = _c(c2w, f32).reshape(-1, 16); B = c2w.shape[0]
    dt = f16 if tri.dtype == np.float16 else f32
    tri = _c(tri, dt).copy(); vn = None if vn is None else _c(vn, dt).copy()
    n_verts = tri.size // (3 * B)
    fn = lib().oracle_world_to_cam_f16 if dt == f16 else lib().oracle_world_to_cam_f32
    fn(_ptr(c2w), _ptr(tri), _ptr(vn), I(B), I(n_verts))
    return tri, vn


def center_pos(c2w, center, nr):
    out = np.empty((nr, 9), f16)
    lib().oracle_center_pos(_ptr(_c(c2w, f32)), _ptr(_c(center, f32)), _ptr(out), I(nr)); return out


# ----------------------------------------------------------------- layouts


def transpose_bshd_to_bhsd(x):
    x = _c(x, f16); B, S, Hh, D = x.shape; o = np.empty((B, Hh, S, D), f16)
    lib().oracle_transpose_bshd_to_bhsd(_ptr(x), _ptr(o), I(B), I(S), I(Hh), I(D)); return o


def transpose_bhsd_to_bsd(x):
    x = _c(x, f16); B, Hh, S, D = x.shape; o = np.empty((B, S, Hh * D), f16)
    lib().oracle_transpose_bhsd_to_bsd(_ptr(x), _ptr(o), I(B), I(Hh), I(S), I(D)); return o


def deinterleave_qkv(src, D):
    src = _c(src, f16); M = src.shape[0]
    q = np.empty((M, D), f16); k = np.empty((M, D), f16); v = np.empty((M, D), f16)
    lib().oracle_deinterleave_qkv(_ptr(src), _ptr(q), _ptr(k), _ptr(v), L(M), I(D)); return q, k, v


def cyclic_shift(x, sh, sw):
    x = _c(x, f16); B, Hh, W, C = x.shape; o = np.empty_like(x)
    lib().oracle_cyclic_shift(_ptr(x), _ptr(o), I(B), I(Hh), I(W), I(C), I(sh), I(sw)); return o


def window_partition(x, ws):
    x = _c(x, f16); B, Hh, W, C = x.shape
    o = np.empty((B * (Hh // ws) * (W // ws), ws * ws, C), f16)
    lib().oracle_window_partition(_ptr(x), _ptr(o), I(B), I(Hh), I(W), I(C), I(ws), I(0)); return o


def window_reverse(win, B, Hh, W, ws):
    win = _c(win, f16); C = win.shape[-1]; o = np.empty((B, Hh, W, C), f16)
    lib().oracle_window_partition(_ptr(win), _ptr(o), I(B), I(Hh), I(W), I(C), I(ws), I(1)); return o


def patchify(x, ps):
    x = _c(x, f16); Hh, W, C = x.shape
    o = np.empty(((Hh // ps) * (W // ps), C * ps * ps), f16)
    lib().oracle_patchify(_ptr(x), _ptr(o), I(Hh), I(W), I(C), I(ps)); return o


# ----------------------------------------------- compositions used by tests


def qkv_norm_rope_transpose(qkv, n_parts, gammas, use_rope, cos_vals, sin_vals, B, S, Hh, D, eps):
    """Unfused restatement of the projection epilogue (src/layers/attention.cu:184-210):
    split the [B*S, n_parts*dim] buffer, RMSNorm over the full dim, BSHD->BHSD, RoPE."""
    dim = Hh * D
    outs = []
    for p in range(n_parts):
        part = _c(qkv[:, p * dim:(p + 1) * dim], f16)
        if gammas[p] is not None:
            part = rmsnorm(part, gammas[p], eps)
        t = transpose_bshd_to_bhsd(part.reshape(B, S, Hh, D))
        if use_rope[p]:
            t = apply_rope(t, cos_vals, sin_vals)
        outs.append(t)
    return outs
