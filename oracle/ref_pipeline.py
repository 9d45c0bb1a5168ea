"""The reference engine's scene encoding and per-view decoder pipeline, driven through
oracle/_ref/libref_layers.so (the reference's own kernels and layer functions, compiled
unchanged) from Python.

TEST INFRASTRUCTURE ONLY: used by the GPU parity tests and by the reference arm of the
benchmark. Nothing here loads or calls the product's libraries; torch supplies device memory
and a few exact element-wise steps (casts, a copy, a log10) whose reference kernels are
file-local to src/pipeline/render_session.cu.

    state = ref_pipeline.encode_scene(model, tri, vn, tex)      # render_session.cu:296-416
    pipe  = ref_pipeline.ViewPipeline(model, state, n_tris, img_res)   # :177-238, graph replay
    pipe.render(host_ptr_to_16_floats, fov); ms = pipe.wait(); pipe.download(pinned_tensor)

`model` is any object with the attributes of renderformer_cuda_b200.session.Model (shape
fields and the dict `t` of weight tensors); the scene state has the layout the product
documents for rfk_scene_state_bytes: [dec_layers][K,V][heads][Se_pad][head_dim] fp16, then
256-byte-aligned fp16 triangles, fp16 normals and the fp32 scene centre.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import ref

VP = ctypes.c_void_p


def _up(v: int, a: int = 256) -> int:
    return (v + a - 1) // a * a


def state_layout(model, n_tris: int) -> dict:
    Se = model.num_register_tokens + n_tris
    Se_pad = (Se + 7) & ~7
    kv_layer = Se_pad * model.dim * 2
    tri_off = _up(2 * model.dec_layers * kv_layer)
    vn_off = _up(tri_off + n_tris * 18)
    c_off = _up(vn_off + n_tris * 18)
    return dict(Se=Se, Se_pad=Se_pad, kv_layer=kv_layer, tri_off=tri_off, vn_off=vn_off, c_off=c_off,
                total=_up(c_off + 12))


def decoder_record(model, i: int) -> "ref.DecoderLayerW":
    t, p = model.t, f"dec{i}."
    w = ref.DecoderLayerW()
    for k, v in dict(query_norm_gamma=t[p + "query_norm"], kv_norm_gamma=t[p + "kv_norm"], q_proj_w=t[p + "q_proj_w"],
                     k_proj_w=t[p + "k_proj_w"], v_proj_w=t[p + "v_proj_w"], cross_out_w=t[p + "cross_out_w"],
                     cross_q_norm=t[p + "cq_norm"], cross_k_norm=t[p + "ck_norm"],
                     self_attn_norm_gamma=t[p + "self_attn_norm"], swin_in_w=t[p + "swin_in_w"],
                     swin_out_w=t[p + "swin_out_w"], swin_q_norm=t[p + "sq_norm"], swin_k_norm=t[p + "sk_norm"],
                     ffn_norm_gamma=t[p + "ffn_norm"], w2=t[p + "w2"]).items():
        setattr(w, k, v.data_ptr())
    w13 = t[p + "w13"]
    w.w1 = w13.data_ptr()
    w.w3 = w13.data_ptr() + model.ffn_hidden * model.dim * 2
    return w


def shift_mask(pH: int, ws: int, shift: int) -> torch.Tensor:
    """[windows, ws*ws, ws*ws] bool-as-bytes: same pre-shift region (render_session.cu:99-116)."""
    n = pH // ws
    reg = np.array([[((i + shift) % pH // ws) * n + ((j + shift) % pH // ws) for j in range(pH)] for i in range(pH)])
    mask = np.zeros((n * n, ws * ws, ws * ws), np.uint8)
    for wi in range(n):
        for wj in range(n):
            r = reg[wi * ws:(wi + 1) * ws, wj * ws:(wj + 1) * ws].reshape(-1)
            mask[wi * n + wj] = (r[:, None] == r[None, :])
    return torch.from_numpy(mask).cuda()


def encode_scene(model, tri: torch.Tensor, vn: torch.Tensor, tex: torch.Tensor, state: torch.Tensor | None = None) -> torch.Tensor:
    """Scene preprocessing, the mixed-precision encoder and the per-layer cross-attention K/V
    cache with the reference's own functions, in the order of RenderSession::create
    (src/pipeline/render_session.cu:296-416). tri, vn [N,3,3] fp32; tex [N,13] fp16 (first texel)."""
    R, L = ref, ref.layers()
    if L is None:
        raise RuntimeError("oracle/_ref/libref_layers.so is not built")
    m, t = model, model.t
    N, dim, nh, ffn, nr = tri.shape[0], m.dim, m.num_heads, m.ffn_hidden, m.num_register_tokens
    hd = dim // nh
    lay = state_layout(m, N)
    Se, Se_pad = lay["Se"], lay["Se_pad"]
    if state is None:
        state = torch.zeros(lay["total"], dtype=torch.uint8, device="cuda")
    blas = R.cublas_create()
    f16, f32 = torch.float16, torch.float32
    e = lambda *s, dt=f16: torch.empty(*s, device="cuda", dtype=dt)
    try:
        # texture: last three channels log-encoded (k_log_encode_s :33-38); geometry cast to fp16 (:301-304)
        texb = tex.clone()
        texb[:, -3:] = torch.log10(texb[:, -3:].float() + 1.0).half()
        tri16, vn16 = tri.half().contiguous(), vn.half().contiguous()
        # world-space centroid on the host in double (compute_world_centroid :62-70)
        h = tri16.reshape(N, 9).cpu().numpy().astype(np.float32).astype(np.float64)
        mean9 = h.sum(0) / N
        c = np.array([(mean9[j] + mean9[3 + j] + mean9[6 + j]) / 3.0 for j in range(3)], dtype=np.float32)
        center = torch.from_numpy(c).cuda()
        # normals: nerf_pe_f32 -> linear -> fp32 RMSNorm (:310-318)
        pe_dim = 9 + 9 * m.vn_pe_num_freqs * 2
        vn_pe = e(N, pe_dim)
        R.call("ref_nerf_pe_f32", vn.contiguous(), vn_pe, 1, N, 9, m.vn_pe_num_freqs, 0.0, float(m.vn_pe_num_freqs - 1), 1)
        emb = e(N, dim)
        R.call("ref_linear", R.Raw(blas), vn_pe, t["vn_proj_w"], t["vn_proj_b"], emb, N, dim, pe_dim, lib=L)
        vn_n = emb.float()
        R.call("ref_rmsnorm_f32", vn_n, t["vn_enc_norm"], vn_n, N, dim, 2.0 ** -10)
        # texture: linear -> fp32 RMSNorm (:321-327)
        R.call("ref_linear", R.Raw(blas), texb.contiguous(), t["tex_enc_w"], t["tex_enc_b"], emb, N, dim, m.texture_channels, lib=L)
        tex_n = emb.float()
        R.call("ref_rmsnorm_f32", tex_n, t["tex_enc_norm"], tex_n, N, dim, 2.0 ** -10)
        # sequence = [register tokens | texture + normal + triangle token], fp32 (k_add3_bc_f32_s :39-43, :330-339)
        seq = e(Se, dim, dt=f32)
        seq[:nr] = t["reg_tokens"].float()
        seq[nr:] = (tex_n + vn_n) + t["tri_token"].float()
        # encoder positions and rotary tables (:342-350)
        pos = e(1, Se, 9)
        pos[0, :nr] = center.half().repeat(3)
        pos[0, nr:] = tri16.reshape(N, 9)
        ec, es = e(1, 1, Se, hd), e(1, 1, Se, hd)
        R.call("ref_triangle_rope_freqs", pos, t["enc_rope_freqs"], ec, es, 1, Se, m.rope_num_freqs, hd)
        # encoder (:356-371)
        temp, qkv, ffnb = e(Se * dim), e(Se * max(3 * dim, 2 * ffn)), e(Se * max(dim, ffn))
        score = e(nh * Se * Se_pad, dt=f32)
        for i in range(m.enc_layers):
            p = f"enc{i}."
            w13 = t[p + "w13"]
            R.call("ref_encoder_layer_forward_mixed", R.Raw(blas), t[p + "query_norm"], t[p + "in_proj_w"], t[p + "out_proj_w"],
                   t[p + "q_norm"], t[p + "k_norm"], t[p + "ffn_norm"], R.Raw(w13.data_ptr()), t[p + "w2"],
                   R.Raw(w13.data_ptr() + ffn * dim * 2), seq, temp, qkv, ffnb, score, 1, Se, dim, nh, ffn, ec, es, lib=L)
        del score
        ctx16 = seq.half()
        # K/V cache per decoder layer, padded to Se_pad rows per head (:377-416)
        ctx_n, kvp = e(Se, dim), e(2 * Se * dim)
        Kt, Vt = e(nh, Se, hd), e(nh, Se, hd)
        kv = state[:2 * m.dec_layers * lay["kv_layer"]].view(f16).view(m.dec_layers, 2, nh, Se_pad, hd)
        kv.zero_()
        for i in range(m.dec_layers):
            w = decoder_record(m, i)
            R.call("ref_rmsnorm", ctx16, t[f"dec{i}.kv_norm"], ctx_n, Se, dim, 2.0 ** -10)
            R.call("ref_precompute_cross_kv", R.Raw(blas), ctypes.byref(w), ctx_n, Kt, Vt, kvp, 1, Se, dim, dim, nh, lib=L)
            kv[i, 0, :, :Se] = Kt
            kv[i, 1, :, :Se] = Vt
        state[lay["tri_off"]:lay["tri_off"] + N * 18].view(f16).copy_(tri16.reshape(-1))
        state[lay["vn_off"]:lay["vn_off"] + N * 18].view(f16).copy_(vn16.reshape(-1))
        state[lay["c_off"]:lay["c_off"] + 12].view(f32).copy_(center)
        torch.cuda.synchronize()
    finally:
        R.cublas_destroy(blas)
    return state


class ViewPipeline:
    """Per-view decoder pipeline of the reference (oracle/ref_shim_layers.cu: ref_view_*):
    its world_to_cam / RoPE-table / ray_gen front end and its decoder_layer_forward_cached per
    layer, captured and replayed as one CUDA graph as the reference does."""

    def __init__(self, model, state: torch.Tensor, n_tris: int, img_res: int, use_graph: bool = True):
        if not ref.layers_available():
            raise RuntimeError("oracle/_ref/libref_layers.so is not built")
        self.L = ref.layers()
        m, t = model, model.t
        lay = state_layout(m, n_tris)
        base, kvl = state.data_ptr(), lay["kv_layer"]
        K = (VP * m.dec_layers)(*[base + (2 * i) * kvl for i in range(m.dec_layers)])
        V = (VP * m.dec_layers)(*[base + (2 * i + 1) * kvl for i in range(m.dec_layers)])
        W = (ref.DecoderLayerW * m.dec_layers)()
        for i in range(m.dec_layers):
            W[i] = decoder_record(m, i)
        pH = img_res // m.patch_size
        self.mask = shift_mask(pH, m.window_size, m.shift_size)
        cfg = (ctypes.c_int * 11)(n_tris, img_res, m.dim, m.num_heads, m.ffn_hidden, m.num_register_tokens,
                                  m.rope_num_freqs, m.patch_size, m.window_size, m.shift_size, m.dec_layers)
        fn = self.L.ref_view_create
        fn.restype = VP
        self.keep = (K, V, W, cfg, state)
        self.h = fn(cfg, VP(base + lay["tri_off"]), VP(base + lay["vn_off"]), VP(base + lay["c_off"]),
                    VP(t["vt_rope_freqs"].data_ptr()), VP(t["ray_enc_w"].data_ptr()), VP(t["ray_enc_b"].data_ptr()),
                    VP(t["ray_enc_norm"].data_ptr()), VP(t["ray_map_patch_token"].data_ptr()), W, K, V,
                    VP(self.mask.data_ptr()), ctypes.c_int(1 if use_graph else 0))
        self.L.ref_view_wait.restype = ctypes.c_float
        self.n_tokens, self.dim = pH * pH, m.dim

    def graph_nodes(self) -> int:
        return int(self.L.ref_view_graph_nodes(VP(self.h)))

    def render(self, c2w_host_ptr: int, fov: float):
        self.L.ref_view_render(VP(self.h), VP(c2w_host_ptr), ctypes.c_float(fov))

    def wait(self) -> float:
        return float(self.L.ref_view_wait(VP(self.h)))

    def download(self, host: torch.Tensor):
        rc = self.L.ref_view_download(VP(self.h), VP(host.data_ptr()), ctypes.c_size_t(host.numel() * 2))
        assert rc == 0

    def taps(self):
        out = (VP * 4)()
        self.L.ref_view_taps(VP(self.h), out)
        return [int(v) for v in out]

    def stream(self) -> int:
        self.L.ref_view_stream.restype = VP
        return int(self.L.ref_view_stream(VP(self.h)))

    def close(self):
        if self.h:
            self.L.ref_view_destroy(VP(self.h))
            self.h = None


class ImageHead:
    """The reference's DPT head and image post-process after a view (src/pipeline/render_session.cu:239-253):
    rf::dpt_forward over the pipeline's feature taps, elu, cast to fp32, pow10_minus1, launched on the pipeline's
    stream. rf::dpt_forward allocates and frees its intermediates per call (stream-ordered)."""

    def __init__(self, model, pipe: ViewPipeline, img_res: int):
        self.pipe, self.m, self.res = pipe, model, img_res
        self.blas = ref.cublas_create()
        n = model.dpt_out_dim * img_res * img_res
        self.out16 = torch.empty(n, device="cuda", dtype=torch.float16)
        self.out32 = torch.empty(n, device="cuda", dtype=torch.float32)
        self.col = torch.empty(1 << 29, device="cuda", dtype=torch.float16)      # cuDNN workspace (the reference reserves 4.8 GB)
        self.taps = pipe.taps()
        self.ts = torch.cuda.ExternalStream(pipe.stream())

    def run(self):
        m, p = self.m, self.pipe
        R = ref
        st = p.stream()
        pH = self.res // m.patch_size
        R.call("ref_dpt_forward", R.Raw(self.blas), ctypes.byref(m.dpt_c), R.Raw(self.taps[0]), R.Raw(self.taps[1]),
               R.Raw(self.taps[2]), R.Raw(self.taps[3]), self.out16, self.col, 1, m.dim, pH, pH, m.patch_size, lib=ref.layers(),
               stream=st)
        R.call("ref_elu", self.out16, self.out16, self.out16.numel(), 1e-3, stream=st)
        with torch.cuda.stream(self.ts):
            self.out32.copy_(self.out16)                                           # k_fp16_to_fp32_s (:251-252)
        R.call("ref_pow10_minus1", self.out32, self.out32, self.out32.numel(), stream=st)

    def download(self, host: torch.Tensor):
        with torch.cuda.stream(self.ts):
            host.copy_(self.out32.view_as(host), non_blocking=True)
        self.ts.synchronize()

    def close(self):
        ref.cublas_destroy(self.blas)
