"""Python side of the layer library (include/rfk_layers.h): weight records, the per-scene
render session and the multi-GPU view scheduler.

torch supplies device memory, streams and (for the scheduler) `torch.distributed`; all
compute happens behind the C ABI in librfk_layers.so / librfk.so.

    model   = Model.random(seed=4)                    # renderformer-v1.1-swin-large shapes
    session = RenderSession(model, n_tris=5633, img_res=512)
    session.encode_scene(tri, vn, tex); session.finalize()
    session.render_frame(c2w, fov); tokens = session.download()

    sched = ViewScheduler(model, scene, img_res=512)  # one process per GPU (torchrun)
    sched.render(c2ws, fovs, out=pinned_host_buffer)
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _abi

VP = ctypes.c_void_p
MAX_LAYERS = 32


class FfnW(ctypes.Structure):
    _fields_ = [("w1", VP), ("w2", VP), ("w3", VP)]


class MhaW(ctypes.Structure):
    _fields_ = [(n, VP) for n in ("in_proj_w", "in_proj_b", "out_proj_w", "out_proj_b", "q_norm_gamma", "k_norm_gamma")]


class CrossW(ctypes.Structure):
    _fields_ = [(n, VP) for n in ("q_proj_w", "q_proj_b", "k_proj_w", "k_proj_b", "v_proj_w", "v_proj_b",
                                  "out_proj_w", "out_proj_b", "q_norm_gamma", "k_norm_gamma")]


class EncLayerW(ctypes.Structure):
    _fields_ = [("query_norm_gamma", VP), ("attn", MhaW), ("ffn_norm_gamma", VP), ("ffn", FfnW)]


class DecLayerW(ctypes.Structure):
    _fields_ = [("query_norm_gamma", VP), ("kv_norm_gamma", VP), ("cross_attn", CrossW),
                ("self_attn_norm_gamma", VP), ("self_attn", MhaW), ("ffn_norm_gamma", VP), ("ffn", FfnW)]


class RcuW(ctypes.Structure):
    _fields_ = [(n, VP) for n in ("conv1_w", "conv1_b", "conv2_w", "conv2_b")]


class FfbW(ctypes.Structure):
    _fields_ = [("rcu1", RcuW), ("rcu2", RcuW), ("out_conv_w", VP), ("out_conv_b", VP), ("has_resconv1", ctypes.c_int)]


class DptW(ctypes.Structure):
    """rfk_dpt_weights (include/rfk_layers.h); oracle/ref_shim_layers.cu mirrors the same layout."""
    _fields_ = [("project_w", VP * 4), ("project_b", VP * 4), ("resize_w", VP * 4), ("resize_b", VP * 4),
                ("layer_rn_w", VP * 4), ("refinenet", FfbW * 4),
                ("output_conv1_w", VP), ("output_conv1_b", VP), ("output_conv2a_w", VP), ("output_conv2a_b", VP),
                ("output_conv2b_w", VP), ("output_conv2b_b", VP),
                ("features_dim", ctypes.c_int), ("out_dim", ctypes.c_int), ("out_channels", ctypes.c_int * 4)]


class ModelW(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_int) for n in ("dim", "num_heads", "ffn_hidden", "num_register_tokens", "enc_layers",
                                             "dec_layers", "rope_num_freqs", "patch_size", "window_size", "shift_size",
                                             "texture_channels", "vn_pe_num_freqs")]
                + [(n, VP) for n in ("tri_token", "reg_tokens", "tex_enc_w", "tex_enc_b", "tex_enc_norm", "vn_proj_w",
                                     "vn_proj_b", "vn_enc_norm", "enc_rope_freqs", "ray_map_patch_token", "ray_enc_w",
                                     "ray_enc_b", "ray_enc_norm", "vt_rope_freqs")]
                + [("enc", EncLayerW * MAX_LAYERS), ("dec", DecLayerW * MAX_LAYERS), ("dpt", ctypes.POINTER(DptW))])


RFK_SESSION_PAD_KEYS_ATTEND = 1
RFK_SESSION_NO_GRAPH = 2


def _lib():
    return _abi.load("rfk_layers.h")


class RfkLayersError(RuntimeError):
    pass


def _check(name, rc):
    if rc != 0:
        text = _abi.load("rfk.h").rfk_status_string(rc).decode() if rc < 1000 else f"cuBLAS status {rc - 1000}"
        raise RfkLayersError(f"{name} failed with status {rc}: {text}")


def _ptr(t):
    return None if t is None else t.data_ptr()


class Model:
    """Device weights + the C record that points at them. Shapes follow the reference's
    RenderFormerModel (src/model/renderformer.h:12-44) with runtime dimensions."""

    def __init__(self, dim=1024, num_heads=16, ffn_hidden=4096, num_register_tokens=32, enc_layers=12, dec_layers=12,
                 patch_size=8, window_size=8, shift_size=4, texture_channels=13, vn_pe_num_freqs=6, device="cuda",
                 with_dpt=False, dpt_features=256, dpt_out_channels=(256, 512, 1024, 1024), dpt_out_dim=3):
        # DPT image head (src/model/config.h:38-42); without it a view ends at the decoder's token map
        self.with_dpt, self.dpt_features, self.dpt_out_dim = with_dpt, dpt_features, dpt_out_dim
        self.dpt_out_channels = tuple(dpt_out_channels)
        self.dpt_c = None
        self.dim, self.num_heads, self.ffn_hidden = dim, num_heads, ffn_hidden
        self.head_dim = dim // num_heads
        # frequencies per coordinate: as many as fit, 9*nf <= head_dim/2, at most 6 (src/model/config.h:28)
        self.rope_num_freqs = max(1, min(6, (self.head_dim // 2) // 9))
        self.num_register_tokens, self.enc_layers, self.dec_layers = num_register_tokens, enc_layers, dec_layers
        self.patch_size, self.window_size, self.shift_size = patch_size, window_size, shift_size
        self.texture_channels, self.vn_pe_num_freqs = texture_channels, vn_pe_num_freqs
        self.device = device
        self.t: dict[str, torch.Tensor] = {}
        self.c = ModelW()

    # -- construction -------------------------------------------------------------------
    @classmethod
    def random(cls, seed=4, weight_std=0.02, **kw) -> "Model":
        """Random-init weights of the given architecture: N(0, weight_std) matrices, gains
        N(1, 0.02), geometric rotary frequencies (stand-ins for the learned ones)."""
        m = cls(**kw)
        g = torch.Generator(device=m.device).manual_seed(seed)
        dim, ffn = m.dim, m.ffn_hidden

        def W(*shape):
            return (torch.randn(*shape, device=m.device, generator=g) * weight_std).half().contiguous()

        def G(n):
            return (1 + 0.02 * torch.randn(n, device=m.device, generator=g)).float().contiguous()

        t = m.t
        t["tri_token"], t["reg_tokens"] = W(dim), W(m.num_register_tokens, dim)
        t["tex_enc_w"], t["tex_enc_b"], t["tex_enc_norm"] = W(dim, m.texture_channels), W(dim), G(dim)
        vn_pe = 9 + 9 * m.vn_pe_num_freqs * 2
        t["vn_proj_w"], t["vn_proj_b"], t["vn_enc_norm"] = W(dim, vn_pe), W(dim), G(dim)
        nf = m.rope_num_freqs
        freqs = torch.tensor([math.pi * 10000.0 ** (-i / nf) for i in range(nf)], device=m.device, dtype=torch.float32)
        t["enc_rope_freqs"], t["vt_rope_freqs"] = freqs.clone(), freqs.clone()
        t["ray_map_patch_token"] = W(dim)
        t["ray_enc_w"], t["ray_enc_b"], t["ray_enc_norm"] = W(dim, 3 * m.patch_size ** 2), W(dim), G(dim)
        for i in range(m.enc_layers):
            p = f"enc{i}."
            t[p + "query_norm"], t[p + "ffn_norm"] = G(dim), G(dim)
            t[p + "in_proj_w"], t[p + "out_proj_w"] = W(3 * dim, dim), W(dim, dim)
            t[p + "q_norm"], t[p + "k_norm"] = G(dim), G(dim)
            t[p + "w13"], t[p + "w2"] = W(2 * ffn, dim), W(dim, ffn)   # w1 and w3 stored back to back
        for i in range(m.dec_layers):
            p = f"dec{i}."
            for n in ("query_norm", "kv_norm", "self_attn_norm", "ffn_norm", "cq_norm", "ck_norm", "sq_norm", "sk_norm"):
                t[p + n] = G(dim)
            for n in ("q_proj_w", "k_proj_w", "v_proj_w", "cross_out_w", "swin_out_w"):
                t[p + n] = W(dim, dim)
            t[p + "swin_in_w"] = W(3 * dim, dim)
            t[p + "w13"], t[p + "w2"] = W(2 * ffn, dim), W(dim, ffn)
        if m.with_dpt:
            # convolution weights scaled so that activations keep their magnitude through the head: N(0, 1/sqrt(fan_in))
            def C(cout, cin, k):
                return (torch.randn(cout, cin, k, k, device=m.device, generator=g) * (cin * k * k) ** -0.5).half().contiguous()

            def Bv(n):
                return (0.02 * torch.randn(n, device=m.device, generator=g)).half().contiguous()

            F, oc = m.dpt_features, m.dpt_out_channels
            for i in range(4):
                t[f"dpt.project{i}_w"], t[f"dpt.project{i}_b"] = C(oc[i], dim, 1), Bv(oc[i])
                t[f"dpt.layer_rn{i}_w"] = C(F, oc[i], 3)
                for u in ("rcu1", "rcu2"):
                    if u == "rcu1" and i == 3:
                        continue        # the deepest fusion block has no skip input (has_resconv1 = false)
                    for c_ in ("conv1", "conv2"):
                        t[f"dpt.ref{i}.{u}.{c_}_w"], t[f"dpt.ref{i}.{u}.{c_}_b"] = C(F, F, 3), Bv(F)
                t[f"dpt.ref{i}.out_w"], t[f"dpt.ref{i}.out_b"] = C(F, F, 1), Bv(F)
            # transposed convolutions store [Cin, Cout, k, k]
            t["dpt.resize0_w"], t["dpt.resize0_b"] = (torch.randn(oc[0], oc[0], 4, 4, device=m.device, generator=g) * oc[0] ** -0.5).half(), Bv(oc[0])
            t["dpt.resize1_w"], t["dpt.resize1_b"] = (torch.randn(oc[1], oc[1], 2, 2, device=m.device, generator=g) * oc[1] ** -0.5).half(), Bv(oc[1])
            t["dpt.resize3_w"], t["dpt.resize3_b"] = C(oc[3], oc[3], 3), Bv(oc[3])
            t["dpt.out1_w"], t["dpt.out1_b"] = C(F // 2, F, 3), Bv(F // 2)
            t["dpt.out2a_w"], t["dpt.out2a_b"] = C(32, F // 2, 3), Bv(32)
            t["dpt.out2b_w"], t["dpt.out2b_b"] = C(m.dpt_out_dim, 32, 1), Bv(m.dpt_out_dim)
        m._fill_record()
        return m

    def dpt_record(self) -> DptW:
        t, d = self.t, DptW()
        P = lambda k: t[k].data_ptr() if k in t else None
        for i in range(4):
            d.project_w[i], d.project_b[i] = P(f"dpt.project{i}_w"), P(f"dpt.project{i}_b")
            d.resize_w[i], d.resize_b[i] = P(f"dpt.resize{i}_w"), P(f"dpt.resize{i}_b")
            d.layer_rn_w[i] = P(f"dpt.layer_rn{i}_w")
            f = d.refinenet[i]
            f.has_resconv1 = int(f"dpt.ref{i}.rcu1.conv1_w" in t)
            for u, rec in (("rcu1", f.rcu1), ("rcu2", f.rcu2)):
                rec.conv1_w, rec.conv1_b = P(f"dpt.ref{i}.{u}.conv1_w"), P(f"dpt.ref{i}.{u}.conv1_b")
                rec.conv2_w, rec.conv2_b = P(f"dpt.ref{i}.{u}.conv2_w"), P(f"dpt.ref{i}.{u}.conv2_b")
            f.out_conv_w, f.out_conv_b = P(f"dpt.ref{i}.out_w"), P(f"dpt.ref{i}.out_b")
            d.out_channels[i] = self.dpt_out_channels[i]
        d.output_conv1_w, d.output_conv1_b = P("dpt.out1_w"), P("dpt.out1_b")
        d.output_conv2a_w, d.output_conv2a_b = P("dpt.out2a_w"), P("dpt.out2a_b")
        d.output_conv2b_w, d.output_conv2b_b = P("dpt.out2b_w"), P("dpt.out2b_b")
        d.features_dim, d.out_dim = self.dpt_features, self.dpt_out_dim
        return d

    def _fill_record(self):
        c, t = self.c, self.t
        for n in ("dim", "num_heads", "ffn_hidden", "num_register_tokens", "enc_layers", "dec_layers", "rope_num_freqs",
                  "patch_size", "window_size", "shift_size", "texture_channels", "vn_pe_num_freqs"):
            setattr(c, n, getattr(self, n))
        for n in ("tri_token", "reg_tokens", "tex_enc_w", "tex_enc_b", "tex_enc_norm", "vn_proj_w", "vn_proj_b",
                  "vn_enc_norm", "enc_rope_freqs", "ray_map_patch_token", "ray_enc_w", "ray_enc_b", "ray_enc_norm",
                  "vt_rope_freqs"):
            setattr(c, n, t[n].data_ptr())
        half_w13 = self.ffn_hidden * self.dim * 2  # bytes of w1
        for i in range(self.enc_layers):
            p, e = f"enc{i}.", c.enc[i]
            e.query_norm_gamma, e.ffn_norm_gamma = t[p + "query_norm"].data_ptr(), t[p + "ffn_norm"].data_ptr()
            e.attn = self.mha_record(t[p + "in_proj_w"], t[p + "out_proj_w"], t[p + "q_norm"], t[p + "k_norm"])
            e.ffn = FfnW(t[p + "w13"].data_ptr(), t[p + "w2"].data_ptr(), t[p + "w13"].data_ptr() + half_w13)
        for i in range(self.dec_layers):
            c.dec[i] = self.decoder_record(i)
        if self.with_dpt:
            self.dpt_c = self.dpt_record()
            c.dpt = ctypes.pointer(self.dpt_c)

    @staticmethod
    def mha_record(in_w, out_w, qn, kn) -> MhaW:
        return MhaW(in_w.data_ptr(), None, out_w.data_ptr(), None, _ptr(qn), _ptr(kn))

    def decoder_record(self, i) -> DecLayerW:
        t, p = self.t, f"dec{i}."
        d = DecLayerW()
        d.query_norm_gamma, d.kv_norm_gamma = t[p + "query_norm"].data_ptr(), t[p + "kv_norm"].data_ptr()
        d.cross_attn = CrossW(t[p + "q_proj_w"].data_ptr(), None, t[p + "k_proj_w"].data_ptr(), None,
                              t[p + "v_proj_w"].data_ptr(), None, t[p + "cross_out_w"].data_ptr(), None,
                              t[p + "cq_norm"].data_ptr(), t[p + "ck_norm"].data_ptr())
        d.self_attn_norm_gamma = t[p + "self_attn_norm"].data_ptr()
        d.self_attn = self.mha_record(t[p + "swin_in_w"], t[p + "swin_out_w"], t[p + "sq_norm"], t[p + "sk_norm"])
        d.ffn_norm_gamma = t[p + "ffn_norm"].data_ptr()
        w13 = t[p + "w13"]
        d.ffn = FfnW(w13.data_ptr(), t[p + "w2"].data_ptr(), w13.data_ptr() + self.ffn_hidden * self.dim * 2)
        return d

    def num_params(self) -> int:
        return sum(v.numel() for v in self.t.values())


class Ctx:
    """One cuBLAS context per device (rfk_ctx)."""

    def __init__(self):
        self.h = VP()
        _check("rfk_ctx_create", _lib().rfk_ctx_create(ctypes.byref(self.h)))

    def close(self):
        if self.h:
            _lib().rfk_ctx_destroy(self.h)
            self.h = VP()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class RenderSession:
    """Mirror of the reference's RenderSession (src/pipeline/render_session.h:10-39): create
    for a scene, then render_frame / wait / download per camera view."""

    def __init__(self, model: Model, n_tris: int, img_res: int = 512, scene_state: torch.Tensor | None = None,
                 pad_keys_attend: bool = False, use_graph: bool = True, views_per_frame: int = 1):
        """views_per_frame > 1: a frame is that many views rendered together as one batch (rfk_session_create_batched);
        cameras go in through render_frames, results come back as [views_per_frame, n_tokens, dim]."""
        self.model, self.n_tris, self.img_res = model, n_tris, img_res
        self.views_per_frame = int(views_per_frame)
        lib = _lib()
        lib.rfk_scene_state_bytes.restype = ctypes.c_size_t
        nbytes = lib.rfk_scene_state_bytes(ctypes.byref(model.c), n_tris)
        if nbytes == 0:
            raise RfkLayersError("invalid model or triangle count")
        if scene_state is None:
            scene_state = torch.zeros(nbytes, dtype=torch.uint8, device=model.device)
        if scene_state.numel() < nbytes or not scene_state.is_cuda:
            raise ValueError("scene_state must be a CUDA byte tensor of rfk_scene_state_bytes() bytes")
        self.scene_state = scene_state
        flags = (RFK_SESSION_PAD_KEYS_ATTEND if pad_keys_attend else 0) | (0 if use_graph else RFK_SESSION_NO_GRAPH)
        self.h = VP()
        _check("rfk_session_create_batched", lib.rfk_session_create_batched(ctypes.byref(model.c), n_tris, img_res,
                                                                            scene_state.data_ptr(), flags, self.views_per_frame,
                                                                            ctypes.byref(self.h)))
        self.n_tokens = (img_res // model.patch_size) ** 2
        self.result_bytes = self.n_tokens * model.dim * 2          # per view

    def encode_scene(self, tri: torch.Tensor, vn: torch.Tensor, tex: torch.Tensor):
        """tri, vn [N,3,3] fp32 (world space), tex [N, texture_channels] fp16. Runs the scene
        preprocessing, the encoder and the K/V cache build into the scene state."""
        assert tri.dtype == torch.float32 and vn.dtype == torch.float32 and tex.dtype == torch.float16
        tri, vn, tex = tri.contiguous(), vn.contiguous(), tex.contiguous()
        torch.cuda.synchronize()
        _check("rfk_session_encode_scene", _lib().rfk_session_encode_scene(self.h, tri.data_ptr(), vn.data_ptr(),
                                                                           tex.data_ptr()))

    def finalize(self):
        torch.cuda.synchronize()
        _check("rfk_session_finalize", _lib().rfk_session_finalize(self.h))

    def render_frame(self, c2w, fov_rad: float):
        """c2w: 16 floats (row-major 4x4, host: list / numpy / CPU tensor)."""
        arr = (ctypes.c_float * 16)(*[float(v) for v in (c2w.reshape(-1).tolist() if hasattr(c2w, "reshape") else c2w)])
        _check("rfk_session_render_frame", _lib().rfk_session_render_frame(self.h, arr, ctypes.c_float(fov_rad)))

    def render_frame_raw(self, c2w_ptr: int, fov_rad: float):
        """Same with a raw host pointer to 16 floats (no per-call conversion)."""
        _check("rfk_session_render_frame", _lib().rfk_session_render_frame(self.h, VP(c2w_ptr), ctypes.c_float(fov_rad)))

    def render_frames(self, c2ws, fovs):
        """One frame of views_per_frame views: c2ws [V, 4, 4] (or [V, 16]) and fovs [V], host arrays / CPU tensors."""
        V = self.views_per_frame
        flat = [float(x) for x in (c2ws.reshape(-1).tolist() if hasattr(c2ws, "reshape") else c2ws)]
        fv = [float(x) for x in (fovs.tolist() if hasattr(fovs, "tolist") else fovs)]
        if len(flat) != 16 * V or len(fv) != V:
            raise ValueError(f"render_frames takes {V} cameras")
        _check("rfk_session_render_frames", _lib().rfk_session_render_frames(self.h, (ctypes.c_float * (16 * V))(*flat),
                                                                             (ctypes.c_float * V)(*fv)))

    def render_frames_raw(self, c2w_ptr: int, fov_ptr: int):
        """Same with raw host pointers to [V][16] and [V] floats."""
        _check("rfk_session_render_frames", _lib().rfk_session_render_frames(self.h, VP(c2w_ptr), VP(fov_ptr)))

    def wait(self) -> float:
        ms = ctypes.c_float()
        _check("rfk_session_wait", _lib().rfk_session_wait(self.h, ctypes.byref(ms)))
        return ms.value

    def result_tensor(self) -> torch.Tensor:
        """The last frame's token map [n_tokens, dim] fp16 as a device tensor (via the host)."""
        return self.download().to(self.model.device)

    def _frame_shape(self, *per_view):
        return per_view if self.views_per_frame == 1 else (self.views_per_frame, *per_view)

    def download(self, host: torch.Tensor | None = None) -> torch.Tensor:
        if host is None:
            host = torch.empty(*self._frame_shape(self.n_tokens, self.model.dim), dtype=torch.float16).pin_memory()
        _check("rfk_session_download", _lib().rfk_session_download(self.h, host.data_ptr(), host.numel() * 2))
        return host

    def download_image(self, host: torch.Tensor | None = None) -> torch.Tensor:
        """The last frame's image [out_dim, img_res, img_res] fp32 (models with a DPT head), waits for the frame."""
        m = self.model
        if host is None:
            host = torch.empty(*self._frame_shape(m.dpt_out_dim, self.img_res, self.img_res), dtype=torch.float32).pin_memory()
        _check("rfk_session_download_image", _lib().rfk_session_download_image(self.h, host.data_ptr(), host.numel() * 4))
        return host

    def download_async(self, host: torch.Tensor):
        _check("rfk_session_download_async", _lib().rfk_session_download_async(self.h, host.data_ptr(), host.numel() * 2))

    def drain(self):
        _check("rfk_session_drain", _lib().rfk_session_drain(self.h))

    def mark_begin(self):
        _check("rfk_session_mark_begin", _lib().rfk_session_mark_begin(self.h))

    def mark_end(self) -> float:
        ms = ctypes.c_float()
        _check("rfk_session_mark_end", _lib().rfk_session_mark_end(self.h, ctypes.byref(ms)))
        return ms.value

    @property
    def graph_nodes(self) -> int:
        return _lib().rfk_session_graph_nodes(self.h)

    @property
    def kernels_per_view(self) -> int:
        return _lib().rfk_session_kernels_per_view(self.h)

    def close(self):
        if self.h:
            _lib().rfk_session_destroy(self.h)
            self.h = VP()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def shard_views(n_views: int, rank: int, world: int) -> list[int]:
    """Static round-robin: view v is rendered by rank v mod world."""
    return list(range(rank, n_views, world))


class SchedulerError(RuntimeError):
    pass


class ViewScheduler:
    """Data-parallel view scheduler: one process per GPU. Rank 0 encodes the scene; the scene
    state (cross-attention K/V cache + fp16 geometry) is broadcast once over NCCL into every
    GPU's own memory; each rank then renders its share of the camera views from its local
    copy through its own captured graph. No collective runs on the per-view path.

    `streams_per_gpu` > 1 keeps that many views in flight on the GPU: that many sessions (each with its
    own stream, buffers and captured graphs) share one scene state and take this rank's views in turn,
    so that one view's partial last wave of CTAs and its bandwidth-bound kernels overlap with another
    view's compute-bound ones.

    Failure handling is host-side only and happens between views: a session call that raises marks this
    rank as failed for the rest of the `render` call; after the local pass the ranks exchange (one object
    all-gather on the host) which views are still undone, and the surviving ranks render them. Nothing is
    in flight on a rank when it joins that exchange (its sessions are drained first).

    `session_factory(scene_state_or_None)` builds one session; the default builds a RenderSession. Tests
    inject a host-only stand-in to drive this class without a GPU."""

    def __init__(self, model: Model, n_tris: int, img_res: int = 512, process_group=None, pad_keys_attend=False,
                 streams_per_gpu: int = 1, session_factory=None, views_per_frame: int = 1):
        import torch.distributed as dist
        self.dist = dist if (dist.is_available() and dist.is_initialized()) else None
        self.group = process_group
        self.rank = self.dist.get_rank(process_group) if self.dist else 0
        self.world = self.dist.get_world_size(process_group) if self.dist else 1
        if streams_per_gpu < 1:
            raise ValueError("streams_per_gpu must be at least 1")
        if views_per_frame < 1:
            raise ValueError("views_per_frame must be at least 1")
        self.views_per_frame = views_per_frame
        if session_factory is None:
            def session_factory(scene_state):
                return RenderSession(model, n_tris, img_res, scene_state=scene_state, pad_keys_attend=pad_keys_attend,
                                     views_per_frame=views_per_frame)
        self.session = session_factory(None)
        self.sessions = [self.session] + [session_factory(self.session.scene_state) for _ in range(streams_per_gpu - 1)]
        self.broadcast_ms = 0.0
        self.failed = False          # this rank hit an error in its last render() call
        self.last_error = None

    # -- scene ---------------------------------------------------------------------------
    def encode_scene(self, tri, vn, tex):
        """Runs the scene encoder on this rank (the source of the broadcast)."""
        self.session.encode_scene(tri, vn, tex)

    def broadcast_scene(self, src: int = 0, warm: bool = True) -> float:
        """Broadcasts the scene state from rank `src` into every rank's own buffer; returns the device time of
        that one broadcast in ms (0 for a single rank). With `warm`, two broadcasts of a scratch buffer of the
        same size go first: the communicator allocates its channels and staging buffers on its first large
        message, which otherwise costs an order of magnitude more than the transfer itself."""
        if not (self.dist and self.world > 1):
            return 0.0
        state = self.session.scene_state
        if warm:
            scratch = torch.empty_like(state)
            for _ in range(2):
                self.dist.broadcast(scratch, src=src, group=self.group)
            del scratch
        if state.is_cuda:
            st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            st.record()
            self.dist.broadcast(state, src=src, group=self.group)
            en.record()
            torch.cuda.synchronize()
            self.broadcast_ms = st.elapsed_time(en)
        else:
            import time
            t0 = time.perf_counter()
            self.dist.broadcast(state, src=src, group=self.group)
            self.broadcast_ms = (time.perf_counter() - t0) * 1e3
        return self.broadcast_ms

    def finalize(self):
        for ses in self.sessions:
            ses.finalize()

    def load_scene(self, tri=None, vn=None, tex=None, src: int = 0):
        """Rank `src` passes the scene tensors and runs the encoder; every rank receives the
        scene state. Returns the broadcast time in ms (device events, this rank)."""
        if self.rank == src:
            self.encode_scene(tri, vn, tex)
        self.broadcast_scene(src)
        self.finalize()
        return self.broadcast_ms

    # -- views ---------------------------------------------------------------------------
    def my_views(self, n_views: int) -> list[int]:
        return shard_views(n_views, self.rank, self.world)

    def _render_list(self, views, base, stride, fl, out, out_pos) -> list[int]:
        """Renders `views` in order; returns those NOT rendered because a session call raised."""
        if self.views_per_frame > 1:
            return self._render_list_batched(views, base, stride, fl, out, out_pos)
        n = len(self.sessions)
        for j, v in enumerate(views):
            if self.failed:
                return list(views[j:])
            ses = self.sessions[j % n]
            try:
                ses.render_frame_raw(base + v * stride, fl[v])
                if out is not None:
                    ses.download_async(out[out_pos + j])
            except Exception as e:  # a failing rank keeps running on the host: it reports, the others take over
                self.failed, self.last_error = True, e
                return list(views[j:])
        return []

    def _render_list_batched(self, views, base, stride, fl, out, out_pos) -> list[int]:
        """The same for sessions that take views_per_frame views per frame: the list is cut into frames (the last one
        padded by repeating its last view; the padding's results are dropped). A frame's cameras are gathered first,
        because a rank's views are strided in the caller's array."""
        V, n = self.views_per_frame, len(self.sessions)
        n_frames = (len(views) + V - 1) // V
        self._tail_rows = None
        for f in range(n_frames):
            ids = list(views[f * V:(f + 1) * V])
            real = len(ids)
            ids += [ids[-1]] * (V - real)
            if self.failed:
                return list(views[f * V:])
            ses = self.sessions[f % n]
            try:
                cams = (ctypes.c_float * (16 * V))()          # the call copies them into the session's pinned slot
                for i, v in enumerate(ids):
                    ctypes.memmove(ctypes.addressof(cams) + i * 64, base + v * stride, 64)
                fovs = (ctypes.c_float * V)(*[fl[v] for v in ids])
                ses.render_frames_raw(ctypes.addressof(cams), ctypes.addressof(fovs))
                if out is not None:
                    if real == V:
                        ses.download_async(out[out_pos + f * V: out_pos + (f + 1) * V])
                    else:                      # partial last frame: through a scratch frame, copied out after the drain
                        if getattr(self, "_tail", None) is None:
                            self._tail = torch.empty(V, *out.shape[1:], dtype=out.dtype)
                            if out.is_pinned():
                                self._tail = self._tail.pin_memory()
                        ses.download_async(self._tail)
                        self._tail_rows = (out, out_pos + f * V, real)
            except Exception as e:
                self.failed, self.last_error = True, e
                return list(views[f * V:])
        return []

    def _drain(self):
        for ses in self.sessions:
            try:
                ses.drain()
            except Exception as e:
                self.failed, self.last_error = True, e
        rows = getattr(self, "_tail_rows", None)
        if rows is not None and not self.failed:
            out, pos, real = rows
            out[pos:pos + real].copy_(self._tail[:real])
        self._tail_rows = None

    def render(self, c2ws: torch.Tensor, fovs: torch.Tensor, out: torch.Tensor | None = None) -> list[int]:
        """c2ws [V,4,4] fp32 and fovs [V] fp32 (radians) on the HOST. Renders this rank's views;
        if `out` (pinned host [n_local (+ spare rows for re-issued views), n_tokens, dim] fp16) is given, each
        frame is downloaded into it while the next one renders. Returns the view ids rendered here, in the
        order of the rows of `out`. If a rank fails, its undone views are re-issued to the surviving ranks
        (round-robin) and appended to their lists; SchedulerError if views remain that nobody could render."""
        mine = self.my_views(c2ws.shape[0])
        c2ws = c2ws.contiguous()
        base, stride = c2ws.data_ptr(), 16 * 4
        fl = fovs.tolist()
        self.failed, self.last_error = False, None
        undone = self._render_list(mine, base, stride, fl, out, 0)
        self._drain()
        if self.failed and not undone:
            undone = list(mine)          # the error surfaced while draining: none of this pass can be trusted
        done = [v for v in mine if v not in set(undone)]
        if not (self.dist and self.world > 1):
            if undone:
                raise SchedulerError(f"views {undone} could not be rendered: {self.last_error}") from self.last_error
            return done
        # host-side exchange between passes: who survived, which views are left
        reports = [None] * self.world
        self.dist.all_gather_object(reports, (not self.failed, undone), group=self.group)
        survivors = [r for r, (ok, _) in enumerate(reports) if ok]
        pool = sorted(v for _, u in reports for v in u)
        if pool and not survivors:
            raise SchedulerError(f"views {pool} could not be rendered: every rank failed") from self.last_error
        if pool and not self.failed:
            extra = [v for i, v in enumerate(pool) if survivors[i % len(survivors)] == self.rank]
            if out is not None and len(done) + len(extra) > out.shape[0]:
                raise SchedulerError("`out` has no spare rows for the views re-issued from a failed rank")
            left = self._render_list(extra, base, stride, fl, out, len(done))
            self._drain()
            if left or self.failed:
                raise SchedulerError(f"re-issued views {left or extra} failed on rank {self.rank}") from self.last_error
            done += extra
        return done

    def close(self):
        for ses in self.sessions:
            ses.close()
