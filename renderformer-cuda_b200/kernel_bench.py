"""Per-kernel HBM microbenchmark of the hot-path operators at the benchmark shapes.

For every operator it reports the algorithmic bytes one launch must move (inputs read once
+ outputs written once), the average launch duration measured with CUDA events on the
launching stream, and the achieved GB/s. Cache effects are defeated by rotating each launch
through enough independent buffer sets that the working set exceeds twice the 126 MB L2
(`config: "l2": "rotating buffer sets > 2x L2"`), so consecutive launches never touch lines
the previous ones left in cache.

The suite is backend-neutral: a backend is an object with one method per operator taking
torch CUDA tensors (see `RfkBackend`). The benchmark driver supplies a second backend that
wraps the reference engine's kernels to time them with the same harness.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable

import torch

L2_BYTES = 126 * 1024 * 1024
T, D, HEADS, HD, NF = 5633, 1024, 16, 64, 3
RES, NP = 512, 4096
SOFTMAX_ROWS = HEADS * NP   # 65536 score rows; the CLI can shrink it for profiler captures


@dataclass
class Entry:
    name: str
    config: int
    bytes_per_launch: int
    make: Callable[[], tuple]        # () -> argument tuple (one buffer set)
    op: str                          # backend method name
    launches: int = 1                # kernels per call for the rfk backend


def _r(shape, dtype=torch.float32, scale=1.0):
    return (torch.randn(shape, device="cuda") * scale).to(dtype)


def _cams(n):
    g = torch.Generator().manual_seed(3)
    d = torch.nn.functional.normalize(torch.randn(n, 3, generator=g), dim=-1)
    pos = d * (2 + 2 * torch.rand(n, 1, generator=g))
    fwd = -torch.nn.functional.normalize(pos, dim=-1)
    up = torch.tensor([0.0, 0.0, 1.0]).expand(n, 3)
    right = torch.nn.functional.normalize(torch.cross(fwd, up, dim=-1), dim=-1)
    up2 = torch.cross(right, fwd, dim=-1)
    c2w = torch.zeros(n, 4, 4)
    c2w[:, :3, 0], c2w[:, :3, 1], c2w[:, :3, 2], c2w[:, :3, 3], c2w[:, 3, 3] = right, up2, -fwd, pos, 1.0
    fov = torch.deg2rad(30 + 30 * torch.rand(n, generator=g))
    return c2w.cuda().contiguous(), fov.cuda().contiguous()


def suite() -> list[Entry]:
    H16 = torch.float16
    e: list[Entry] = []
    # config 1: h fp32 (r+w), r fp32 (r), y16 (w), gamma
    e.append(Entry("rmsnorm_residual_f32_cast16 [5633x1024]", 1, 3 * 4 * T * D + 2 * T * D + 4 * D,
                   lambda: (_r((T, D)), _r((T, D)), 1 + 0.02 * _r((D,)), torch.empty((T, D), device="cuda", dtype=H16)),
                   "fused_rmsnorm"))
    e.append(Entry("rmsnorm_residual_f32_cast16 x8 batch [45064x1024]", 1, 8 * (3 * 4 * T * D + 2 * T * D) + 4 * D,
                   lambda: (_r((8 * T, D)), _r((8 * T, D)), 1 + 0.02 * _r((D,)), torch.empty((8 * T, D), device="cuda", dtype=H16)),
                   "fused_rmsnorm"))
    # config 2
    def rope_set():
        pos = (torch.rand(1, T, 9, device="cuda") * 2 - 1).half()
        c = torch.empty(1, 1, T, HD, device="cuda", dtype=H16); s = torch.empty_like(c)
        return (_r((1, HEADS, T, HD), H16), _r((1, HEADS, T, HD), H16), c, s, pos)
    e.append(Entry("apply_rope q,k [16x5633x64]", 2, 4 * 2 * HEADS * T * HD + 2 * 2 * T * HD, rope_set, "rope"))

    def rope_set8():
        c = torch.empty(8, 1, T, HD, device="cuda", dtype=H16).normal_(); s = torch.empty_like(c).normal_()
        return (_r((8, HEADS, T, HD), H16), _r((8, HEADS, T, HD), H16), c, s, None)
    e.append(Entry("apply_rope q,k x8 batch", 2, 8 * (4 * 2 * HEADS * T * HD + 2 * 2 * T * HD), rope_set8, "rope"))
    e.append(Entry("triangle_rope_freqs [5633x9 -> 2x5633x64]", 2, 2 * 9 * T + 2 * 2 * T * HD, rope_set, "rope_tables"))

    def pe_normals(b):
        def mk():
            n = torch.nn.functional.normalize(torch.randn(b, T, 3, 3, device="cuda"), dim=-1).reshape(b, T, 9).contiguous()
            return (n, torch.empty(b, T, 117, device="cuda", dtype=H16))
        return mk
    e.append(Entry("nerf_pe_f32 normals [5633x9 -> 117]", 2, T * (9 * 4 + 117 * 2), pe_normals(1), "nerf_pe_f32"))
    e.append(Entry("nerf_pe_f32 normals x64 batch", 2, 64 * T * (9 * 4 + 117 * 2), pe_normals(64), "nerf_pe_f32"))
    # config 3
    rows, cols, stride = SOFTMAX_ROWS, 5633, 5640
    def sm_set():
        x = torch.empty(rows, stride, device="cuda")
        x.normal_(0.0, 3.0 / 8.0)
        x[:, cols:] = float("-inf")
        return (x, torch.empty(rows, stride, device="cuda", dtype=H16), rows, cols, stride)
    e.append(Entry(f"softmax_cast_fp16 [{rows}x5633 stride 5640]", 3, rows * (cols * 4 + stride * 2), sm_set, "softmax"))
    # config 4
    def ray_set(b):
        def mk():
            c2w, fov = _cams(b)
            return (c2w, fov, torch.empty(b, 3, device="cuda"), torch.empty(b, RES, RES, 3, device="cuda", dtype=H16), b)
        return mk
    e.append(Entry("ray_gen 512x512", 4, RES * RES * 6 + 64 + 4 + 12, ray_set(1), "ray_gen"))
    e.append(Entry("ray_gen 512x512 x64 batch", 4, 64 * (RES * RES * 6 + 80), ray_set(64), "ray_gen"))

    def w2c_set(b):
        def mk():
            c2w, _ = _cams(b)
            tri = (torch.rand(b, T, 3, 3, device="cuda") * 2 - 1).half()
            vn = torch.nn.functional.normalize(torch.randn(b, T, 3, 3, device="cuda"), dim=-1).half()
            return (c2w, tri, vn, b)
        return mk
    e.append(Entry("world_to_cam 5633 tris (tri+vn fp16)", 4, 2 * 2 * T * 9 * 2 + 64, w2c_set(1), "world_to_cam"))
    e.append(Entry("world_to_cam 5633 tris x64 batch", 4, 64 * (2 * 2 * T * 9 * 2 + 64), w2c_set(64), "world_to_cam"))
    e.append(Entry("world_to_cam 5633 tris x512 batch", 4, 512 * (2 * 2 * T * 9 * 2 + 64), w2c_set(512), "world_to_cam"))

    def pe_dirs(b):
        def mk():
            d = torch.nn.functional.normalize(torch.randn(b, RES * RES, 3, device="cuda"), dim=-1).half()
            return (d, torch.empty(b, RES * RES, 39, device="cuda", dtype=H16))
        return mk
    e.append(Entry("nerf_pe ray dirs [262144x3 -> 39]", 4, RES * RES * (3 + 39) * 2, pe_dirs(1), "nerf_pe_f16"))
    e.append(Entry("nerf_pe ray dirs x8 batch", 4, 8 * RES * RES * (3 + 39) * 2, pe_dirs(8), "nerf_pe_f16"))
    # decoder-layer kernels that have no counterpart among the reference's src/kernels (library batches + glue there)
    def win_set():
        q = _r((64, HEADS, 64, HD), H16); k = _r((64, HEADS, 64, HD), H16); v = _r((64, HEADS, 64, HD), H16)
        mask = (torch.rand(64, 64, 64, device="cuda") > 0.3).to(torch.uint8)
        return (q, k, v, torch.empty(64 * 64, HEADS * HD, device="cuda", dtype=H16), mask)
    e.append(Entry("window_attention [64 windows x 16 heads x 64x64x64, masked]", 5, 4 * 64 * HEADS * 64 * HD * 2 + 64 * 64 * 64,
                   win_set, "window_attention"))

    def winnorm_set():
        q, k, v, o, mask = win_set()
        ss = torch.rand(2, 64 * 64, HEADS * HD // 256, device="cuda") * 256 + 1
        g = torch.ones(HEADS * HD, device="cuda")
        return (q, k, v, o, mask, ss, g)
    e.append(Entry("window_attention_normed [same; q, k normalised while staged]", 5,
                   4 * 64 * HEADS * 64 * HD * 2 + 64 * 64 * 64 + 2 * 64 * 64 * (HEADS * HD // 256) * 4, winnorm_set, "window_attention_normed"))

    def normwin_set():
        return (_r((4096, 1024), H16), _r((4096, 1024), H16), torch.ones(1024, device="cuda"), torch.empty(4096, 1024, device="cuda", dtype=H16))
    e.append(Entry("rmsnorm_residual_f16 -> windows [4096x1024]", 5, 4 * 4096 * 1024 * 2 + 4096, normwin_set, "rmsnorm_windows"))
    def qproj_set(parts):
        def mk():
            x = _r((4096, parts * 1024), H16)
            outs = [torch.empty(HEADS, 4096, HD, device="cuda", dtype=H16) for _ in range(parts)]
            c = torch.rand(4096, HD, device="cuda").half(); s_ = torch.rand(4096, HD, device="cuda").half()
            return (x, outs, torch.ones(1024, device="cuda"), c, s_)
        return mk
    e.append(Entry("qkv_norm_rope_transpose cross q [4096x1024 -> 16x4096x64, norm + rope]", 5,
                   2 * 4096 * 1024 * 2 + 2 * 4096 * HD * 2 + 4096, qproj_set(1), "qkv_epilogue"))
    e.append(Entry("qkv_norm_rope_transpose swin q,k,v [4096x3072 -> 3x16x4096x64, q,k norm]", 5,
                   2 * 4096 * 3072 * 2 + 2 * 4096, qproj_set(3), "qkv_epilogue"))
    # element-wise operators of the DPT head at the sizes of a 512x512 view (src/layers/dpt.cu)
    def up_set(C, hi, ho):
        return lambda: (_r((1, C, hi, hi), H16), torch.empty(1, C, ho, ho, device="cuda", dtype=H16), C, hi, ho)
    e.append(Entry("bilinear_upsample [256 x 128^2 -> 256^2]", 5, 256 * (128 * 128 + 256 * 256) * 2, up_set(256, 128, 256), "bilinear_upsample"))
    e.append(Entry("bilinear_upsample [256 x 256^2 -> 512^2]", 5, 256 * (256 * 256 + 512 * 512) * 2, up_set(256, 256, 512), "bilinear_upsample"))
    e.append(Entry("silu_inplace [256 x 256^2]", 5, 2 * 256 * 256 * 256 * 2, lambda: (_r((256 * 256 * 256,), H16),), "silu_inplace"))
    e.append(Entry("add_bias_nchw [256 x 256^2]", 5, 2 * 256 * 256 * 256 * 2 + 512,
                   lambda: (_r((1, 256, 256, 256), H16), _r((256,), H16)), "add_bias_nchw"))
    e.append(Entry("permute_bsd_to_nchw [4096 x 1024]", 5, 2 * 4096 * 1024 * 2,
                   lambda: (_r((1, 4096, 1024), H16), torch.empty(1, 1024, 4096, device="cuda", dtype=H16)), "permute_bsd_to_nchw"))
    e.append(Entry("fused_silu_mul [4096x4096] fp16", 4, 3 * 4096 * 4096 * 2,
                   lambda: (_r((4096, 4096), H16), _r((4096, 4096), H16), torch.empty(4096, 4096, device="cuda", dtype=H16)),
                   "silu_mul"))
    return e


class RfkBackend:
    """The operators of this package (C ABI -> CUDA kernels)."""
    name = "rfk"

    def __init__(self):
        from . import ops
        self.o = ops

    def fused_rmsnorm(self, h, r, g, y):
        self.o.rmsnorm_residual_f32_cast16(h, r, g, y, h.shape[0], h.shape[1], 1e-6)

    def rope(self, q, k, c, s, pos):
        self.o.apply_rope(q, k, c, s, q.shape[0], HEADS, T, HD)

    def rope_tables(self, q, k, c, s, pos):
        self.o.triangle_rope_freqs(pos, self.freqs(), c, s, 1, T, NF, HD)

    def freqs(self):
        if not hasattr(self, "_f"):
            self._f = torch.tensor([math.pi * 10000.0 ** (-i / NF) for i in range(NF)], device="cuda", dtype=torch.float32)
        return self._f

    def nerf_pe_f32(self, x, out):
        self.o.nerf_pe_f32(x, out, x.shape[0], x.shape[1], x.shape[2], 6, 0.0, 5.0, True)

    def nerf_pe_f16(self, x, out):
        self.o.nerf_pe(x, out, x.shape[0], x.shape[1], x.shape[2], 6, 0.0, 5.0, True)

    def softmax(self, x, p, rows, cols, stride):
        self.o.softmax_cast_fp16(x, p, rows, cols, stride, stride)

    def ray_gen(self, c2w, fov, ro, rd, b):
        self.o.ray_gen(c2w, fov, ro, rd, b, RES)

    def world_to_cam(self, c2w, tri, vn, b):
        self.o.world_to_cam(c2w, tri, vn, b, T)

    def silu_mul(self, a, b, out):
        self.o.fused_silu_mul(a, b, out, a.numel())

    def window_attention(self, q, k, v, o, mask):
        self.o.window_attention(q, k, v, o, mask, 64, HEADS, 64)

    def window_attention_normed(self, q, k, v, o, mask, ss, g):
        self.o.window_attention_normed(q, k, v, o, mask, ss[0], ss[1], ss.shape[-1], g, g, g.numel(), 64, HEADS, 64)

    def qkv_epilogue(self, x, outs, gamma, c, s):
        n = len(outs)
        if n == 1:
            self.o.qkv_norm_rope_transpose(x, 1024, [gamma], outs, [1], c, s, 1, 4096, HEADS, HD)
        else:
            self.o.qkv_norm_rope_transpose(x, 3072, [gamma, gamma, None], outs, [0, 0, 0], None, None, 1, 4096, HEADS, HD)

    def bilinear_upsample(self, x, o, C, hi, ho):
        self.o.bilinear_upsample(x, o, 1, C, hi, hi, ho, ho)

    def silu_inplace(self, x):
        self.o.silu_inplace(x, x.numel())

    def add_bias_nchw(self, x, b):
        self.o.add_bias_nchw(x, b, 1, x.shape[1], x.shape[2] * x.shape[3])

    def permute_bsd_to_nchw(self, x, o):
        self.o.permute_bsd_to_nchw(x, o, 1, x.shape[1], x.shape[2])

    def rmsnorm_windows(self, x, r, gamma, y):
        self.o.rmsnorm_residual_f16_windows(x, r, gamma, y, 1, 64, 64, 1024, 8, 4, 1)


def time_entry(entry: Entry, backend, iters: int = 20, warmup: int = 3, budget_bytes: int = 3 * L2_BYTES):
    """Average launch duration (ms) of one operator over `iters` launches on rotating sets.

    The launches are captured once into a CUDA graph and the graph is replayed between two
    CUDA events, so the figure is device time (kernel + the few hundred ns between graph
    nodes) and not the host's launch rate. Operators that cannot be captured (the
    reference's nerf_pe wrappers allocate) are launched eagerly with one event pair per launch.
    """
    nsets = max(2, min(64, math.ceil(budget_bytes / max(entry.bytes_per_launch, 1))))
    sets = [entry.make() for _ in range(nsets)]
    fn = getattr(backend, entry.op)
    for w in range(max(warmup, 3)):
        fn(*sets[w % nsets])
    torch.cuda.synchronize()
    if entry.op in getattr(backend, "not_capturable", ()):
        total = 0.0
        for i in range(iters):
            st = torch.cuda.Event(enable_timing=True); en = torch.cuda.Event(enable_timing=True)
            st.record(); fn(*sets[i % nsets]); en.record()
            torch.cuda.synchronize()
            total += st.elapsed_time(en)
        ms = total / iters
        mode = "eager, event pair per launch"
    else:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(iters):
                fn(*sets[i % nsets])
        graph.replay()  # warm replay
        torch.cuda.synchronize()
        st = torch.cuda.Event(enable_timing=True); en = torch.cuda.Event(enable_timing=True)
        st.record()
        graph.replay()
        en.record()
        torch.cuda.synchronize()
        ms = st.elapsed_time(en) / iters
        mode = "cuda graph replay"
        del graph
    del sets
    return ms, nsets, mode


def run_suite(backend, peak_gbs: float, iters: int = 20, warmup: int = 3, only: set | None = None) -> list[dict]:
    rows = []
    for entry in suite():
        if (only and entry.op not in only) or not hasattr(backend, entry.op):
            continue
        ms, nsets, mode = time_entry(entry, backend, iters, warmup)
        gbs = entry.bytes_per_launch / (ms * 1e-3) / 1e9
        rows.append({"kernel": entry.name, "config": entry.config, "op": entry.op,
                     "bytes": entry.bytes_per_launch, "us": round(ms * 1e3, 2), "gbs": round(gbs, 1),
                     "frac_measured_peak": round(gbs / peak_gbs, 3), "frac_8tbs": round(gbs / 8000.0, 3),
                     "buffer_sets": nsets, "timing": mode})
        torch.cuda.empty_cache()
    return rows


def _time_graph(fn, nsets, iters):
    for i in range(3):
        fn(i % nsets)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fn(i % nsets)
    graph.replay()
    torch.cuda.synchronize()
    st = torch.cuda.Event(enable_timing=True); en = torch.cuda.Event(enable_timing=True)
    st.record(); graph.replay(); en.record()
    torch.cuda.synchronize()
    return st.elapsed_time(en) / iters


def gemm_table(iters: int = 20, nsets: int = 6) -> list[dict]:
    """The projections of one decoder layer at the benchmark shape (4096 tokens, dim 1024, FFN 4096), each timed
    through rfk_gemm_f16 (tcgen05 kernel, fused epilogue) and through the library route the layer functions fall
    back to (cublasGemmEx, plus the separate gate / residual kernel the fused epilogue replaces), on rotating
    weight and activation sets (graph replay, CUDA events)."""
    import ctypes
    from . import _abi, ops, session
    L = _abi.load("rfk_layers.h")
    VP = ctypes.c_void_p
    ctx = session.Ctx()
    H16 = torch.float16
    M, dim, ffn = NP, D, 4096
    rows = []

    def P(t):
        return VP(t.data_ptr())

    def st():
        return VP(torch.cuda.current_stream().cuda_stream)

    def case(name, N, K, epi, flop):
        a = [_r((M, K), H16) for _ in range(nsets)]
        w = [_r((N, K), H16, K ** -0.5) for _ in range(nsets)]
        wu = [_r((N, K), H16, K ** -0.5) for _ in range(nsets)] if epi == "swiglu" else None
        c = [torch.empty(M, N, device="cuda", dtype=H16) for _ in range(nsets)]
        r = [_r((M, N), H16) for _ in range(nsets)] if epi == "residual" else None
        gu = torch.empty(M, 2 * N, device="cuda", dtype=H16) if epi == "swiglu" else None
        wcat = [torch.cat([w[i], wu[i]]) for i in range(nsets)] if epi == "swiglu" else None

        def fused(i):
            ops.gemm_f16(a[i], w[i], c[i], M, N, K, w_up=wu[i] if wu else None, residual=r[i] if r else None)

        def library(i):
            if epi == "swiglu":   # one [M, 2N] product + the in-place gate kernel
                assert L.rfk_linear(ctx.h, P(a[i]), P(wcat[i]), None, P(gu), M, 2 * N, K, st()) == 0
                ops.swiglu_inplace(gu, M, N)
            else:
                assert L.rfk_linear(ctx.h, P(a[i]), P(w[i]), None, P(c[i]), M, N, K, st()) == 0
                if epi == "residual":
                    ops.residual_add(c[i], r[i], M * N)

        ops.gemm_set_path(2)
        t_f = _time_graph(fused, nsets, iters)
        ops.gemm_set_path(3)
        t_s = _time_graph(fused, nsets, iters)
        ops.gemm_set_path(1)
        t_l = _time_graph(library, nsets, iters)
        ops.gemm_set_path(0)
        rows.append({"gemm": name, "M": M, "N": N, "K": K, "epilogue": epi, "us_tcgen05": round(t_f * 1e3, 2),
                     "tflops_tcgen05": round(flop / (t_f * 1e-3) / 1e12, 1), "us_tcgen05_single_cta": round(t_s * 1e3, 2), "us_library": round(t_l * 1e3, 2),
                     "tflops_library": round(flop / (t_l * 1e-3) / 1e12, 1), "speedup": round(t_l / t_f, 3)})
        torch.cuda.empty_cache()

    def heads_case(name, parts):
        """Projection stored head-split with the rows' sums of squares (rfk_gemm_f16_heads) against the route it
        replaces: the plain projection followed by the QK-norm + head-split kernel (rfk_qkv_norm_rope_transpose)."""
        N, K = parts * dim, dim
        a = [_r((M, K), H16) for _ in range(nsets)]
        w = [_r((N, K), H16, K ** -0.5) for _ in range(nsets)]
        c = [torch.empty(M, N, device="cuda", dtype=H16) for _ in range(nsets)]
        out = [torch.empty(parts, M * dim, device="cuda", dtype=H16) for _ in range(nsets)]
        outs = [[o[p] for p in range(parts)] for o in out]
        ss = torch.empty(parts, M, dim // 256, device="cuda")
        g = torch.ones(dim, device="cuda")
        gam = [g, g, None][:parts] if parts == 3 else [g]
        seq = M if parts == 1 else 64
        heads = dim // HD

        def fused(i):
            ops.gemm_f16_heads(a[i], w[i], out[i], ss, 3 if parts == 3 else 1, M, N, K, seq, heads, part_stride=M * dim)

        def separate(i):
            ops.gemm_f16(a[i], w[i], c[i], M, N, K)
            ops.qkv_norm_rope_transpose(c[i], N, gam, outs[i], [False] * parts, None, None, M // seq, seq, heads, HD)

        ops.gemm_set_path(0)
        t_f = _time_graph(fused, nsets, iters)
        t_l = _time_graph(separate, nsets, iters)
        flop = 2.0 * M * N * K
        rows.append({"gemm": name, "M": M, "N": N, "K": K, "epilogue": "heads + row statistics", "us_tcgen05": round(t_f * 1e3, 2),
                     "tflops_tcgen05": round(flop / (t_f * 1e-3) / 1e12, 1), "us_projection_then_norm_kernel": round(t_l * 1e3, 2),
                     "speedup": round(t_l / t_f, 3)})
        torch.cuda.empty_cache()

    case("q / out projection", dim, dim, "none", 2.0 * M * dim * dim)
    heads_case("cross q projection -> heads", 1)
    heads_case("swin in projection -> heads", 3)
    case("out projection + residual", dim, dim, "residual", 2.0 * M * dim * dim)
    case("swin in projection", 3 * dim, dim, "none", 2.0 * M * 3 * dim * dim)
    case("FFN w1|w3 + SwiGLU", ffn, dim, "swiglu", 2.0 * M * 2 * ffn * dim)
    case("FFN w2 + residual", dim, ffn, "residual", 2.0 * M * dim * ffn)
    err = ops.gemm_error(clear=False)
    ctx.close()
    if err:
        raise RuntimeError(f"tcgen05 GEMM kernel reported error word {err}")
    return rows


def _main():
    """python -m renderformer_cuda_b200.kernel_bench [--op NAME ...] [--iters N] [--eager]

    Prints one JSON object per operator. --eager launches without graph capture (what a
    profiler wants: a few plain launches of the selected operator); --rows scales the
    softmax case down so that a profiler capture stays small."""
    import argparse
    import json
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", action="append", help="operator(s) to run (default: all)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--peak", type=float, default=6455.6, help="HBM GB/s used for the fraction column")
    ap.add_argument("--softmax-rows", type=int, default=SOFTMAX_ROWS)
    ap.add_argument("--gemm", action="store_true", help="print the tcgen05-vs-library GEMM table instead")
    ap.add_argument("--profile", choices=["attention", "gemm", "dpt"],
                    help="a few plain launches of the fused cross-attention (16 x 4096 queries x 5665 keys) or of the "
                         "decoder layer's projections through rfk_gemm_f16, for a profiler capture")
    ap.add_argument("--views", type=int, default=1, help="--profile attention: views per launch (a frame of the batched session)")
    a = ap.parse_args()
    if a.gemm:
        for row in gemm_table(a.iters):
            print(json.dumps(row))
        return
    if a.profile:
        from . import ops
        H16 = torch.float16
        if a.profile == "dpt":
            # the DPT image head alone at the benchmark size (four [4096, 1024] token maps -> [3, 512, 512]), random weights
            import ctypes
            from . import _abi, session
            L = _abi.load("rfk_layers.h")
            model = session.Model.random(seed=4, dim=D, num_heads=HEADS, ffn_hidden=64, enc_layers=0, dec_layers=0, with_dpt=True)
            ctx = session.Ctx()
            head = ctypes.c_void_p()
            rc = L.rfk_dpt_create(ctx.h, ctypes.byref(model.dpt_c), 1, D, RES // 8, RES // 8, 8, ctypes.byref(head))
            assert rc == 0, rc
            feats = [_r((NP, D), H16) for _ in range(4)]
            taps = (ctypes.c_void_p * 4)(*[f.data_ptr() for f in feats])
            img = torch.empty(3, RES, RES, device="cuda", dtype=H16)
            st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
            for i in range(a.iters + 1):
                if i == 1:
                    t0.record()
                assert L.rfk_dpt_forward(head, taps, ctypes.c_void_p(img.data_ptr()), st) == 0
            t1.record()
            torch.cuda.synchronize()
            print(json.dumps({"kernel": "rfk_dpt_forward 4 x [4096,1024] -> [3,512,512]", "launched": a.iters + 1,
                              "us_per_forward_eager": round(t0.elapsed_time(t1) * 1e3 / max(a.iters, 1), 1),
                              "convolutions": L.rfk_dpt_num_convolutions(head), "finite": bool(torch.isfinite(img.float()).all())}))
            L.rfk_dpt_destroy(head)
            ctx.close()
            return
        if a.profile == "attention":
            Se = 5665; Sp = (Se + 7) & ~7
            V = a.views
            if V < 1:
                ap.error("--views must be at least 1")
            if V == 1:
                q, k, v = _r((1, HEADS, NP, HD), H16), _r((1, HEADS, Sp, HD), H16), _r((1, HEADS, Sp, HD), H16)
                o = torch.empty(1, NP, HEADS * HD, device="cuda", dtype=H16)
                for _ in range(a.iters):
                    ops.flash_attention(q, k, v, o, 1, HEADS, NP, Sp, Se, HD, o_bshd=True)
            else:
                # a frame of V views as the session launches it: own queries and rotated keys per view, one set of
                # values, the queries' RMSNorm applied from their row statistics
                q, k, v = _r((V, HEADS, NP, HD), H16), _r((V, HEADS, Sp, HD), H16), _r((HEADS, Sp, HD), H16)
                o = torch.empty(V, NP, HEADS * HD, device="cuda", dtype=H16)
                ss = torch.rand(V, NP, D // 256, device="cuda") * 256.0 + 1.0
                for _ in range(a.iters):
                    ops.flash_attention_ex(q, k, v, o, V, HEADS, NP, Sp, Se, HD, q_row_ss=ss, ss_tiles=D // 256, norm_dim=D,
                                           o_bshd=True, v_shared=True)
            torch.cuda.synchronize()
            print(json.dumps({"kernel": f"flash_attention {V}x16x4096x5665 d64", "launched": a.iters, "error_word": ops.flash_attention_error()}))
        else:
            M, dim, ffn = NP, D, 4096
            x, xh = _r((M, dim), H16), _r((M, ffn), H16)
            w_q, w_in, w1, w3, w2 = (_r(s_, H16, 0.03) for s_ in ((dim, dim), (3 * dim, dim), (ffn, dim), (ffn, dim), (dim, ffn)))
            y, y3, act, res = (torch.empty(M, n, device="cuda", dtype=H16) for n in (dim, 3 * dim, ffn, dim))
            res.normal_()
            ss = torch.empty(3, M, dim // 256, device="cuda")
            for _ in range(a.iters):
                ops.gemm_f16_heads(x, w_q, y, ss, 1, M, dim, dim, M, HEADS)                              # cross q -> heads + statistics
                ops.gemm_f16_heads(x, w_in, y3, ss, 3, M, 3 * dim, dim, 64, HEADS, part_stride=M * dim)  # swin q|k|v -> heads
                ops.gemm_f16(x, w_q, y, M, dim, dim)                       # q / out projection
                ops.gemm_f16(x, w_in, y3, M, 3 * dim, dim)                 # swin in projection
                ops.gemm_f16(x, w1, act, M, ffn, dim, w_up=w3)             # FFN w1 | w3 + SwiGLU
                ops.gemm_f16(xh, w2, res, M, dim, ffn, residual=res)       # FFN w2 + residual, in place
            torch.cuda.synchronize()
            print(json.dumps({"kernel": "rfk_gemm_f16_heads x2 + rfk_gemm_f16 x4 shapes", "launched": 6 * a.iters, "error_word": ops.gemm_error()}))
        return
    globals()["SOFTMAX_ROWS"] = a.softmax_rows
    backend = RfkBackend()
    if a.eager:
        for entry in suite():
            if a.op and entry.op not in a.op:
                continue
            sets = [entry.make() for _ in range(2)]
            fn = getattr(backend, entry.op)
            for i in range(a.iters):
                fn(*sets[i % 2])
            torch.cuda.synchronize()
            print(json.dumps({"kernel": entry.name, "launched": a.iters}))
        return
    for row in run_suite(backend, a.peak, a.iters, 3, set(a.op) if a.op else None):
        print(json.dumps(row))


if __name__ == "__main__":
    _main()
