"""Data-driven parity cases shared by the CPU tests, the GPU tests and the golden-fixture
generator.

A case names one operator at one (small) shape and knows how to
  * build its seeded inputs as numpy arrays                      -> make()
  * run the CPU oracle on them                                   -> oracle()
  * run the CUDA kernels of this repo through the C ABI          -> rfk()
  * run the reference engine's own CUDA kernels (oracle/_ref)    -> ref()   (may be absent)
and how each output is compared ("f16", "f32" or "exact").

Tolerances (north-star statement): bit-exact for ray_gen / world_to_cam / pure data
movement; <= 1e-3 relative for fp32 outputs; <= 2e-3 absolute for fp16 outputs. An fp16
output whose magnitude exceeds 2 has a rounding step above 2e-3, so for those the bound is
one fp16 rounding step (2^-10 relative), which is what "the same fp32 value rounded once"
can differ by when the fp32 values differ in their last bits.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import oracle as O  # noqa: E402  (test infrastructure)

F16_ABS = 2e-3
F16_ULP_REL = 2.0 ** -10
F32_REL = 1e-3
F32_ABS = 1e-6


def compare(kind: str, got: np.ndarray, want: np.ndarray, name: str = "") -> None:
    """Raise AssertionError with a short report if `got` is outside the tolerance of `want`."""
    assert got.shape == want.shape, f"{name}: shape {got.shape} != {want.shape}"
    if kind == "exact":
        g = got.view(np.uint16) if got.dtype == np.float16 else got
        w = want.view(np.uint16) if want.dtype == np.float16 else want
        if got.dtype == np.float32:
            g, w = got.view(np.uint32), want.view(np.uint32)
        bad = g != w
        assert not bad.any(), f"{name}: {int(bad.sum())} of {bad.size} elements differ bitwise"
        return
    g = got.astype(np.float64)
    w = want.astype(np.float64)
    assert np.isfinite(g).all() or not np.isfinite(w).all(), f"{name}: non-finite output"
    diff = np.abs(g - w)
    if kind == "f16":
        tol = np.maximum(F16_ABS, F16_ULP_REL * np.abs(w))
    elif kind == "f16_1ulp":  # CPU libm vs GPU intrinsics on a bit-exact target: one fp16 step
        tol = np.maximum(2.0 ** -24, F16_ULP_REL * np.abs(w))
    elif kind == "f32":
        tol = F32_REL * np.abs(w) + F32_ABS
    else:
        raise ValueError(kind)
    bad = diff > tol
    if bad.any():
        i = np.unravel_index(np.argmax(diff - tol), diff.shape)
        raise AssertionError(
            f"{name}: {int(bad.sum())} of {bad.size} outside tolerance ({kind}); worst at {i}: "
            f"got {g[i]!r} want {w[i]!r}")


@dataclass
class Case:
    name: str
    make: Callable[[np.random.Generator], dict]
    oracle: Callable[[dict], dict]
    rfk: Callable[[dict], dict]
    kinds: dict
    ref: Callable[[dict], dict] | None = None
    seed: int = 0
    # comparison kind of the CPU oracle against GPU results when it differs from `kinds`
    # (bit-exact targets are exact GPU-vs-GPU but only to one fp16 step against libm)
    oracle_kinds: dict = field(default_factory=dict)

    def inputs(self) -> dict:
        import zlib
        return self.make(np.random.default_rng([self.seed, zlib.crc32(self.name.encode())]))


# --------------------------------------------------------------------- helpers

def _t(a):
    """numpy -> fresh CUDA tensor (bool arrays travel as uint8)."""
    import torch
    if isinstance(a, np.ndarray):
        if a.dtype == np.bool_:
            a = a.astype(np.uint8)
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return a


def _n(t):
    import torch
    torch.cuda.synchronize()
    return t.detach().cpu().numpy()


def _empty(shape, dtype):
    import torch
    return torch.empty(shape, dtype=dtype, device="cuda")


def _ops():
    import renderformer_cuda_b200 as pkg
    return pkg.ops


def _ref():
    from oracle import ref
    return ref


def normal(rng, shape, dtype, scale=1.0, loc=0.0):
    return (rng.standard_normal(shape) * scale + loc).astype(dtype)


def uniform(rng, shape, dtype, lo=-1.0, hi=1.0):
    return rng.uniform(lo, hi, shape).astype(dtype)


def look_at_c2w(rng, n):
    """Random pinhole cameras: position on a sphere of radius 2..4 looking at the origin
    (recipe of the reference's trackball camera, src/app/camera.h:31-54), fov 30..60 deg."""
    c2w = np.zeros((n, 4, 4), np.float32)
    fov = np.deg2rad(rng.uniform(30.0, 60.0, n)).astype(np.float32)
    for i in range(n):
        d = rng.standard_normal(3)
        d /= np.linalg.norm(d)
        pos = d * rng.uniform(2.0, 4.0)
        fwd = -pos / np.linalg.norm(pos)
        up = np.array([0.0, 0.0, 1.0]) if abs(fwd[2]) < 0.99 else np.array([0.0, 1.0, 0.0])
        right = np.cross(fwd, up); right /= np.linalg.norm(right)
        up2 = np.cross(right, fwd)
        c2w[i, :3, 0], c2w[i, :3, 1], c2w[i, :3, 2], c2w[i, :3, 3] = right, up2, -fwd, pos
        c2w[i, 3, 3] = 1.0
    return c2w, fov


CASES: list[Case] = []


def case(**kw):
    CASES.append(Case(**kw))


# --------------------------------------------------------------------- RMSNorm

def _rms_make(rows, dim, dtype):
    def make(rng):
        return dict(x=normal(rng, (rows, dim), dtype), gamma=normal(rng, (dim,), np.float32, 0.02, 1.0),
                    eps=1e-6 if dtype == np.float32 else 2.0 ** -10)
    return make


def _rms16_rfk(i):
    import torch
    x, g = _t(i["x"]), _t(i["gamma"]); y = torch.empty_like(x)
    _ops().rmsnorm(x, g, y, x.shape[0], x.shape[1], i["eps"])
    x2 = x.clone(); _ops().rmsnorm(x2, g, x2, x.shape[0], x.shape[1], i["eps"])  # in-place form
    return dict(y=_n(y), y_inplace=_n(x2))


def _rms16_ref(i):
    import torch
    x, g = _t(i["x"]), _t(i["gamma"]); y = torch.empty_like(x)
    _ref().call("ref_rmsnorm", x, g, y, x.shape[0], x.shape[1], float(i["eps"]))
    return dict(y=_n(y), y_inplace=_n(y))


def _rms32_rfk(i):
    import torch
    x, g = _t(i["x"]), _t(i["gamma"]); y = torch.empty_like(x)
    _ops().rmsnorm_f32(x, g, y, x.shape[0], x.shape[1], i["eps"])
    return dict(y=_n(y))


def _rms32_ref(i):
    import torch
    x, g = _t(i["x"]), _t(i["gamma"]); y = torch.empty_like(x)
    _ref().call("ref_rmsnorm_f32", x, g, y, x.shape[0], x.shape[1], float(i["eps"]))
    return dict(y=_n(y))


for rows, dim in [(37, 1024), (5, 96), (3, 100), (9, 2048), (2, 4096), (1, 8), (4, 512)]:
    case(name=f"rmsnorm_f16_{rows}x{dim}", make=_rms_make(rows, dim, np.float16),
         oracle=lambda i: (lambda y: dict(y=y, y_inplace=y))(O.rmsnorm(i["x"], i["gamma"], i["eps"])),
         rfk=_rms16_rfk, ref=_rms16_ref if dim % 32 == 0 else None,  # ref assumes whole warps
         kinds=dict(y="f16", y_inplace="f16"))
    case(name=f"rmsnorm_f32_{rows}x{dim}", make=_rms_make(rows, dim, np.float32),
         oracle=lambda i: dict(y=O.rmsnorm_f32(i["x"], i["gamma"], i["eps"])),
         rfk=_rms32_rfk, ref=_rms32_ref if dim % 32 == 0 else None, kinds=dict(y="f32"))


def _fused_make(rows, dim, rdtype, hdtype=np.float32):
    def make(rng):
        return dict(h=normal(rng, (rows, dim), hdtype), r=normal(rng, (rows, dim), rdtype),
                    gamma=normal(rng, (dim,), np.float32, 0.02, 1.0),
                    eps=1e-6 if hdtype == np.float32 else 2.0 ** -10)
    return make


def _fused32_rfk(i):
    h, r, g = _t(i["h"]), _t(i["r"]), _t(i["gamma"])
    y = _empty(h.shape, __import__("torch").float16)
    fn = _ops().rmsnorm_residual_f32_cast16 if i["r"].dtype == np.float32 else _ops().rmsnorm_residual_mixed_cast16
    fn(h, r, g, y, h.shape[0], h.shape[1], i["eps"])
    return dict(h=_n(h), y16=_n(y))


def _fused32_ref(i):
    import torch
    h, r, g = _t(i["h"]), _t(i["r"]), _t(i["gamma"])
    n = h.numel(); rows, dim = h.shape
    tmp = torch.empty_like(h); y = _empty(h.shape, torch.float16)
    R = _ref()
    if i["r"].dtype == np.float32:
        R.call("ref_residual_rmsnorm_cast", h, r, g, tmp, y, rows, dim, float(i["eps"]), lib=R.layers())
    else:
        R.call("ref_residual_add_mixed", h, r, n, lib=R.layers())
        R.call("ref_rmsnorm_f32", h, g, tmp, rows, dim, float(i["eps"]))
        R.call("ref_cast_fp32_to_fp16", tmp, y, n, lib=R.layers())
    return dict(h=_n(h), y16=_n(y))


def _fused32_oracle(i):
    h, y = O.rmsnorm_residual_f32_cast16(i["h"], i["r"], i["gamma"], i["eps"])
    return dict(h=h, y16=y)


for rows, dim in [(64, 1024), (7, 256), (3, 100), (5, 2048)]:
    for rdt, tag in [(np.float32, "f32"), (np.float16, "mixed")]:
        case(name=f"rmsnorm_residual_{tag}_cast16_{rows}x{dim}", make=_fused_make(rows, dim, rdt),
             oracle=_fused32_oracle, rfk=_fused32_rfk, ref=_fused32_ref if dim % 32 == 0 else None,
             kinds=dict(h="f32", y16="f16"))


def _fused16_rfk(i):
    import torch
    x, r, g = _t(i["h"]), _t(i["r"]), _t(i["gamma"]); y = torch.empty_like(x)
    _ops().rmsnorm_residual_f16(x, r, g, y, x.shape[0], x.shape[1], i["eps"])
    return dict(x=_n(x), y=_n(y))


def _fused16_ref(i):
    import torch
    x, r, g = _t(i["h"]), _t(i["r"]), _t(i["gamma"]); y = torch.empty_like(x)
    R = _ref()
    R.call("ref_residual_add", x, r, x.numel(), lib=R.layers())
    R.call("ref_rmsnorm", x, g, y, x.shape[0], x.shape[1], float(i["eps"]))
    return dict(x=_n(x), y=_n(y))


for rows, dim in [(33, 1024), (3, 100)]:
    case(name=f"rmsnorm_residual_f16_{rows}x{dim}", make=_fused_make(rows, dim, np.float16, np.float16),
         oracle=lambda i: dict(zip(("x", "y"), O.rmsnorm_residual_f16(i["h"], i["r"], i["gamma"], i["eps"]))),
         rfk=_fused16_rfk, ref=_fused16_ref if dim % 32 == 0 else None, kinds=dict(x="exact", y="f16"),
         oracle_kinds=dict(x="exact"))

# ------------------------------------------------------ residual / cast plumbing

def _ew_case(name, adt, bdt, op_rfk, op_ref, op_oracle, kind):
    def make(rng):
        n = 1003
        return dict(a=normal(rng, (n,), adt), b=normal(rng, (n,), bdt))

    def rfk(i):
        a, b = _t(i["a"]), _t(i["b"])
        getattr(_ops(), op_rfk)(a, b, a.numel())
        return dict(a=_n(a))

    def ref(i):
        a, b = _t(i["a"]), _t(i["b"])
        _ref().call(op_ref, a, b, a.numel(), lib=_ref().layers())
        return dict(a=_n(a))

    case(name=name, make=make, oracle=lambda i: dict(a=op_oracle(i["a"], i["b"])), rfk=rfk, ref=ref,
         kinds=dict(a=kind), oracle_kinds=dict(a=kind))


_ew_case("residual_add", np.float16, np.float16, "residual_add", "ref_residual_add", O.residual_add, "exact")
_ew_case("residual_add_f32", np.float32, np.float32, "residual_add_f32", "ref_residual_add_f32", O.residual_add_f32, "exact")
_ew_case("residual_add_mixed", np.float32, np.float16, "residual_add_mixed", "ref_residual_add_mixed", O.residual_add_mixed, "exact")


def _cast_case(name, sdt, ddt, op_rfk, op_ref, op_oracle):
    def make(rng):
        return dict(a=normal(rng, (1003,), sdt, 3.0))

    def rfk(i):
        import torch
        a = _t(i["a"]); o = _empty(a.shape, torch.float16 if ddt == np.float16 else torch.float32)
        getattr(_ops(), op_rfk)(a, o, a.numel())
        return dict(o=_n(o))

    def ref(i):
        import torch
        a = _t(i["a"]); o = _empty(a.shape, torch.float16 if ddt == np.float16 else torch.float32)
        _ref().call(op_ref, a, o, a.numel(), lib=_ref().layers())
        return dict(o=_n(o))

    case(name=name, make=make, oracle=lambda i: dict(o=op_oracle(i["a"])), rfk=rfk, ref=ref,
         kinds=dict(o="exact"), oracle_kinds=dict(o="exact"))


_cast_case("cast_fp32_to_fp16", np.float32, np.float16, "cast_fp32_to_fp16", "ref_cast_fp32_to_fp16", O.cast_fp32_to_fp16)
_cast_case("cast_fp16_to_fp32", np.float16, np.float32, "cast_fp16_to_fp32", "ref_cast_fp16_to_fp32", O.cast_fp16_to_fp32)


def _bcast_rfk(i):
    o, bc = _t(i["out"]), _t(i["bc"])
    _ops().broadcast_add(o, bc, o.numel(), bc.numel())
    return dict(out=_n(o))


for rows, dim in [(13, 1024), (5, 100)]:
    case(name=f"broadcast_add_{rows}x{dim}",
         make=(lambda rows, dim: lambda rng: dict(out=normal(rng, (rows, dim), np.float16), bc=normal(rng, (dim,), np.float16)))(rows, dim),
         oracle=lambda i: dict(out=O.broadcast_add(i["out"], i["bc"])), rfk=_bcast_rfk,
         kinds=dict(out="exact"), oracle_kinds=dict(out="exact"))

# ------------------------------------------------------------------------ RoPE

def _geo_freqs(nf, base=10000.0):
    """nf rotary frequencies, geometric with base 10000 (stand-in for the learned weights)."""
    return (base ** (-np.arange(nf, dtype=np.float64) / max(nf, 1))).astype(np.float32) * np.float32(np.pi)


def _table_make(B, S, nf, hd):
    def make(rng):
        return dict(pos=uniform(rng, (B, S, 9), np.float16), freqs=_geo_freqs(nf), nf=nf, hd=hd)
    return make


def _table_rfk(i):
    import torch
    pos, fr = _t(i["pos"]), _t(i["freqs"]); B, S, _ = pos.shape
    c = _empty((B, 1, S, i["hd"]), torch.float16); s = torch.empty_like(c)
    _ops().triangle_rope_freqs(pos, fr, c, s, B, S, i["nf"], i["hd"])
    return dict(cos=_n(c), sin=_n(s))


def _table_ref(i):
    import torch
    pos, fr = _t(i["pos"]), _t(i["freqs"]); B, S, _ = pos.shape
    c = _empty((B, 1, S, i["hd"]), torch.float16); s = torch.empty_like(c)
    _ref().call("ref_triangle_rope_freqs", pos, fr, c, s, B, S, i["nf"], i["hd"])
    return dict(cos=_n(c), sin=_n(s))


def _table_oracle(i):
    c, s = O.triangle_rope_freqs(i["pos"], i["freqs"], i["hd"])
    B, S, hd = c.shape
    return dict(cos=c.reshape(B, 1, S, hd), sin=s.reshape(B, 1, S, hd))


for B, S, nf, hd in [(1, 70, 3, 64), (2, 33, 6, 128), (1, 17, 1, 24), (1, 9, 3, 54)]:
    case(name=f"triangle_rope_freqs_b{B}_s{S}_nf{nf}_hd{hd}", make=_table_make(B, S, nf, hd),
         oracle=_table_oracle, rfk=_table_rfk, ref=_table_ref, kinds=dict(cos="f16", sin="f16"))


def _rope_make(B, Hh, S, D, dtype, nf):
    def make(rng):
        pos = uniform(rng, (B, S, 9), np.float16)
        c, s = O.triangle_rope_freqs(pos, _geo_freqs(nf), D)
        return dict(q=normal(rng, (B, Hh, S, D), dtype), k=normal(rng, (B, Hh, S, D), dtype),
                    cos=c.reshape(B, 1, S, D), sin=s.reshape(B, 1, S, D))
    return make


def _rope_rfk(i):
    q, k, c, s = _t(i["q"]), _t(i["k"]), _t(i["cos"]), _t(i["sin"])
    B, Hh, S, D = q.shape
    one = q.clone()
    if i["q"].dtype == np.float16:
        _ops().apply_rope(q, k, c, s, B, Hh, S, D)
        _ops().apply_rope_one(one, c, s, B, Hh, S, D)
    else:
        _ops().apply_rope_f32(q, k, c, s, B, Hh, S, D)
        _ops().apply_rope_one_f32(one, c, s, B, Hh, S, D)
    return dict(q=_n(q), k=_n(k), one=_n(one))


def _rope_ref(i):
    q, k, c, s = _t(i["q"]), _t(i["k"]), _t(i["cos"]), _t(i["sin"])
    B, Hh, S, D = q.shape
    one = q.clone()
    sfx = "" if i["q"].dtype == np.float16 else "_f32"
    _ref().call("ref_apply_rope" + sfx, q, k, c, s, B, Hh, S, D)
    _ref().call("ref_apply_rope_one" + sfx, one, c, s, B, Hh, S, D)
    return dict(q=_n(q), k=_n(k), one=_n(one))


def _rope_oracle(i):
    q = O.apply_rope(i["q"], i["cos"], i["sin"])
    return dict(q=q, k=O.apply_rope(i["k"], i["cos"], i["sin"]), one=q)


for B, Hh, S, D, nf in [(2, 4, 33, 64, 3), (1, 8, 19, 128, 6), (1, 3, 11, 24, 1), (1, 16, 40, 64, 3)]:
    for dt, tag in [(np.float16, "f16"), (np.float32, "f32")]:
        kind = "f16" if dt == np.float16 else "f32"
        case(name=f"apply_rope_{tag}_b{B}h{Hh}s{S}d{D}", make=_rope_make(B, Hh, S, D, dt, nf),
             # the reference updates in place with one thread per element and no ordering between
             # the partner's load and this thread's store; with head_dim 24 a rotation pair can
             # straddle a warp boundary and the race shows (observed on B200), so that shape is
             # checked against the oracle only.
             oracle=_rope_oracle, rfk=_rope_rfk, ref=_rope_ref if D % 64 == 0 else None,
             kinds=dict(q=kind, k=kind, one=kind))


def _oop_make(rng):
    B, Hh, S, D, pad = 1, 4, 29, 64, 3
    pos = uniform(rng, (B, S, 9), np.float16)
    c, s = O.triangle_rope_freqs(pos, _geo_freqs(3), D)
    return dict(src=normal(rng, (B, Hh, S + pad, D), np.float16), cos=c.reshape(B, 1, S, D),
                sin=s.reshape(B, 1, S, D), S=S, pad=pad)


def _oop_rfk(i):
    import torch
    src, c, s = _t(i["src"]), _t(i["cos"]), _t(i["sin"])
    B, Hh, SP, D = src.shape
    dst = torch.full_like(src, 7.0)
    _ops().rope_one_oop(src, dst, c, s, B, Hh, i["S"], D, SP, SP, copy_tail=True)
    return dict(dst=_n(dst))


def _oop_oracle(i):
    S = i["S"]
    out = i["src"].copy()
    out[:, :, :S] = O.apply_rope(np.ascontiguousarray(i["src"][:, :, :S]), i["cos"], i["sin"])
    return dict(dst=out)


case(name="rope_one_oop_tail", make=_oop_make, oracle=_oop_oracle, rfk=_oop_rfk, kinds=dict(dst="f16"))


def _qkv_make(B, S, Hh, D, nf):
    def make(rng):
        dim = Hh * D
        pos = uniform(rng, (B, S, 9), np.float16)
        c, s = O.triangle_rope_freqs(pos, _geo_freqs(nf), D)
        return dict(qkv=normal(rng, (B * S, 3 * dim), np.float16),
                    gq=normal(rng, (dim,), np.float32, 0.02, 1.0), gk=normal(rng, (dim,), np.float32, 0.02, 1.0),
                    cos=c.reshape(B, 1, S, D), sin=s.reshape(B, 1, S, D), B=B, S=S, H=Hh, D=D)
    return make


def _qkv_rfk(i):
    import torch
    qkv, gq, gk, c, s = _t(i["qkv"]), _t(i["gq"]), _t(i["gk"]), _t(i["cos"]), _t(i["sin"])
    B, S, Hh, D = i["B"], i["S"], i["H"], i["D"]
    outs = [_empty((B, Hh, S, D), torch.float16) for _ in range(3)]
    _ops().qkv_norm_rope_transpose(qkv, 3 * Hh * D, [gq, gk, None], outs, [1, 1, 0], c, s, B, S, Hh, D)
    return dict(q=_n(outs[0]), k=_n(outs[1]), v=_n(outs[2]))


def _qkv_ref(i):
    """The unfused sequence with the reference kernels; pure copies are done by torch."""
    import torch
    qkv, c, s = _t(i["qkv"]), _t(i["cos"]), _t(i["sin"])
    B, S, Hh, D = i["B"], i["S"], i["H"], i["D"]; dim = Hh * D
    q, k, v = [qkv[:, p * dim:(p + 1) * dim].contiguous() for p in range(3)]
    _ref().call("ref_rmsnorm", q, _t(i["gq"]), q, B * S, dim, 2.0 ** -10)
    _ref().call("ref_rmsnorm", k, _t(i["gk"]), k, B * S, dim, 2.0 ** -10)
    q, k, v = [t.view(B, S, Hh, D).permute(0, 2, 1, 3).contiguous() for t in (q, k, v)]
    _ref().call("ref_apply_rope", q, k, c, s, B, Hh, S, D)
    return dict(q=_n(q), k=_n(k), v=_n(v))


def _qkv_oracle(i):
    q, k, v = O.qkv_norm_rope_transpose(i["qkv"], 3, [i["gq"], i["gk"], None], [1, 1, 0], i["cos"], i["sin"],
                                        i["B"], i["S"], i["H"], i["D"], 2.0 ** -10)
    return dict(q=q, k=k, v=v)


for B, S, Hh, D, nf in [(1, 45, 16, 64, 3), (2, 21, 8, 128, 6), (1, 10, 4, 32, 1)]:
    case(name=f"qkv_norm_rope_transpose_b{B}s{S}h{Hh}d{D}", make=_qkv_make(B, S, Hh, D, nf),
         oracle=_qkv_oracle, rfk=_qkv_rfk, ref=_qkv_ref, kinds=dict(q="f16", k="f16", v="exact"),
         oracle_kinds=dict(v="exact"))
# 2048-wide rows: two chunk pairs per thread, two warps per row (no reference output stored for this shape)
case(name="qkv_norm_rope_transpose_b1s19h16d128", make=_qkv_make(1, 19, 16, 128, 6),
     oracle=_qkv_oracle, rfk=_qkv_rfk, ref=None, kinds=dict(q="f16", k="f16", v="exact"),
     oracle_kinds=dict(v="exact"))

# --------------------------------------------------------------------- NeRF PE

def _pe_make(rows, in_dim, dtype, nf, mn, mx, inc, unit):
    def make(rng):
        x = rng.standard_normal((1, rows, in_dim))
        if unit:
            x = x.reshape(1, rows, -1, 3)
            x /= np.linalg.norm(x, axis=-1, keepdims=True)
            x = x.reshape(1, rows, in_dim)
        return dict(x=x.astype(dtype), nf=nf, mn=mn, mx=mx, inc=inc)
    return make


def _pe_rfk(i):
    import torch
    x = _t(i["x"]); B, S, D = x.shape
    od = D * i["nf"] * 2 + (D if i["inc"] else 0)
    out = _empty((B, S, od), torch.float16)
    fn = _ops().nerf_pe if i["x"].dtype == np.float16 else _ops().nerf_pe_f32
    fn(x, out, B, S, D, i["nf"], i["mn"], i["mx"], i["inc"])
    return dict(out=_n(out))


def _pe_ref(i):
    import torch
    x = _t(i["x"]); B, S, D = x.shape
    od = D * i["nf"] * 2 + (D if i["inc"] else 0)
    out = _empty((B, S, od), torch.float16)
    name = "ref_nerf_pe" if i["x"].dtype == np.float16 else "ref_nerf_pe_f32"
    _ref().call(name, x, out, B, S, D, i["nf"], float(i["mn"]), float(i["mx"]), int(i["inc"]))
    return dict(out=_n(out))


for rows, in_dim, dt, nf, mn, mx, inc, unit, tag in [
        (50, 9, np.float32, 6, 0.0, 5.0, True, True, "normals_f32"),
        (101, 3, np.float16, 6, 0.0, 5.0, True, True, "raydirs_f16"),
        (23, 9, np.float16, 12, 0.0, 11.0, True, False, "nf12_f16"),
        (23, 5, np.float32, 4, -1.0, 2.5, False, False, "noinput_f32"),
        (7, 2, np.float32, 1, 3.0, 3.0, True, False, "nf1_f32")]:
    case(name=f"nerf_pe_{tag}", make=_pe_make(rows, in_dim, dt, nf, mn, mx, inc, unit),
         oracle=lambda i: dict(out=O.nerf_pe(i["x"], i["nf"], i["mn"], i["mx"], i["inc"])),
         rfk=_pe_rfk, ref=_pe_ref, kinds=dict(out="f16"))

# --------------------------------------------------------------------- softmax

def _sm_make(rows, cols, in_stride, out_stride, masked, mask_rows, scale_in=3.0 / 8.0):
    def make(rng):
        x = np.full((rows, in_stride), -np.inf, np.float32)  # pad columns hold -inf, never to be read
        x[:, :cols] = normal(rng, (rows, cols), np.float32, scale_in)
        d = dict(x=x, cols=cols, out_stride=out_stride)
        if masked:
            m = rng.random((mask_rows, cols)) > 0.3
            m[0, :] = False  # a fully masked row
            if mask_rows > 1:
                m[1, :] = True
            d["mask"] = m
        return d
    return make


def _sm_rfk(i):
    import torch
    x = _t(i["x"]); rows, ist = x.shape
    out = torch.full((rows, i["out_stride"]), 9.0, dtype=torch.float16, device="cuda")
    if "mask" in i:
        m = _t(i["mask"])
        _ops().softmax_cast_fp16_masked(x, out, m, rows, i["cols"], ist, i["out_stride"], m.shape[0])
    else:
        _ops().softmax_cast_fp16(x, out, rows, i["cols"], ist, i["out_stride"])
    return dict(p=_n(out))


def _sm_ref(i):
    import torch
    x = _t(i["x"]); rows, ist = x.shape
    out = torch.full((rows, i["out_stride"]), 9.0, dtype=torch.float16, device="cuda")
    if "mask" in i:
        m = _t(i["mask"])
        _ref().call("ref_softmax_cast_fp16_masked", x, out, m, rows, i["cols"], ist, i["out_stride"], m.shape[0])
    else:
        _ref().call("ref_softmax_cast_fp16", x, out, rows, i["cols"], ist, i["out_stride"])
    return dict(p=_n(out))


for rows, cols, ist, ost, masked, mr, tag in [
        (6, 5633, 5640, 5640, False, 1, "cross_5633"),
        (5, 64, 64, 64, False, 1, "c64"),
        (7, 300, 304, 304, False, 1, "c300"),
        (4, 1000, 1001, 1003, False, 1, "unaligned"),
        (3, 8192, 8192, 8192, False, 1, "c8192"),
        (2, 9001, 9001, 9008, False, 1, "long"),
        (3, 1, 1, 8, False, 1, "c1"),
        (9, 333, 336, 336, True, 3, "masked_c333"),
        (6, 64, 64, 64, True, 2, "masked_c64"),
        (4, 5633, 5640, 5640, True, 2, "masked_cross"),
        (2, 9001, 9001, 9001, True, 2, "masked_long")]:
    case(name=f"softmax_cast_fp16_{tag}", make=_sm_make(rows, cols, ist, ost, masked, mr),
         oracle=lambda i: dict(p=O.softmax_cast_fp16(i["x"], i["cols"], i["out_stride"], i.get("mask"))),
         # the reference needs >= 1 full warp, and its unmasked kernel issues float4 loads and
         # half2 stores on every row: it faults (misaligned address) unless in_stride % 4 == 0
         # and out_stride % 2 == 0. Those shapes are checked against the oracle only.
         rfk=_sm_rfk, ref=_sm_ref if cols >= 32 and (masked or (ist % 4 == 0 and ost % 2 == 0)) else None,
         kinds=dict(p="f16"))


def _sm_scaled_rfk(i):
    import torch
    x = _t(i["x"]); rows, ist = x.shape
    out = _empty((rows, i["out_stride"]), torch.float16)
    _ops().softmax_cast_fp16_scaled(x, out, rows, i["cols"], ist, i["out_stride"], 0.125)
    return dict(p=_n(out))


case(name="softmax_cast_fp16_scaled", make=_sm_make(5, 777, 784, 784, False, 1, 3.0),
     oracle=lambda i: dict(p=O.softmax_cast_fp16(i["x"], i["cols"], i["out_stride"], None, 0.125)),
     rfk=_sm_scaled_rfk, kinds=dict(p="f16"))


def _smi_make(rows, cols, mode, heads=2, nW=3):
    def make(rng):
        d = dict(x=normal(rng, (rows, cols), np.float32, 2.0), mode=mode, heads=heads, nW=nW)
        if mode == "masked":
            m = rng.random((3, cols)) > 0.3; m[0, :] = False; d["mask"] = m
        if mode == "swin":
            m = rng.random((nW, cols, cols)) > 0.4; m[:, :, 0] = True; d["mask"] = m
        return d
    return make


def _smi_rfk(i):
    x = _t(i["x"]); rows, cols = x.shape
    if i["mode"] == "plain":
        _ops().softmax_inplace(x, rows, cols)
    elif i["mode"] == "masked":
        _ops().masked_softmax_inplace(x, _t(i["mask"]), rows, cols, 3)
    else:
        _ops().swin_masked_softmax_inplace(x, _t(i["mask"]), rows // (i["heads"] * cols), i["heads"], cols, i["nW"])
    return dict(p=_n(x))


def _smi_ref(i):
    x = _t(i["x"]); rows, cols = x.shape
    if i["mode"] == "plain":
        _ref().call("ref_softmax_inplace", x, rows, cols)
    elif i["mode"] == "masked":
        _ref().call("ref_masked_softmax_inplace", x, _t(i["mask"]), rows, cols, 3)
    else:
        _ref().call("ref_swin_masked_softmax_inplace", x, _t(i["mask"]), rows // (i["heads"] * cols), i["heads"], cols, i["nW"])
    return dict(p=_n(x))


def _smi_oracle(i):
    if i["mode"] == "plain":
        return dict(p=O.softmax_inplace(i["x"]))
    if i["mode"] == "masked":
        return dict(p=O.softmax_inplace(i["x"], i["mask"]))
    return dict(p=O.softmax_inplace(i["x"], i["mask"], swin=(i["heads"], i["nW"])))


for rows, cols, mode in [(11, 64, "plain"), (5, 1000, "plain"), (3, 10000, "plain"), (7, 50, "masked"),
                         (6, 777, "masked"), (2 * 3 * 2 * 16, 16, "swin"), (1 * 3 * 2 * 64, 64, "swin")]:
    case(name=f"softmax_inplace_{mode}_{rows}x{cols}", make=_smi_make(rows, cols, mode),
         oracle=_smi_oracle, rfk=_smi_rfk, ref=_smi_ref, kinds=dict(p="f32"))


def _swinf_rfk(i):
    import torch
    x = _t(i["x"]); rows, cols = x.shape
    out = _empty((rows, cols), torch.float16)
    m = _t(i["mask"]) if i["mode"] == "swin" else None
    _ops().swin_softmax_cast_fp16(x, out, m, rows // (i["heads"] * cols), i["heads"], cols, i["nW"])
    return dict(p=_n(out))


def _swinf_ref(i):
    """swin_masked_softmax_inplace | softmax_inplace, then the fp32->fp16 cast (torch: a pure cast)."""
    r = _smi_ref(i)
    return dict(p=r["p"].astype(np.float16))


for mode in ("swin", "plain"):
    case(name=f"swin_softmax_cast_fp16_{mode}", make=_smi_make(2 * 3 * 2 * 64, 64, mode),
         oracle=lambda i: dict(p=_smi_oracle(i)["p"].astype(np.float16)),
         rfk=_swinf_rfk, ref=_swinf_ref, kinds=dict(p="f16"))

# ----------------------------------------------------------------- activations

def _silu_rfk(i):
    import torch
    a, b = _t(i["a"]), _t(i["b"]); o = torch.empty_like(a)
    fn = _ops().fused_silu_mul if i["a"].dtype == np.float16 else _ops().fused_silu_mul_f32
    fn(a, b, o, a.numel())
    a2 = a.clone(); fn(a2, b, a2, a.numel())  # in place on a, as ffn_swiglu calls it
    return dict(o=_n(o), o_inplace=_n(a2))


def _silu_ref(i):
    import torch
    a, b = _t(i["a"]), _t(i["b"]); o = torch.empty_like(a)
    name = "ref_fused_silu_mul" if i["a"].dtype == np.float16 else "ref_fused_silu_mul_f32"
    _ref().call(name, a, b, o, a.numel())
    return dict(o=_n(o), o_inplace=_n(o))


for n, dt, tag in [(4099, np.float16, "f16"), (4099, np.float32, "f32"), (64, np.float16, "f16_small")]:
    kind = "f16" if dt == np.float16 else "f32"
    case(name=f"fused_silu_mul_{tag}",
         make=(lambda n, dt: lambda rng: dict(a=normal(rng, (n,), dt, 2.0), b=normal(rng, (n,), dt)))(n, dt),
         oracle=lambda i: (lambda o: dict(o=o, o_inplace=o))(O.fused_silu_mul(i["a"], i["b"])),
         rfk=_silu_rfk, ref=_silu_ref, kinds=dict(o=kind, o_inplace=kind))


def _swiglu_rfk(i):
    import torch
    gu = _t(i["gu"]); rows, th = gu.shape
    o = _empty((rows, th // 2), torch.float16)
    _ops().swiglu(gu, o, rows, th // 2)
    return dict(o=_n(o))


def _swiglu_ref(i):
    import torch
    gu = _t(i["gu"]); rows, th = gu.shape
    g = gu[:, :th // 2].contiguous(); u = gu[:, th // 2:].contiguous()
    _ref().call("ref_fused_silu_mul", g, u, g, g.numel())
    return dict(o=_n(g))


for rows, hidden in [(9, 4096), (5, 100)]:
    case(name=f"swiglu_{rows}x{hidden}",
         make=(lambda r, h: lambda rng: dict(gu=normal(rng, (r, 2 * h), np.float16, 1.5)))(rows, hidden),
         oracle=lambda i: dict(o=O.swiglu(i["gu"])), rfk=_swiglu_rfk, ref=_swiglu_ref, kinds=dict(o="f16"))


def _post_make(rng):
    return dict(x=normal(rng, (3 * 37 * 37,), np.float16, 1.0))


def _post_rfk(i):
    import torch
    x = _t(i["x"]); n = x.numel()
    e = torch.empty_like(x); _ops().elu(x, e, n, 1e-3)
    e32 = e.float(); p = torch.empty_like(e32); _ops().pow10_minus1(e32, p, n)
    fused = torch.empty_like(e32); _ops().post_elu_pow10(x, fused, n, 1e-3)
    return dict(elu=_n(e), pow10=_n(p), fused=_n(fused))


def _post_ref(i):
    import torch
    x = _t(i["x"]); n = x.numel()
    e = torch.empty_like(x); _ref().call("ref_elu", x, e, n, 1e-3)
    e32 = e.float(); p = torch.empty_like(e32); _ref().call("ref_pow10_minus1", e32, p, n)
    return dict(elu=_n(e), pow10=_n(p), fused=_n(p))


def _post_oracle(i):
    e = O.elu(i["x"])
    p = O.pow10_minus1(e.astype(np.float32))
    return dict(elu=e, pow10=p, fused=O.post_elu_pow10(i["x"]))


# same expf/powf calls as the reference: exact GPU-vs-GPU, libm-close against the CPU
case(name="post_elu_pow10", make=_post_make, oracle=_post_oracle, rfk=_post_rfk, ref=_post_ref,
     kinds=dict(elu="exact", pow10="exact", fused="exact"),
     oracle_kinds=dict(elu="f16", pow10="f32", fused="f32"))

# ------------------------------------------------------ DPT head glue (src/layers/dpt.cu)

def _up_make(N, C, Hi, Wi, Ho, Wo):
    def make(rng):
        return dict(x=normal(rng, (N, C, Hi, Wi), np.float16, 1.0), Ho=Ho, Wo=Wo)
    return make


def _up_rfk(i):
    import torch
    x = _t(i["x"]); N, C, Hi, Wi = x.shape
    o = torch.empty(N, C, i["Ho"], i["Wo"], device="cuda", dtype=torch.float16)
    _ops().bilinear_upsample(x, o, N, C, Hi, Wi, i["Ho"], i["Wo"])
    return dict(o=_n(o))


def _up_ref(i):
    import torch
    x = _t(i["x"]); N, C, Hi, Wi = x.shape
    o = torch.empty(N, C, i["Ho"], i["Wo"], device="cuda", dtype=torch.float16)
    _ref().call("ref_bilinear_upsample", x, o, N, C, Hi, Wi, i["Ho"], i["Wo"])
    return dict(o=_n(o))


# the same expression compiled by the same compiler: exact GPU-vs-GPU; the CPU oracle does not contract to FMAs
for shp in [(1, 3, 8, 8, 16, 16), (2, 5, 7, 9, 13, 20), (1, 4, 16, 16, 16, 16), (1, 2, 5, 6, 1, 1), (1, 6, 32, 32, 64, 64),
            (1, 2, 40, 150, 70, 300), (1, 1, 300, 40, 300, 264), (1, 2, 20, 30, 9, 44)]:
    case(name="bilinear_upsample_" + "x".join(map(str, shp)), make=_up_make(*shp),
         oracle=lambda i: dict(o=O.bilinear_upsample(i["x"], i["Ho"], i["Wo"])), rfk=_up_rfk, ref=_up_ref,
         kinds=dict(o="exact"), oracle_kinds=dict(o="f16"))


def _silu_rfk(i):
    x = _t(i["x"]).clone(); _ops().silu_inplace(x, x.numel()); return dict(y=_n(x))


def _silu_ref(i):
    x = _t(i["x"]).clone(); _ref().call("ref_silu_inplace", x, x.numel()); return dict(y=_n(x))


for n in (1, 1001, 32 * 24 * 24):
    case(name=f"silu_inplace_n{n}", make=(lambda n: lambda rng: dict(x=normal(rng, (n,), np.float16, 2.0)))(n),
         oracle=lambda i: dict(y=O.silu(i["x"])), rfk=_silu_rfk, ref=_silu_ref, kinds=dict(y="f16"))


def _bias_rfk(i):
    x = _t(i["x"]).clone(); N, C = x.shape[:2]
    _ops().add_bias_nchw(x, _t(i["b"]), N, C, x.numel() // (N * C)); return dict(y=_n(x))


for shp in [(2, 5, 7, 9), (1, 32, 16, 16), (3, 1, 1, 1)]:
    case(name="add_bias_nchw_" + "x".join(map(str, shp)),
         make=(lambda shp: lambda rng: dict(x=normal(rng, shp, np.float16, 1.0), b=normal(rng, (shp[1],), np.float16, 1.0)))(shp),
         oracle=lambda i: dict(y=O.add_bias_nchw(i["x"], i["b"])), rfk=_bias_rfk, ref=None, kinds=dict(y="exact"),
         oracle_kinds=dict(y="exact"))


def _perm_rfk(i):
    import torch
    x = _t(i["x"]); B, S, D = x.shape
    o = torch.empty(B, D, S, device="cuda", dtype=torch.float16)
    _ops().permute_bsd_to_nchw(x, o, B, S, D); return dict(o=_n(o))


for shp in [(1, 64, 64), (2, 49, 100), (1, 130, 33), (3, 1, 7)]:
    case(name="permute_bsd_to_nchw_" + "x".join(map(str, shp)),
         make=(lambda shp: lambda rng: dict(x=normal(rng, shp, np.float16, 1.0)))(shp),
         oracle=lambda i: dict(o=O.permute_bsd_to_nchw(i["x"])), rfk=_perm_rfk, ref=None, kinds=dict(o="exact"),
         oracle_kinds=dict(o="exact"))

# ------------------------------------------------------ per-view ray front end

def _ray_make(B, res):
    def make(rng):
        c2w, fov = look_at_c2w(rng, B)
        return dict(c2w=c2w, fov=fov, res=res)
    return make


def _ray_rfk(i):
    import torch
    c2w, fov = _t(i["c2w"]), _t(i["fov"]); B, res = fov.numel(), i["res"]
    ro = _empty((B, 3), torch.float32); rd = _empty((B, res, res, 3), torch.float16)
    _ops().ray_gen(c2w, fov, ro, rd, B, res)
    out = dict(rays_o=_n(ro), rays_d=_n(rd))
    if res % 8 == 0:
        pat = _empty((B, (res // 8) ** 2, 192), torch.float16)
        _ops().ray_gen_patchify(c2w, fov, None, pat, B, res, 8)
        out["tokens"] = _n(pat)
    return out


def _ray_ref(i):
    import torch
    c2w, fov = _t(i["c2w"]), _t(i["fov"]); B, res = fov.numel(), i["res"]
    ro = _empty((B, 3), torch.float32); rd = _empty((B, res, res, 3), torch.float16)
    _ref().call("ref_ray_gen", c2w, fov, ro, rd, B, res)
    out = dict(rays_o=_n(ro), rays_d=_n(rd))
    if res % 8 == 0:  # patch layout of k_patchify_s, a pure permutation
        p = res // 8
        t = out["rays_d"].reshape(B, p, 8, p, 8, 3).transpose(0, 1, 3, 5, 2, 4).reshape(B, p * p, 192)
        out["tokens"] = np.ascontiguousarray(t)
    return out


def _ray_oracle(i):
    ro, rd = O.ray_gen(i["c2w"], i["fov"], i["res"])
    out = dict(rays_o=ro, rays_d=rd)
    if i["res"] % 8 == 0:
        out["tokens"] = O.ray_gen(i["c2w"], i["fov"], i["res"], 8)[1]
    return out


for B, res in [(2, 64), (1, 20), (1, 8)]:
    kinds = dict(rays_o="exact", rays_d="exact")
    okinds = dict(rays_o="exact", rays_d="f16_1ulp")
    if res % 8 == 0:
        kinds["tokens"] = "exact"; okinds["tokens"] = "f16_1ulp"
    case(name=f"ray_gen_b{B}_res{res}", make=_ray_make(B, res), oracle=_ray_oracle, rfk=_ray_rfk,
         ref=_ray_ref, kinds=kinds, oracle_kinds=okinds, seed=3)


def _w2c_make(B, N, with_vn, dtype):
    def make(rng):
        c2w, _ = look_at_c2w(rng, B)
        vn = rng.standard_normal((B, N, 3, 3)); vn /= np.linalg.norm(vn, axis=-1, keepdims=True)
        return dict(c2w=c2w, tri=uniform(rng, (B, N, 3, 3), dtype), vn=vn.astype(dtype) if with_vn else None)
    return make


def _w2c_rfk(i):
    c2w, tri = _t(i["c2w"]), _t(i["tri"]); vn = None if i["vn"] is None else _t(i["vn"])
    B, N = tri.shape[:2]
    if i["tri"].dtype == np.float16:
        _ops().world_to_cam(c2w, tri, vn, B, N)
    else:
        _ops().world_to_cam_f32(c2w, tri, vn, B, N * 3)
    out = dict(tri=_n(tri))
    if vn is not None:
        out["vn"] = _n(vn)
    return out


def _w2c_ref(i):
    c2w, tri = _t(i["c2w"]), _t(i["tri"]); vn = None if i["vn"] is None else _t(i["vn"])
    B, N = tri.shape[:2]
    _ref().call("ref_world_to_cam", c2w, tri, vn, B, N)
    out = dict(tri=_n(tri))
    if vn is not None:
        out["vn"] = _n(vn)
    return out


def _w2c_oracle(i):
    tri, vn = O.world_to_cam(i["c2w"], i["tri"], i["vn"])
    out = dict(tri=tri)
    if vn is not None:
        out["vn"] = vn
    return out


for B, N, with_vn, dt, tag in [(2, 100, True, np.float16, "f16"), (1, 77, False, np.float16, "f16_novn"),
                                (2, 100, True, np.float32, "f32")]:
    ks = dict(tri="exact", vn="exact") if with_vn else dict(tri="exact")
    oks = {k: ("f16_1ulp" if dt == np.float16 else "f32") for k in ks}
    case(name=f"world_to_cam_{tag}", make=_w2c_make(B, N, with_vn, dt), oracle=_w2c_oracle, rfk=_w2c_rfk,
         ref=_w2c_ref if dt == np.float16 else None, kinds=ks, oracle_kinds=oks, seed=3)


def _vg_make(N, nr, pad, nf, hd):
    def make(rng):
        c2w, _ = look_at_c2w(rng, 1)
        vn = rng.standard_normal((N, 3, 3)); vn /= np.linalg.norm(vn, axis=-1, keepdims=True)
        tri = uniform(rng, (N, 3, 3), np.float16)
        center = tri.astype(np.float64).reshape(N, 9).mean(0).reshape(3, 3).mean(0).astype(np.float32)
        return dict(c2w=c2w[0], tri=tri, vn=vn.astype(np.float16), center=center, freqs=_geo_freqs(nf),
                    nr=nr, seq_pad=nr + N + pad, nf=nf, hd=hd)
    return make


def _vg_rfk(i):
    import torch
    N = i["tri"].shape[0]; sp, hd = i["seq_pad"], i["hd"]
    vtri = _empty((N, 3, 3), torch.float16); vvn = torch.empty_like(vtri)
    vpos = _empty((sp, 9), torch.float16); kc = _empty((sp, hd), torch.float16); ks = torch.empty_like(kc)
    _ops().view_geometry(_t(i["c2w"]), _t(i["tri"]), _t(i["vn"]), _t(i["center"]), _t(i["freqs"]),
                         vtri, vvn, vpos, kc, ks, N, i["nr"], sp, i["nf"], hd)
    return dict(vtri=_n(vtri), vvn=_n(vvn), vpos=_n(vpos), k_cos=_n(kc), k_sin=_n(ks))


def _vg_ref(i):
    """The reference's per-view sequence (src/pipeline/render_session.cu:192-203); the
    register-token rows come from the CPU restatement of k_center_pos_from_c2w, which the
    reference library does not export."""
    import torch
    N = i["tri"].shape[0]; sp, hd, nr = i["seq_pad"], i["hd"], i["nr"]
    vtri, vvn = _t(i["tri"]), _t(i["vn"])
    _ref().call("ref_world_to_cam", _t(i["c2w"]), vtri, vvn, 1, N)
    vpos = torch.zeros((sp, 9), dtype=torch.float16, device="cuda")
    vpos[:nr] = _t(O.center_pos(i["c2w"], i["center"], nr))
    vpos[nr:nr + N] = vtri.view(N, 9)
    kc = _empty((sp, hd), torch.float16); ks = torch.empty_like(kc)
    _ref().call("ref_triangle_rope_freqs", vpos, _t(i["freqs"]), kc, ks, 1, sp, i["nf"], hd)
    return dict(vtri=_n(vtri), vvn=_n(vvn), vpos=_n(vpos), k_cos=_n(kc), k_sin=_n(ks))


def _vg_oracle(i):
    N = i["tri"].shape[0]; sp, hd, nr = i["seq_pad"], i["hd"], i["nr"]
    vtri, vvn = O.world_to_cam(i["c2w"], i["tri"][None], i["vn"][None])
    vpos = np.zeros((sp, 9), np.float16)
    vpos[:nr] = O.center_pos(i["c2w"], i["center"], nr)
    vpos[nr:nr + N] = vtri.reshape(N, 9)
    c, s = O.triangle_rope_freqs(vpos, i["freqs"], hd)
    return dict(vtri=vtri[0], vvn=vvn[0], vpos=vpos, k_cos=c, k_sin=s)


for N, nr, pad, nf, hd in [(61, 32, 3, 3, 64), (40, 4, 0, 6, 128)]:
    case(name=f"view_geometry_n{N}_hd{hd}", make=_vg_make(N, nr, pad, nf, hd), oracle=_vg_oracle,
         rfk=_vg_rfk, ref=_vg_ref, seed=3,
         kinds=dict(vtri="exact", vvn="exact", vpos="exact", k_cos="f16", k_sin="f16"),
         oracle_kinds=dict(vtri="f16_1ulp", vvn="f16_1ulp", vpos="f16_1ulp", k_cos="f16", k_sin="f16"))

# --------------------------------------------------------------------- layouts

def _tr_make(B, S, Hh, D):
    return lambda rng: dict(x=normal(rng, (B, S, Hh, D), np.float16))


def _tr_rfk(i):
    import torch
    x = _t(i["x"]); B, S, Hh, D = x.shape
    o = _empty((B, Hh, S, D), torch.float16); _ops().transpose_bshd_to_bhsd(x, o, B, S, Hh, D)
    back = _empty((B, S, Hh * D), torch.float16); _ops().transpose_bhsd_to_bsd(o, back, B, Hh, S, D)
    return dict(bhsd=_n(o), back=_n(back))


for B, S, Hh, D in [(2, 13, 4, 64), (1, 7, 3, 20)]:
    case(name=f"transpose_b{B}s{S}h{Hh}d{D}", make=_tr_make(B, S, Hh, D),
         oracle=lambda i: dict(bhsd=O.transpose_bshd_to_bhsd(i["x"]),
                               back=O.transpose_bhsd_to_bsd(O.transpose_bshd_to_bhsd(i["x"]))),
         rfk=_tr_rfk, kinds=dict(bhsd="exact", back="exact"), oracle_kinds=dict(bhsd="exact", back="exact"))


def _win_make(B, Hh, W, C, ws, shift):
    return lambda rng: dict(x=normal(rng, (B, Hh, W, C), np.float16), y=normal(rng, (B, Hh, W, C), np.float16),
                            ws=ws, shift=shift)


def _win_rfk(i):
    import torch
    x, y = _t(i["x"]), _t(i["y"]); B, Hh, W, C = x.shape; ws, sh = i["ws"], i["shift"]
    win = _empty((B * (Hh // ws) * (W // ws), ws * ws, C), torch.float16)
    _ops().window_gather(x, win, B, Hh, W, C, ws, sh)
    back = torch.empty_like(x); _ops().window_scatter(win, back, B, Hh, W, C, ws, sh, False)
    acc = y.clone(); _ops().window_scatter(win, acc, B, Hh, W, C, ws, sh, True)
    return dict(win=_n(win), back=_n(back), acc=_n(acc))


def _win_ref(i):
    import torch
    x, y = _t(i["x"]), _t(i["y"]); B, Hh, W, C = x.shape; ws, sh = i["ws"], i["shift"]
    R = _ref(); L = R.layers()
    shifted = x
    if sh > 0:
        shifted = torch.empty_like(x); R.call("ref_cyclic_shift_2d", x, shifted, B, Hh, W, C, -sh, -sh, lib=L)
    win = _empty((B * (Hh // ws) * (W // ws), ws * ws, C), torch.float16)
    R.call("ref_window_partition", shifted, win, B, Hh, W, C, ws, lib=L)
    rev = torch.empty_like(x); R.call("ref_window_reverse", win, rev, B, Hh, W, C, ws, lib=L)
    back = rev
    if sh > 0:
        back = torch.empty_like(x); R.call("ref_cyclic_shift_2d", rev, back, B, Hh, W, C, sh, sh, lib=L)
    acc = y.clone(); R.call("ref_residual_add", acc, back, acc.numel(), lib=L)
    return dict(win=_n(win), back=_n(back), acc=_n(acc))


def _win_oracle(i):
    x, ws, sh = i["x"], i["ws"], i["shift"]; B, Hh, W, C = x.shape
    shifted = O.cyclic_shift(x, -sh, -sh) if sh > 0 else x
    win = O.window_partition(shifted, ws)
    rev = O.window_reverse(win, B, Hh, W, ws)
    back = O.cyclic_shift(rev, sh, sh) if sh > 0 else rev
    return dict(win=win, back=back, acc=O.residual_add(i["y"], back))


for B, Hh, W, C, ws, sh in [(1, 16, 16, 64, 8, 4), (2, 8, 16, 24, 4, 0), (1, 8, 8, 20, 4, 2)]:
    k = dict(win="exact", back="exact", acc="exact")
    case(name=f"window_b{B}_{Hh}x{W}x{C}_ws{ws}_s{sh}", make=_win_make(B, Hh, W, C, ws, sh),
         oracle=_win_oracle, rfk=_win_rfk, ref=_win_ref, kinds=k, oracle_kinds=k)


def _patch_rfk(i):
    import torch
    x = _t(i["x"]); Hh, W, C = x.shape
    o = _empty(((Hh // 8) * (W // 8), C * 64), torch.float16)
    _ops().patchify(x, o, Hh, W, C, 8)
    return dict(o=_n(o))


case(name="patchify_24x16x3", make=lambda rng: dict(x=normal(rng, (24, 16, 3), np.float16)),
     oracle=lambda i: dict(o=O.patchify(i["x"], 8)), rfk=_patch_rfk, kinds=dict(o="exact"),
     oracle_kinds=dict(o="exact"))


# ------------------------------------------------- fused attention (no score matrix)

def _attn_make(B, Hh, Sq, Sk, D, n_keys):
    def make(rng):
        K = normal(rng, (B, Hh, Sk, D), np.float16); V = normal(rng, (B, Hh, Sk, D), np.float16)
        K[:, :, n_keys:] = 0; V[:, :, n_keys:] = 0  # pad keys as the K/V cache builder leaves them
        return dict(Q=normal(rng, (B, Hh, Sq, D), np.float16), K=K, V=V, n_keys=n_keys)
    return make


def _attn_oracle(i):
    return dict(o=O.sdpa(i["Q"], i["K"], i["V"], n_keys=i["n_keys"]),
                o_bshd=O.sdpa(i["Q"], i["K"], i["V"], n_keys=i["n_keys"], o_bshd=True))


def _attn_rfk(i):
    import torch
    Q, K, V = _t(i["Q"]), _t(i["K"]), _t(i["V"]); B, Hh, Sq, D = Q.shape; Sk = K.shape[2]
    o = _empty(Q.shape, torch.float16); ob = _empty((B, Sq, Hh * D), torch.float16)
    _ops().flash_attention(Q, K, V, o, B, Hh, Sq, Sk, i["n_keys"], D)
    _ops().flash_attention(Q, K, V, ob, B, Hh, Sq, Sk, i["n_keys"], D, o_bshd=True)
    torch.cuda.synchronize()
    assert _ops().flash_attention_error() == 0
    return dict(o=_n(o), o_bshd=_n(ob))


def _attn_ref(i):
    """rf::sdpa (cuDNN fused kernel when it takes the shape, else cuBLAS + softmax_cast_fp16); it attends all Sk keys."""
    import torch
    R = _ref()
    Q, K, V = _t(i["Q"]), _t(i["K"]), _t(i["V"]); B, Hh, Sq, D = Q.shape; Sk = K.shape[2]
    o = _empty(Q.shape, torch.float16); ws = _empty((B * Hh * Sq * Sk,), torch.float32)
    h = R.cublas_create()
    R.call("ref_sdpa", R.Raw(h), Q, K, V, o, ws, None, B, Hh, Sq, Sk, D, lib=R.layers())
    torch.cuda.synchronize()
    R.cublas_destroy(h)
    ob = o.permute(0, 2, 1, 3).contiguous().view(B, Sq, Hh * D)
    return dict(o=_n(o), o_bshd=_n(ob))


for B, Hh, Sq, Sk, D, nk in [(1, 2, 128, 128, 64, 128), (1, 3, 200, 328, 64, 328), (2, 2, 77, 200, 64, 193),
                             (1, 2, 130, 72, 128, 72), (1, 1, 5, 40, 64, 33)]:
    case(name=f"flash_attention_b{B}h{Hh}_{Sq}x{Sk}_d{D}_k{nk}", make=_attn_make(B, Hh, Sq, Sk, D, nk),
         oracle=_attn_oracle, rfk=_attn_rfk, ref=_attn_ref if nk == Sk else None, kinds=dict(o="f16", o_bshd="f16"))


def _winattn_make(BnW, Hh, nW, masked):
    def make(rng):
        m = None
        if masked:
            m = (rng.uniform(size=(nW, 64, 64)) > 0.4).astype(np.uint8)
            m[nW - 1, 5, :] = 0  # one fully masked row: the -FLT_MAX fill makes it the plain mean of V
        return dict(Q=normal(rng, (BnW, Hh, 64, 64), np.float16), K=normal(rng, (BnW, Hh, 64, 64), np.float16),
                    V=normal(rng, (BnW, Hh, 64, 64), np.float16), mask=m, nW=nW)
    return make


def _winattn_rfk(i):
    import torch
    Q, K, V = _t(i["Q"]), _t(i["K"]), _t(i["V"]); BnW, Hh = Q.shape[:2]
    o = _empty((BnW * 64, Hh * 64), torch.float16)
    _ops().window_attention(Q, K, V, o, None if i["mask"] is None else _t(i["mask"]), BnW, Hh, i["nW"])
    return dict(o=_n(o))


for BnW, Hh, nW, masked in [(4, 2, 4, False), (8, 3, 4, True)]:
    case(name=f"window_attention_{BnW}x{Hh}_{'masked' if masked else 'plain'}", make=_winattn_make(BnW, Hh, nW, masked),
         oracle=lambda i: dict(o=O.sdpa(i["Q"], i["K"], i["V"], mask=i["mask"], o_bshd=True).reshape(-1, i["Q"].shape[1] * 64)),
         rfk=_winattn_rfk, kinds=dict(o="f16"))


# ---------------------------- residual + RMSNorm with one operand in swin window order

def _normwin_make(B, Hh, W, C, ws, sh):
    def make(rng):
        return dict(x=normal(rng, (B, Hh, W, C), np.float16), r=normal(rng, (B, Hh, W, C), np.float16),
                    gamma=normal(rng, (C,), np.float32, 0.1, 1.0), ws=ws, shift=sh)
    return make


def _normwin_oracle(i):
    x, r, ws, sh = i["x"], i["r"], i["ws"], i["shift"]; B, Hh, W, C = x.shape
    to_win = lambda a: O.window_partition(O.cyclic_shift(a, -sh, -sh) if sh > 0 else a, ws)
    # (1) x += r; y = norm(x); y leaves in window order
    x1, y1 = O.rmsnorm_residual_f16(x.reshape(-1, C), r.reshape(-1, C), i["gamma"], 2.0 ** -10)
    y1w = to_win(y1.reshape(B, Hh, W, C)).reshape(-1, C)
    # (2) r arrives in window order: x += unwindow(r); y = norm(x)
    rev = O.window_reverse(r.reshape(-1, ws * ws, C), B, Hh, W, ws)
    back = O.cyclic_shift(rev, sh, sh) if sh > 0 else rev
    x2, y2 = O.rmsnorm_residual_f16(x.reshape(-1, C), back.reshape(-1, C), i["gamma"], 2.0 ** -10)
    return dict(x1=x1, y1=y1w, x2=x2, y2=y2)


def _normwin_rfk(i):
    import torch
    x, r, g = _t(i["x"]), _t(i["r"]), _t(i["gamma"]); B, Hh, W, C = x.shape
    out = {}
    for which in (1, 2):
        xx = x.clone().view(-1, C); y = torch.empty_like(xx)
        _ops().rmsnorm_residual_f16_windows(xx, r.view(-1, C), g, y, B, Hh, W, C, i["ws"], i["shift"], which)
        out[f"x{which}"] = _n(xx); out[f"y{which}"] = _n(y)
    return out


for B, Hh, W, C, ws, sh in [(1, 16, 16, 256, 8, 4), (2, 8, 16, 64, 4, 0), (1, 8, 8, 1024, 4, 3)]:
    k = dict(x1="exact", y1="f16", x2="exact", y2="f16")
    case(name=f"rmsnorm_windows_b{B}_{Hh}x{W}x{C}_ws{ws}_s{sh}", make=_normwin_make(B, Hh, W, C, ws, sh),
         oracle=_normwin_oracle, rfk=_normwin_rfk, kinds=k)


BY_NAME = {c.name: c for c in CASES}
assert len(BY_NAME) == len(CASES), "duplicate case names"
