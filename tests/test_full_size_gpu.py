"""GPU tests at the full sizes of the benchmark configurations, through size-independent
properties plus a comparison with the reference's own kernels where they are present."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

T, D = 5633, 1024


def _ops():
    import renderformer_cuda_b200 as pkg
    return pkg.ops


def _ref():
    from oracle import ref
    return ref if (ref.available() and ref.layers_available()) else None


def _close16(a, b):
    """fp16 tolerance: 2e-3 absolute, or one fp16 rounding step for magnitudes above 2."""
    import torch
    a, b = a.float(), b.float()
    tol = torch.maximum(torch.full_like(b, 2e-3), b.abs() * 2.0 ** -10)
    bad = (a - b).abs() > tol
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} outside fp16 tolerance"


def test_config1_fused_rmsnorm_residual_full_size():
    import torch
    g = torch.Generator(device="cuda").manual_seed(0)
    h = torch.randn(T, D, device="cuda", generator=g); r = torch.randn(T, D, device="cuda", generator=g)
    gamma = 1 + 0.02 * torch.randn(D, device="cuda", generator=g)
    h0 = h.clone(); y = torch.empty(T, D, device="cuda", dtype=torch.float16)
    _ops().rmsnorm_residual_f32_cast16(h, r, gamma, y, T, D, 1e-6)
    assert torch.equal(h, h0 + r)                                  # residual add is exact fp32
    hs = (h0 + r).double()
    want = hs / torch.sqrt((hs ** 2).mean(1, keepdim=True) + 1e-6) * gamma.double()
    _close16(y, want.float())
    # scale invariance of the norm: y(2h) == y(h) up to rounding
    h2 = (h0 + r) * 2; y2 = torch.empty_like(y)
    _ops().rmsnorm_residual_f32_cast16(h2, None, gamma, y2, T, D, 4e-6)
    _close16(y2, y)
    R = _ref()
    if R:
        hr = h0.clone(); tmp = torch.empty_like(hr); yr = torch.empty_like(y)
        R.call("ref_residual_rmsnorm_cast", hr, r, gamma, tmp, yr, T, D, 1e-6, lib=R.layers())
        assert torch.equal(hr, h)
        _close16(y, yr)


def test_config2_rope_full_size_is_norm_preserving_and_matches_reference():
    import torch
    Hh, hd, nf = 16, 64, 3
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(1, Hh, T, hd, device="cuda", generator=g).half()
    k = torch.randn(1, Hh, T, hd, device="cuda", generator=g).half()
    pos = (torch.rand(1, T, 9, device="cuda", generator=g) * 2 - 1).half()
    freqs = torch.tensor([np.pi, np.pi * 10000 ** (-1 / 3), np.pi * 10000 ** (-2 / 3)], device="cuda", dtype=torch.float32)
    c = torch.empty(1, 1, T, hd, device="cuda", dtype=torch.float16); s = torch.empty_like(c)
    _ops().triangle_rope_freqs(pos, freqs, c, s, 1, T, nf, hd)
    assert torch.equal(c[..., :32], c[..., 32:]) and (c[..., 27:32] == 1).all() and (s[..., 27:32] == 0).all()
    q0, k0 = q.clone(), k.clone()
    _ops().apply_rope(q, k, c, s, 1, Hh, T, hd)
    n0 = q0.float()[..., :32] ** 2 + q0.float()[..., 32:] ** 2
    n1 = q.float()[..., :32] ** 2 + q.float()[..., 32:] ** 2
    assert ((n1 - n0).abs() <= 1e-2 + 4e-3 * n0).all()           # each pair is rotated
    assert torch.equal(q[..., 27:32], q0[..., 27:32])              # pad region: cos=1, sin=0
    # rotating by the table and then by its inverse (sin -> -sin) restores the input
    qi = q.clone(); _ops().apply_rope_one(qi, c, -s, 1, Hh, T, hd)
    err = (qi.float() - q0.float()).abs()                          # two fp16 roundings + table rounding
    assert (err <= 4e-3 + 3 * 2.0 ** -10 * q0.float().abs()).all()
    # the rotation itself, from the stored fp16 tables, in fp32 (rope.cu:75-88 restated in torch)
    def rot(x):
        xf = x.float()
        rh = torch.cat([-xf[..., 32:], xf[..., :32]], dim=-1)
        return (xf * c.float() + rh * s.float()).half()
    _close16(q, rot(q0)); _close16(k, rot(k0))
    R = _ref()
    if R:
        cr = torch.empty_like(c); sr = torch.empty_like(s)
        R.call("ref_triangle_rope_freqs", pos, freqs, cr, sr, 1, T, nf, hd)
        _close16(c, cr); _close16(s, sr)
        qr, kr = q0.clone(), k0.clone()
        R.call("ref_apply_rope", qr, kr, cr, sr, 1, Hh, T, hd)
        # The reference rotates in place with one thread per element and no ordering between a
        # thread's store and its partner's load (src/kernels/rope.cu:84-92): at this size a few
        # hundred of the 5.8 M elements come out rotated from an already-updated partner. Where
        # the two disagree, this library must be the one that matches the formula.
        for mine, theirs, x0 in ((q, qr, q0), (k, kr, k0)):
            tol = torch.maximum(torch.full_like(mine.float(), 2e-3), theirs.float().abs() * 2.0 ** -10)
            bad = (mine.float() - theirs.float()).abs() > tol
            assert bad.float().mean() < 1e-3, "more disagreement than a sporadic race explains"
            want = rot(x0)
            assert ((mine.float() - want.float()).abs()[bad] <= 2e-3 + 2.0 ** -10 * want.float().abs()[bad]).all()


def test_config2_nerf_pe_normals_full_size():
    import torch
    g = torch.Generator(device="cuda").manual_seed(1)
    n = torch.randn(1, T, 3, 3, device="cuda", generator=g)
    n = (n / n.norm(dim=-1, keepdim=True)).reshape(1, T, 9).contiguous()
    out = torch.empty(1, T, 117, device="cuda", dtype=torch.float16)
    _ops().nerf_pe_f32(n, out, 1, T, 9, 6, 0.0, 5.0, True)
    o = out.float()
    assert torch.equal(out[..., :9], n.half())
    sin, cos = o[..., 9:63], o[..., 63:]
    assert ((sin ** 2 + cos ** 2 - 1).abs() < 4e-3).all()          # sin^2 + cos^2 = 1
    f = 2.0 ** torch.arange(6, device="cuda")
    want = torch.sin((n.double()[..., :, None] * f.double()).reshape(1, T, 54))
    assert (sin.double() - want).abs().max() < 2e-3
    R = _ref()
    if R:
        outr = torch.empty_like(out)
        R.call("ref_nerf_pe_f32", n, outr, 1, T, 9, 6, 0.0, 5.0, 1)
        _close16(out, outr)


def test_config3_softmax_full_size():
    import torch
    rows, cols, stride = 16 * 4096, 5633, 5640
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.full((rows, stride), float("-inf"), device="cuda")
    x[:, :cols] = torch.randn(rows, cols, device="cuda", generator=g) * (3.0 / 8.0)
    p = torch.full((rows, stride), 7.0, device="cuda", dtype=torch.float16)
    _ops().softmax_cast_fp16(x, p, rows, cols, stride, stride)
    assert (p[:, cols:] == 0).all()                                 # pad written as zero
    sums = p.float().sum(1)
    assert ((sums - 1).abs() < 2e-3).all()                          # rows are distributions
    # shift invariance: softmax(x + c) == softmax(x)
    sub = slice(0, 2048)
    p2 = torch.empty_like(p[sub])
    xs = (x[sub] + 5.0).contiguous()
    _ops().softmax_cast_fp16(xs, p2, 2048, cols, stride, stride)
    assert ((p2.float() - p[sub].float()).abs() <= 2e-3).all()
    # argmax is preserved
    want = torch.softmax(x[sub, :cols].double(), dim=1)
    assert (p[sub, :cols].double() - want).abs().max() < 2e-3
    R = _ref()
    if R:
        pr = torch.empty_like(p)
        R.call("ref_softmax_cast_fp16", x, pr, rows, cols, stride, stride)
        assert ((p.float() - pr.float()).abs() <= 2e-3).all()


def test_config4_front_end_full_size():
    import torch
    import cases
    rng = np.random.default_rng(3)
    c2w_np, fov_np = cases.look_at_c2w(rng, 2)
    c2w = torch.from_numpy(c2w_np).cuda(); fov = torch.from_numpy(fov_np).cuda()
    res = 512
    ro = torch.empty(2, 3, device="cuda"); rd = torch.empty(2, res, res, 3, device="cuda", dtype=torch.float16)
    _ops().ray_gen(c2w, fov, ro, rd, 2, res)
    assert torch.equal(ro, c2w[:, :3, 3])
    assert ((rd.float().norm(dim=-1) - 1).abs() < 2e-3).all()
    tok = torch.empty(2, 4096, 192, device="cuda", dtype=torch.float16)
    _ops().ray_gen_patchify(c2w, fov, None, tok, 2, res, 8)
    want_tok = rd.view(2, 64, 8, 64, 8, 3).permute(0, 1, 3, 5, 2, 4).reshape(2, 4096, 192)
    assert torch.equal(tok, want_tok)                               # fused patch layout is a permutation
    R = _ref()
    if R:
        ror = torch.empty_like(ro); rdr = torch.empty_like(rd)
        R.call("ref_ray_gen", c2w, fov, ror, rdr, 2, res)
        assert torch.equal(rd.view(torch.int16), rdr.view(torch.int16))  # bit-exact
    # world -> camera of 5633 triangles, then back with the inverse pose: round trip in fp32
    v = (torch.rand(1, T * 3, 3, device="cuda") * 2 - 1)
    v0 = v.clone()
    _ops().world_to_cam_f32(c2w[:1], v, None, 1, T * 3)
    back = v @ c2w[0, :3, :3].T + c2w[0, :3, 3]
    assert (back - v0).abs().max() < 1e-5
    tri = v0.half().view(1, T, 3, 3).contiguous(); vn = torch.nn.functional.normalize(torch.randn(1, T, 3, 3, device="cuda"), dim=-1).half()
    tri_r, vn_r = tri.clone(), vn.clone()
    _ops().world_to_cam(c2w[:1], tri, vn, 1, T)
    assert ((vn.float().norm(dim=-1) - 1).abs() < 3e-3).all()       # rotations keep unit normals
    if R:
        R.call("ref_world_to_cam", c2w[:1], tri_r, vn_r, 1, T)
        assert torch.equal(tri.view(torch.int16), tri_r.view(torch.int16))
        assert torch.equal(vn.view(torch.int16), vn_r.view(torch.int16))
    # nerf_pe of the ray directions [262144,3] -> [262144,39]
    dirs = rd[0].reshape(1, res * res, 3).contiguous()
    pe = torch.empty(1, res * res, 39, device="cuda", dtype=torch.float16)
    _ops().nerf_pe(dirs, pe, 1, res * res, 3, 6, 0.0, 5.0, True)
    assert torch.equal(pe[..., :3], dirs)
    assert ((pe.float()[..., 3:21] ** 2 + pe.float()[..., 21:] ** 2 - 1).abs() < 4e-3).all()
    if R:
        per = torch.empty_like(pe)
        R.call("ref_nerf_pe", dirs, per, 1, res * res, 3, 6, 0.0, 5.0, 1)
        _close16(pe, per)
    # SwiGLU gate on [4096,4096]
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(4096, 4096, device="cuda", generator=g).half(); b = torch.randn(4096, 4096, device="cuda", generator=g).half()
    o = torch.empty_like(a)
    _ops().fused_silu_mul(a, b, o, a.numel())
    want = torch.nn.functional.silu(a.float()) * b.float()
    _close16(o, want)
    if R:
        orf = torch.empty_like(a)
        R.call("ref_fused_silu_mul", a, b, orf, a.numel())
        _close16(o, orf)


def test_batched_world_to_cam_and_ray_gen_paths_equal_the_single_view_kernels():
    """Large batches take other kernels (8 vertices per thread with 128-bit accesses; ray strips with stores staged
    through shared memory). Both must give the bits of the one-view kernels, which are checked against the reference."""
    import torch
    import renderformer_cuda_b200 as pkg
    import cases
    ops = pkg.ops
    B, n_tris, res = 40, 5633, 512        # 16899 vertices per view: threads straddle view boundaries
    c2w_np, fov_np = cases.look_at_c2w(np.random.default_rng(11), B)
    c2w, fov = torch.from_numpy(c2w_np).cuda(), torch.from_numpy(fov_np).cuda()
    g = torch.Generator(device="cuda").manual_seed(3)
    tri = (torch.rand(B, n_tris, 3, 3, device="cuda", generator=g) * 2 - 1).half()
    vn = torch.nn.functional.normalize(torch.randn(B, n_tris, 3, 3, device="cuda", generator=g), dim=-1).half()
    t_all, v_all = tri.clone(), vn.clone()
    ops.world_to_cam(c2w, t_all, v_all, B, n_tris)
    for b in range(B):
        t1, v1 = tri[b:b + 1].clone(), vn[b:b + 1].clone()
        ops.world_to_cam(c2w[b:b + 1].contiguous(), t1, v1, 1, n_tris)
        assert torch.equal(t1[0], t_all[b]) and torch.equal(v1[0], v_all[b]), f"view {b}"
    ro_all = torch.empty(B, 3, device="cuda"); rd_all = torch.empty(B, res, res, 3, device="cuda", dtype=torch.float16)
    ops.ray_gen(c2w, fov, ro_all, rd_all, B, res)
    for b in range(0, B, 5):
        ro1 = torch.empty(1, 3, device="cuda"); rd1 = torch.empty(1, res, res, 3, device="cuda", dtype=torch.float16)
        ops.ray_gen(c2w[b:b + 1].contiguous(), fov[b:b + 1].contiguous(), ro1, rd1, 1, res)
        assert torch.equal(rd1[0], rd_all[b]) and torch.equal(ro1[0], ro_all[b]), f"view {b}"


# ----------------------------------------------------------------------------------------------
# BASELINE configs[4] at full size: dim 1024, 16 heads x 64, FFN 4096, 12 decoder layers, 5633
# triangles (5665 keys padded to 5672), 512x512 -> 4096 patch tokens.

def _config5():
    """Model, scene state (encoded by this library) and one camera, shared by the tests below."""
    import torch
    import cases
    from renderformer_cuda_b200 import session as S
    if "c5" not in _config5.__dict__:
        model = S.Model.random(seed=4)
        g = torch.Generator(device="cuda").manual_seed(4)
        n = 5633
        tri = (torch.rand(n, 3, 3, device="cuda", generator=g) * 2 - 1).contiguous()
        vn = torch.nn.functional.normalize(torch.randn(n, 3, 3, device="cuda", generator=g), dim=-1).contiguous()
        tex = torch.rand(n, 13, device="cuda", generator=g).half().contiguous()
        ses = S.RenderSession(model, n, 512, pad_keys_attend=True)   # the reference attends its 7 zero pad keys
        ses.encode_scene(tri, vn, tex)
        ses.finalize()
        c2w, fov = cases.look_at_c2w(np.random.default_rng(4), 2)
        _config5.c5 = dict(model=model, ses=ses, c2w=torch.from_numpy(c2w).contiguous().pin_memory(), fov=fov, n=n,
                           scene=(tri, vn, tex))
    return _config5.c5


def _fp32_view(c5, cam):
    """fp32 torch evaluation of one view from the same scene state: ray-token front end (the patchified rays come
    from this library's ray generator, bit-identical to the reference's), then the 12 decoder layers."""
    import torch
    import renderformer_cuda_b200 as pkg
    import torch_layers as TL
    from oracle import ref_pipeline as RP
    m, ses, n = c5["model"], c5["ses"], c5["n"]
    lay = RP.state_layout(m, n)
    st, H16 = ses.scene_state, torch.float16
    Se_pad, hd, nr, dim, heads = lay["Se_pad"], m.head_dim, m.num_register_tokens, m.dim, m.num_heads
    kv = st[:2 * m.dec_layers * lay["kv_layer"]].view(H16).view(m.dec_layers, 2, heads, Se_pad, hd)
    tri16 = st[lay["tri_off"]:lay["tri_off"] + n * 18].view(H16); vn16 = st[lay["vn_off"]:lay["vn_off"] + n * 18].view(H16)
    center = st[lay["c_off"]:lay["c_off"] + 12].view(torch.float32)
    c2w = c5["c2w"][cam].reshape(16).cuda(); fv = torch.tensor([float(c5["fov"][cam])], device="cuda")
    vtri = torch.empty(n * 9, device="cuda", dtype=H16); vvn = torch.empty_like(vtri)
    vpos = torch.empty(Se_pad * 9, device="cuda", dtype=H16)
    kc = torch.empty(Se_pad, hd, device="cuda", dtype=H16); ks = torch.empty_like(kc)
    pkg.ops.view_geometry(c2w, tri16, vn16, center, m.t["vt_rope_freqs"], vtri, vvn, vpos, kc, ks, n, nr, Se_pad,
                          m.rope_num_freqs, hd)
    pat = torch.empty(4096, 192, device="cuda", dtype=H16)
    pkg.ops.ray_gen_patchify(torch.eye(4, device="cuda").reshape(16).contiguous(), fv, None, pat, 1, 512, 8)
    t = m.t
    x = pat.float() @ t["ray_enc_w"].float().t() + t["ray_enc_b"].float()
    x = TL.rms(x, t["ray_enc_norm"]) + t["ray_map_patch_token"].float()
    mask = RP.shift_mask(64, 8, 4)
    for i in range(m.dec_layers):
        shift = 4 if i % 2 else 0
        x = TL.decoder_layer(x, TL.layer_weights(m, i), kv[i, 0], kv[i, 1], kc, ks, mask, shift, heads, 64, 64, 8)
    return x, (kv, kc, ks, mask)


def test_config5_view_matches_reference_pipeline_with_fp32_arbiter():
    """One 512x512 view of the 5633-triangle scene at renderformer-v1.1-swin-large shapes through rfk_session_*
    and through the reference's own per-view pipeline (its kernels, layer functions, cuBLAS + cuDNN attention,
    composed as RenderSession::render_view, src/pipeline/render_session.cu:177-238) from the same scene state;
    the two token maps [4096, 1024] are compared element-wise and both are measured against an fp32 torch
    evaluation of the same view. Asserted: this library is at most 1.5x as far from the fp32 result as the
    reference (mean and max), the two arms differ by at most 2.5x the reference's own error, and the fraction of
    elements outside the per-kernel fp16 tolerance (2e-3 or one fp16 step) is reported."""
    import torch
    import torch_layers as TL
    R = _ref()
    if not R:
        pytest.skip("oracle/_ref libraries not present")
    from oracle import ref_pipeline as RP
    c5 = _config5()
    m, ses = c5["model"], c5["ses"]
    cam = 0
    ses.render_frame_raw(c5["c2w"][cam].data_ptr(), float(c5["fov"][cam]))
    got = ses.download().clone().cuda()
    pipe = RP.ViewPipeline(m, ses.scene_state, c5["n"], 512)
    host = torch.empty(4096, m.dim, dtype=torch.float16).pin_memory()
    pipe.render(c5["c2w"][cam].data_ptr(), float(c5["fov"][cam])); pipe.wait(); pipe.download(host)
    want = host.cuda()
    pipe.close()
    truth, _ = _fp32_view(c5, cam)
    assert torch.isfinite(got.float()).all() and torch.isfinite(want.float()).all()
    (rfk_mean, rfk_max), (ref_mean, ref_max) = TL.err_stats(got, truth), TL.err_stats(want, truth)
    d = (got.float() - want.float()).abs()
    tol = torch.maximum(torch.full_like(d, 2e-3), want.float().abs() * 2.0 ** -10)
    outside = float((d > tol).float().mean())
    print(f"config 5 view: |x| mean {float(want.float().abs().mean()):.4f}; vs fp32: rfk mean {rfk_mean:.3e} max {rfk_max:.3e} | "
          f"reference mean {ref_mean:.3e} max {ref_max:.3e} | rfk vs reference: mean {float(d.mean()):.3e} "
          f"max {float(d.max()):.3e}, {outside:.4%} of elements outside 2e-3 / one fp16 step")
    assert rfk_mean <= 1.5 * ref_mean + 1e-5 and rfk_max <= 1.5 * ref_max + 1e-3
    assert float(d.mean()) <= 2.5 * ref_mean + 1e-5 and float(d.max()) <= 2.5 * ref_max + 1e-3
    assert ref_mean < 1e-2 and rfk_mean < 1e-2          # 12 layers of fp16 steps on |x| = O(1) values


def test_config5_scene_state_matches_reference_encoder():
    """The scene state (12-layer mixed-precision encoder + K/V cache build) computed by this library and by the
    reference's own functions (oracle/ref_pipeline.encode_scene: its nerf_pe, linear, rmsnorm_f32,
    encoder_layer_forward_mixed, precompute_cross_kv) on the same 5633-triangle scene: geometry and centre
    bit-identical, K/V caches within the layer tolerance (mean error against the reference below 2e-3 of a
    unit-scale tensor: keys are RMS-normalised, values O(1))."""
    import torch
    R = _ref()
    if not R:
        pytest.skip("oracle/_ref libraries not present")
    from oracle import ref_pipeline as RP
    c5 = _config5()
    m, ses, n = c5["model"], c5["ses"], c5["n"]
    lay = RP.state_layout(m, n)
    assert lay["total"] == ses.scene_state.numel()
    ref_state = RP.encode_scene(m, *c5["scene"])
    a, b = ses.scene_state, ref_state
    assert torch.equal(a[lay["tri_off"]:lay["c_off"] + 12], b[lay["tri_off"]:lay["c_off"] + 12])   # fp16 geometry + fp32 centre
    H16 = torch.float16
    ka = a[:2 * m.dec_layers * lay["kv_layer"]].view(H16).float(); kb = b[:2 * m.dec_layers * lay["kv_layer"]].view(H16).float()
    d = (ka - kb).abs()
    print(f"K/V cache, 24 slabs of [16, 5672, 64]: |ref| mean {float(kb.abs().mean()):.4f}, diff mean {float(d.mean()):.3e} "
          f"max {float(d.max()):.3e}")
    assert torch.isfinite(ka).all()
    assert float(d.mean()) < 2e-3 and float(d.max()) < 0.25
    del ref_state


def test_config5_single_decoder_layer_full_shape_matches_reference():
    """One rfk_decoder_layer_forward_cached call at the full shape (4096 x 1024 tokens, 5672 keys, shift 4) against
    rf::decoder_layer_forward_cached on the same input, arbitrated by the fp32 evaluation of that layer."""
    import ctypes
    import torch
    import torch_layers as TL
    from renderformer_cuda_b200 import _abi, session as S
    R = _ref()
    if not R:
        pytest.skip("oracle/_ref libraries not present")
    from oracle import ref_pipeline as RP
    c5 = _config5()
    m, ses, n = c5["model"], c5["ses"], c5["n"]
    L = _abi.load("rfk_layers.h")
    VP = ctypes.c_void_p
    P = lambda t: VP(t.data_ptr()) if t is not None else VP(0)
    lay = RP.state_layout(m, n)
    Se_pad, hd, dim, heads, ffn, nP = lay["Se_pad"], m.head_dim, m.dim, m.num_heads, m.ffn_hidden, 4096
    H16 = torch.float16
    kv = ses.scene_state[:2 * m.dec_layers * lay["kv_layer"]].view(H16).view(m.dec_layers, 2, heads, Se_pad, hd)
    layer, shift = 1, 4
    K, V = kv[layer, 0].contiguous(), kv[layer, 1].contiguous()
    g = torch.Generator(device="cuda").manual_seed(9)
    x0 = torch.randn(nP, dim, device="cuda", generator=g).half()
    pos = (torch.rand(1, Se_pad, 9, device="cuda", generator=g) * 2 - 1).half(); pos[:, lay["Se"]:] = 0
    import renderformer_cuda_b200 as pkg
    kc = torch.empty(1, 1, Se_pad, hd, device="cuda", dtype=H16); ks = torch.empty_like(kc)
    pkg.ops.triangle_rope_freqs(pos, m.t["vt_rope_freqs"], kc, ks, 1, Se_pad, m.rope_num_freqs, hd)
    qc = torch.ones(1, 1, nP, hd, device="cuda", dtype=H16); qs = torch.zeros_like(qc)   # tables of zero positions
    mask = RP.shift_mask(64, 8, 4)
    e = lambda k, dt=H16: torch.zeros(k, device="cuda", dtype=dt)
    nWin = 64
    def bufs():
        return dict(temp=e(nP * dim), proj=e(max(2 * nP * dim + heads * Se_pad * hd, 3 * nP * dim + nWin * heads * 8 ** 4)),
                    qkv=e(nP * max(3 * dim, 2 * ffn)), ffn=e(nP * max(dim, ffn)), win=e(nP * dim),
                    cross=e(heads * nP * Se_pad, torch.float32), selfs=e(nWin * heads * 8 ** 4, torch.float32))
    ctx = S.Ctx()
    b = bufs()
    x = x0.clone()
    w = m.decoder_record(layer)
    s_ = VP(torch.cuda.current_stream().cuda_stream)
    rc = L.rfk_decoder_layer_forward_cached(ctx.h, ctypes.byref(w), P(x), VP(0), None, P(b["temp"]), P(b["proj"]), P(b["qkv"]),
                                            P(b["ffn"]), P(b["win"]), VP(0), VP(0), P(K), P(V), 1, nP, Se_pad, Se_pad, dim, heads,
                                            ffn, 64, 64, 8, shift, P(mask), VP(0), VP(0), P(kc), P(ks), s_)
    assert rc == 0, rc
    torch.cuda.synchronize()
    blas = R.cublas_create()
    xr = x0.clone()
    rw = RP.decoder_record(m, layer)
    R.call("ref_decoder_layer_forward_cached", R.Raw(blas), ctypes.byref(rw), xr, b["temp"], b["proj"], b["qkv"], b["ffn"],
           b["win"], b["cross"], b["selfs"], K, V, 1, nP, Se_pad, dim, heads, ffn, 64, 64, 8, shift, mask, qc, qs, kc, ks,
           lib=R.layers())
    torch.cuda.synchronize()
    R.cublas_destroy(blas)
    ctx.close()
    truth = TL.decoder_layer(x0, TL.layer_weights(m, layer), K, V, kc[0, 0], ks[0, 0], mask, shift, heads, 64, 64, 8)
    (rfk_mean, rfk_max), (ref_mean, ref_max) = TL.err_stats(x, truth), TL.err_stats(xr, truth)
    d_mean, d_max = TL.err_stats(x, xr)
    print(f"decoder layer [4096x1024, 5672 keys] vs fp32: rfk mean {rfk_mean:.3e} max {rfk_max:.3e} | reference mean "
          f"{ref_mean:.3e} max {ref_max:.3e} | rfk vs reference mean {d_mean:.3e} max {d_max:.3e}")
    assert rfk_mean <= 1.5 * ref_mean + 1e-5 and rfk_max <= 1.5 * ref_max + 1e-3
    assert d_mean <= 2.5 * ref_mean + 1e-5 and d_max <= 2.5 * ref_max + 1e-3
    assert ref_mean < 2e-3 and rfk_mean < 2e-3          # one layer on N(0,1) input: within the fp16 figure on average


def test_config5_teardown():
    c5 = _config5.__dict__.pop("c5", None)
    if c5:
        c5["ses"].close()
