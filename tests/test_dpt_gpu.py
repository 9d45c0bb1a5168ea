"""GPU parity tests of the DPT image head (rfk_dpt_*, include/rfk_layers.h) and of the session's image output:
against rf::dpt_forward of the reference (oracle/_ref, its cuDNN / cuBLAS calls and its own element-wise kernels,
allocating per call) on the same features and weights, arbitrated by an fp32 torch evaluation of the same head
(tests/torch_layers.py:dpt_forward): this library may be at most 1.5x as far from the fp32 result as the reference."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
H16 = torch.float16
VP = ctypes.c_void_p


def _mods():
    from renderformer_cuda_b200 import _abi, session
    return _abi.load("rfk_layers.h"), session


def _ref():
    from oracle import ref
    if not (ref.available() and ref.layers_available()):
        pytest.skip("oracle/_ref libraries not present")
    return ref


def _head(model, pH, ps, seed):
    """rfk head output, reference head output, fp32 evaluation, for random feature taps of unit scale."""
    import torch_layers as TL
    L, session = _mods()
    R = _ref()
    g = torch.Generator(device="cuda").manual_seed(seed)
    S = pH * pH
    feats = [torch.randn(S, model.dim, device="cuda", generator=g).half() for _ in range(4)]
    fp = (VP * 4)(*[f.data_ptr() for f in feats])
    res = pH * ps
    ctx = session.Ctx()
    dpt = VP()
    rc = L.rfk_dpt_create(ctx.h, ctypes.byref(model.dpt_c), 1, model.dim, pH, pH, ps, ctypes.byref(dpt))
    assert rc == 0, rc
    out = torch.empty(model.dpt_out_dim, res, res, device="cuda", dtype=H16)
    st = VP(torch.cuda.current_stream().cuda_stream)
    assert L.rfk_dpt_forward(dpt, fp, VP(out.data_ptr()), st) == 0
    torch.cuda.synchronize()
    first = out.clone()
    assert L.rfk_dpt_forward(dpt, fp, VP(out.data_ptr()), st) == 0      # same buffers, same result
    torch.cuda.synchronize()
    assert torch.equal(first, out)
    n_conv = L.rfk_dpt_num_convolutions(dpt)
    blas = R.cublas_create()
    outr = torch.empty_like(out)
    col = torch.empty(1 << 29, device="cuda", dtype=H16)                 # 1 GiB of workspace for the reference's cuDNN calls
    R.call("ref_dpt_forward", R.Raw(blas), ctypes.byref(model.dpt_c), feats[0], feats[1], feats[2], feats[3], outr, col, 1,
           model.dim, pH, pH, ps, lib=R.layers())
    torch.cuda.synchronize()
    R.cublas_destroy(blas)
    truth = TL.dpt_forward(feats, model.t, pH, pH, ps, model.dpt_out_channels)
    L.rfk_dpt_destroy(dpt)
    ctx.close()
    return out, outr, truth, n_conv


@pytest.mark.parametrize("dim,pH,features,channels", [(256, 16, 64, (32, 64, 128, 128)), (1024, 64, 256, (256, 512, 1024, 1024))])
def test_dpt_head_matches_reference_with_fp32_arbiter(dim, pH, features, channels):
    import torch_layers as TL
    _, session = _mods()
    model = session.Model.random(seed=3, dim=dim, num_heads=dim // 64, ffn_hidden=4 * dim, enc_layers=0, dec_layers=1,
                                 with_dpt=True, dpt_features=features, dpt_out_channels=channels)
    out, outr, truth, n_conv = _head(model, pH, 8, seed=dim)
    assert n_conv == 32                                                    # 4 + 3 + 4, 7 RCUs x 2, 4 fusion outputs, 3 in the output head
    assert torch.isfinite(out.float()).all() and torch.isfinite(outr.float()).all()
    (e_mean, e_max), (r_mean, r_max) = TL.err_stats(out, truth), TL.err_stats(outr, truth)
    d_mean, d_max = TL.err_stats(out, outr)
    print(f"DPT head dim {dim}, {pH * 8}^2: |image| mean {float(truth.abs().mean()):.3f}; vs fp32: rfk mean {e_mean:.3e} max {e_max:.3e} | "
          f"reference mean {r_mean:.3e} max {r_max:.3e} | rfk vs reference mean {d_mean:.3e} max {d_max:.3e}")
    assert e_mean <= 1.5 * r_mean + 1e-5 and e_max <= 1.5 * r_max + 1e-3
    assert d_mean <= 2.5 * r_mean + 1e-5 and d_max <= 2.5 * r_max + 1e-3


def test_session_with_dpt_head_renders_an_image_and_replays_it():
    """A session whose model carries a DPT head ends in the post-processed image [3, res, res] fp32 (ELU(1e-3), then
    10^x - 1): graph replay equals eager launches bit for bit, the image equals the head + post-process applied to the
    frame's own feature taps, and the token map is unchanged by the head's presence."""
    L, session = _mods()
    import cases
    model = session.Model.random(seed=4, dim=256, num_heads=4, ffn_hidden=1024, enc_layers=2, dec_layers=4, num_register_tokens=5,
                                 with_dpt=True, dpt_features=64, dpt_out_channels=(32, 64, 128, 128))
    g = torch.Generator(device="cuda").manual_seed(4)
    n_tris, res = 60, 128
    tri = (torch.rand(n_tris, 3, 3, device="cuda", generator=g) * 2 - 1).contiguous()
    vn = torch.nn.functional.normalize(torch.randn(n_tris, 3, 3, device="cuda", generator=g), dim=-1).contiguous()
    tex = torch.rand(n_tris, 13, device="cuda", generator=g).half().contiguous()
    c2w, fov = cases.look_at_c2w(np.random.default_rng(4), 2)
    imgs, toks = {}, {}
    for use_graph in (True, False):
        s = session.RenderSession(model, n_tris, res, use_graph=use_graph)
        s.encode_scene(tri, vn, tex); s.finalize()
        frames = []
        for v in range(2):
            s.render_frame(c2w[v], float(fov[v]))
            frames.append((s.download_image().clone(), s.download().clone()))
        imgs[use_graph], toks[use_graph] = [f[0] for f in frames], [f[1] for f in frames]
        if use_graph:
            # the head + post-process over the last frame's own taps, driven call by call
            taps = (VP * 4)()
            assert L.rfk_session_feature_taps(s.h, taps) == 0
            ctx = session.Ctx(); dpt = VP()
            assert L.rfk_dpt_create(ctx.h, ctypes.byref(model.dpt_c), 1, model.dim, res // 8, res // 8, 8, ctypes.byref(dpt)) == 0
            img16 = torch.empty(3, res, res, device="cuda", dtype=H16)
            st = VP(torch.cuda.current_stream().cuda_stream)
            assert L.rfk_dpt_forward(dpt, taps, VP(img16.data_ptr()), st) == 0
            torch.cuda.synchronize()
            x = img16.float()
            want = torch.pow(10.0, torch.where(x > 0, x, 1e-3 * torch.expm1(x))) - 1.0
            got = frames[1][0].cuda()
            assert torch.allclose(got, want, rtol=2e-3, atol=2e-3)
            L.rfk_dpt_destroy(dpt); ctx.close()
        s.close()
    for a, b in zip(imgs[True], imgs[False]):
        assert torch.isfinite(a).all() and torch.equal(a, b)
    assert not torch.equal(imgs[True][0], imgs[True][1])
    # the same model without the head gives the same token maps
    model.c.dpt = ctypes.POINTER(session.DptW)()
    s = session.RenderSession(model, n_tris, res)
    s.encode_scene(tri, vn, tex); s.finalize()
    s.render_frame(c2w[0], float(fov[0]))
    assert torch.equal(s.download(), toks[True][0])
    s.close()


# ---------------------------------------------------------------- channels-last companions (what the head runs on)

def _ops():
    import renderformer_cuda_b200 as pkg
    return pkg.ops


def _nhwc(t):   # [N, C, H, W] -> [N, H, W, C] contiguous
    return t.permute(0, 2, 3, 1).contiguous()


@pytest.mark.parametrize("bias,silu,res", [(True, False, False), (True, True, False), (True, False, True), (False, True, True),
                                           (False, False, True), (True, True, True)])
def test_fused_bias_activation_residual_equals_the_separate_operators(bias, silu, res):
    """One channels-last pass against add_bias_nchw -> silu_inplace -> residual_add on the same values: bit-identical,
    because every intermediate is still rounded to fp16."""
    o = _ops()
    g = torch.Generator(device="cuda").manual_seed(11)
    N, C, Hh, Ww = 2, 48, 9, 13
    x = torch.randn(N, C, Hh, Ww, device="cuda", generator=g).half()
    b = torch.randn(C, device="cuda", generator=g).half()
    r = torch.randn(N, C, Hh, Ww, device="cuda", generator=g).half()
    want = x.clone()
    if bias:
        o.add_bias_nchw(want, b, N, C, Hh * Ww)
    if silu:
        o.silu_inplace(want, want.numel())
    if res:
        o.residual_add(want, r, want.numel())
    got = _nhwc(x)
    o.bias_act_residual_nhwc(got, b if bias else None, _nhwc(r) if res else None, N * Hh * Ww, C, silu)
    torch.cuda.synchronize()
    assert torch.equal(got, _nhwc(want))


def test_out_of_place_silu_and_channels_last_upsample_equal_the_nchw_operators():
    o = _ops()
    g = torch.Generator(device="cuda").manual_seed(12)
    N, C, Hi, Wi, Ho, Wo = 2, 24, 7, 5, 16, 11
    x = torch.randn(N, C, Hi, Wi, device="cuda", generator=g).half()
    want = torch.empty(N, C, Ho, Wo, device="cuda", dtype=H16)
    o.bilinear_upsample(x, want, N, C, Hi, Wi, Ho, Wo)
    got = torch.empty(N, Ho, Wo, C, device="cuda", dtype=H16)
    o.bilinear_upsample_nhwc(_nhwc(x), got, N, Hi, Wi, Ho, Wo, C)
    y = torch.empty_like(x)
    o.silu(x, y, x.numel())
    x2 = x.clone()
    o.silu_inplace(x2, x2.numel())
    torch.cuda.synchronize()
    assert torch.equal(got, _nhwc(want))
    assert torch.equal(y, x2)
    # the same doubling as inside the head: 64 -> 128 at 256 channels
    big = torch.randn(1, 256, 64, 64, device="cuda", generator=g).half()
    w2 = torch.empty(1, 256, 128, 128, device="cuda", dtype=H16)
    o.bilinear_upsample(big, w2, 1, 256, 64, 64, 128, 128)
    g2 = torch.empty(1, 128, 128, 256, device="cuda", dtype=H16)
    o.bilinear_upsample_nhwc(_nhwc(big), g2, 1, 64, 64, 128, 128, 256)
    torch.cuda.synchronize()
    assert torch.equal(g2, _nhwc(w2))


@pytest.mark.parametrize("f,Cin,Cout", [(4, 32, 32), (2, 64, 40)])
def test_transposed_convolution_as_gemm_and_scatter(f, Cin, Cout):
    """kernel = stride transposed convolution = GEMM with the re-laid-out filter + depth-to-space (+ bias), against torch's
    conv_transpose2d in fp32 (tolerance: one fp16 rounding of the product plus one of the bias add)."""
    o = _ops()
    g = torch.Generator(device="cuda").manual_seed(f)
    N, Hh, Ww = 2, 6, 5
    x = torch.randn(N, Cin, Hh, Ww, device="cuda", generator=g).half()
    w = (torch.randn(Cin, Cout, f, f, device="cuda", generator=g) * Cin ** -0.5).half()
    b = torch.randn(Cout, device="cuda", generator=g).half()
    wg = torch.empty(f * f * Cout, Cin, device="cuda", dtype=H16)
    o.permute_filter(w, wg, Cin, Cout, f * f, 1)
    torch.cuda.synchronize()
    assert torch.equal(wg.view(f * f, Cout, Cin), w.permute(2, 3, 1, 0).reshape(f * f, Cout, Cin))
    xr = _nhwc(x).view(N * Hh * Ww, Cin)
    blocks = (xr.float() @ wg.float().t()).half()                      # the GEMM the head runs through rfk_linear
    got = torch.empty(N, Hh * f, Ww * f, Cout, device="cuda", dtype=H16)
    o.depth_to_space_bias_nhwc(blocks, b, got, N, Hh, Ww, Cout, f)
    torch.cuda.synchronize()
    want = torch.nn.functional.conv_transpose2d(x.float(), w.float(), b.float(), stride=f)
    err = (got.permute(0, 3, 1, 2).float() - want).abs()
    assert (err <= 2e-3 + 2.0 ** -9 * want.abs()).all(), err.max().item()


def test_filter_and_image_permutes_are_exact():
    o = _ops()
    g = torch.Generator(device="cuda").manual_seed(13)
    w = torch.randn(24, 16, 3, 3, device="cuda", generator=g).half()
    out = torch.empty(24, 3, 3, 16, device="cuda", dtype=H16)
    o.permute_filter(w, out, 24, 16, 9, 0)
    img = torch.randn(2, 10, 7, 3, device="cuda", generator=g).half()
    planar = torch.empty(2, 3, 10, 7, device="cuda", dtype=H16)
    o.permute_nhwc_to_nchw(img, planar, 2, 70, 3)
    torch.cuda.synchronize()
    assert torch.equal(out, w.permute(0, 2, 3, 1).contiguous())
    assert torch.equal(planar, img.permute(0, 3, 1, 2).contiguous())
    with pytest.raises(o.RfkError) as e:           # channel counts that are not multiples of 8 are refused, not mangled
        o.bias_act_residual_nhwc(torch.zeros(4, 12, device="cuda", dtype=H16), None, None, 4, 12, True)
    assert e.value.status == -2


@pytest.mark.parametrize("C_in,C_out", [(32, 3), (64, 1), (8, 4)])
def test_pointwise_convolution_to_planes(C_in, C_out):
    """The head's last layer as one kernel against fp32 torch: product rounded to fp16, then the bias (tolerance: those
    two roundings)."""
    o = _ops()
    g = torch.Generator(device="cuda").manual_seed(C_in)
    N, HW = 2, 1000
    x = torch.randn(N * HW, C_in, device="cuda", generator=g).half()
    w = (torch.randn(C_out, C_in, device="cuda", generator=g) * C_in ** -0.5).half()
    b = torch.randn(C_out, device="cuda", generator=g).half()
    out = torch.full((N, C_out, HW), 7.0, device="cuda", dtype=H16)
    o.pointwise_conv_to_planar(x, w, b, out, N, HW, C_in, C_out)
    torch.cuda.synchronize()
    want = ((x.float() @ w.float().t()).half().float() + b.float()).view(N, HW, C_out).permute(0, 2, 1)
    err = (out.float() - want).abs()
    assert (err <= 1e-3 + 2.0 ** -9 * want.abs()).all(), err.max().item()
    with pytest.raises(o.RfkError) as e:
        o.pointwise_conv_to_planar(x, w, b, out, N, HW, C_in, 5)
    assert e.value.status == -2
