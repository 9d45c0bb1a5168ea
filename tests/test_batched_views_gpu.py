"""GPU tests of frames of several views (rfk_session_create_batched / rfk_session_render_frames): the views of a
frame go through the decoder as one batch - their own cameras, geometry, rotary tables and rotated keys, shared values -
and must come out bit-identical to the same views rendered one at a time; through the scheduler too, including a view
count that does not fill the last frame."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mods():
    import renderformer_cuda_b200 as pkg  # noqa: F401
    from renderformer_cuda_b200 import session
    import cases
    return session, cases


def _scene(n_tris, seed=4):
    g = torch.Generator(device="cuda").manual_seed(seed)
    tri = (torch.rand(n_tris, 3, 3, device="cuda", generator=g) * 2 - 1).contiguous()
    vn = torch.nn.functional.normalize(torch.randn(n_tris, 3, 3, device="cuda", generator=g), dim=-1).contiguous()
    tex = torch.rand(n_tris, 13, device="cuda", generator=g).half().contiguous()
    return tri, vn, tex


@pytest.mark.parametrize("V,with_dpt", [(4, False), (3, True)])
def test_frame_of_views_equals_views_one_by_one(V, with_dpt):
    session, cases = _mods()
    model = session.Model.random(seed=4, dim=256, num_heads=4, ffn_hidden=1024, enc_layers=2, dec_layers=4, num_register_tokens=5,
                                 with_dpt=with_dpt, dpt_features=64, dpt_out_channels=(32, 64, 128, 128))
    n_tris, res = 60, 128
    tri, vn, tex = _scene(n_tris)
    c2w, fov = cases.look_at_c2w(np.random.default_rng(7), V)
    one = session.RenderSession(model, n_tris, res)
    one.encode_scene(tri, vn, tex); one.finalize()
    singles, images = [], []
    for v in range(V):
        one.render_frame(c2w[v], float(fov[v]))
        singles.append(one.download().clone())
        if with_dpt:
            images.append(one.download_image().clone())
    for use_graph in (True, False):
        many = session.RenderSession(model, n_tris, res, scene_state=one.scene_state, views_per_frame=V, use_graph=use_graph)
        many.finalize()
        assert many.views_per_frame == V
        with pytest.raises(session.RfkLayersError):
            many.render_frame(c2w[0], float(fov[0]))                    # a batched session takes its cameras V at a time
        many.render_frames(torch.as_tensor(np.asarray(c2w[:V], dtype=np.float32)), torch.as_tensor(np.asarray(fov[:V], dtype=np.float32)))
        got = many.download()
        assert got.shape == (V, one.n_tokens, model.dim)
        for v in range(V):
            assert torch.isfinite(got[v].float()).all()
            assert torch.equal(got[v], singles[v]), f"view {v} of the frame differs from the single render (graph={use_graph})"
        if with_dpt:
            img = many.download_image()
            for v in range(V):
                assert torch.equal(img[v], images[v]), f"image {v} differs (graph={use_graph})"
        # a second frame with the cameras in another order: no state leaks from frame to frame
        order = list(reversed(range(V)))
        many.render_frames(torch.as_tensor(np.asarray([c2w[i] for i in order], dtype=np.float32)),
                           torch.as_tensor(np.asarray([fov[i] for i in order], dtype=np.float32)))
        got2 = many.download()
        for k, i in enumerate(order):
            assert torch.equal(got2[k], singles[i])
        many.close()
    one.close()


def test_scheduler_with_frames_of_views_matches_the_single_view_scheduler():
    session, cases = _mods()
    model = session.Model.random(seed=5, dim=256, num_heads=4, ffn_hidden=1024, enc_layers=2, dec_layers=2, num_register_tokens=5)
    n_tris, res, n_views = 40, 128, 7                                  # 7 views in frames of 3: the last frame is padded
    tri, vn, tex = _scene(n_tris, seed=5)
    c2w, fov = cases.look_at_c2w(np.random.default_rng(9), n_views)
    c2w_t = torch.as_tensor(np.asarray(c2w, dtype=np.float32)); fov_t = torch.as_tensor(np.asarray(fov, dtype=np.float32))
    outs = []
    for V, streams in ((1, 1), (3, 2)):
        sched = session.ViewScheduler(model, n_tris, res, streams_per_gpu=streams, views_per_frame=V)
        sched.load_scene(tri, vn, tex)
        out = torch.zeros(n_views, (res // 8) ** 2, model.dim, dtype=torch.float16).pin_memory()
        assert sched.render(c2w_t, fov_t, out) == list(range(n_views))
        outs.append(out.clone())
        sched.close()
    assert torch.equal(outs[0], outs[1])


def test_batched_session_refuses_models_without_the_fused_route():
    session, _ = _mods()
    model = session.Model.random(seed=6, dim=384, num_heads=6, ffn_hidden=512, enc_layers=1, dec_layers=1)   # dim % 256 != 0
    with pytest.raises(session.RfkLayersError):
        session.RenderSession(model, 20, 128, views_per_frame=2)
    session.RenderSession(model, 20, 128).close()                      # one view per frame still works
