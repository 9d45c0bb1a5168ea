"""GPU tests of the file side: the pinned double-buffered upload of a safetensors data section, and a model that goes
out under the reference checkpoint's key names (src/model/renderformer.cpp:35-172), comes back through load_model
and renders the same frame."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mods():
    import renderformer_cuda_b200 as pkg
    from renderformer_cuda_b200 import session
    return pkg.assets, session


def test_upload_spans_several_staging_chunks(tmp_path):
    """100 MB of data: four 32 MB chunks through the two pinned buffers; every byte must arrive, at its offset,
    including a tensor whose offset is not a multiple of its element size."""
    A, _ = _mods()
    rng = np.random.default_rng(0)
    arrays = {"lead": rng.integers(0, 255, size=(3,)).astype(np.uint8),           # 3 bytes: misaligns what follows
              "big": rng.standard_normal((25, 1024, 1024)).astype(np.float32),
              "half": rng.standard_normal((1000, 77)).astype(np.float16),
              "tail": rng.integers(-9, 9, size=(5, 5)).astype(np.int64)}
    p = str(tmp_path / "big.safetensors")
    A.save_safetensors(p, arrays)
    with A.SafeTensors(p) as f:
        buf = f.to_device()
        assert buf.numel() == f.data_bytes == sum(v.nbytes for v in arrays.values())
        for k, v in arrays.items():
            got = f.tensor(k)
            assert tuple(got.shape) == v.shape
            assert np.array_equal(got.cpu().numpy(), v), k


def test_model_round_trip_through_checkpoint_names(tmp_path):
    A, session = _mods()
    kw = dict(dim=256, num_heads=4, ffn_hidden=512, enc_layers=2, dec_layers=2, with_dpt=True,
              dpt_features=32, dpt_out_channels=(32, 64, 128, 128), num_register_tokens=5)
    m = session.Model.random(seed=9, **kw)
    named = A.export_model(m)
    assert all(v.dtype == np.float32 for v in named.values())
    p = str(tmp_path / "model.safetensors")
    A.save_safetensors(p, named)
    m2 = A.load_model(p, num_heads=4)
    assert (m2.dim, m2.ffn_hidden, m2.enc_layers, m2.dec_layers, m2.num_register_tokens, m2.patch_size, m2.texture_channels,
            m2.vn_pe_num_freqs, m2.with_dpt, m2.dpt_features, m2.dpt_out_channels) == \
           (m.dim, m.ffn_hidden, m.enc_layers, m.dec_layers, m.num_register_tokens, m.patch_size, m.texture_channels,
            m.vn_pe_num_freqs, True, m.dpt_features, m.dpt_out_channels)
    assert set(m2.t) == set(m.t)
    for k, v in m.t.items():
        assert m2.t[k].dtype == v.dtype and m2.t[k].shape == v.shape and torch.equal(m2.t[k], v), k
    # and the same frame out of both
    import cases
    g = torch.Generator(device="cuda").manual_seed(1)
    n_tris, res = 60, 128
    tri = (torch.rand(n_tris, 3, 3, device="cuda", generator=g) * 2 - 1).contiguous()
    vn = torch.nn.functional.normalize(torch.randn(n_tris, 3, 3, device="cuda", generator=g), dim=-1).contiguous()
    tex = torch.rand(n_tris, 13, device="cuda", generator=g).half().contiguous()
    c2ws, fovs = cases.look_at_c2w(np.random.default_rng(1), 1)
    c2w, fov = c2ws[0], float(fovs[0])
    frames = []
    for model in (m, m2):
        s = session.RenderSession(model, n_tris, res)
        s.encode_scene(tri, vn, tex)
        s.finalize()
        s.render_frame(c2w, fov)
        frames.append((s.download().clone(), s.download_image().clone()))
        s.close()
    assert torch.isfinite(frames[0][0].float()).all() and torch.isfinite(frames[0][1]).all()
    assert torch.equal(frames[0][0], frames[1][0]), "token maps differ"
    d = (frames[0][1] - frames[1][1]).abs().max().item()
    assert d == 0.0, f"images differ by {d}"
    # the image goes out as EXR + PNG
    A.save_view(str(tmp_path / "view_0"), frames[0][1].cpu().numpy())
    assert (tmp_path / "view_0.exr").stat().st_size > 3 * res * res * 4 and (tmp_path / "view_0.png").stat().st_size > 100
