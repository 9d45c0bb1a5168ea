"""CPU tests of the file side (include/rfk_io.h through renderformer_cuda_b200.assets): the safetensors reader and
writer against the `safetensors` package's own files and against files broken on purpose, the PNG writer against
PIL's decoder, the EXR writer against a reader of the format written here from the specification, the tone-mapping
curve against its formula (src/io/image_writer.cpp:61-72 of the reference), and the scene container."""
import json
import struct

import numpy as np
import pytest


def _assets():
    import renderformer_cuda_b200 as pkg
    return pkg.assets


def _arrays(rng):
    return {
        "a.weight": rng.standard_normal((7, 5)).astype(np.float32),
        "b/half": rng.standard_normal((3, 4, 2)).astype(np.float16),
        "scalar": np.array(3.5, dtype=np.float64),
        "empty": np.zeros((0, 4), dtype=np.float32),
        "ints": rng.integers(-5, 5, size=(11,)).astype(np.int64),
        "bytes \"quoted\"": rng.integers(0, 255, size=(13,)).astype(np.uint8),
        "odd": rng.standard_normal((3,)).astype(np.float16),       # 6 bytes: what follows is not 4-byte aligned
        "after_odd": rng.standard_normal((2, 2)).astype(np.float32),
    }


def test_safetensors_round_trip_and_package_interop(tmp_path):
    A = _assets()
    rng = np.random.default_rng(1)
    arrays = _arrays(rng)
    mine = tmp_path / "mine.safetensors"
    A.save_safetensors(str(mine), arrays)
    with A.SafeTensors(str(mine)) as f:
        assert set(f.entries) == set(arrays)
        offsets = [f.entries[k][2] for k in f.entries]
        assert offsets == sorted(offsets)                           # entries come in file order
        for k, v in arrays.items():
            got = f.numpy(k)
            assert got.dtype == v.dtype and got.shape == v.shape and np.array_equal(got, v), k
        assert f.data_bytes == sum(v.nbytes for v in arrays.values())
        assert not f.has("nope")
        with pytest.raises(A.IoError) as e:
            f.numpy("nope")
        assert e.value.status == -12
    # a file of the package's writer (with metadata) read here, and this writer's file read by the package
    from safetensors.numpy import load_file, save_file
    theirs = tmp_path / "theirs.safetensors"
    plain = {k: v for k, v in arrays.items() if v.size}              # the package refuses nothing here, but keep it simple
    save_file(plain, str(theirs), metadata={"format": "pt", "note": "line\nbreak é"})
    with A.SafeTensors(str(theirs)) as f:
        assert f.metadata("format") == "pt" and f.metadata("note") == "line\nbreak é" and f.metadata("x") is None
        for k, v in plain.items():
            assert np.array_equal(f.numpy(k), v), k
    back = load_file(str(mine))
    for k, v in arrays.items():
        assert np.array_equal(back[k], v), k


def _file(tmp_path, header: dict | bytes, data: bytes = b"", name="x.safetensors", hlen=None):
    h = header if isinstance(header, bytes) else json.dumps(header).encode()
    p = tmp_path / name
    p.write_bytes(struct.pack("<Q", len(h) if hlen is None else hlen) + h + data)
    return str(p)


def test_safetensors_rejects_malformed_files(tmp_path):
    A = _assets()
    ok = {"t": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}
    with A.SafeTensors(_file(tmp_path, ok, b"\0" * 16)) as f:       # the well-formed baseline
        assert f.entries["t"] == (0, (2, 2), 0, 16)
    with A.SafeTensors(_file(tmp_path, {"t": {"data_offsets": [0, 16], "extra": {"a": [1, {"b": None}]}, "shape": [2, 2], "dtype": "F32"}},
                             b"\0" * 16)) as f:                      # field order is free, unknown fields are skipped
        assert f.entries["t"][1] == (2, 2)
    bad = [
        _file(tmp_path, ok, b"\0" * 15),                                                        # data section too short
        _file(tmp_path, {"t": {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 16]}}, b"\0" * 16),   # bytes != dtype x shape
        _file(tmp_path, {"t": {"dtype": "F33", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 16),      # unknown dtype
        _file(tmp_path, {"t": {"dtype": "F32", "shape": [4], "data_offsets": [16, 0]}}, b"\0" * 16),      # end before begin
        _file(tmp_path, {"t": {"dtype": "F32", "shape": [4]}}, b"\0" * 16),                               # no offsets
        _file(tmp_path, b'{"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}', b"\0" * 16),    # unterminated object
        _file(tmp_path, b'{"t": {"dtype": "F32", "shape": [-4], "data_offsets": [0, 16]}}', b"\0" * 16),  # negative extent
        _file(tmp_path, ok, b"", hlen=1 << 40),                                                           # header longer than the file
        _file(tmp_path, b'{"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}, "t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}', b"\0" * 16),
    ]
    for path in bad:
        with pytest.raises(A.IoError) as e:
            A.SafeTensors(path)
        assert e.value.status == -11, path
    short = tmp_path / "short.safetensors"
    short.write_bytes(b"\1\2\3")
    with pytest.raises(A.IoError) as e:
        A.SafeTensors(str(short))
    assert e.value.status == -11
    with pytest.raises(A.IoError) as e:
        A.SafeTensors(str(tmp_path / "does_not_exist.safetensors"))
    assert e.value.status == -10


@pytest.mark.parametrize("channels", [1, 2, 3, 4])
def test_png_decodes_to_the_same_pixels(tmp_path, channels):
    A = _assets()
    from PIL import Image
    rng = np.random.default_rng(channels)
    img = rng.integers(0, 256, size=(37, 53, channels), dtype=np.uint8)
    img[:8] = 200                                                    # a flat band, so the deflate stream has matches
    p = tmp_path / f"i{channels}.png"
    A.write_png(str(p), img)
    got = np.asarray(Image.open(str(p)))
    if got.ndim == 2:
        got = got[:, :, None]
    assert got.shape == img.shape and np.array_equal(got, img)
    assert p.stat().st_size < img.size + 200                        # compressed, not stored


def _read_exr(path):
    """Reader for the subset written by rfk_write_exr: version 2, single part, scan lines, no compression."""
    b = open(path, "rb").read()
    assert struct.unpack_from("<I", b, 0)[0] == 20000630 and struct.unpack_from("<I", b, 4)[0] == 2
    pos, attrs = 8, {}
    while b[pos] != 0:
        e = b.index(b"\0", pos); name = b[pos:e].decode(); pos = e + 1
        e = b.index(b"\0", pos); typ = b[pos:e].decode(); pos = e + 1
        n = struct.unpack_from("<i", b, pos)[0]; pos += 4
        attrs[name] = (typ, b[pos:pos + n]); pos += n
    pos += 1
    chans, v, q = [], attrs["channels"][1], 0
    while v[q] != 0:
        e = v.index(b"\0", q); nm = v[q:e].decode(); q = e + 1
        ptype, _plin, xs, ys = struct.unpack_from("<iB3xii", v, q); q += 16
        assert ptype == 2 and xs == 1 and ys == 1
        chans.append(nm)
    assert attrs["compression"] == ("compression", b"\0") and attrs["lineOrder"] == ("lineOrder", b"\0")
    x0, y0, x1, y1 = struct.unpack("<4i", attrs["dataWindow"][1])
    w, h = x1 - x0 + 1, y1 - y0 + 1
    assert attrs["displayWindow"][1] == attrs["dataWindow"][1]
    for need in ("pixelAspectRatio", "screenWindowCenter", "screenWindowWidth"):
        assert need in attrs
    offs = struct.unpack_from(f"<{h}Q", b, pos)
    planes = {c: np.empty((h, w), np.float32) for c in chans}
    for y in range(h):
        yy, n = struct.unpack_from("<ii", b, offs[y])
        assert yy == y and n == w * 4 * len(chans)
        for i, c in enumerate(chans):
            planes[c][y] = np.frombuffer(b, np.float32, w, offs[y] + 8 + i * w * 4)
    assert offs[-1] + 8 + w * 4 * len(chans) == len(b)
    return chans, planes


@pytest.mark.parametrize("channels", [1, 3, 4])
def test_exr_holds_the_same_floats(tmp_path, channels):
    A = _assets()
    rng = np.random.default_rng(10 + channels)
    img = (rng.standard_normal((19, 31, channels)) * 100).astype(np.float32)
    img[0, 0] = [np.float32(65504.0 * 4)] * channels               # beyond fp16: FLOAT channels must keep it
    p = tmp_path / f"i{channels}.exr"
    A.write_exr(str(p), img)
    chans, planes = _read_exr(str(p))
    assert chans == sorted(chans)                                   # the format wants channels in alphabetical order
    names = {1: "Y", 3: "RGB", 4: "RGBA"}[channels]
    assert sorted(names) == chans
    for i, c in enumerate(names):
        assert np.array_equal(planes[c], img[:, :, i]), c


def test_tonemap_is_the_reference_curve():
    A = _assets()
    rng = np.random.default_rng(3)
    hdr = np.concatenate([rng.standard_normal(4000).astype(np.float32) * 3, np.array([0, -1, 1e-8, 1, 1e6, np.inf], np.float32)])
    hdr = hdr[:4002].reshape(29, 46, 3)
    got = A.tonemap(hdr)
    v = np.maximum(hdr.astype(np.float64), 0)
    with np.errstate(invalid="ignore"):
        v = np.where(np.isinf(v), 1.0, v / (v + 1.0))
    want = np.clip(v ** (1 / 2.2) * 255.0, 0, 255)
    assert got.dtype == np.uint8 and got.shape == hdr.shape
    finite = np.isfinite(hdr)
    # truncation of a float32 evaluation against a float64 one: equal except where the value sits on an integer
    assert (np.abs(got[finite].astype(np.float64) - np.floor(want[finite])) <= 1).all()
    assert (got[finite] == np.floor(want[finite])).mean() > 0.99
    assert got[hdr <= 0].max() == 0


def test_scene_container_round_trip(tmp_path):
    A = _assets()
    rng = np.random.default_rng(5)
    n, k = 17, 3
    scene = dict(triangles=rng.standard_normal((n, 3, 3)).astype(np.float32), texture=rng.standard_normal((n, 13, 32, 32)).astype(np.float16),
                 vn=rng.standard_normal((n, 3, 3)).astype(np.float32), c2w=rng.standard_normal((k, 4, 4)).astype(np.float32),
                 fov=np.array([30, 45, 60], np.float32))
    p = str(tmp_path / "scene.safetensors")
    A.save_scene(p, **scene)
    back = A.load_scene(p)
    assert all(np.array_equal(back[key], scene[key]) for key in A.SCENE_KEYS)
    A.save_safetensors(p, {key: scene[key] for key in ("triangles", "vn")})
    with pytest.raises(A.IoError):
        A.load_scene(p)


def test_checkpoint_key_map_covers_the_reference_names():
    A = _assets()
    m = A.reference_key_map(12, 12, True)
    for key in ("tri_token", "texture_encoder_norm.weight", "transformer.rope_emb.freqs", "transformer.layers.11.multihead_attn.in_proj.weight",
                "transformer.layers.0.ffn.w3.weight", "view_transformer.ray_map_encoder.bias",
                "view_transformer.transformer.layers.7.self_attn.k_norm.weight", "view_transformer.transformer.layers.0.kv_norm.weight",
                "view_transformer.out_dpt.resize_layers.3.bias", "view_transformer.out_dpt.scratch.refinenet4.resConvUnit2.conv2.weight",
                "view_transformer.out_dpt.scratch.output_conv2.2.bias", "view_transformer.out_dpt.scratch.layer4_rn.weight"):
        assert key in m, key
    assert "view_transformer.out_dpt.resize_layers.2.weight" not in m                 # identity
    assert "view_transformer.out_dpt.scratch.refinenet4.resConvUnit1.conv1.weight" not in m   # the deepest block has no skip input
    # 14 top-level + 9 per encoder layer + 17 per decoder layer + the head: 4 projections (w, b), 4 layer_rn, 3 resize
    # (w, b), 4 out_conv (w, b), 7 residual units of 4 tensors, 3 output convolutions (w, b)
    assert len(m) == 14 + 12 * 9 + 12 * 17 + (4 * 2 + 4 + 3 * 2 + 4 * 2 + 7 * 4 + 3 * 2)
    targets = [v if isinstance(v, str) else v for v in m.values()]
    assert len(set(targets)) == len(targets)                                          # nothing mapped twice
