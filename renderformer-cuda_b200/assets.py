"""Files either side of the render path, bound to librfk_io.so (include/rfk_io.h): safetensors weights and
scenes in, EXR / PNG images out. Host-side mirror of the reference's src/io and of the key mapping of
src/model/renderformer.cpp (BANANASJIM/renderformer-cuda):

  SafeTensors            rf::SafeTensorsFile (src/io/safetensors.h:10-32): open, has / get, one bulk upload
  load_model             rf::RenderFormerModel::load (src/model/renderformer.cpp:35-172): the checkpoint's key names ->
                         the weight records of the session; matrices are cast to fp16 on the device (the reference
                         converts on the host, renderformer.cpp:15-33), norm weights and rotary frequencies stay fp32
  load_scene/save_scene  rf::Scene (src/io/hdf5_reader.h:9-26) as five named arrays in a safetensors file; the
                         reference's HDF5 reader has no counterpart here (no libhdf5 in this build)
  write_exr, write_png, tonemap, save_view
                         src/io/image_writer.h:8-15 and the tail of the render loop (src/pipeline/renderer.cu:36-40)

There is no fallback: if librfk_io.so is missing, loading raises.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np

from . import _abi

_NP = {0: np.float32, 1: np.float16, 3: np.float64, 4: np.int64, 5: np.int32, 6: np.int16, 7: np.int8, 8: np.uint8,
       9: np.bool_, 10: np.uint16, 11: np.uint32, 12: np.uint64}
_CODE = {np.dtype(v): k for k, v in _NP.items()}
DTYPE_BF16 = 2


class IoError(RuntimeError):
    def __init__(self, fn, rc):
        self.status = rc
        names = {-1: "invalid argument", -2: "unsupported", -10: "i/o error", -11: "malformed file", -12: "no such tensor"}
        super().__init__(f"{fn} failed with status {rc}: {names.get(rc, 'CUDA error' if rc > 0 else 'error')}")


def _lib():
    return _abi.load("rfk_io.h")


def _check(fn, rc):
    if rc != 0:
        raise IoError(fn, rc)


class TensorInfo(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("dtype", ctypes.c_int), ("ndim", ctypes.c_int),
                ("shape", ctypes.POINTER(ctypes.c_int64)), ("offset", ctypes.c_size_t), ("bytes", ctypes.c_size_t),
                ("host", ctypes.c_void_p)]


class SafeTensors:
    """A mapped safetensors file. `entries`: name -> (dtype code, shape tuple, offset, bytes), in file order."""

    def __init__(self, path: str):
        self.h = ctypes.c_void_p()
        _check("rfk_safetensors_open", _lib().rfk_safetensors_open(str(path).encode(), ctypes.byref(self.h)))
        self.entries: dict[str, tuple] = {}
        info = TensorInfo()
        for i in range(_lib().rfk_safetensors_count(self.h)):
            _check("rfk_safetensors_entry", _lib().rfk_safetensors_entry(self.h, i, ctypes.byref(info)))
            self.entries[info.name.decode()] = (info.dtype, tuple(info.shape[k] for k in range(info.ndim)), info.offset, info.bytes)
        self.data_bytes = int(_lib().rfk_safetensors_data_bytes(self.h))
        self._device = None

    def close(self):
        if self.h:
            _lib().rfk_safetensors_close(self.h)
            self.h = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def has(self, name: str) -> bool:
        return name in self.entries

    def metadata(self, key: str):
        v = _lib().rfk_safetensors_metadata(self.h, key.encode())
        return None if v is None else v.decode()

    def numpy(self, name: str) -> np.ndarray:
        """A host copy of one tensor (bf16 comes back as its raw uint16 words)."""
        info = TensorInfo()
        _check("rfk_safetensors_find", _lib().rfk_safetensors_find(self.h, name.encode(), ctypes.byref(info)))
        dt = np.uint16 if info.dtype == DTYPE_BF16 else _NP[info.dtype]
        shape = tuple(info.shape[k] for k in range(info.ndim))
        if info.bytes == 0:
            return np.zeros(shape, dtype=dt)
        raw = (ctypes.c_ubyte * info.bytes).from_address(info.host)
        return np.frombuffer(raw, dtype=dt).reshape(shape).copy()

    def to_device(self, device="cuda"):
        """One bulk upload of the data section (pinned double buffering inside the library); returns the uint8
        device tensor that `tensor()` slices."""
        import torch
        if self._device is None:
            buf = torch.empty(max(self.data_bytes, 1), dtype=torch.uint8, device=device)
            with torch.cuda.device(buf.device):
                _check("rfk_safetensors_upload", _lib().rfk_safetensors_upload(self.h, buf.data_ptr(), torch.cuda.current_stream().cuda_stream))
            self._device = buf
        return self._device

    def tensor(self, name: str):
        """The tensor as a view of the uploaded data section (a copy only if its offset is not a multiple of the
        element size, which the format allows)."""
        import torch
        tdt = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16, 3: torch.float64, 4: torch.int64, 5: torch.int32,
               6: torch.int16, 7: torch.int8, 8: torch.uint8, 9: torch.bool}
        code, shape, off, nbytes = self.entries[name]
        if code not in tdt:
            raise IoError("tensor", -2)
        raw = self.to_device()[off:off + nbytes]
        es = torch.empty(0, dtype=tdt[code]).element_size()
        if (raw.data_ptr() % es) != 0:
            raw = raw.clone()
        return raw.view(tdt[code]).reshape(shape)


def save_safetensors(path: str, arrays: dict[str, np.ndarray]) -> None:
    """Writes host arrays as a safetensors file (rfk_safetensors_write)."""
    names = list(arrays)
    n = len(names)
    arrs = [np.asarray(arrays[k], order="C") for k in names]   # (ascontiguousarray would turn a scalar into [1])
    c_names = (ctypes.c_char_p * n)(*[k.encode() for k in names])
    c_dt = (ctypes.c_int * n)(*[_CODE[a.dtype] for a in arrs])
    c_nd = (ctypes.c_int * n)(*[a.ndim for a in arrs])
    shapes = [(ctypes.c_int64 * max(a.ndim, 1))(*a.shape) for a in arrs]
    c_sh = (ctypes.c_void_p * n)(*[ctypes.cast(s, ctypes.c_void_p) for s in shapes])
    c_da = (ctypes.c_void_p * n)(*[a.ctypes.data for a in arrs])
    _check("rfk_safetensors_write", _lib().rfk_safetensors_write(str(path).encode(), n, ctypes.cast(c_names, ctypes.POINTER(ctypes.c_void_p)),
                                                                  c_dt, c_nd, c_sh, c_da))


# ------------------------------------------------------------------------------------- images

def write_exr(path: str, image_hwc: np.ndarray) -> None:
    a = np.ascontiguousarray(image_hwc, dtype=np.float32)
    if a.ndim == 2:
        a = a[:, :, None]
    h, w, c = a.shape
    _check("rfk_write_exr", _lib().rfk_write_exr(str(path).encode(), a.ctypes.data, w, h, c))


def write_png(path: str, image_hwc: np.ndarray) -> None:
    a = np.ascontiguousarray(image_hwc, dtype=np.uint8)
    if a.ndim == 2:
        a = a[:, :, None]
    h, w, c = a.shape
    _check("rfk_write_png", _lib().rfk_write_png(str(path).encode(), a.ctypes.data, w, h, c))


def tonemap(image_hwc: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(image_hwc, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint8)
    h, w = a.shape[0], a.shape[1]
    c = int(np.prod(a.shape[2:])) if a.ndim > 2 else 1
    _check("rfk_tonemap", _lib().rfk_tonemap(a.ctypes.data, out.ctypes.data, w, h, c))
    return out


def save_view(base: str, image_chw) -> None:
    """One rendered view [3, res, res] fp32 (host tensor or array) -> base.exr + base.png, as the reference's render loop
    does per camera (src/pipeline/renderer.cu:36-40)."""
    a = np.asarray(image_chw, dtype=np.float32)
    hwc = np.ascontiguousarray(a.transpose(1, 2, 0))
    write_exr(base + ".exr", hwc)
    write_png(base + ".png", tonemap(hwc))


# ------------------------------------------------------------------------------------- scene

SCENE_KEYS = ("triangles", "texture", "vn", "c2w", "fov")  # rf::Scene, src/io/hdf5_reader.h:10-15


def save_scene(path: str, triangles, texture, vn, c2w, fov) -> None:
    """triangles [N,3,3] fp32, texture [N,13,32,32] fp16, vn [N,3,3] fp32, c2w [K,4,4] fp32, fov [K] fp32 (degrees)."""
    save_safetensors(path, {"triangles": np.asarray(triangles, np.float32), "texture": np.asarray(texture, np.float16),
                            "vn": np.asarray(vn, np.float32), "c2w": np.asarray(c2w, np.float32), "fov": np.asarray(fov, np.float32)})


def load_scene(path: str) -> dict[str, np.ndarray]:
    with SafeTensors(path) as f:
        missing = [k for k in SCENE_KEYS if not f.has(k)]
        if missing:
            raise IoError(f"load_scene: missing {missing}", -11)
        s = {k: f.numpy(k) for k in SCENE_KEYS}
    n, k = s["triangles"].shape[0], s["c2w"].shape[0]
    if s["triangles"].shape != (n, 3, 3) or s["vn"].shape != (n, 3, 3) or s["texture"].shape[0] != n or s["c2w"].shape != (k, 4, 4) or s["fov"].shape != (k,):
        raise IoError("load_scene: shapes", -11)
    return s


# ------------------------------------------------------------------------------------- model

def reference_key_map(enc_layers: int, dec_layers: int, with_dpt: bool) -> dict[str, str | tuple]:
    """checkpoint key -> name in session.Model.t (a tuple for the two halves of the packed FFN matrix).
    Follows rf::RenderFormerModel::load, src/model/renderformer.cpp:35-172."""
    m: dict[str, str | tuple] = {
        "tri_token": "tri_token", "reg_tokens": "reg_tokens",
        "texture_encoder.weight": "tex_enc_w", "texture_encoder.bias": "tex_enc_b", "texture_encoder_norm.weight": "tex_enc_norm",
        "vn_encoding_proj.weight": "vn_proj_w", "vn_encoding_proj.bias": "vn_proj_b", "vn_encoder_norm.weight": "vn_enc_norm",
        "transformer.rope_emb.freqs": "enc_rope_freqs",
        "view_transformer.ray_map_patch_token": "ray_map_patch_token",
        "view_transformer.ray_map_encoder.weight": "ray_enc_w", "view_transformer.ray_map_encoder.bias": "ray_enc_b",
        "view_transformer.ray_map_encoder_norm.weight": "ray_enc_norm",
        "view_transformer.transformer.rope_emb.freqs": "vt_rope_freqs",
    }
    for i in range(enc_layers):
        p, q = f"transformer.layers.{i}.", f"enc{i}."
        m.update({p + "query_norm.weight": q + "query_norm", p + "ffn_norm.weight": q + "ffn_norm",
                  p + "multihead_attn.in_proj.weight": q + "in_proj_w", p + "multihead_attn.out_proj.weight": q + "out_proj_w",
                  p + "multihead_attn.q_norm.weight": q + "q_norm", p + "multihead_attn.k_norm.weight": q + "k_norm",
                  p + "ffn.w1.weight": (q + "w13", 0), p + "ffn.w3.weight": (q + "w13", 1), p + "ffn.w2.weight": q + "w2"})
    for i in range(dec_layers):
        p, q = f"view_transformer.transformer.layers.{i}.", f"dec{i}."
        m.update({p + "query_norm.weight": q + "query_norm", p + "kv_norm.weight": q + "kv_norm",
                  p + "multihead_attn.q_proj.weight": q + "q_proj_w", p + "multihead_attn.k_proj.weight": q + "k_proj_w",
                  p + "multihead_attn.v_proj.weight": q + "v_proj_w", p + "multihead_attn.out_proj.weight": q + "cross_out_w",
                  p + "multihead_attn.q_norm.weight": q + "cq_norm", p + "multihead_attn.k_norm.weight": q + "ck_norm",
                  p + "self_attn_norm.weight": q + "self_attn_norm",
                  p + "self_attn.in_proj.weight": q + "swin_in_w", p + "self_attn.out_proj.weight": q + "swin_out_w",
                  p + "self_attn.q_norm.weight": q + "sq_norm", p + "self_attn.k_norm.weight": q + "sk_norm",
                  p + "ffn_norm.weight": q + "ffn_norm",
                  p + "ffn.w1.weight": (q + "w13", 0), p + "ffn.w3.weight": (q + "w13", 1), p + "ffn.w2.weight": q + "w2"})
    if with_dpt:
        dp, sc = "view_transformer.out_dpt.", "view_transformer.out_dpt.scratch."
        for i in range(4):
            m[dp + f"projects.{i}.weight"], m[dp + f"projects.{i}.bias"] = f"dpt.project{i}_w", f"dpt.project{i}_b"
            m[sc + f"layer{i + 1}_rn.weight"] = f"dpt.layer_rn{i}_w"
            rn = sc + f"refinenet{i + 1}."
            m[rn + "out_conv.weight"], m[rn + "out_conv.bias"] = f"dpt.ref{i}.out_w", f"dpt.ref{i}.out_b"
            for u, v in (("resConvUnit1.", "rcu1"), ("resConvUnit2.", "rcu2")):
                if v == "rcu1" and i == 3:
                    continue
                for c in ("conv1", "conv2"):
                    m[rn + u + c + ".weight"], m[rn + u + c + ".bias"] = f"dpt.ref{i}.{v}.{c}_w", f"dpt.ref{i}.{v}.{c}_b"
        for i in (0, 1, 3):   # resize layer 2 is the identity
            m[dp + f"resize_layers.{i}.weight"], m[dp + f"resize_layers.{i}.bias"] = f"dpt.resize{i}_w", f"dpt.resize{i}_b"
        m[sc + "output_conv1.weight"], m[sc + "output_conv1.bias"] = "dpt.out1_w", "dpt.out1_b"
        m[sc + "output_conv2.0.weight"], m[sc + "output_conv2.0.bias"] = "dpt.out2a_w", "dpt.out2a_b"
        m[sc + "output_conv2.2.weight"], m[sc + "output_conv2.2.bias"] = "dpt.out2b_w", "dpt.out2b_b"
    return m


def _keeps_fp32(internal: str) -> bool:
    """Norm weights and rotary frequencies stay fp32 (the reference's f(...)), everything else becomes fp16 (its h(...))."""
    leaf = internal.split(".")[-1]
    return leaf.endswith("_norm") or leaf.endswith("rope_freqs")


def load_model(path: str, num_heads: int, device="cuda", window_size=8, shift_size=4):
    """Builds a session.Model from a checkpoint in the reference's key layout. Everything but the head count and the
    window geometry is read off the tensors' shapes."""
    import torch
    from . import ops, session
    with SafeTensors(path) as f:
        names = set(f.entries)
        enc_layers = 1 + max((int(k.split(".")[2]) for k in names if k.startswith("transformer.layers.")), default=-1)
        dec_layers = 1 + max((int(k.split(".")[3]) for k in names if k.startswith("view_transformer.transformer.layers.")), default=-1)
        with_dpt = any(k.startswith("view_transformer.out_dpt.") for k in names)
        shape = lambda k: f.entries[k][1]
        dim = int(np.prod(shape("tri_token")))
        ray_in = shape("view_transformer.ray_map_encoder.weight")[1]
        vn_in = shape("vn_encoding_proj.weight")[1]
        kw = dict(dim=dim, num_heads=num_heads, ffn_hidden=shape("transformer.layers.0.ffn.w1.weight")[0],
                  num_register_tokens=shape("reg_tokens")[-2] if len(shape("reg_tokens")) > 1 else 1,
                  enc_layers=enc_layers, dec_layers=dec_layers, patch_size=int(round(math.sqrt(ray_in / 3))),
                  window_size=window_size, shift_size=shift_size, texture_channels=shape("texture_encoder.weight")[1],
                  vn_pe_num_freqs=(vn_in - 9) // 18, device=device, with_dpt=with_dpt)
        if with_dpt:
            oc = tuple(shape(f"view_transformer.out_dpt.projects.{i}.weight")[0] for i in range(4))
            kw.update(dpt_out_channels=oc, dpt_features=shape("view_transformer.out_dpt.scratch.layer1_rn.weight")[0],
                      dpt_out_dim=shape("view_transformer.out_dpt.scratch.output_conv2.2.weight")[0])
        m = session.Model(**kw)
        keymap = reference_key_map(enc_layers, dec_layers, with_dpt)
        missing = [k for k in keymap if k not in names]
        if missing:
            raise IoError(f"load_model: checkpoint lacks {missing[:4]}{'...' if len(missing) > 4 else ''}", -12)
        f.to_device(device)

        def fetch(key, internal):
            src = f.tensor(key)
            want = torch.float32 if _keeps_fp32(internal) else torch.float16
            if src.dtype == want:
                return src.clone()        # own storage: the upload buffer is released below
            if src.dtype == torch.float32 and want == torch.float16:
                out = torch.empty(src.shape, dtype=torch.float16, device=src.device)
                ops.cast_fp32_to_fp16(src.contiguous(), out, src.numel())   # on the device; the reference converts on the host
                return out
            return src.to(want)

        packed: dict[str, list] = {}
        for key, internal in keymap.items():
            if isinstance(internal, tuple):
                packed.setdefault(internal[0], [None, None])[internal[1]] = fetch(key, internal[0])
            else:
                m.t[internal] = fetch(key, internal).reshape(-1) if internal in ("tri_token", "ray_map_patch_token") else fetch(key, internal)
        for internal, (w1, w3) in packed.items():
            m.t[internal] = torch.cat([w1, w3], dim=0).contiguous()   # w1 and w3 back to back: one GEMM operand pair
        if "reg_tokens" in m.t:
            m.t["reg_tokens"] = m.t["reg_tokens"].reshape(-1, dim).contiguous()
        f._device = None
    nf = m.rope_num_freqs
    for k in ("enc_rope_freqs", "vt_rope_freqs"):
        if m.t[k].numel() != nf:
            raise IoError(f"load_model: {k} has {m.t[k].numel()} frequencies, head size {m.head_dim} takes {nf}", -11)
    m._fill_record()
    return m


def export_model(model) -> dict[str, np.ndarray]:
    """The inverse of load_model: a session.Model's tensors under the checkpoint's key names (host arrays, matrices as
    fp32 like the published checkpoint). For round trips and for handing random-init weights to the reference."""
    out: dict[str, np.ndarray] = {}
    ffn = model.ffn_hidden
    for key, internal in reference_key_map(model.enc_layers, model.dec_layers, model.with_dpt).items():
        if isinstance(internal, tuple):
            t = model.t[internal[0]][internal[1] * ffn:(internal[1] + 1) * ffn]
        else:
            t = model.t[internal]
        out[key] = t.detach().float().cpu().numpy()
    return out
