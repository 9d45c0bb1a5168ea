"""fp32 / fp64 torch evaluation of the view decoder's layers: the third party that arbitrates
between this library and the reference engine in the layer-level parity tests.

It computes the same function as rf::decoder_layer_forward_cached
(src/layers/transformer.cu:151-194 with cross_attention_cached, src/layers/attention.cu:326-373,
swin_self_attention, :476-576, and ffn_swiglu, transformer.cu:63-79) without any fp16
rounding between the steps: weights and inputs are the fp16 values widened, everything else
stays in `dtype`. Both fp16 pipelines are then measured against it, so that the layer
tolerance of the tests is a statement about both arms' distance from the exact result
instead of a number picked by hand. Test infrastructure only.
"""
from __future__ import annotations

import math

import torch

EPS = 2.0 ** -10   # kEpsFp16 of the reference (src/kernels/rmsnorm.h:9)


def rms(v, g, eps=EPS):
    return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * g


def rope_rotate(x, cos, sin):
    """HF rotate-half form (src/kernels/rope.cu:75-88); x [..., S, D], tables [S, D]."""
    h = x.shape[-1] // 2
    rot = torch.cat([-x[..., h:], x[..., :h]], dim=-1)
    return x * cos + rot * sin


def decoder_layer(x, w, K, V, k_cos, k_sin, mask, shift, heads, pH, pW, ws, dtype=torch.float32):
    """x [Sq, dim]; w: dict of this layer's weights (any float dtype); K, V [heads, Sk, hd] cached keys
    (unrotated) and values, every row takes part in the softmax (the reference attends its zero pad
    rows); k_cos/k_sin [Sk, hd]; mask [windows, ws*ws, ws*ws] bytes, used when shift > 0."""
    f = lambda t: t.to(dtype)
    x = f(x)
    Sq, dim = x.shape
    hd = dim // heads
    # 1) cached cross-attention
    t = rms(x, f(w["query_norm"]))
    q = rms(t @ f(w["q_proj_w"]).t(), f(w["cq_norm"])).view(Sq, heads, hd).permute(1, 0, 2)
    kr = rope_rotate(f(K), f(k_cos), f(k_sin))
    att = torch.softmax(q @ kr.transpose(-1, -2) / math.sqrt(hd), dim=-1)
    o = (att @ f(V)).permute(1, 0, 2).reshape(Sq, dim)
    x = x + o @ f(w["cross_out_w"]).t()
    # 2) shifted-window self-attention
    t = rms(x, f(w["self_attn_norm"])).view(pH, pW, dim)
    if shift:
        t = torch.roll(t, (shift, shift), (0, 1))              # out[h] = in[h - shift]: cyclic_shift_2d(-shift)
    nH, nW, ws2 = pH // ws, pW // ws, ws * ws
    win = t.view(nH, ws, nW, ws, dim).permute(0, 2, 1, 3, 4).reshape(nH * nW, ws2, dim)
    qkv = win @ f(w["swin_in_w"]).t()
    qw = rms(qkv[..., :dim], f(w["sq_norm"])).view(-1, ws2, heads, hd).permute(0, 2, 1, 3)
    kw = rms(qkv[..., dim:2 * dim], f(w["sk_norm"])).view(-1, ws2, heads, hd).permute(0, 2, 1, 3)
    vw = qkv[..., 2 * dim:].view(-1, ws2, heads, hd).permute(0, 2, 1, 3)
    s = qw @ kw.transpose(-1, -2) / math.sqrt(hd)
    if shift and mask is not None:
        s = torch.where(mask.bool()[:, None], s, torch.full_like(s, torch.finfo(torch.float32).min))
    o = (torch.softmax(s, dim=-1) @ vw).permute(0, 2, 1, 3).reshape(-1, ws2, dim) @ f(w["swin_out_w"]).t()
    o = o.view(nH, nW, ws, ws, dim).permute(0, 2, 1, 3, 4).reshape(pH, pW, dim)
    if shift:
        o = torch.roll(o, (-shift, -shift), (0, 1))
    x = x + o.reshape(Sq, dim)
    # 3) SwiGLU feed-forward
    t = rms(x, f(w["ffn_norm"]))
    gu = t @ f(w["w13"]).t()
    hidden = gu.shape[-1] // 2
    x = x + (torch.nn.functional.silu(gu[:, :hidden]) * gu[:, hidden:]) @ f(w["w2"]).t()
    return x


def layer_weights(model, i):
    t, p = model.t, f"dec{i}."
    return {k: t[p + k] for k in ("query_norm", "q_proj_w", "cq_norm", "cross_out_w", "self_attn_norm", "swin_in_w",
                                  "sq_norm", "sk_norm", "swin_out_w", "ffn_norm", "w13", "w2")}


def err_stats(a, truth):
    e = (a.double() - truth.double()).abs()
    return float(e.mean()), float(e.max())
