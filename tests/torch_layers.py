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


def dpt_forward(feats, t, pH, pW, ps, out_channels, dtype=torch.float32):
    """fp32 evaluation of the DPT image head (rf::dpt_forward, src/layers/dpt.cu:322-461): feats = four token maps
    [S, dim]; t = the model's weight dict ("dpt.*" entries of session.Model); returns [out_dim, pH*ps, pW*ps]."""
    import torch.nn.functional as F
    f = lambda k: t[k].to(dtype)
    has = lambda k: k in t
    up = lambda x, h, w: F.interpolate(x, size=(h, w), mode="bilinear", align_corners=True)
    resized = []
    for i in range(4):
        x = feats[i].to(dtype).t().reshape(1, -1, pH, pW)                    # [1, dim, pH, pW]
        x = F.conv2d(x, f(f"dpt.project{i}_w"), f(f"dpt.project{i}_b"))
        if i == 0:
            x = F.conv_transpose2d(x, f("dpt.resize0_w"), f("dpt.resize0_b"), stride=4)
        elif i == 1:
            x = F.conv_transpose2d(x, f("dpt.resize1_w"), f("dpt.resize1_b"), stride=2)
        elif i == 3:
            x = F.conv2d(x, f("dpt.resize3_w"), f("dpt.resize3_b"), stride=2, padding=1)
        resized.append(x)
    rn = [F.conv2d(resized[i], f(f"dpt.layer_rn{i}_w"), None, padding=1) for i in range(4)]

    def rcu(x, p):
        y = F.conv2d(F.silu(x), f(p + "conv1_w"), f(p + "conv1_b"), padding=1)
        return F.conv2d(F.silu(y), f(p + "conv2_w"), f(p + "conv2_b"), padding=1) + x

    def refine(i, path, lr, th, tw):
        if has(f"dpt.ref{i}.rcu1.conv1_w"):
            path = path + rcu(lr, f"dpt.ref{i}.rcu1.")
        path = rcu(path, f"dpt.ref{i}.rcu2.")
        return F.conv2d(up(path, th, tw), f(f"dpt.ref{i}.out_w"), f(f"dpt.ref{i}.out_b"))

    p4 = refine(3, rn[3], None, rn[2].shape[2], rn[2].shape[3])
    p3 = refine(2, p4, rn[2], rn[1].shape[2], rn[1].shape[3])
    p2 = refine(1, p3, rn[1], rn[0].shape[2], rn[0].shape[3])
    p1 = refine(0, p2, rn[0], rn[0].shape[2] * 2, rn[0].shape[3] * 2)
    x = F.conv2d(p1, f("dpt.out1_w"), f("dpt.out1_b"), padding=1)
    x = up(x, pH * ps, pW * ps)
    x = F.silu(F.conv2d(x, f("dpt.out2a_w"), f("dpt.out2a_b"), padding=1))
    return F.conv2d(x, f("dpt.out2b_w"), f("dpt.out2b_b"))[0]
