"""GPU parity tests of the deferred QK-RMSNorm chain through the C ABI: the projection that stores its output
head-split together with the rows' sums of squares (rfk_gemm_f16_heads), the key rotation that folds the query
norm's weight into the keys (col_scale of rfk_rope_one_oop_strided), and the two attention kernels that apply the
row statistic (rfk_flash_attention_ex, rfk_window_attention_normed). Each is checked against a torch fp32
evaluation of the unfused sequence it replaces (linear -> rmsnorm -> head split -> attention,
src/layers/attention.cu:336-366 and :511-566 of the reference), with the tolerance of the corresponding unfused
kernel's own test."""

import pytest
import torch

pytestmark = pytest.mark.gpu
H16 = torch.float16
EPS = 2.0 ** -10


def _ops():
    import renderformer_cuda_b200 as pkg
    return pkg.ops


@pytest.fixture(autouse=True)
def _error_words_clear():
    o = _ops()
    o.gemm_error(clear=True)
    o.flash_attention_error(clear=True)
    yield
    torch.cuda.synchronize()
    assert o.gemm_error(clear=True) == 0, "the tcgen05 GEMM kernel reported a time-out"
    assert o.flash_attention_error(clear=True) == 0, "the tcgen05 attention kernel reported a time-out"


def _rand(g, *shape, scale=1.0):
    return (torch.randn(*shape, device="cuda", generator=g) * scale).half()


def _close(got, want, what, atol, rtol, mean_tol=None):
    got, want = got.float(), want.float()
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    err = (got - want).abs()
    bad = err > atol + rtol * want.abs()
    assert not bad.any(), f"{what}: {int(bad.sum())}/{bad.numel()} outside tolerance, max err {err.max().item():.4g}"
    if mean_tol is not None:
        assert err.mean().item() < mean_tol, f"{what}: mean err {err.mean().item():.4g}"


def _head_split(c, groups, seq, heads):
    """[groups * seq, heads * 64] -> [groups, heads, seq, 64]"""
    return c.view(groups, seq, heads, 64).permute(0, 2, 1, 3).contiguous()


@pytest.mark.parametrize("M,seq,heads,parts,K,mask", [
    (2304, 2304, 12, 1, 768, 1),      # query projection of the view decoder (config 5)
    (2304, 64, 12, 3, 768, 3),        # packed q | k | v of its window attention
    (4096, 4096, 16, 1, 1024, 1),     # query projection at 512 x 512
    (4096, 64, 16, 3, 1024, 3),
    (64, 32, 4, 1, 64, 1),            # one tile, two groups
    (192, 64, 4, 3, 72, 2),           # statistics of the middle part only, K not a multiple of the K block
    (320, 64, 8, 3, 256, 0),          # no statistics at all
])
def test_heads_projection_equals_plain_projection_head_split(M, seq, heads, parts, K, mask):
    """The head-split store is a permutation of the plain kernel's output (bit-exact: same accumulation, same one
    rounding), and the statistic is the sum of squares of those rounded values per 256 columns (fp32, rel 1e-5)."""
    o = _ops()
    dim = heads * 64
    N = parts * dim
    g = torch.Generator(device="cuda").manual_seed(M + 13 * K + parts)
    a, w = _rand(g, M, K), _rand(g, N, K, scale=K ** -0.5)
    plain = torch.empty(M, N, device="cuda", dtype=H16)
    o.gemm_f16(a, w, plain, M, N, K)
    out = torch.full((parts, M * dim), 7.0, device="cuda", dtype=H16)
    tiles = dim // 256
    ss = torch.full((parts, M, tiles), -1.0, device="cuda", dtype=torch.float32)
    o.gemm_f16_heads(a, w, out, ss if mask else None, mask, M, N, K, seq, heads, part_stride=M * dim)
    torch.cuda.synchronize()
    groups = M // seq
    for p in range(parts):
        want = _head_split(plain[:, p * dim:(p + 1) * dim].contiguous(), groups, seq, heads)
        assert torch.equal(out[p].view(groups, heads, seq, 64), want), f"part {p}: head-split output differs"
        if mask >> p & 1:
            want_ss = plain[:, p * dim:(p + 1) * dim].float().pow(2).view(M, tiles, 256).sum(-1)
            assert torch.allclose(ss[p], want_ss, rtol=1e-5, atol=1e-6), f"part {p}: row statistics differ"
        else:
            assert (ss[p] == -1.0).all(), f"part {p}: statistics written although not asked for"


def test_heads_projection_refuses_shapes_it_cannot_tile():
    o = _ops()
    a = torch.zeros(96, 64, device="cuda", dtype=H16)
    w = torch.zeros(192, 64, device="cuda", dtype=H16)
    out = torch.zeros(96 * 192, device="cuda", dtype=H16)
    ss = torch.zeros(96, 1, device="cuda", dtype=torch.float32)
    with pytest.raises(o.RfkError) as e:      # three heads: a 256-column tile would straddle parts
        o.gemm_f16_heads(a, w, out, ss, 1, 96, 192, 64, 32, 3)
    assert e.value.status == -2
    w4 = torch.zeros(256, 64, device="cuda", dtype=H16)
    out4 = torch.zeros(96 * 256, device="cuda", dtype=H16)
    with pytest.raises(o.RfkError) as e:      # sequence length not a multiple of 32
        o.gemm_f16_heads(a, w4, out4, ss, 1, 96, 256, 64, 48, 4)
    assert e.value.status == -2
    with pytest.raises(o.RfkError) as e:      # statistics asked for without a buffer
        o.gemm_f16_heads(a, w4, out4, None, 1, 96, 256, 64, 32, 4)
    assert e.value.status == -1


@pytest.mark.parametrize("layers,heads,rows,pad", [(1, 12, 1537, 1600), (3, 4, 200, 256), (11, 6, 64, 64)])
def test_rotation_with_folded_norm_weight(layers, heads, rows, pad):
    """dst[l] = half(rotate(src[l]) * gamma[l]) with one shared table: fp32 torch evaluation, half an fp16 step of
    slack for the fused multiply-add order."""
    o = _ops()
    hd = 64
    g = torch.Generator(device="cuda").manual_seed(layers * 100 + rows)
    src = _rand(g, layers, 2, heads, pad, hd)                       # [layer][K|V][heads][rows][hd]: the key slabs
    ang = torch.rand(pad, hd // 2, device="cuda", generator=g) * 6.28
    cos = torch.cat([ang.cos(), ang.cos()], -1).half()
    sin = torch.cat([ang.sin(), ang.sin()], -1).half()
    gamma = (torch.rand(layers, heads * hd, device="cuda", generator=g) + 0.5).float()
    dst = torch.full((layers, heads, pad, hd), 7.0, device="cuda", dtype=H16)
    slab = heads * pad * hd
    o.rope_one_oop_strided(src, dst, cos, sin, layers, 2 * slab, slab, 0, heads, rows, hd, pad, pad, gamma, heads * hd)
    torch.cuda.synchronize()
    x = src[:, 0, :, :rows].float()
    rot = torch.cat([-x[..., hd // 2:], x[..., :hd // 2]], -1)
    want = (x * cos[:rows].float() + rot * sin[:rows].float()) * gamma.view(layers, heads, 1, hd)
    _close(dst[:, :, :rows], want, "scaled rotation", atol=1e-4, rtol=2.0 ** -10)
    assert (dst[:, :, rows:] == 7.0).all(), "rows beyond seq_len were written"
    # without the factor the same entry point equals the plain rotation kernel
    plain = torch.empty_like(dst)
    o.rope_one_oop_strided(src, plain, cos, sin, layers, 2 * slab, slab, 0, heads, rows, hd, pad, pad)
    ref = torch.empty(heads, pad, hd, device="cuda", dtype=H16)
    o.rope_one_oop(src[layers - 1, 0].contiguous(), ref, cos, sin, 1, heads, rows, hd, pad, pad)
    torch.cuda.synchronize()
    assert torch.equal(plain[layers - 1, :, :rows], ref[:, :rows])


@pytest.mark.parametrize("B,Hh,Sq,Sk,n_keys", [(1, 12, 2304, 1600, 1537), (2, 4, 96, 200, 193), (1, 8, 4096, 4096, 4096),
                                               (1, 4, 32, 64, 5)])
def test_rowscale_attention_equals_attention_over_normalised_queries(B, Hh, Sq, Sk, n_keys):
    """projection -> statistics -> attention with row scale and weight-carrying keys, against fp32 torch attention
    over rmsnorm(q) * gamma. Tolerance of the flash attention test (4e-3 abs + 4e-3 rel, mean 5e-4)."""
    o = _ops()
    D, dim = 64, Hh * 64
    g = torch.Generator(device="cuda").manual_seed(Sq + Sk)
    a, w = _rand(g, B * Sq, dim), _rand(g, dim, dim, scale=dim ** -0.5)
    gamma = (torch.rand(dim, device="cuda", generator=g) + 0.5).float()
    K = _rand(g, B, Hh, Sk, D)
    V = _rand(g, B, Hh, Sk, D)
    q = torch.empty(B, Hh, Sq, D, device="cuda", dtype=H16)
    tiles = dim // 256
    ss = torch.empty(B * Sq, tiles, device="cuda", dtype=torch.float32)
    o.gemm_f16_heads(a, w, q, ss, 1, B * Sq, dim, dim, Sq, Hh)
    Kg = (K.float() * gamma.view(1, Hh, 1, D)).half()              # what the rotation kernel's col_scale produces
    O = torch.full((B, Sq, dim), 7.0, device="cuda", dtype=H16)
    o.flash_attention_ex(q, Kg, V, O, B, Hh, Sq, Sk, n_keys, D, q_row_ss=ss, ss_tiles=tiles, norm_dim=dim, o_bshd=True)
    torch.cuda.synchronize()
    proj = (a.float() @ w.float().t()).half().float()              # the projection's one rounding, as the reference has it
    qn = proj * torch.rsqrt(proj.pow(2).mean(-1, keepdim=True) + EPS) * gamma
    qn = qn.view(B, Sq, Hh, D).permute(0, 2, 1, 3)
    want = torch.nn.functional.scaled_dot_product_attention(qn, K[:, :, :n_keys].float(), V[:, :, :n_keys].float())
    _close(O.view(B, Sq, Hh, D).permute(0, 2, 1, 3), want, "row-scaled attention", atol=4e-3, rtol=4e-3, mean_tol=5e-4)


@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("BnW,Hh,nW", [(36, 12, 36), (8, 4, 4)])
def test_normed_window_attention_equals_norm_then_window_attention(masked, BnW, Hh, nW):
    """packed projection -> statistics -> window attention that normalises while staging, against the separate
    sequence on the same projection: rmsnorm (torch, the norm kernel's formula half((x * inv) * gamma)) -> plain
    window attention kernel. The two differ only by the last bit of inv, so almost every output is identical and
    the rest is within the window attention test's tolerance."""
    o = _ops()
    dim, M = Hh * 64, BnW * 64
    g = torch.Generator(device="cuda").manual_seed(BnW + Hh)
    a, w = _rand(g, M, dim), _rand(g, 3 * dim, dim, scale=dim ** -0.5)
    gq = (torch.rand(dim, device="cuda", generator=g) + 0.5).float()
    gk = (torch.rand(dim, device="cuda", generator=g) + 0.5).float()
    mask = (torch.rand(nW, 64, 64, device="cuda", generator=g) > 0.3).to(torch.uint8) if masked else None
    tiles = dim // 256
    qkv = torch.empty(3, BnW, Hh, 64, 64, device="cuda", dtype=H16)
    ss = torch.empty(2, M, tiles, device="cuda", dtype=torch.float32)
    o.gemm_f16_heads(a, w, qkv, ss, 3, M, 3 * dim, dim, 64, Hh, part_stride=M * dim)
    O = torch.full((M, dim), 7.0, device="cuda", dtype=H16)
    o.window_attention_normed(qkv[0], qkv[1], qkv[2], O, mask, ss[0], ss[1], tiles, gq, gk, dim, BnW, Hh, nW)
    torch.cuda.synchronize()

    def normed(x, gamma):                                           # x [BnW, Hh, 64, 64] -> token rows -> norm -> back
        rows = x.permute(0, 2, 1, 3).reshape(M, dim).float()
        inv = torch.rsqrt(rows.pow(2).mean(-1, keepdim=True) + EPS)
        y = ((rows * inv) * gamma).half()
        return y.view(BnW, 64, Hh, 64).permute(0, 2, 1, 3).contiguous()

    O2 = torch.empty_like(O)
    o.window_attention(normed(qkv[0], gq), normed(qkv[1], gk), qkv[2].contiguous(), O2, mask, BnW, Hh, nW)
    torch.cuda.synchronize()
    same = (O == O2).float().mean().item()
    assert same > 0.98, f"only {same:.3f} of the outputs are identical to the separate sequence"
    _close(O, O2, "normed window attention", atol=3e-3, rtol=3e-3, mean_tol=3e-5)


@pytest.mark.parametrize("B,Hh,Sq,Sk,n_keys,cut", [
    (1, 16, 1024, 5696, 5672, True),     # a 256 x 256 view: 64 units for 148 SMs, every unit cut
    (2, 3, 300, 2048, 2001, True),       # 12 ragged units, many pieces per unit
    (1, 1, 77, 4096, 4096, True),        # one unit: eight pieces (the merge is serial in one CTA, so pieces per unit are capped)
    (1, 16, 4096, 5696, 5672, False),    # the 512 x 512 view fills the SMs: left whole
    (1, 12, 2304, 1600, 1537, False),    # 108 short units: the pieces' overhead would eat the gain
    (1, 4, 256, 64, 33, False),          # one tile per unit: nothing to cut
])
def test_key_split_equals_unsplit_attention(B, Hh, Sq, Sk, n_keys, cut):
    """The key split changes the schedule, not the function. Where the launcher cuts, the outputs differ from the
    unsplit kernel's by the fp32 merge and by the probabilities' fp16 rounding relative to each piece's own running
    maximum (a few fp16 steps at most where the output is a small difference, less than one on average), the fp32 torch
    attention is met with the flash attention test's tolerance, the unit counters are back to zero, and a second launch
    on the same workspace gives the same bits as the first. Where it does not cut, the workspace changes nothing."""
    o = _ops()
    D = 64
    g = torch.Generator(device="cuda").manual_seed(Sq * 3 + Sk)
    Q = _rand(g, B, Hh, Sq, D)
    K = _rand(g, B, Hh, Sk, D)
    V = _rand(g, B, Hh, Sk, D)
    ws = o.flash_attention_workspace()
    whole = torch.full((B, Sq, Hh * D), 7.0, device="cuda", dtype=H16)
    split = torch.full_like(whole, 7.0)
    again = torch.full_like(whole, 7.0)
    o.flash_attention_ex(Q, K, V, whole, B, Hh, Sq, Sk, n_keys, D, o_bshd=True)
    o.flash_attention_ex(Q, K, V, split, B, Hh, Sq, Sk, n_keys, D, workspace=ws, o_bshd=True)
    torch.cuda.synchronize()
    assert int(ws[:1024].view(torch.int32).abs().sum()) == 0, "unit counters not returned to zero"
    o.flash_attention_ex(Q, K, V, again, B, Hh, Sq, Sk, n_keys, D, workspace=ws, o_bshd=True)
    torch.cuda.synchronize()
    want = torch.nn.functional.scaled_dot_product_attention(Q.float(), K[:, :, :n_keys].float(), V[:, :, :n_keys].float())
    _close(split.view(B, Sq, Hh, D).permute(0, 2, 1, 3), want, "split attention", atol=4e-3, rtol=4e-3, mean_tol=5e-4)
    if not cut:
        assert torch.equal(split, whole)
    else:
        assert not torch.equal(split, whole), "expected the launcher to cut this grid"
        d = (split.float() - whole.float()).abs()
        assert (d <= 2.0 ** -9 * whole.float().abs() + 2e-4).all(), f"split and unsplit outputs apart: {d.max().item():.3g}"
        assert d.mean().item() < 2.0 ** -10 * whole.float().abs().mean().item(), "on average more than one fp16 step apart"
    # which CTA merges depends on timing, the order of the merge's additions does not
    assert torch.equal(again, split), "second launch on the same workspace differs"
    o.flash_attention_set_split(False)
    try:
        off = torch.full_like(whole, 7.0)
        o.flash_attention_ex(Q, K, V, off, B, Hh, Sq, Sk, n_keys, D, workspace=ws, o_bshd=True)
        torch.cuda.synchronize()
        assert torch.equal(off, whole)
    finally:
        o.flash_attention_set_split(True)
