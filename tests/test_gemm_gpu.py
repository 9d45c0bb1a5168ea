"""GPU parity tests of rfk_gemm_f16, the tcgen05 / tensor-memory GEMM with fused epilogues, through
the C ABI: against an fp32 torch evaluation of the same product (tolerance: one fp16 rounding step of
the result, 2^-10 relative, plus 1e-3 absolute for cancellation near zero), against the reference's
rf::linear / rf::ffn_swiglu where oracle/_ref is present, and on ragged shapes (rows, columns and
K that are not multiples of the tile). The kernel's error word must stay clear."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
H16 = torch.float16


def _ops():
    import renderformer_cuda_b200 as pkg
    return pkg.ops


@pytest.fixture(autouse=True, params=[2, 3], ids=["cta_pair", "single_cta"])
def _error_word_clear(request):
    """Every test runs once through the CTA-pair kernel (tcgen05.mma.cta_group::2, the default) and once through
    the single-CTA kernel."""
    o = _ops()
    o.gemm_error(clear=True)
    o.gemm_set_path(request.param)
    yield
    o.gemm_set_path(0)
    torch.cuda.synchronize()
    assert o.gemm_error(clear=True) == 0, "the tcgen05 GEMM kernel reported a time-out"


def _close(got, want, what, rel=2.0 ** -10, atol=1e-3):
    got, want = got.float(), want.float()
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    err = (got - want).abs()
    bad = err > atol + rel * want.abs()
    assert not bad.any(), f"{what}: {int(bad.sum())}/{bad.numel()} outside tolerance, max err {err.max().item():.4g}"


def _rand(g, *shape, scale=1.0):
    return (torch.randn(*shape, device="cuda", generator=g) * scale).half()


SHAPES = [(128, 256, 64), (128, 256, 1024), (4096, 1024, 1024), (4096, 3072, 1024), (4096, 1024, 4096), (4096, 1024, 192),
          (5665, 1024, 1024), (300, 264, 200), (1, 8, 8), (77, 1000, 136), (257, 520, 72)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_plain_matches_fp32_product(M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a, w = _rand(g, M, K), _rand(g, N, K, scale=K ** -0.5)
    c = torch.full((M, N), 7.0, device="cuda", dtype=H16)
    _ops().gemm_f16(a, w, c, M, N, K)
    _close(c, a.float() @ w.float().t(), f"gemm {M}x{N}x{K}")


@pytest.mark.parametrize("M,N,K", [(4096, 1024, 4096), (300, 264, 200), (4096, 1024, 1024)])
def test_gemm_bias_and_residual_epilogues(M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a, w = _rand(g, M, K), _rand(g, N, K, scale=K ** -0.5)
    bias, r = _rand(g, N, scale=0.3), _rand(g, M, N)
    prod = a.float() @ w.float().t()
    c = torch.empty(M, N, device="cuda", dtype=H16)
    _ops().gemm_f16(a, w, c, M, N, K, bias=bias)
    _close(c, prod.half().float() + bias.float(), "gemm + bias", atol=2e-3)   # product rounded before the add, as the unfused pair
    _ops().gemm_f16(a, w, c, M, N, K, residual=r)
    _close(c, prod + r.float(), "gemm + residual", atol=2e-3)
    x = r.clone()                                                              # in place: C is R
    _ops().gemm_f16(a, w, x, M, N, K, residual=x)
    torch.cuda.synchronize()
    assert torch.equal(x, c)
    _ops().gemm_f16(a, w, c, M, N, K, bias=bias, residual=r)
    _close(c, prod.half().float() + bias.float() + r.float(), "gemm + bias + residual", atol=3e-3)


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 1024), (256, 1024, 256), (300, 136, 72), (5665, 4096, 1024)])
def test_gemm_swiglu_epilogue(M, N, K):
    """silu(a wg^T) * (a wu^T) with the gate and up weights in separate arrays and back to back."""
    g = torch.Generator(device="cuda").manual_seed(M + 2 * N + K)
    a = _rand(g, M, K)
    w13 = _rand(g, 2 * N, K, scale=K ** -0.5)
    wg, wu = w13[:N], w13[N:]
    want = torch.nn.functional.silu(a.float() @ wg.float().t()) * (a.float() @ wu.float().t())
    c = torch.full((M, N), 7.0, device="cuda", dtype=H16)
    _ops().gemm_f16(a, wg, c, M, N, K, w_up=wu)
    _close(c, want, "gemm + swiglu", atol=2e-3)
    c2 = torch.empty_like(c)
    _ops().gemm_f16(a, wg.clone(), c2, M, N, K, w_up=wu.clone())
    torch.cuda.synchronize()
    assert torch.equal(c, c2)


def test_gemm_strided_operands_and_repeatability():
    """Row pitches larger than the row (a column block of a wider matrix on every operand), and bit-identical
    results from launch to launch (tile order and accumulation order are fixed)."""
    g = torch.Generator(device="cuda").manual_seed(5)
    M, N, K = 513, 384, 320
    abig, wbig, cbig = _rand(g, M, K + 64), _rand(g, N, K + 8, scale=K ** -0.5), torch.zeros(M, N + 24, device="cuda", dtype=H16)
    a, w = abig[:, 64:], wbig[:, :K]
    L = __import__("renderformer_cuda_b200")._abi.load("rfk.h")
    VP = ctypes.c_void_p
    st = VP(torch.cuda.current_stream().cuda_stream)
    rc = L.rfk_gemm_f16(VP(abig.data_ptr() + 128), K + 64, VP(wbig.data_ptr()), K + 8, None, None, None, 0,
                        VP(cbig.data_ptr() + 16), N + 24, M, N, K, 0, st)
    assert rc == 0
    _close(cbig[:, 8:8 + N], a.float() @ w.float().t(), "strided gemm")
    assert bool((cbig[:, :8] == 0).all()) and bool((cbig[:, 8 + N:] == 0).all())
    first = cbig.clone()
    for _ in range(3):
        assert L.rfk_gemm_f16(VP(abig.data_ptr() + 128), K + 64, VP(wbig.data_ptr()), K + 8, None, None, None, 0,
                              VP(cbig.data_ptr() + 16), N + 24, M, N, K, 0, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(first, cbig)


def test_gemm_rejects_what_it_cannot_serve():
    L = __import__("renderformer_cuda_b200")._abi.load("rfk.h")
    VP = ctypes.c_void_p
    a = torch.zeros(64, 64, device="cuda", dtype=H16)
    p = VP(a.data_ptr())
    assert L.rfk_gemm_f16(p, 13, p, 13, None, None, None, 0, p, 64, 4, 64, 13, 0, None) == -2      # K % 8
    assert L.rfk_gemm_f16(p, 64, p, 64, None, None, None, 0, p, 60, 4, 60, 64, 0, None) == -2      # N % 8
    assert L.rfk_gemm_f16(VP(a.data_ptr() + 2), 64, p, 64, None, None, None, 0, p, 64, 4, 64, 56, 0, None) == -2
    assert L.rfk_gemm_f16(p, 64, p, 64, None, None, None, 0, p, 64, 4, 64, 64, 1, None) == -1      # residual epilogue without R
    assert L.rfk_gemm_f16(p, 64, p, 64, None, None, None, 0, p, 64, 4, 64, 64, 2, None) == -1      # SwiGLU without up weights
    assert L.rfk_gemm_f16(None, 64, p, 64, None, None, None, 0, p, 64, 4, 64, 64, 0, None) == -1
    _ops().gemm_set_path(1)
    assert L.rfk_gemm_f16(p, 64, p, 64, None, None, None, 0, p, 64, 4, 64, 64, 0, None) == -2      # switched off


def test_linear_and_ffn_through_both_gemm_paths_match_reference():
    """rfk_linear / rfk_ffn_swiglu with the tcgen05 kernel and with the library GEMM (path 1) against rf::linear and
    rf::ffn_swiglu at the decoder's FFN shape."""
    from oracle import ref as R
    if not (R.available() and R.layers_available()):
        pytest.skip("oracle/_ref libraries not present")
    from renderformer_cuda_b200 import _abi, session
    L = _abi.load("rfk_layers.h")
    VP = ctypes.c_void_p
    P = lambda t: VP(t.data_ptr())
    st = lambda: VP(torch.cuda.current_stream().cuda_stream)
    M, dim, ffn = 4096, 1024, 4096
    g = torch.Generator(device="cuda").manual_seed(12)
    x = _rand(g, M, dim)
    w13, w2 = _rand(g, 2 * ffn, dim, scale=0.02), _rand(g, dim, ffn, scale=0.02)
    bias = _rand(g, 2 * ffn, scale=0.1)
    ctx = session.Ctx()
    blas = R.cublas_create()
    yr = torch.empty(M, 2 * ffn, device="cuda", dtype=H16)
    R.call("ref_linear", R.Raw(blas), x, w13, bias, yr, M, 2 * ffn, dim, lib=R.layers())
    outr = torch.empty(M, dim, device="cuda", dtype=H16); bufr = torch.empty(M * 2 * ffn, device="cuda", dtype=H16)
    R.call("ref_ffn_swiglu", R.Raw(blas), R.Raw(w13.data_ptr()), R.Raw(w2.data_ptr()), R.Raw(w13.data_ptr() + ffn * dim * 2), x,
           outr, bufr, M, dim, ffn, lib=R.layers())
    truth = (torch.nn.functional.silu(x.float() @ w13[:ffn].float().t()) * (x.float() @ w13[ffn:].float().t())) @ w2.float().t()
    w = session.FfnW(w13.data_ptr(), w2.data_ptr(), w13.data_ptr() + ffn * dim * 2)
    errs = {}
    for path in (2, 1):
        _ops().gemm_set_path(path)   # (this test drives the path itself: tcgen05 on CTA pairs, then the library)
        y = torch.empty_like(yr)
        assert L.rfk_linear(ctx.h, P(x), P(w13), P(bias), P(y), M, 2 * ffn, dim, st()) == 0
        out = torch.empty_like(outr); buf = torch.empty_like(bufr)
        assert L.rfk_ffn_swiglu(ctx.h, ctypes.byref(w), P(x), P(out), P(buf), M, dim, ffn, st()) == 0
        torch.cuda.synchronize()
        if path == 1:
            assert torch.equal(y, yr)                       # same library call, same bias kernel semantics
        else:
            _close(y, yr, "linear + bias vs reference", atol=2e-3)
        errs[path] = float((out.float() - truth).abs().mean())
    err_ref = float((outr.float() - truth).abs().mean())
    print(f"ffn_swiglu mean |err| vs fp32: tcgen05 {errs[2]:.3e}, library path {errs[1]:.3e}, reference {err_ref:.3e}")
    assert errs[2] <= 1.2 * err_ref + 1e-6 and errs[1] <= 1.5 * err_ref + 1e-6
    R.cublas_destroy(blas)
    ctx.close()
