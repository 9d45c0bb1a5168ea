"""GPU test of rfk_sdpa_static, the attention entry point for callers that cannot allocate
device memory (stream-capture code, stream callbacks, hosts with a fixed memory budget): its
score matrix lives in a fixed 32 MiB array inside the library. Called through the C ABI, twice
in a row with different inputs, it must give the same result as rfk_sdpa with a caller-supplied
workspace (the arithmetic is the same launch sequence, so the match is bit for bit), must leave
the allocator untouched, and must reject shapes that do not fit. The file name sorts last so
that a run stopping at the first failure has already executed every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
VP = ctypes.c_void_p


def _p(t):
    return VP(t.data_ptr())


def _stream():
    return VP(torch.cuda.current_stream().cuda_stream)


def test_static_scratch_sdpa_matches_workspace_sdpa_on_two_calls():
    from renderformer_cuda_b200 import _abi, session
    L = _abi.load("rfk_layers.h")
    ctx = session.Ctx()
    B, H, Sq, Sk, D = 1, 4, 256, 77, 64                      # 77 keys: rows padded to 80 floats
    ld = (Sk + 7) & ~7
    g = torch.Generator(device="cuda").manual_seed(11)
    ws = torch.empty(B * H * Sq * ld, device="cuda")
    for call in range(2):                                     # second call reuses the array's old contents
        Q = torch.randn(B, H, Sq, D, device="cuda", generator=g).half()
        K = torch.randn(B, H, Sk, D, device="cuda", generator=g).half()
        V = torch.randn(B, H, Sk, D, device="cuda", generator=g).half()
        n_keys = Sk if call == 0 else Sk - 5
        want = torch.empty_like(Q); got = torch.empty_like(Q)
        assert L.rfk_sdpa(ctx.h, _p(Q), _p(K), _p(V), _p(want), _p(ws), VP(0), B, H, Sq, Sk, n_keys, D, 0, _stream()) == 0
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        assert L.rfk_sdpa_static(ctx.h, _p(Q), _p(K), _p(V), _p(got), B, H, Sq, Sk, n_keys, D, 0, _stream()) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # same GEMMs and the same softmax kernel on the same values: tolerance of the other attention
        # tests (4e-3), and in fact identical bits
        assert (got.float() - want.float()).abs().max().item() <= 4e-3
        assert torch.equal(got, want)
        ref = torch.nn.functional.scaled_dot_product_attention(Q.float(), K[:, :, :n_keys].float(), V[:, :, :n_keys].float())
        assert (got.float() - ref).abs().max().item() <= 4e-3 + 4e-3 * ref.abs().max().item()
    # beyond the fixed maximum (8 Mi floats) the call is refused, nothing is launched
    assert L.rfk_sdpa_static(ctx.h, _p(Q), _p(K), _p(V), _p(got), 1, 16, 4096, 5672, 5672, 64, 0, _stream()) == -3
    ctx.close()
