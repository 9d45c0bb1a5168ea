"""GPU test of rfk_sdpa_static, the attention entry point for callers that cannot allocate
device memory (stream host callbacks, code that must not call cudaMalloc, hosts with a fixed
memory budget): its score matrix lives in a fixed 32 MiB array inside the library. Called through the C ABI, twice
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


@pytest.mark.parametrize("B,H,Sq,Sk,D,o_bshd", [(1, 4, 256, 77, 64, 0), (2, 3, 130, 200, 64, 1)])
def test_static_scratch_sdpa_matches_workspace_sdpa_on_two_calls(B, H, Sq, Sk, D, o_bshd):
    from renderformer_cuda_b200 import _abi, session
    L = _abi.load("rfk_layers.h")
    ctx = session.Ctx()
    ld = (Sk + 7) & ~7                                        # 77 keys: rows padded to 80 floats
    g = torch.Generator(device="cuda").manual_seed(11)
    ws = torch.empty(B * H * Sq * ld, device="cuda")
    for call in range(2):                                     # second call reuses the array's old contents
        Q = torch.randn(B, H, Sq, D, device="cuda", generator=g).half()
        K = torch.randn(B, H, Sk, D, device="cuda", generator=g).half()
        V = torch.randn(B, H, Sk, D, device="cuda", generator=g).half()
        n_keys = Sk if call == 0 else Sk - 5
        shape = (B, Sq, H * D) if o_bshd else (B, H, Sq, D)
        want = torch.empty(shape, device="cuda", dtype=torch.float16); got = torch.empty_like(want)
        assert L.rfk_sdpa(ctx.h, _p(Q), _p(K), _p(V), _p(want), _p(ws), VP(0), B, H, Sq, Sk, n_keys, D, o_bshd, _stream()) == 0
        torch.cuda.synchronize()
        if call == 0:   # the documented first call on a device: looks up the array's address, launches the same work
            assert L.rfk_sdpa_static(ctx.h, _p(Q), _p(K), _p(V), _p(got), B, H, Sq, Sk, n_keys, D, o_bshd, _stream()) == 0
            torch.cuda.synchronize()
        # device memory as the driver sees it (cudaMemGetInfo covers cudaMalloc, pool allocations and library
        # workspaces, which torch's own counter does not) and torch's counter, around one call
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        assert L.rfk_sdpa_static(ctx.h, _p(Q), _p(K), _p(V), _p(got), B, H, Sq, Sk, n_keys, D, o_bshd, _stream()) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before
        # same GEMMs and the same softmax kernel on the same values: tolerance of the other attention
        # tests (4e-3), and in fact identical bits
        assert (got.float() - want.float()).abs().max().item() <= 4e-3
        assert torch.equal(got, want)
        ref = torch.nn.functional.scaled_dot_product_attention(Q.float(), K[:, :, :n_keys].float(), V[:, :, :n_keys].float())
        if o_bshd:
            ref = ref.permute(0, 2, 1, 3).reshape(B, Sq, H * D)
        assert (got.float() - ref).abs().max().item() <= 4e-3 + 4e-3 * ref.abs().max().item()
    # beyond the fixed maximum (8 Mi floats) the call is refused, nothing is launched
    assert L.rfk_sdpa_static(ctx.h, _p(Q), _p(K), _p(V), _p(got), 1, 16, 4096, 5672, 5672, 64, 0, _stream()) == -3
    # a product of sizes that would wrap around 2^64 is refused as well, not mistaken for a small one
    assert L.rfk_sdpa_static(ctx.h, _p(Q), _p(K), _p(V), _p(got), 65536, 65536, 65536, 8192, 8192, 64, 0, _stream()) == -3
    # rows longer than the register-resident softmax serves are refused before anything is launched
    assert L.rfk_sdpa_static(ctx.h, _p(Q), _p(K), _p(V), _p(got), 1, 1, 1, 8200, 8200, 64, 0, _stream()) == -2
    ctx.close()
