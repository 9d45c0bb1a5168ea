"""GPU parity tests: every kernel, called through the C ABI, against
  (1) the CPU oracle on the same seeded inputs,
  (2) the reference engine's own CUDA kernels run live on the same device, when the
      oracle/_ref libraries travelled with the tree, and
  (3) the committed outputs of those reference kernels (tests/golden/)."""
from pathlib import Path

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden" / "reference_outputs.npz"


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN) if GOLDEN.exists() else None


@pytest.fixture(scope="module", autouse=True)
def _library_is_native():
    import renderformer_cuda_b200 as pkg
    from renderformer_cuda_b200 import _abi
    assert _abi.library_path("rfk.h").exists(), "librfk.so missing: the CUDA path must be the one that runs"
    assert "sm_100a" in pkg.version()


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.name)
def test_kernel_matches_oracle(case):
    i = case.inputs()
    got = case.rfk(i)
    want = case.oracle(i)
    for k, kind in case.kinds.items():
        cases.compare(case.oracle_kinds.get(k, kind), got[k], want[k], f"{case.name}.{k} vs oracle")


@pytest.mark.parametrize("case", [c for c in cases.CASES if c.ref is not None], ids=lambda c: c.name)
def test_kernel_matches_reference_kernels_live(case):
    from oracle import ref
    if not (ref.available() and ref.layers_available()):
        pytest.skip("oracle/_ref libraries not present")
    i = case.inputs()
    got = case.rfk(i)
    want = case.ref(i)
    for k, kind in case.kinds.items():
        cases.compare(kind, got[k], want[k], f"{case.name}.{k} vs reference kernels")


@pytest.mark.parametrize("case", [c for c in cases.CASES if c.ref is not None], ids=lambda c: c.name)
def test_kernel_matches_reference_golden(case, golden):
    if golden is None:
        pytest.skip("golden fixtures not generated yet")
    got = case.rfk(case.inputs())
    for k, kind in case.kinds.items():
        cases.compare(kind, got[k], golden[f"{case.name}::{k}"], f"{case.name}.{k} vs golden")


def test_launch_counter_counts():
    import torch
    import renderformer_cuda_b200 as pkg
    x = torch.randn(8, 1024, device="cuda").half()
    g = torch.ones(1024, device="cuda")
    n0 = pkg.ops.launch_count()
    pkg.ops.rmsnorm(x, g, x, 8, 1024)
    assert pkg.ops.launch_count() == n0 + 1


def test_kernels_run_on_a_side_stream_and_in_a_graph():
    """The entry points neither allocate nor synchronise: they can be captured."""
    import torch
    import renderformer_cuda_b200 as pkg
    x = torch.randn(64, 1024, device="cuda").half(); g = torch.ones(1024, device="cuda")
    y = torch.empty_like(x); pe_in = torch.randn(1, 64, 9, device="cuda")
    pe_out = torch.empty(1, 64, 117, device="cuda", dtype=torch.float16)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        pkg.ops.rmsnorm(x, g, y, 64, 1024)
    s.synchronize()
    want = y.clone()
    y.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        pkg.ops.rmsnorm(x, g, y, 64, 1024)
        pkg.ops.nerf_pe_f32(pe_in, pe_out, 1, 64, 9, 6, 0.0, 5.0, True)   # the reference form mallocs here
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, want)
    assert torch.isfinite(pe_out.float()).all()


@pytest.mark.gpu
@pytest.mark.parametrize("B,Hh,W,dim,ws,shift", [(1, 16, 16, 256, 8, 0), (1, 16, 16, 256, 8, 4), (2, 8, 24, 1024, 4, 3),
                                                 (1, 64, 64, 1024, 8, 4), (1, 8, 8, 2048, 8, 1)])
def test_rmsnorm_residual_with_window_ordered_operand_equals_the_separate_kernels(B, Hh, W, dim, ws, shift):
    """The fused norm that writes its output in swin window order (or reads its residual out of it) is bit-identical
    to residual+norm followed by window_gather, and to window_scatter(+residual) followed by the norm."""
    import torch
    import renderformer_cuda_b200 as pkg
    ops = pkg.ops
    rows = B * Hh * W
    g = torch.Generator(device="cuda").manual_seed(rows + dim + shift)
    x0 = torch.randn(rows, dim, device="cuda", generator=g).half()
    r = torch.randn(rows, dim, device="cuda", generator=g).half()
    gamma = torch.rand(dim, device="cuda", generator=g) + 0.5
    # (1) y in window order
    xa, xb = x0.clone(), x0.clone()
    ya, tmp, yb = torch.empty_like(x0), torch.empty_like(x0), torch.empty_like(x0)
    ops.rmsnorm_residual_f16(xa, r, gamma, tmp, rows, dim)
    ops.window_gather(tmp, ya, B, Hh, W, dim, ws, shift)
    ops.rmsnorm_residual_f16_windows(xb, r, gamma, yb, B, Hh, W, dim, ws, shift, 1)
    torch.cuda.synchronize()
    assert torch.equal(xa, xb) and torch.equal(ya, yb)
    # (2) r in window order
    xa, xb = x0.clone(), x0.clone()
    ops.window_scatter(r, xa, B, Hh, W, dim, ws, shift, residual_into=True)
    ops.rmsnorm(xa, gamma, ya, rows, dim)
    ops.rmsnorm_residual_f16_windows(xb, r, gamma, yb, B, Hh, W, dim, ws, shift, 2)
    torch.cuda.synchronize()
    assert torch.equal(xa, xb) and torch.equal(ya, yb)
