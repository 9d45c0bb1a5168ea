"""CPU tests of the oracle: it must reproduce the committed outputs of the reference's own
CUDA kernels (tests/golden/reference_outputs.npz) and agree with float64 numpy formulas."""
from pathlib import Path

import numpy as np
import pytest

import cases
from oracle import oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden" / "reference_outputs.npz"


@pytest.fixture(scope="module")
def golden():
    if not GOLDEN.exists():
        pytest.skip("golden fixtures not generated yet")
    return np.load(GOLDEN)


def test_golden_covers_reference_cases(golden):
    want = {f"{c.name}::{k}" for c in cases.CASES if c.ref is not None for k in c.kinds}
    assert want <= set(golden.files), sorted(want - set(golden.files))[:5]


@pytest.mark.parametrize("case", [c for c in cases.CASES if c.ref is not None], ids=lambda c: c.name)
def test_oracle_matches_reference_golden(case, golden):
    out = case.oracle(case.inputs())
    for k, kind in case.kinds.items():
        kind = case.oracle_kinds.get(k, kind)
        cases.compare(kind, out[k], golden[f"{case.name}::{k}"], f"{case.name}.{k}")


def test_rmsnorm_against_float64():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((16, 1024)).astype(np.float32)
    g = rng.normal(1.0, 0.02, 1024).astype(np.float32)
    y = O.rmsnorm_f32(x, g, 1e-6)
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 ** 2).mean(1, keepdims=True) + 1e-6) * g
    np.testing.assert_allclose(y, want, rtol=2e-6)


def test_fused_residual_norm_cast_is_the_three_step_sequence():
    rng = np.random.default_rng(1)
    h = rng.standard_normal((8, 256)).astype(np.float32)
    r = rng.standard_normal((8, 256)).astype(np.float32)
    g = rng.normal(1.0, 0.02, 256).astype(np.float32)
    h2, y16 = O.rmsnorm_residual_f32_cast16(h, r, g, 1e-6)
    step = O.residual_add_f32(h, r)
    np.testing.assert_array_equal(h2, step)
    np.testing.assert_array_equal(y16, O.cast_fp32_to_fp16(O.rmsnorm_f32(step, g, 1e-6)))


def test_softmax_rows_sum_to_one_and_pad_is_zero():
    rng = np.random.default_rng(2)
    x = np.full((4, 5640), -np.inf, np.float32)
    x[:, :5633] = rng.normal(0, 3 / 8, (4, 5633))
    p = O.softmax_cast_fp16(x, 5633, 5640)
    assert (p[:, 5633:] == 0).all()
    np.testing.assert_allclose(p.astype(np.float64).sum(1), 1.0, atol=2e-3)
    x64 = x[:, :5633].astype(np.float64)
    want = np.exp(x64 - x64.max(1, keepdims=True)); want /= want.sum(1, keepdims=True)
    np.testing.assert_allclose(p[:, :5633].astype(np.float64), want, atol=2e-6 + 2.0 ** -11 * want.max())


def test_masked_softmax_empty_row_is_zero():
    x = np.zeros((1, 8), np.float32)
    p = O.softmax_cast_fp16(x, 8, 8, mask=np.zeros((1, 8), bool))
    assert (p == 0).all()


def test_rope_is_a_rotation():
    rng = np.random.default_rng(3)
    pos = rng.uniform(-1, 1, (1, 10, 9)).astype(np.float16)
    c, s = O.triangle_rope_freqs(pos, np.array([1.0, 0.1, 0.01], np.float32), 64)
    assert (c[..., 27:32] == 1).all() and (s[..., 27:32] == 0).all()       # zero-pad region
    np.testing.assert_array_equal(c[..., :32], c[..., 32:])                  # duplicated halves
    x = rng.standard_normal((1, 2, 10, 64)).astype(np.float32)
    y = O.apply_rope(x, c, s)
    n0 = (x[..., :32] ** 2 + x[..., 32:] ** 2)
    n1 = (y[..., :32] ** 2 + y[..., 32:] ** 2)
    np.testing.assert_allclose(n1, n0, rtol=5e-3, atol=1e-3)                 # pairs keep their norm


def test_nerf_pe_layout():
    x = np.array([[[0.5, -0.25, 1.0]]], np.float32)
    o = O.nerf_pe(x, 2, 0.0, 1.0, True).astype(np.float64)[0, 0]
    want = np.concatenate([x[0, 0], np.sin([0.5, 1.0, -0.25, -0.5, 1.0, 2.0]), np.cos([0.5, 1.0, -0.25, -0.5, 1.0, 2.0])])
    np.testing.assert_allclose(o, want, atol=1e-3)


def test_ray_gen_center_ray_and_unit_length():
    c2w = np.eye(4, dtype=np.float32)[None]
    ro, rd = O.ray_gen(c2w, np.array([0.8], np.float32), 64)
    d = rd.astype(np.float64)
    np.testing.assert_allclose(np.linalg.norm(d, axis=-1), 1.0, atol=2e-3)
    assert (d[..., 2] < 0).all()                                             # -Z forward
    assert d[0, 0, 0, 0] < 0 < d[0, 0, 0, 1]                                 # top-left pixel: -x, +y
    _, tok = O.ray_gen(c2w, np.array([0.8], np.float32), 64, 8)
    np.testing.assert_array_equal(tok[0], O.patchify(rd[0], 8))


def test_world_to_cam_inverts_camera_pose():
    rng = np.random.default_rng(4)
    c2w, _ = cases.look_at_c2w(rng, 1)
    cam = rng.uniform(-1, 1, (1, 50, 3)).astype(np.float32)
    world = cam @ c2w[0, :3, :3].T + c2w[0, :3, 3]
    back, _ = O.world_to_cam(c2w, world.astype(np.float32))
    np.testing.assert_allclose(back, cam, atol=1e-5)


def test_window_gather_matches_shift_then_partition():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, 8, 8, 4)).astype(np.float16)
    win = O.window_partition(O.cyclic_shift(x, -2, -2), 4)
    back = O.cyclic_shift(O.window_reverse(win, 1, 8, 8, 4), 2, 2)
    np.testing.assert_array_equal(back, x)


def test_threads_do_not_change_results():
    rng = np.random.default_rng(6)
    x = rng.standard_normal((64, 512)).astype(np.float32)
    g = np.ones(512, np.float32)
    O.set_threads(1); a = O.rmsnorm_f32(x, g, 1e-6)
    O.set_threads(O.max_threads()); b = O.rmsnorm_f32(x, g, 1e-6)
    O.set_threads(1)
    np.testing.assert_array_equal(a, b)


def test_timed_port_functions_agree_with_the_checker():
    """oracle_linear_f16 and oracle_sdpa_f32acc carry the host-core baseline that bench.py times; they must
    compute what the checked oracle functions compute: linear = fp32-accumulated product rounded to fp16
    (+ bias added after the rounding), attention = oracle_sdpa within one fp16 step."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((37, 264)).astype(np.float16)[:, :200]            # row pitch larger than the row
    w = (rng.standard_normal((56, 200)) * 0.1).astype(np.float16)
    b = rng.standard_normal(56).astype(np.float16)
    prod = x.astype(np.float64) @ w.astype(np.float64).T
    got = O.linear(x, w).astype(np.float64)
    assert np.abs(got - prod).max() <= 2.0 ** -10 * np.abs(prod).max() + 1e-6
    want_b = (prod.astype(np.float16).astype(np.float32) + b.astype(np.float32)).astype(np.float16)
    got_b = O.linear(x, w, b)
    assert np.abs(got_b.astype(np.float32) - want_b.astype(np.float32)).max() <= 2.0 ** -9 * np.abs(prod).max()
    Q = rng.standard_normal((2, 3, 70, 64)).astype(np.float16)
    K = rng.standard_normal((2, 3, 93, 64)).astype(np.float16)
    V = rng.standard_normal((2, 3, 93, 64)).astype(np.float16)
    a = O.sdpa(Q, K, V, n_keys=90, o_bshd=True).astype(np.float32)
    f = O.sdpa_f32acc(Q, K, V, n_keys=90).astype(np.float32)
    assert np.abs(a - f).max() <= 1e-3
    O.set_threads(O.max_threads())
    f2 = O.sdpa_f32acc(Q, K, V, n_keys=90).astype(np.float32)
    O.set_threads(1)
    assert np.array_equal(f, f2)                                               # threads split rows, not sums
