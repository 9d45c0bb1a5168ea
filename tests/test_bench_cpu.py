"""CPU checks of bench.py's outer contract: without a CUDA device it refuses to run (no CPU fallback) and writes
nothing to standard output, which is reserved for the one JSON line; the roofline's traffic table and the flags the
driver passes are present."""
import importlib.util
import pathlib
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _load():
    spec = importlib.util.spec_from_file_location("rfk_bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_bench_refuses_to_run_without_a_gpu_and_keeps_stdout_empty():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a CUDA device is present: the refusal path is not taken")
    for extra in ([], ["--impl", "reference"], ["--gpus", "1", "--steps", "20", "--warmup", "5"]):
        r = subprocess.run([sys.executable, str(ROOT / "bench.py"), *extra], capture_output=True, text=True, timeout=600)
        assert r.returncode != 0
        assert r.stdout == ""
        assert "no CPU fallback" in r.stderr


def test_bench_constants_match_the_headline_configuration():
    b = _load()
    assert (b.N_TRIS, b.IMG_RES, b.N_CAMERAS) == (5633, 512, 64)
    assert b.N_REPS >= 7
    assert set(b.ATTENTION_TRAFFIC) >= {1, 4} and all(v > 0 for v in b.ATTENTION_TRAFFIC.values())
