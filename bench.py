"""Benchmark of the hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl rfk|reference] [--workload W]

Prints ONE JSON line on rank 0. For N > 1 launch with
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N ...
(one process per GPU; RANK / LOCAL_RANK / WORLD_SIZE are read from the environment).

Workloads
  kernels  one step = every hot-path operator once at its benchmark shape (fused
           residual+RMSNorm+cast, RoPE, RoPE tables, NeRF PE, softmax, ray generation,
           world->camera, SwiGLU gate); metric = algorithmic GB/s over the whole step.
Arms
  rfk        this repository's CUDA kernels through the C ABI.
  reference  the reference engine's own CUDA kernels (oracle/_ref, built unchanged from the
             reference sources) under the same harness. The reference has no CPU
             implementation; its host-core stand-in is the scalar oracle port, reported as
             `cpu_baseline`.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.path = Path(f"/tmp/rfk_clocks_{os.getpid()}.csv")

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.path.read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.path.unlink(missing_ok=True)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


def dist_setup(n_gpus: int):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier_sync(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms: float, world: int) -> float:
    import torch
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ------------------------------------------------------------------ backends

def rfk_backend():
    import renderformer_cuda_b200 as pkg  # noqa: F401
    from renderformer_cuda_b200.kernel_bench import RfkBackend
    return RfkBackend()


class RefBackend:
    """The reference engine's own CUDA kernels (oracle/_ref), same operator surface."""
    name = "reference"
    not_capturable = ("nerf_pe_f32", "nerf_pe_f16")  # its wrappers cudaMalloc/cudaFree per call

    def __init__(self):
        import math
        import torch
        from oracle import ref
        if not (ref.available() and ref.layers_available()):
            raise RuntimeError("oracle/_ref libraries are not built")
        self.R = ref
        self.freqs_t = torch.tensor([math.pi * 10000.0 ** (-i / 3) for i in range(3)], device="cuda", dtype=torch.float32)
        self.tmp = None

    def fused_rmsnorm(self, h, r, g, y):
        import torch
        if self.tmp is None or self.tmp.shape != h.shape:
            self.tmp = torch.empty_like(h)
        self.R.call("ref_residual_rmsnorm_cast", h, r, g, self.tmp, y, h.shape[0], h.shape[1], 1e-6, lib=self.R.layers())

    def rope(self, q, k, c, s, pos):
        self.R.call("ref_apply_rope", q, k, c, s, q.shape[0], q.shape[1], q.shape[2], q.shape[3])

    def rope_tables(self, q, k, c, s, pos):
        self.R.call("ref_triangle_rope_freqs", pos, self.freqs_t, c, s, 1, pos.shape[1], 3, c.shape[-1])

    def nerf_pe_f32(self, x, out):
        self.R.call("ref_nerf_pe_f32", x, out, x.shape[0], x.shape[1], x.shape[2], 6, 0.0, 5.0, 1)

    def nerf_pe_f16(self, x, out):
        self.R.call("ref_nerf_pe", x, out, x.shape[0], x.shape[1], x.shape[2], 6, 0.0, 5.0, 1)

    def softmax(self, x, p, rows, cols, stride):
        self.R.call("ref_softmax_cast_fp16", x, p, rows, cols, stride, stride)

    def ray_gen(self, c2w, fov, ro, rd, b):
        self.R.call("ref_ray_gen", c2w, fov, ro, rd, b, rd.shape[1])

    def world_to_cam(self, c2w, tri, vn, b):
        self.R.call("ref_world_to_cam", c2w, tri, vn, b, tri.shape[1])

    def silu_mul(self, a, b, out):
        self.R.call("ref_fused_silu_mul", a, b, out, a.numel())


# -------------------------------------------------------------- CPU baseline

def cpu_baseline_kernels(budget_s: float = 20.0) -> dict:
    """Scalar C port of the same operators (oracle/), timed on this host's cores on a bounded
    sample: config 1 in full and a slice of the config-3 rows, all threads, then 1 thread."""
    import numpy as np
    from oracle import oracle as O
    rng = np.random.default_rng(0)
    T, D = 5633, 1024
    h = rng.standard_normal((T, D), dtype=np.float32); r = rng.standard_normal((T, D), dtype=np.float32)
    g = np.ones(D, np.float32)
    rows, cols, stride = 1024, 5633, 5640
    x = rng.standard_normal((rows, stride), dtype=np.float32) * 0.375
    bytes_done = (3 * 4 * T * D + 2 * T * D) + rows * (cols * 4 + stride * 2)
    out = {}
    for label, threads in (("all", O.max_threads()), ("one", 1)):
        O.set_threads(threads)
        best = float("inf")
        t_end = time.time() + budget_s / 2
        while True:
            t0 = time.perf_counter()
            O.rmsnorm_residual_f32_cast16(h, r, g, 1e-6)
            O.softmax_cast_fp16(x, cols, stride)
            best = min(best, time.perf_counter() - t0)
            if time.time() > t_end:
                break
        out[label] = bytes_done / best / 1e9
    O.set_threads(1)
    return {"value": round(out["all"], 3), "unit": "GB/s", "cores": O.max_threads(), "kind": "port",
            "single_thread_value": round(out["one"], 3),
            "sample": "fused residual+RMSNorm+cast [5633x1024] in full + 1024 of the 65536 softmax rows "
                      "(5633 cols), best of repeated runs"}


# ------------------------------------------------------------------ workloads

def run_kernels(args, backend, rank, world, peak, peak_src):
    import torch
    from renderformer_cuda_b200 import kernel_bench as kb
    import renderformer_cuda_b200 as pkg
    entries = kb.suite()
    step_entries = [e for e in entries if " batch" not in e.name]
    # one buffer set per entry and rotation slot, sized so the step's working set is >> L2
    sets = {e.name: [e.make() for _ in range(2 if e.bytes_per_launch > kb.L2_BYTES else 4)] for e in step_entries}
    fns = {e.name: getattr(backend, e.op) for e in step_entries}

    def step(i):
        for e in step_entries:
            s = sets[e.name]
            fns[e.name](*s[i % len(s)])

    for w in range(args.warmup):
        step(w)
    barrier_sync(world)
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    n0 = pkg.ops.launch_count()
    graph = None
    if not getattr(backend, "not_capturable", ()):
        # the K steps are captured once and replayed: device time, not the host's launch rate
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(args.steps):
                step(i)
        graph.replay()
    launches = pkg.ops.launch_count() - n0   # kernels in the captured K steps (replayed as is)
    st = torch.cuda.Event(enable_timing=True); en = torch.cuda.Event(enable_timing=True)
    barrier_sync(world)
    st.record()
    if graph is not None:
        graph.replay()
    else:
        for i in range(args.steps):
            step(i)
    en.record()
    barrier_sync(world)
    ms = max_over_ranks(st.elapsed_time(en), world)
    clocks = sampler.stop() if rank == 0 else None
    del sets
    torch.cuda.empty_cache()
    step_bytes = sum(e.bytes_per_launch for e in step_entries)
    value = world * step_bytes * args.steps / (ms * 1e-3) / 1e9

    table = kb.run_suite(backend, peak, iters=max(args.steps, 10), warmup=max(args.warmup, 3)) if rank == 0 else None
    if rank != 0:
        return None
    dom = next(r for r in table if r["op"] == "softmax")
    line = {
        "metric": "hot-path kernel suite, algorithmic HBM GB/s", "value": round(value, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32/f16", "data": "synthetic",
        "config": {"workload": "kernels: configs 1-4 of BASELINE.json, one launch each per step",
                   "l2": "rotating buffer sets > 2x L2 per operator", "impl": backend.name},
        "roofline": {"bound": "hbm", "kernel": dom["kernel"], "achieved": dom["gbs"], "peak": peak,
                     "unit": "GB/s", "frac": round(dom["gbs"] / peak, 3), "peak_source": peak_src,
                     "frac_of_8tbs_nominal": dom["frac_8tbs"], "traffic": None},
        "kernels": table,
        "gpu_launches": int(launches) if backend.name == "rfk" else 0,
        "clocks": clocks,
        "e2e": None,
    }
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="rfk", choices=["rfk", "reference"])
    ap.add_argument("--workload", default="kernels", choices=["kernels"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    import torch
    if not torch.cuda.is_available():
        sys.exit("bench.py needs a CUDA device: there is no CPU fallback")
    rank, world, local = dist_setup(args.gpus)
    peak, peak_src = measured_peaks()

    if args.impl == "reference":
        try:
            backend = RefBackend()
        except Exception as e:  # reference libraries did not travel / did not build
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"}))
            return
    else:
        backend = rfk_backend()

    line = run_kernels(args, backend, rank, world, peak, peak_src)
    if rank == 0:
        if args.impl == "reference":
            line["impl"] = "reference"
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_kernels()
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
