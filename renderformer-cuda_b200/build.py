"""Build the native libraries of this package in-tree with nvcc for sm_100a.

    python renderformer-cuda_b200/build.py [--force] [--verbose]

Produces, next to this file:
    librfk.so         the kernel library behind include/rfk.h (CUDA runtime only)
    librfk_layers.so  layer boundaries, render session (include/rfk_layers.h; cuBLAS + librfk.so)

nvcc cross-compiles without a GPU, so this also runs on a CPU-only machine.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-O3,-Wall,-Wno-unused-function",
    "--expt-relaxed-constexpr",
]

LAYER_SOURCES = ["layers.cu", "session.cu", "dpt.cu"]
IO_SOURCES = ["io.cpp"]   # host code (safetensors, EXR, PNG); needs the CUDA runtime for the upload, zlib for the PNG

KERNEL_SOURCES = [
    "abi.cu", "rmsnorm.cu", "softmax.cu", "rope.cu", "layout.cu",
    "activations.cu", "nerf_pe.cu", "raygen.cu", "geometry.cu", "attention.cu", "attention_tc.cu", "gemm_tc.cu", "dpt_glue.cu", "dpt_nhwc.cu",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the rfk libraries cannot be built")
    return exe


def _newer(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(d.stat().st_mtime <= t for d in deps)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"build step failed: {' '.join(cmd[:3])} ...")
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout + proc.stderr)


def build_library(name: str, sources: list[str], extra: list[str], force: bool,
                  verbose: bool, ptxas_info: bool = False) -> Path:
    """Compile each .cu to an object (in build/), then link lib<name>.so."""
    out = PKG / f"lib{name}.so"
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sorted(INCLUDE.glob("*.h"))
    objs = []
    for src in sources:
        s = CSRC / src
        o = objdir / (s.stem + ".o")
        if force or not _newer(o, [s] + headers):
            cmd = [nvcc(), *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", f"-I{cudnn_include()}", "-c", str(s), "-o", str(o)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            _run(cmd, verbose or ptxas_info)
        objs.append(o)
    if force or not _newer(out, objs):
        _run([nvcc(), "-shared", "-o", str(out), *map(str, objs), "-cudart", "shared", *extra],
             verbose)
    return out


def cudnn_include() -> str:
    """cudnn.h ships with the Python environment's cuDNN package; the library itself is the system's libcudnn.so.9."""
    import sysconfig
    return os.path.join(sysconfig.get_paths()["purelib"], "nvidia", "cudnn", "include")


def build_all(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> dict[str, Path]:
    libs = {"rfk": build_library("rfk", KERNEL_SOURCES, [], force, verbose, ptxas_info)}
    # layer boundaries + session + DPT head: cuBLAS for the fallback GEMMs, cuDNN for the head's convolutions,
    # librfk.so (same directory) for everything else
    libs["rfk_layers"] = build_library(
        "rfk_layers", LAYER_SOURCES,
        ["-lcublas", "-lcudnn", f"-L{PKG}", "-lrfk", "-Xlinker", "-rpath=$ORIGIN"], force, verbose, ptxas_info)
    libs["rfk_io"] = build_library("rfk_io", IO_SOURCES, ["-lz"], force, verbose, False)
    return libs


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true", help="rebuild everything")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true",
                    help="print registers / spills / shared memory per kernel (implies --force)")
    a = ap.parse_args()
    for k, v in build_all(a.force or a.ptxas_info, a.verbose, a.ptxas_info).items():
        print(f"{k}: {v}")
