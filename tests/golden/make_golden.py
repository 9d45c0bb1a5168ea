"""Generate tests/golden/reference_outputs.npz: outputs of the reference engine's OWN CUDA
kernels (oracle/_ref/*.so, built unchanged from the reference sources by oracle/Makefile)
on the seeded inputs of tests/cases.py.

Run on a machine with a B200 and the built oracle/_ref libraries:

    python tests/golden/make_golden.py [--out tests/golden/reference_outputs.npz]

The inputs are not stored: they are regenerated from the case name and seed. Only cases that
have a reference implementation contribute. The file also records the GPU name and the
CUDA runtime version it was produced with.
"""
import argparse
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

import cases  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(HERE / "reference_outputs.npz"))
    a = ap.parse_args()
    import torch
    from oracle import ref
    if not torch.cuda.is_available():
        sys.exit("needs a CUDA device")
    if not (ref.available() and ref.layers_available()):
        sys.exit("oracle/_ref libraries are not built (make -C oracle ref)")
    store = {}
    for c in cases.CASES:
        if c.ref is None:
            continue
        out = c.ref(c.inputs())
        for k, v in out.items():
            store[f"{c.name}::{k}"] = v
    store["__meta__"] = np.array([torch.cuda.get_device_name(0), torch.version.cuda,
                                  f"{len(store)} arrays"])
    np.savez_compressed(a.out, **store)
    size = Path(a.out).stat().st_size
    print(f"wrote {a.out}: {len(store) - 1} arrays, {size / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
