"""Writes tests/golden/ref_kernels.npz: outputs of the reference's OWN kernels (resource/<model>/<model>.cu, compiled
unchanged and run on the CPU by oracle/refkernels) for the cases of tests/ref_cases.py, on seeded inputs.

Run where the reference tree is present:
    make -C oracle ref && python tests/golden/make_ref_kernel_golden.py
The fixture pins the C oracle on every machine, including those without the reference tree: the test regenerates the
same seeded inputs, runs the oracle and compares with the stored reference outputs (a fixed-stride subsample of at most
32768 values per case keeps the file small).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import ref_cases as RC  # noqa: E402
from oracle import ref_kernels as R  # noqa: E402


def main():
    out = {}
    for cid, case in RC.CASES.items():
        d = RC.case_inputs(cid)
        y = case["ref"](R, d)
        out[cid] = RC.subsample(y).astype(np.float32)
        out[cid + "__shape"] = np.asarray(y.shape, dtype=np.int64)
        out[cid + "__input_checksum"] = np.asarray([RC.input_checksum(d)], dtype=np.float64)
        print(f"{cid:40s} shape {tuple(y.shape)} stored {out[cid].size} values")
    path = os.path.join(HERE, "ref_kernels.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    for m in ("resnet152", "bert", "inception"):
        if not R.available(m):
            raise SystemExit(f"oracle/_ref/libref_{m}.so is missing: run `make -C oracle ref` where the reference tree is present")
    main()
