"""Regenerates the golden fixtures in this directory.

The reference cannot be imported or built here (HIP-only host, TVM-generated gfx906 kernels), and its
own golden vector needs a .param file it does not ship, so the fixtures are produced by the two
independent CPU implementations this repository has — the plain-C oracle accumulating in double and a
PyTorch float64 interpretation of the same schedule graph — and are written only when the two agree to
1e-6.  Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

from oracle import oracle  # noqa: E402
from reef_b200 import resources  # noqa: E402
from torch_ref import run_graph  # noqa: E402


def main():
    root = os.environ.get("REEF_RESOURCE_DIR", "/tmp/reef_b200_resources")
    # the exact-fp32 schedule (unrounded weights, CUDA-core convolutions)
    d = resources.generate("resnet18_64", root, variant="_fp32")
    base = os.path.join(d, "resnet18_64_fp32")
    x = np.full(3 * 64 * 64, 10.0, np.float32)
    o = oracle.OracleExecutor(base + ".json", base + ".param", acc64=True)
    o.set_input("data", x)
    o.execute()
    st, names = run_graph(base + ".json", base + ".param", {"data": x}, double=True)
    j = json.load(open(base + ".json"))
    li = j["kernels"][-1]["args"][0]
    err = np.abs(o.storage[li] - st[li]).max() / np.abs(st[li]).max()
    assert err < 1e-6, err
    np.savez(os.path.join(HERE, "resnet18_64_fp32_const10.npz"), logits=st[li].astype(np.float32),
             probs=st[names.index("output")].astype(np.float32))
    print("wrote resnet18_64_const10.npz; oracle(acc64) vs torch(float64) rel err", err)


if __name__ == "__main__":
    main()
