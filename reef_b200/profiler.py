"""Kernel profiler: measures `<model>.profile.json` on the current GPU.

Replaces the `profiler` binary that the reference's resource/Makefile:32-36 invokes but does not ship.
The file feeds the dynamic-kernel-padding policy (reference: src/reef/server/scheduler.cpp:566-595):
``total_latency`` of a kernel and ``latency[j]`` = one persistent wave at occupancy j+1, here in
nanoseconds (``"latency_unit_ns": 1``; the reference wrote microseconds, too coarse for B200).

    python -m reef_b200.profiler --model resnet152 [--dir DIR] [--iters 20]
"""
from __future__ import annotations

import argparse
import os

import numpy as np


def profile_model(base: str, iters: int = 20, device: int = 0) -> str:
    """`base` = path without extension; rewrites base + '.profile.json' and returns its path."""
    from . import capi
    e = capi.HybridExecutor(device)
    e.load_model_from_file(base + ".json", None)
    if os.path.exists(base + ".param"):
        e.load_param_from_file(base + ".param")
    out = base + ".profile.json"
    e.write_profile(out, iters)
    e.close()
    return out


def main():
    from . import resources
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", required=True)
    ap.add_argument("--variant", default="")
    ap.add_argument("--dir", default=None)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    d = resources.generate(a.model, a.dir, variant=a.variant)
    base = os.path.join(d, os.path.basename(d))
    print(profile_model(base, a.iters))


if __name__ == "__main__":
    main()
