"""Offline estimate of how much of the GPU a model's kernels occupy, weighted by their latency.

The reference's ``script/estimate_resource_usage.py`` (lines 21-33) answers "how many compute units does a
real-time model leave idle?" from ``<model>.json`` and ``<model>.profile.json``: per kernel, the compute units a
launch covers x its profiled latency, over all compute units x latency.  Same question here for a B200, in the
units the padding policy uses: an SM holds two tensor-core CTAs (two slots), or four 256-thread logical blocks
per slot for the other kernels; a real-time kernel also holds the slots of its successor's parked prologue.

    python -m reef_b200.estimate MODEL_DIR [MODEL_DIR ...]      (a directory holding <name>.json and .profile.json)
"""
from __future__ import annotations

import argparse
import json
import math
import os

from . import capi

NUM_SMS = 148
SLOTS = 2 * NUM_SMS


def estimate(model_dir: str) -> dict:
    name = os.path.basename(os.path.normpath(model_dir))
    sched = json.load(open(os.path.join(model_dir, name + ".json")))
    prof = json.load(open(os.path.join(model_dir, name + ".profile.json")))
    total = used = used_with_prologue = 0.0
    slots = []
    for k in sched["kernels"]:
        lp = k["launch_params"]
        blocks = lp[0] * lp[1] * lp[2]
        _, _, tc = capi.kernel_cost(k["name"])
        slots.append(min(SLOTS, blocks if tc else math.ceil(blocks / 4)))
    for i, k in enumerate(sched["kernels"]):
        lat = prof["kernel_latency"][k["name"]]["total_latency"]
        nxt = slots[i + 1] if i + 1 < len(slots) else 0
        total += lat * SLOTS
        used += lat * slots[i]
        used_with_prologue += lat * min(SLOTS, slots[i] + nxt)
    return dict(model=name, kernels=len(slots), busy_pct=100.0 * used / total,
                busy_with_parked_successor_pct=100.0 * used_with_prologue / total)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("model_dirs", nargs="+")
    args = ap.parse_args(argv)
    for d in args.model_dirs:
        r = estimate(d)
        print("%s: %.1f%% of the SM slots busy (%.1f%% with the parked prologue of the next kernel), %d kernels"
              % (r["model"], r["busy_pct"], r["busy_with_parked_successor_pct"], r["kernels"]))


if __name__ == "__main__":
    main()
