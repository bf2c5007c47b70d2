"""Per-kernel roofline table of a model: every distinct kernel name of the schedule timed alone on the GPU.

    python -m reef_b200.kernel_table --model vgg16 [--json out.json]

For each distinct kernel: microseconds per launch (a CUDA graph of back-to-back launches of that kernel, CUDA events),
its algorithmic bytes and flops (reef_kernel_cost), the achieved GB/s and the fraction of the HBM peak, or TFLOP/s for
the kernels whose floor is arithmetic.  The peak is the measured copy bandwidth in MEASURED_PEAKS.json at the
repository root when that file exists, else 6650 GB/s.  The reference has per-kernel latencies only
(<model>.profile.json, reference: src/reef/executor/model.cpp:57-82); this adds the bytes behind them.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np


def peak_gbs():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def kernel_table(model: str, device: int = 0, variant: str = "", reps: int = 20, iters: int = 20):
    from . import capi, resources
    d = resources.generate(model, variant=variant)
    base = os.path.join(d, model + variant)
    j = json.load(open(base + ".json"))
    e = capi.HybridExecutor(device)
    e.load_model_from_file(base + ".json", base + ".profile.json")
    e.load_param_from_file(base + ".param")
    st = j["storage"][0]
    rng = np.random.default_rng(1)
    x = rng.integers(0, 30522, st["size"]).astype(np.int64) if st["stype"] == "int64" else rng.normal(0, 1, st["size"]).astype(np.float32)
    e.set_input(st["name"], x)
    e.execute()     # every buffer holds real activations
    peak, kind = peak_gbs()
    rows, seen = [], {}
    for i, k in enumerate(j["kernels"]):
        if k["name"] in seen:
            seen[k["name"]]["launches"] += 1
            continue
        flops, nbytes, tc = capi.kernel_cost(k["name"])
        us = e.time_kernel(i, reps=reps, iters=iters)
        row = dict(name=k["name"], launches=1, us=us, bytes=nbytes, flops=flops, tensor_core=tc,
                   gbs=nbytes / us * 1e-3, frac_hbm=nbytes / us * 1e-3 / peak, tflops=flops / us * 1e-6,
                   blocks=int(np.prod(k["launch_params"][:3])))
        seen[k["name"]] = row
        rows.append(row)
    e.close()
    return dict(model=model + variant, peak_gbs=peak, peak_kind=kind, kernels=rows)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="resnet152")
    ap.add_argument("--variant", default="")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    t = kernel_table(a.model, a.device, a.variant)
    print(f"# {t['model']}: kernels timed alone; HBM peak {t['peak_gbs']:.0f} GB/s ({t['peak_kind']})")
    print(f"{'us':>8} {'MB':>8} {'GB/s':>8} {'of peak':>8} {'TFLOP/s':>8} {'blocks':>7} {'x':>4}  kernel")
    for r in sorted(t["kernels"], key=lambda r: -r["us"] * r["launches"]):
        print(f"{r['us']:8.2f} {r['bytes'] / 1e6:8.2f} {r['gbs']:8.0f} {r['frac_hbm']:8.3f} {r['tflops']:8.2f} {r['blocks']:7d} {r['launches']:4d}  {r['name']}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump(t, f, indent=1)


if __name__ == "__main__":
    main()
