"""Algorithmic work of a model schedule: flops and bytes per kernel family and in total, and the roofline floors.

``python -m reef_b200.flops [model ...] [--dir DIR] [--markdown]`` reads ``<model>.json`` (generated on demand)
and sums ``reef_kernel_cost`` over its kernels.  Formulas (per launch): convolution 2·Cout·Cin·k²·Ho·Wo flops and
4·(Cin·Hi·Wi + Cout·Cin·k² + Cout·Ho·Wo [×2 with a residual] [+ Cout·Ho·Wo for a second output] + Cout·{0,1,2})
bytes; dense 2·N·K and 4·(N·K + K + 2N); attention 4·heads·S²·d and 4·(3·S·H + S·H); everything else bytes only.
Needs no GPU.
"""
from __future__ import annotations

import argparse
import collections
import json
import os

from . import capi, resources

HBM_TBS_NOMINAL = 7.7        # B200 HBM3e, TB/s
TF32_PFLOPS_NOMINAL = 1.1    # dense TF32 tensor peak, PFLOP/s


def model_totals(model: str, out_root: str | None = None, variant: str = "") -> dict:
    d = resources.generate(model, out_root, variant=variant)
    j = json.load(open(os.path.join(d, model + variant + ".json")))
    fam = collections.OrderedDict()
    tot = dict(kernels=0, tensor_core_kernels=0, flops=0.0, bytes=0.0, weight_bytes=0.0)
    for k in j["kernels"]:
        fl, by, tc = capi.kernel_cost(k["name"])
        f = fam.setdefault(k["name"].split("__")[0] + (" (tensor core)" if tc else ""), dict(kernels=0, flops=0.0, bytes=0.0))
        f["kernels"] += 1
        f["flops"] += fl
        f["bytes"] += by
        tot["kernels"] += 1
        tot["tensor_core_kernels"] += tc
        tot["flops"] += fl
        tot["bytes"] += by
    tot["weight_bytes"] = 4.0 * sum(s["size"] for s in j["storage"] if s["name"] not in ("null", "output", "temp", "data")
                                    and not s["name"].startswith("input"))
    tot["hbm_floor_us_nominal"] = tot["bytes"] / (HBM_TBS_NOMINAL * 1e12) * 1e6
    tot["tf32_floor_us_nominal"] = tot["flops"] / (TF32_PFLOPS_NOMINAL * 1e15) * 1e6
    return dict(model=model + variant, totals=tot, families=fam)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("models", nargs="*", default=["resnet18", "resnet50", "resnet152", "vgg16", "densenet201",
                                                  "inception_v3", "bert_base"])
    ap.add_argument("--dir", default=None)
    ap.add_argument("--markdown", action="store_true")
    args = ap.parse_args(argv)
    rows = [model_totals(m, args.dir) for m in args.models]
    if not args.markdown:
        print(json.dumps(rows, indent=1))
        return
    print("| model | kernels (tensor-core) | GFLOP | algorithmic MB | weight MB | HBM floor us (7.7 TB/s) | TF32 floor us (1.1 PF/s) |")
    print("|---|---|---|---|---|---|---|")
    for r in rows:
        t = r["totals"]
        print(f"| {r['model']} | {t['kernels']} ({t['tensor_core_kernels']}) | {t['flops'] / 1e9:.2f} | {t['bytes'] / 1e6:.1f} | "
              f"{t['weight_bytes'] / 1e6:.1f} | {t['hbm_floor_us_nominal']:.1f} | {t['tf32_floor_us_nominal']:.1f} |")


if __name__ == "__main__":
    main()
