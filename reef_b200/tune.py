"""Measured launch plans for the tensor-core kernel (needs a B200).

A batch-1 layer is a tiny GEMM; how it is cut — pixel-tile cap ``tp`` (how many CTAs, how often weights are
re-read from L2) and K splits ``ts`` (cluster size, exchange cost) — decides its latency, and the best cut
depends on the shape.  The reference obtains its per-layer schedules from TVM's auto-tuner (reference:
script/tvm_generate_model.py); here every distinct tensor-core kernel name of a model is timed under each
candidate plan and the fastest is recorded in ``reef_b200/resources/tuned_plans.json``, which the resource
generators read (``tuned_plan``) and write into the kernel names.

Method: one CUDA graph of N launches of the candidate, each launch with its own weight buffer so that weights
come from HBM as in a real pass (N x weights >= 200 MB, more than the L2), replayed 20 times; the launches keep
their programmatic dependencies on one another, as in a model's graph.

    python -m reef_b200.tune --models resnet152 bert_base [--out reef_b200/resources/tuned_plans.json]
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import tempfile

import numpy as np

from . import capi, resources
from .resources.graph import Graph, parse_kname

CAPS = (208, 160, 112, 96, 64, 48, 32)
SPLITS = (1, 2, 4, 8)
DEFAULT_OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "resources", "tuned_plans.json")


NOTE = ("written by python -m reef_b200.tune on one B200: plans = kernel name -> [tile cap tp, K splits ts], kept only "
        "where the whole-model replay gets faster; measured_us = kernel name -> [default plan, best plan] microseconds "
        "per launch on its own; models_ms = model -> [replay ms with default plans, with the kept plans, plans kept, "
        "plans tried]")


def _write_table(table: dict, path: str):
    """One entry per line, sorted, so that a re-tune shows up as a readable diff."""
    def block(name):
        items = sorted(table.get(name, {}).items())
        return f' "{name}": {{\n' + ",\n".join(f'  "{k}": {json.dumps(v)}' for k, v in items) + "\n }"
    with open(path, "w") as f:
        f.write('{\n "note": ' + json.dumps(NOTE) + ",\n" + ",\n".join(block(n) for n in ("models_ms", "plans", "measured_us")) + "\n}\n")


def _arg_sizes(op: str, a: dict):
    """(input size, weight size, output size, [(role, size) of the remaining arguments]) in floats."""
    if op.startswith("reef_matmul_nt"):
        m, n, k = a["m"], a["n"], a["k"]
        extra = [("param", n)] + ([("temp", m * n)] if "_residual" in op else [])
        return m * k, n * k, m * n, extra
    ho = (a["hi"] + 2 * a["ph"] - a["kh"]) // a["sh"] + 1
    wo = (a["wi"] + 2 * a["pw"] - a["kw"]) // a["sw"] + 1
    co, p = a["co"], ho * wo
    ics, ocs = a.get("ics", a["ci"]), a.get("ocs", co)
    tail = op[len("fused_nn_conv2d"):] if op.startswith("fused_nn_conv2d") else None
    if op == "reef_conv2d_add_preact":
        extra = [("temp", p * co), ("param", co), ("temp", p * co)]
    elif tail in ("", "_nn_relu"):
        extra = []
    elif tail == "_add_nn_relu":
        extra = [("param", co)]
    elif tail == "_add":
        extra = [("temp", p * co)]
    elif tail in ("_add_add", "_add_add_nn_relu"):
        extra = [("temp", p * co), ("param", co)]
    elif tail in ("_add_multiply_add", "_add_multiply_add_nn_relu"):
        extra = [("temp", p * co), ("param", co), ("param", co)]
    else:
        raise KeyError(op)
    return a["hi"] * a["wi"] * ics, co * a["kh"] * a["kw"] * a["ci"], p * ocs, extra


def time_name(name: str, workdir: str, min_bytes: float = 200e6, replays: int = 20) -> float:
    """Average microseconds per launch of `name` inside a graph of launches with distinct weights."""
    op, a = parse_kname(name)
    n_in, n_w, n_out, extra = _arg_sizes(op, a)
    copies = int(max(24, min(400, min_bytes // (4 * n_w))))
    g = Graph("tune")
    x = g.input("data", n_in)
    o = g.add_storage("output", n_out)
    rest = [g.add_storage("temp", sz) for _, sz in extra]      # zero-filled arena slices; values do not matter
    for _ in range(copies):
        g.kernel(name, [x, g.add_storage("temp", n_w), o] + rest)
    base = g.write(workdir, capi.plan_fn)
    e = capi.HybridExecutor(0)
    e.load_model_from_file(base + ".json", base + ".profile.json")
    us = e.time(1, 3, replays) * 1000.0 / copies
    e.close()
    return us


def candidates(name: str):
    """Distinct plans reachable for `name`: [(suffix attrs or None for the default plan, grid, smem)]."""
    d, smem, _ = capi.kernel_plan(name)
    out = [(None, tuple(d[:2]), smem)]
    for cap, s in itertools.product(CAPS, SPLITS):
        try:
            d2, sm2, _ = capi.kernel_plan(f"{name}_tp{cap}_ts{s}")
        except capi.ReefError:
            continue
        key = (tuple(d2[:2]), sm2)
        if d2[0] != s and s != 1:
            continue        # the planner could not honour this split count
        if not 24 <= d2[0] * d2[1] <= 300:
            continue        # too few CTAs to stream the weights, or more than the SMs hold at once
        if any(c[1:] == key for c in out[1:]):
            continue
        out.append((dict(tp=cap, ts=s), key[0], key[1]))
    return out


def tune_name(name: str, workdir: str, verbose: bool = True):
    rows = []
    for attrs, grid, smem in candidates(name):
        full = name if attrs is None else f"{name}_tp{attrs['tp']}_ts{attrs['ts']}"
        rows.append((time_name(full, workdir), attrs, grid, smem))
    default_us = rows[0][0]
    best = min(rows, key=lambda r: r[0])
    if verbose:
        print(f"{name}: default {rows[0][2]} {default_us:.2f} us -> best {best[1]} {best[2]} {best[0]:.2f} us", flush=True)
    # keep the default unless a candidate is clearly faster (2 %: below that it is measurement noise)
    if best[1] is None or best[0] > 0.98 * default_us:
        return None, default_us, default_us
    return best[1], best[0], default_us


def tune_models(models, out_path: str = DEFAULT_OUT, variant: str = ""):
    table = json.load(open(out_path)) if os.path.exists(out_path) else {"plans": {}, "measured_us": {}}
    os.environ["REEF_UNTUNED"] = "1"          # generate the schedules with bare names
    names = []
    for m in models:
        d = resources.generate(m, variant=variant)
        for k in json.load(open(os.path.join(d, m + variant + ".json")))["kernels"]:
            fl, by, tc = capi.kernel_cost(k["name"])
            # (the tensor-core attention kernel has one CTA per head: no tile cap or K split to choose)
            if tc and not k["name"].startswith("reef_attention") and k["name"] not in names:
                names.append(k["name"])
    del os.environ["REEF_UNTUNED"]
    with tempfile.TemporaryDirectory() as wd:
        for n in names:
            if n in table["measured_us"]:
                continue
            attrs, us, default_us = tune_name(n, wd)
            table["measured_us"][n] = [round(default_us, 3), round(us, 3)]
            if attrs:
                table["plans"][n] = [attrs["tp"], attrs["ts"]]
            _write_table(table, out_path)
    return table


def _time_schedule(j: dict, plans: dict, workdir: str, tag: str, replays: int = 30) -> float:
    """Whole-model CUDA-graph replay (ms) of schedule `j` with `plans` written into its kernel names.
    Parameters stay zero (the arena is zero-filled): timing does not depend on the values."""
    j = json.loads(json.dumps(j))
    for k in j["kernels"]:
        hit = plans.get(k["name"])
        if hit:
            n2 = f"{k['name']}_tp{hit[0]}_ts{hit[1]}"
            dims, smem, _ = capi.kernel_plan(n2)
            k["name"], k["launch_params"] = n2, dims
            j["shared_memory"][n2] = smem
    base = os.path.join(workdir, tag)
    with open(base + ".json", "w") as f:
        json.dump(j, f)
    e = capi.HybridExecutor(0)
    e.load_model_from_file(base + ".json", None)
    ms = e.time(1, 5, replays)
    e.close()
    return ms


def verify_models(models, out_path: str = DEFAULT_OUT):
    """Second pass: a plan that wins on its own can lose inside a model (its neighbours' early prologues compete
    for the same SMs), so every tuned plan is re-checked where it is used: starting from the default plans of a
    model, plans are applied one name at a time, largest isolated gain first, and kept only if the whole-model
    replay gets faster.  Plans that no model keeps are dropped from the table."""
    table = json.load(open(out_path))
    keep, report = {}, {}
    os.environ["REEF_UNTUNED"] = "1"
    with tempfile.TemporaryDirectory() as wd:
        for m in models:
            d = resources.generate(m)
            j = json.load(open(os.path.join(d, m + ".json")))
            used = [k["name"] for k in j["kernels"]]
            cand = [n for n in dict.fromkeys(used) if n in table["plans"]]
            cand.sort(key=lambda n: (table["measured_us"][n][0] - table["measured_us"][n][1]) * used.count(n), reverse=True)
            applied = {n: keep[n] for n in cand if n in keep}          # accepted for an earlier model
            t0 = _time_schedule(j, {}, wd, m)
            best = _time_schedule(j, applied, wd, m) if applied else t0
            for n in cand:
                if n in applied:
                    continue
                trial = dict(applied)
                trial[n] = table["plans"][n]
                t = _time_schedule(j, trial, wd, m)
                if t < 0.998 * best:
                    applied, best = trial, t
            keep.update(applied)
            report[m] = [round(t0, 4), round(best, 4), len(applied), len(cand)]
            print(f"{m}: default plans {t0:.4f} ms -> {best:.4f} ms with {len(applied)} of {len(cand)} tuned plans", flush=True)
    del os.environ["REEF_UNTUNED"]
    table["plans"] = keep
    table["models_ms"] = report
    _write_table(table, out_path)
    return table


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--models", nargs="+", default=["resnet152"])
    ap.add_argument("--out", default=DEFAULT_OUT)
    ap.add_argument("--verify-only", action="store_true", help="skip the per-kernel pass, re-check the table's plans in the models")
    args = ap.parse_args(argv)
    if args.verify_only:
        verify_models(args.models, args.out)
        return
    t = tune_models(args.models, args.out)
    verify_models(args.models, args.out)
    d = sum(v[0] for v in t["measured_us"].values())
    b = sum(v[1] for v in t["measured_us"].values())
    print(f"{len(t['measured_us'])} kernel names measured, {len(t['plans'])} tuned plans; "
          f"sum of per-launch times {d:.1f} us (default plans) -> {b:.1f} us")


if __name__ == "__main__":
    main()
