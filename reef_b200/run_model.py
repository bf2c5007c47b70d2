"""Run one model through the executor and print its latency.

    python -m reef_b200.run_model --model resnet152 [--variant _fp32] [--mode raw|graph|be|dispatch|chain] [--iters 20]

``raw`` launches the kernels of <model>.json one by one (the reference's ExecutorBase::execute,
src/reef/executor/executor_base.cpp:196-223), ``graph`` replays a CUDA graph of them, ``be`` uses the
best-effort flavour (preempt flag + completion counters), ``dispatch`` sends every kernel through the
dynamic-kernel-padding entry point without a partner, ``chain`` runs every run of consecutive tensor-core layers as
one persistent kernel (``--clusters`` sets its grid) and the other kernels one by one.  The first model output values are printed so that a
run under a profiler can be checked against a plain run.
"""
from __future__ import annotations

import argparse
import os
import time

import numpy as np


def main():
    from . import capi, resources
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet152")
    ap.add_argument("--variant", default="")
    ap.add_argument("--mode", default="raw", choices=["raw", "graph", "be", "dispatch", "chain"])
    ap.add_argument("--clusters", type=int, default=0, help="clusters of a chain kernel's grid (0: the default)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args()
    d = resources.generate(a.model, variant=a.variant)
    base = os.path.join(d, os.path.basename(d))
    e = capi.HybridExecutor(a.device)
    e.load_model_from_file(base + ".json", base + ".profile.json")
    if os.path.exists(base + ".param"):
        e.load_param_from_file(base + ".param")
    for name in ("data", "input0", "a", "b", "c"):
        try:
            n = e.get_data_size(name)
        except capi.ReefError:
            continue
        rng = np.random.default_rng(2001)
        if name == "input0":      # token ids
            e.set_input(name, rng.integers(0, 30522, n // 8).astype(np.int64))
        else:
            e.set_input(name, rng.normal(0, 1, n // 4).astype(np.float32))
    if a.mode == "chain":
        print("chains:", e.build_chains(a.clusters), "first:", e.chain_info(0))
    run = {"chain": e.execute_chained, "raw": e.execute, "graph": e.execute_graph, "be": e.execute_preemptable, "dispatch": e.execute_dispatch}[a.mode]
    t0 = time.perf_counter()
    for _ in range(a.iters):
        run()
    dt = (time.perf_counter() - t0) / max(1, a.iters)
    out = e.get_output()
    print(f"{a.model}{a.variant} mode={a.mode} iters={a.iters} wall_ms_per_iter={dt * 1e3:.3f} kernels={e.num_kernels()} "
          f"launches={capi.launch_count()} device_error={capi.device_error()} out[:4]={out[:4]}")


if __name__ == "__main__":
    main()
