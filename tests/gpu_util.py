"""Helpers shared by the GPU parity tests."""
import json
import os

import numpy as np

from conftest import rel_err
from oracle import oracle
from reef_b200 import capi
from reef_b200.resources.graph import Graph, write_param_file

FP32_TOL = 1e-3    # fp32 kernels: max |y - ref| / max |ref|
TF32_TOL = 1e-2    # TF32 tensor-core kernels


def tol_for(base):
    """1e-2 when the schedule contains tensor-core (TF32) kernels, else 1e-3."""
    j = json.load(open(base + ".json"))
    return TF32_TOL if any("_v1" in k["name"] for k in j["kernels"]) else FP32_TOL


def load_executor(base, params=True):
    e = capi.HybridExecutor(0)
    e.load_model_from_file(base + ".json", base + ".profile.json" if os.path.exists(base + ".profile.json") else None)
    if params and os.path.exists(base + ".param"):
        e.load_param_from_file(base + ".param")
    return e


def all_storage(e, model_json):
    out = []
    for i, s in enumerate(model_json["storage"]):
        item = {"float32": 4, "int64": 8, "int32": 4, "byte": 1, "uint1": 1}[s["stype"]]
        dt = {"float32": np.float32, "int64": np.int64, "int32": np.int32, "byte": np.int8, "uint1": np.int8}[s["stype"]]
        out.append(e.get_data(i, s["size"] * item, dt))
    return out


def compare_layers(e, o, model_json, tol_of=lambda kname: FP32_TOL):
    """Compare every kernel's output buffer on the GPU with the oracle's; returns the worst (err, kernel)."""
    worst = (0.0, "")
    seen = set()
    for k in model_json["kernels"]:
        for a in k["args"]:
            if a in seen or model_json["storage"][a]["name"] not in ("null", "output", "temp"):
                continue
            seen.add(a)
            s = model_json["storage"][a]
            got = e.get_data(a, s["size"] * 4)
            err = rel_err(got, o.storage[a])
            assert err < tol_of(k["name"]), f"{k['name']} storage {a}: rel err {err}"
            if err > worst[0]:
                worst = (err, k["name"])
    return worst


def single_kernel_model(tmpdir, name, kernel_name, arg_specs, seed=0):
    """arg_specs: list of (role, size) with role in {'in','param','out'} in positional order.
    Inputs are named in<i> so both executors can set them."""
    g = Graph(name)
    rng = np.random.default_rng(seed)
    args, inputs = [], {}
    for i, (role, size) in enumerate(arg_specs):
        if role == "in":
            idx = g.input(f"in{i}", size)
            inputs[f"in{i}"] = rng.normal(0, 1, size).astype(np.float32)
        elif role == "param":
            idx = g.param(rng.normal(0, 1, size).astype(np.float32))
        else:
            idx = g.add_storage("output", size)
        args.append(idx)
    g.kernel(kernel_name, args)
    base = g.write(str(tmpdir), capi.plan_fn)
    return base, inputs
