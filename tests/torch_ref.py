"""Independent fp32 interpretation of a schedule graph with PyTorch CPU ops (test helper).

Used to cross-check the plain-C oracle: the two share no arithmetic code.  Layout contract as in
reef_b200/resources/graph.py (NHWC activations, OHWI weights, NCHW model input)."""
from __future__ import annotations

import json

import numpy as np
import torch
import torch.nn.functional as F

from oracle.oracle import parse_kname
from reef_b200.resources.graph import read_param_file


def run_graph(json_path: str, param_path: str | None, inputs: dict, double: bool = False):
    model = json.load(open(json_path))
    dt = torch.float64 if double else torch.float32
    st = [np.zeros(s["size"], dtype=np.float32 if s["stype"] == "float32" else np.int64) for s in model["storage"]]
    names = [s["name"] for s in model["storage"]]
    if param_path:
        params = read_param_file(param_path)
        for i, n in enumerate(names):
            if n in params:
                st[i][: params[n].size] = params[n]
    for k, v in inputs.items():
        st[names.index(k)][:] = np.asarray(v).reshape(-1)

    def T(i):
        return torch.from_numpy(st[i]).to(dt) if st[i].dtype == np.float32 else torch.from_numpy(st[i])

    def put(i, t, view=None):
        st[i][:] = t.to(torch.float32).reshape(-1).numpy()

    for k in model["kernels"]:
        op, a = parse_kname(k["name"])
        args = k["args"]
        if op in ("add", "multiply"):
            x = T(args[0])[:128].repeat(64)
            y = T(args[1])
            put(args[2], x + y if op == "add" else x * y)
        elif op == "fused_add":
            x = T(args[1]).reshape(a["c"], a["hw"])
            put(args[0], x + T(args[2])[:, None])
        elif op == "reef_nchw_to_nhwc4":
            x = T(args[1]).reshape(a["c"], a["hw"]) + T(args[2])[:, None]
            y = torch.zeros(a["hw"], 4, dtype=x.dtype)
            y[:, :a["c"]] = x.T
            put(args[0], y)
        elif op == "fused_add_nn_relu":
            ics, ioff = a.get("ics", a["c"]), a.get("ioff", 0)
            x = T(args[1]).reshape(a["n"], ics)[:, ioff:ioff + a["c"]]
            put(args[0], torch.relu(x + T(args[2])[None, :]))
        elif op.startswith("fused_nn_conv2d") or op == "reef_conv2d_add_preact":
            tail = "_add" if op == "reef_conv2d_add_preact" else op[len("fused_nn_conv2d"):]
            relu = tail.endswith("_nn_relu")
            if relu:
                tail = tail[:-8]
            ci, hi, wi, co = a["ci"], a["hi"], a["wi"], a["co"]
            ics, ioff = a.get("ics", ci), a.get("ioff", 0)
            ocs, ooff = a.get("ocs", co), a.get("ooff", 0)
            if a.get("nchw", 0):
                x = T(args[0]).reshape(1, ci, hi, wi)
            else:
                x = T(args[0]).reshape(hi, wi, ics)[:, :, ioff:ioff + ci].permute(2, 0, 1)[None]
            w = T(args[1]).reshape(co, a["kh"], a["kw"], ci).permute(0, 3, 1, 2)
            y = F.conv2d(x, w, None, (a["sh"], a["sw"]), (a["ph"], a["pw"]))[0].permute(1, 2, 0)  # HWC
            rest = args[3:]
            if tail == "_add":
                if relu:
                    y = y + T(rest[0])
                else:
                    y = y + T(rest[0]).reshape(y.shape)
            elif tail == "_add_add":
                y = y + T(rest[0]).reshape(y.shape) + T(rest[1])
            elif tail == "_add_multiply_add":
                y = (y + T(rest[0]).reshape(y.shape)) * T(rest[1]) + T(rest[2])
            if relu:
                y = torch.relu(y)
            ho, wo = y.shape[0], y.shape[1]
            buf = T(args[2]).reshape(ho * wo, ocs).clone()
            buf[:, ooff:ooff + co] = y.reshape(ho * wo, co)
            put(args[2], buf)
            if op == "reef_conv2d_add_preact":   # second output: the next unit's pre-activation
                put(args[5], torch.relu(y.reshape(ho * wo, co) + T(args[4])[None, :]))
        elif op in ("fused_nn_max_pool2d", "fused_nn_max_pool2d_add_nn_relu", "fused_nn_avg_pool2d"):
            c, hi, wi = a["c"], a["hi"], a["wi"]
            ics, ioff = a.get("ics", c), a.get("ioff", 0)
            ocs, ooff = a.get("ocs", c), a.get("ooff", 0)
            x = T(args[0]).reshape(hi, wi, ics)[:, :, ioff:ioff + c].permute(2, 0, 1)[None]
            ceil = ((hi + 2 * a["p"] - a["k"]) % a["s"]) != 0 and a["ho"] == -(-(hi + 2 * a["p"] - a["k"]) // a["s"]) + 1
            if op == "fused_nn_avg_pool2d":
                y = F.avg_pool2d(x, a["k"], a["s"], a["p"], ceil_mode=ceil, count_include_pad=bool(a.get("cip", 1)))
            else:
                y = F.max_pool2d(x, a["k"], a["s"], a["p"], ceil_mode=ceil)
            y = y[0].permute(1, 2, 0)
            if op.endswith("_add_nn_relu"):
                y = torch.relu(y + T(args[2]))
            buf = T(args[1]).reshape(a["ho"] * a["wo"], ocs).clone()
            buf[:, ooff:ooff + c] = y.reshape(-1, c)
            put(args[1], buf)
        elif op == "fused_nn_global_avg_pool2d":
            put(args[1], T(args[0]).reshape(a["hw"], a["c"]).mean(0))
        elif op == "fused_nn_batch_flatten":
            put(args[0], T(args[1]))
        elif op in ("fused_nn_dense_add", "fused_nn_dense_add_nn_relu"):
            y = T(args[1]).reshape(a["n"], a["k"]) @ T(args[0]) + T(args[3])
            put(args[2], torch.relu(y) if op.endswith("_nn_relu") else y)
        elif op == "fused_nn_softmax":
            put(args[1], torch.softmax(T(args[0]).reshape(a.get("rows", 1), a["n"]), dim=-1))
        else:
            raise KeyError(op)
    return st, names
