"""Independent interpretation of a schedule graph with PyTorch CPU ops.

TEST INFRASTRUCTURE ONLY, like the rest of ``oracle/``: the tests cross-check the plain-C oracle against it (the
two share no arithmetic code), and ``bench.py`` times it as the second CPU baseline row (PyTorch on all host cores).
Layout contract as in reef_b200/resources/graph.py (NHWC activations, OHWI weights, NCHW model input).  Per-op math
follows the same reference kernels the C oracle cites (conv / pool / dense / softmax: resource/resnet152/resnet152.cu;
LayerNorm eps 1e-12, exact-erf GELU, clamped embedding ids, masked softmax: resource/bert/bert.cu)."""
from __future__ import annotations

import json
import math

import numpy as np
import torch
import torch.nn.functional as F

from .oracle import parse_kname


def _read_params(path):
    import struct
    out = {}
    with open(path, "rb") as f:
        assert f.read(17) == b"TVM_MODEL_PARAMS\0", "bad .param magic"
        (count,) = struct.unpack("<Q", f.read(8))
        for _ in range(count):
            key = bytearray()
            while True:
                c = f.read(1)
                if c == b"\0":
                    break
                key += c
            (n,) = struct.unpack("<Q", f.read(8))
            out[key.decode()] = np.frombuffer(f.read(4 * n), dtype="<f4")
    return out


class TorchExecutor:
    """set_input / execute / storage, like OracleExecutor.  Weights are converted to PyTorch's layouts once, at
    construction, so that execute() times the operators and not the conversions."""

    def __init__(self, json_path: str, param_path: str | None = None, double: bool = False):
        self.model = json.load(open(json_path))
        self.dt = torch.float64 if double else torch.float32
        self.names = [s["name"] for s in self.model["storage"]]
        self.t = []
        for s in self.model["storage"]:
            self.t.append(torch.zeros(s["size"], dtype=self.dt if s["stype"] == "float32" else torch.int64))
        if param_path:
            for n, v in _read_params(param_path).items():
                if n in self.names:
                    i = self.names.index(n)
                    self.t[i][: v.size] = torch.from_numpy(np.array(v)).to(self.dt)
        self.steps = [self._compile(k) for k in self.model["kernels"]]

    def set_input(self, name, value):
        i = self.names.index(name)
        v = torch.from_numpy(np.ascontiguousarray(np.asarray(value).reshape(-1)))
        self.t[i][:] = v.to(self.t[i].dtype)

    def execute(self):
        with torch.no_grad():
            for f in self.steps:
                f()

    @property
    def storage(self):
        return [x.to(torch.float32).numpy() if x.dtype != torch.int64 else x.numpy() for x in self.t]

    def get_output(self, name="output"):
        return self.t[self.names.index(name)].to(torch.float32).numpy().copy()

    # ---- one closure per kernel ---------------------------------------------------------------------------
    def _compile(self, k):
        op, a = parse_kname(k["name"])
        args = k["args"]
        t = self.t
        if op in ("add", "multiply"):
            def f():
                x = t[args[0]][:128].repeat(64)
                t[args[2]][:] = x + t[args[1]] if op == "add" else x * t[args[1]]
            return f
        if op == "fused_add":
            def f():
                t[args[0]][:] = (t[args[1]].view(a["c"], a["hw"]) + t[args[2]][:, None]).reshape(-1)
            return f
        if op == "reef_nchw_to_nhwc4":
            def f():
                x = t[args[1]].view(a["c"], a["hw"]) + t[args[2]][:, None]
                y = torch.zeros(a["hw"], 4, dtype=x.dtype)
                y[:, :a["c"]] = x.T
                t[args[0]][:] = y.reshape(-1)
            return f
        if op == "reef_im2col_nchw":
            def f():
                c, hi, wi, kh, kw, kp = a["c"], a["hi"], a["wi"], a["kh"], a["kw"], a["kp"]
                x = t[args[1]].view(1, c, hi, wi) + t[args[2]].view(1, c, 1, 1)
                cols = F.unfold(x, (kh, kw), padding=(a["ph"], a["pw"]), stride=(a["sh"], a["sw"]))[0]   # [c*kh*kw][P], (c, ky, kx) order
                P = cols.shape[1]
                cols = cols.view(c, kh * kw, P).permute(2, 1, 0).reshape(P, kh * kw * c)                   # -> (ky, kx, c) order
                y = torch.zeros(P, kp, dtype=x.dtype)
                y[:, :kh * kw * c] = cols
                t[args[0]][:] = y.reshape(-1)
            return f
        if op == "fused_add_nn_relu":
            ics, ioff = a.get("ics", a["c"]), a.get("ioff", 0)

            def f():
                x = t[args[1]].view(a["n"], ics)[:, ioff:ioff + a["c"]]
                t[args[0]][:] = torch.relu(x + t[args[2]][None, :]).reshape(-1)
            return f
        if op.startswith("fused_nn_conv2d") or op == "reef_conv2d_add_preact":
            return self._conv(op, a, args)
        if op in ("fused_nn_max_pool2d", "fused_nn_max_pool2d_add_nn_relu", "fused_nn_avg_pool2d"):
            c, hi, wi = a["c"], a["hi"], a["wi"]
            ics, ioff = a.get("ics", c), a.get("ioff", 0)
            ocs, ooff = a.get("ocs", c), a.get("ooff", 0)
            ceil = ((hi + 2 * a["p"] - a["k"]) % a["s"]) != 0 and a["ho"] == -(-(hi + 2 * a["p"] - a["k"]) // a["s"]) + 1

            def f():
                x = t[args[0]].view(hi, wi, ics)[:, :, ioff:ioff + c].permute(2, 0, 1)[None]
                if op == "fused_nn_avg_pool2d":
                    y = F.avg_pool2d(x, a["k"], a["s"], a["p"], ceil_mode=ceil, count_include_pad=bool(a.get("cip", 1)))
                else:
                    y = F.max_pool2d(x, a["k"], a["s"], a["p"], ceil_mode=ceil)
                y = y[0].permute(1, 2, 0)
                if op.endswith("_add_nn_relu"):
                    y = torch.relu(y + t[args[2]])
                t[args[1]].view(a["ho"] * a["wo"], ocs)[:, ooff:ooff + c] = y.reshape(-1, c)
            return f
        if op == "fused_nn_global_avg_pool2d":
            def f():
                t[args[1]][:] = t[args[0]].view(a["hw"], a["c"]).mean(0)
            return f
        if op == "fused_nn_batch_flatten":
            def f():
                t[args[0]][:] = t[args[1]]
            return f
        if op in ("fused_nn_dense_add", "fused_nn_dense_add_nn_relu"):
            w = t[args[1]].view(a["n"], a["k"])

            def f():
                y = torch.addmv(t[args[3]], w, t[args[0]])
                t[args[2]][:] = torch.relu(y) if op.endswith("_nn_relu") else y
            return f
        if op == "fused_nn_softmax":
            def f():
                t[args[1]][:] = torch.softmax(t[args[0]].view(a.get("rows", 1), a["n"]), dim=-1).reshape(-1)
            return f
        if op == "reef_embedding":      # out, word, ids, pos (reference: bert.cu:313-325, ids clamped)
            s, h, vocab = a["s"], a["h"], a["vocab"]

            def f():
                ids = t[args[2]][:s].clamp(0, vocab - 1)
                t[args[0]][:] = (t[args[1]].view(vocab, h)[ids] + t[args[3]].view(-1, h)[:s]).reshape(-1)
            return f
        if op in ("reef_layernorm", "reef_add_layernorm"):   # two-pass variance, eps 1e-12 inside the sqrt (bert.cu:201)
            rows, h = a["rows"], a["h"]
            has_res = op == "reef_add_layernorm"

            def f():
                x = t[args[1]].view(rows, h)
                if has_res:
                    x = x + t[args[2]].view(rows, h)
                g, b = t[args[3 if has_res else 2]], t[args[4 if has_res else 3]]
                mu = x.mean(1, keepdim=True)
                var = ((x - mu) ** 2).mean(1, keepdim=True)
                t[args[0]][:] = ((x - mu) / torch.sqrt(var + 1e-12) * g + b).reshape(-1)
            return f
        if op.startswith("reef_matmul_nt"):      # A[m][k], B[n][k], out[m][n], [bias], [residual]
            tail = op[len("reef_matmul_nt"):]
            m, n, kk = a["m"], a["n"], a["k"]
            rest = list(args[3:])
            bias = rest.pop(0) if "_bias" in tail else None
            res = rest.pop(0) if "_residual" in tail else None

            def f():
                y = t[args[0]].view(m, kk) @ t[args[1]].view(n, kk).T
                if bias is not None:
                    y = y + t[bias]
                if "_gelu" in tail:   # exact-erf form (bert.cu:170)
                    y = y * (0.5 * torch.erf(y * 0.7071067811865476) + 0.5)
                if res is not None:
                    y = y + t[res].view(m, n)
                t[args[2]][:] = y.reshape(-1)
            return f
        if op == "reef_attention":      # qkv [s][3H], [mask], out [s][H]
            s, heads, d = a["s"], a["heads"], a["d"]
            H = heads * d
            has_mask = bool(a.get("mask", 0))

            def f():
                qkv = t[args[0]].view(s, 3, heads, d)
                q, kx, v = qkv[:, 0].permute(1, 0, 2), qkv[:, 1].permute(1, 0, 2), qkv[:, 2].permute(1, 0, 2)
                sc = (q @ kx.transpose(1, 2)) / math.sqrt(d)
                if has_mask:
                    sc = sc.masked_fill(t[args[1]][None, None, :s] == 0, float("-inf"))
                p = torch.softmax(sc, dim=-1)
                t[args[-1]][:] = (p @ v).permute(1, 0, 2).reshape(-1)
            return f
        raise KeyError(op)

    def _conv(self, op, a, args):
        t = self.t
        tail = "_add" if op == "reef_conv2d_add_preact" else op[len("fused_nn_conv2d"):]
        relu = tail.endswith("_nn_relu")
        if relu:
            tail = tail[:-8]
        ci, hi, wi, co = a["ci"], a["hi"], a["wi"], a["co"]
        ics, ioff = a.get("ics", ci), a.get("ioff", 0)
        ocs, ooff = a.get("ocs", co), a.get("ooff", 0)
        w = t[args[1]].view(co, a["kh"], a["kw"], ci).permute(0, 3, 1, 2).contiguous()   # OHWI -> OIHW, once
        rest = args[3:]
        nchw = bool(a.get("nchw", 0))
        stride, pad = (a["sh"], a["sw"]), (a["ph"], a["pw"])

        def f():
            if nchw:
                x = t[args[0]].view(1, ci, hi, wi)
            else:
                x = t[args[0]].view(hi, wi, ics)[:, :, ioff:ioff + ci].permute(2, 0, 1)[None]
            y = F.conv2d(x, w, None, stride, pad)[0].permute(1, 2, 0)   # HWC
            if tail == "_add":
                y = y + (t[rest[0]] if relu else t[rest[0]].view(y.shape))
            elif tail == "_add_add":
                y = y + t[rest[0]].view(y.shape) + t[rest[1]]
            elif tail == "_add_multiply_add":
                y = (y + t[rest[0]].view(y.shape)) * t[rest[1]] + t[rest[2]]
            if relu:
                y = torch.relu(y)
            y2 = y.reshape(-1, co)
            t[args[2]].view(-1, ocs)[:, ooff:ooff + co] = y2
            if op == "reef_conv2d_add_preact":   # second output: the next unit's pre-activation
                t[args[5]][:] = torch.relu(y2 + t[args[4]][None, :]).reshape(-1)
        return f


def run_graph(json_path: str, param_path: str | None, inputs: dict, double: bool = False):
    """One pass; returns (list of numpy storage buffers, storage names)."""
    e = TorchExecutor(json_path, param_path, double)
    for k, v in inputs.items():
        e.set_input(k, v)
    e.execute()
    return e.storage, e.names
