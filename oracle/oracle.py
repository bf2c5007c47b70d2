"""Python driver of the CPU oracle: interprets a REEF ``<model>.json`` + ``.param``
kernel by kernel, calling the plain-C restatements in ``reef_oracle.c``.

TEST INFRASTRUCTURE ONLY — imported by ``tests/``, ``__graft_entry__.smoke()`` and
``bench.py``'s CPU-baseline legs; the product package never imports it.
Pinned per kernel family against the reference's own kernels run on the CPU
(tests/golden/ref_kernels.npz, see the header of ``reef_oracle.c``) and by the
mocked_kernel known answer (reference: src/reef/test/test.cpp:102-116); a
whole-network golden vector of the reference stays unavailable.

The interpretation of a kernel list mirrors what the reference executor does
with it (reference: src/reef/executor/executor_base.cpp:35-80,196-223): one
zero-filled buffer per storage entry, parameters copied in by name, kernels run
in order with positional storage arguments.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

_STYPE = {"float32": np.float32, "int64": np.int64, "int32": np.int32, "byte": np.int8, "uint1": np.int8}


def build(force: bool = False) -> str:
    so = os.path.join(_HERE, "libreef_oracle.so")
    src = os.path.join(_HERE, "reef_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def parse_kname(name: str):
    if "__" not in name:
        return name, {}
    op, tail = name.split("__", 1)
    attrs = {}
    for tok in tail.split("_"):
        i = 0
        while i < len(tok) and not tok[i].isdigit():
            i += 1
        attrs[tok[:i]] = int(tok[i:])
    return op, attrs


def num_threads() -> int:
    return int(lib().reef_oracle_num_threads())


def set_threads(n: int) -> None:
    lib().reef_oracle_set_threads(int(n))


def im2col_nchw(x, bias, a) -> np.ndarray:
    """[ho*wo][kp] im2col matrix of the planar tensor x [c][hi][wi] + bias[c] (numpy, fp32; attrs of the kernel name)."""
    c, hi, wi, kh, kw, sh, sw, ph, pw, kp = (a[k] for k in ("c", "hi", "wi", "kh", "kw", "sh", "sw", "ph", "pw", "kp"))
    ho, wo = (hi + 2 * ph - kh) // sh + 1, (wi + 2 * pw - kw) // sw + 1
    planar = np.asarray(x, np.float32).reshape(c, hi, wi) + np.asarray(bias, np.float32).reshape(c, 1, 1)
    padded = np.zeros((c, hi + 2 * ph, wi + 2 * pw), np.float32)
    padded[:, ph:ph + hi, pw:pw + wi] = planar
    out = np.zeros((ho, wo, kp), np.float32)
    for ky in range(kh):
        for kx in range(kw):
            tap = padded[:, ky:ky + (ho - 1) * sh + 1:sh, kx:kx + (wo - 1) * sw + 1:sw]   # [c][ho][wo]
            k0 = (ky * kw + kx) * c
            out[:, :, k0:k0 + c] = tap.transpose(1, 2, 0)
    return out.reshape(ho * wo, kp)


def run_kernel(name: str, bufs: list, acc64: bool = False) -> None:
    """Execute one kernel of the schedule on numpy buffers (positional, like the json)."""
    L = lib()
    op, a = parse_kname(name)
    i32 = C.c_int
    if op in ("add", "multiply"):
        fn = L.reef_oracle_mocked_add if op == "add" else L.reef_oracle_mocked_multiply
        fn(_p(bufs[0]), _p(bufs[1]), _p(bufs[2]), i32(64), i32(128))
    elif op == "fused_add":
        L.reef_oracle_fused_add_nchw(_p(bufs[0]), _p(bufs[1]), _p(bufs[2]), i32(a["c"]), i32(a["hw"]))
    elif op == "reef_nchw_to_nhwc4":
        # the reference's fused_add on the planar input (input + per-channel bias), written channels-last with
        # 4 channels per pixel (the 4th zero): bufs = out [hw][4], in [c][hw], bias [c]
        c, hw = a["c"], a["hw"]
        planar = np.empty(c * hw, np.float32)
        L.reef_oracle_fused_add_nchw(_p(planar), _p(bufs[1]), _p(bufs[2]), i32(c), i32(hw))
        out = bufs[0].reshape(hw, 4)
        out[:] = 0.0
        out[:, :c] = planar.reshape(c, hw).T
    elif op == "reef_im2col_nchw":
        # the planar input + per-channel bias (the reference's fused_add), gathered into the im2col matrix of the first
        # convolution: bufs = out [ho*wo][kp], in [c][hi][wi], bias [c]; k = (ky*kw + kx)*c + channel, zero beyond
        # kh*kw*c and where a tap falls into the padding
        bufs[0][:] = im2col_nchw(bufs[1], bufs[2], a).reshape(-1)
    elif op == "fused_add_nn_relu":
        L.reef_oracle_fused_add_nn_relu(_p(bufs[0]), _p(bufs[1]), _p(bufs[2]), i32(a["c"]), i32(a["n"]),
                                        i32(a.get("ics", a["c"])), i32(a.get("ioff", 0)))
    elif op == "reef_conv2d_add_preact":
        # one launch in the product; here the two reference kernels it stands for, one after the other
        # (fused_nn_conv2d_add, then fused_add_nn_relu of the next unit): bufs = in, weight, out, residual, bias2, out2
        conv_name = "fused_nn_conv2d_add__" + name.split("__", 1)[1]
        run_kernel(conv_name, bufs[:4], acc64)
        L.reef_oracle_fused_add_nn_relu(_p(bufs[5]), _p(bufs[2]), _p(bufs[4]), i32(a["co"]),
                                        i32(((a["hi"] + 2 * a["ph"] - a["kh"]) // a["sh"] + 1) *
                                            ((a["wi"] + 2 * a["pw"] - a["kw"]) // a["sw"] + 1)),
                                        i32(a["co"]), i32(0))
    elif op.startswith("fused_nn_conv2d"):
        tail = op[len("fused_nn_conv2d"):]
        relu = tail.endswith("_nn_relu")
        if relu:
            tail = tail[: -len("_nn_relu")]
        res = bias = gamma = beta = None
        inp, w, out = bufs[0], bufs[1], bufs[2]
        rest = list(bufs[3:])
        if tail == "":
            pass
        elif tail == "_add":
            if relu:
                bias = rest[0]
            else:
                res = rest[0]
        elif tail == "_add_add":
            res, bias = rest[0], rest[1]
        elif tail == "_add_multiply_add":
            res, gamma, beta = rest[0], rest[1], rest[2]
        else:
            raise KeyError(f"unknown conv family {op}")
        L.reef_oracle_conv2d(_p(inp), _p(w), _p(out), _p(res), _p(bias), _p(gamma), _p(beta), i32(int(relu)),
                             i32(a["ci"]), i32(a["hi"]), i32(a["wi"]), i32(a["co"]), i32(a["kh"]), i32(a["kw"]),
                             i32(a["sh"]), i32(a["sw"]), i32(a["ph"]), i32(a["pw"]), i32(a.get("nchw", 0)),
                             i32(a.get("ics", a["ci"])), i32(a.get("ioff", 0)),
                             i32(a.get("ocs", a["co"])), i32(a.get("ooff", 0)), i32(int(acc64)))
    elif op in ("fused_nn_max_pool2d", "fused_nn_max_pool2d_add_nn_relu"):
        bias = bufs[2] if op.endswith("_add_nn_relu") else None
        L.reef_oracle_max_pool2d(_p(bufs[0]), _p(bufs[1]), _p(bias), i32(a["c"]), i32(a["hi"]), i32(a["wi"]),
                                 i32(a["k"]), i32(a["s"]), i32(a["p"]), i32(a["ho"]), i32(a["wo"]),
                                 i32(a.get("ics", a["c"])), i32(a.get("ioff", 0)),
                                 i32(a.get("ocs", a["c"])), i32(a.get("ooff", 0)))
    elif op == "fused_nn_avg_pool2d":
        L.reef_oracle_avg_pool2d(_p(bufs[0]), _p(bufs[1]), i32(a["c"]), i32(a["hi"]), i32(a["wi"]),
                                 i32(a["k"]), i32(a["s"]), i32(a["p"]), i32(a["ho"]), i32(a["wo"]), i32(a.get("cip", 1)),
                                 i32(a.get("ics", a["c"])), i32(a.get("ioff", 0)),
                                 i32(a.get("ocs", a["c"])), i32(a.get("ooff", 0)))
    elif op == "fused_nn_global_avg_pool2d":
        L.reef_oracle_global_avg_pool2d(_p(bufs[0]), _p(bufs[1]), i32(a["c"]), i32(a["hw"]))
    elif op == "fused_nn_batch_flatten":
        L.reef_oracle_copy(_p(bufs[0]), _p(bufs[1]), C.c_size_t(a["n"]))
    elif op in ("fused_nn_dense_add", "fused_nn_dense_add_nn_relu"):
        L.reef_oracle_dense(_p(bufs[0]), _p(bufs[1]), _p(bufs[2]), _p(bufs[3]), i32(a["k"]), i32(a["n"]),
                            i32(int(op.endswith("_nn_relu"))), i32(int(acc64)))
    elif op == "fused_nn_softmax":
        L.reef_oracle_softmax(_p(bufs[0]), _p(bufs[1]), i32(a.get("rows", 1)), i32(a["n"]))
    elif op == "reef_embedding":
        L.reef_oracle_embedding(_p(bufs[0]), _p(bufs[1]), _p(bufs[2]), _p(bufs[3]),
                                i32(a["s"]), i32(a["h"]), i32(a["vocab"]))
    elif op in ("reef_layernorm", "reef_add_layernorm"):
        if op == "reef_add_layernorm":
            out, x, res, g, b = bufs[:5]
        else:
            out, x, g, b = bufs[:4]
            res = None
        L.reef_oracle_layernorm(_p(out), _p(x), _p(res), _p(g), _p(b), i32(a["rows"]), i32(a["h"]))
    elif op.startswith("reef_matmul_nt"):
        tail = op[len("reef_matmul_nt"):]
        A, B, out = bufs[0], bufs[1], bufs[2]
        rest = list(bufs[3:])
        bias = rest.pop(0) if "_bias" in tail else None
        res = rest.pop(0) if "_residual" in tail else None
        L.reef_oracle_matmul_nt(_p(A), _p(B), _p(out), _p(bias), _p(res), i32(a["m"]), i32(a["n"]), i32(a["k"]),
                                i32(int("_gelu" in tail)), i32(int(acc64)))
    elif op == "reef_attention":
        # args: qkv, [mask], out (the mask, when the name carries mask1, sits between the two)
        mask = bufs[1] if len(bufs) > 2 and a.get("mask", 0) else None
        out = bufs[-1]
        L.reef_oracle_attention(_p(bufs[0]), _p(mask), _p(out), i32(a["s"]), i32(a["heads"]), i32(a["d"]))
    else:
        raise KeyError(f"oracle: unknown kernel family {op!r}")


class OracleExecutor:
    """Mirror of the reference ExecutorBase surface (set_input / execute / get_output / get_data)."""

    def __init__(self, json_path: str, param_path: str | None = None, acc64: bool = False):
        with open(json_path) as f:
            self.model = json.load(f)
        self.acc64 = acc64
        self.storage = [np.zeros(s["size"], dtype=_STYPE[s["stype"]]) for s in self.model["storage"]]
        self.names = [s["name"] for s in self.model["storage"]]
        if param_path:
            self.load_param_from_file(param_path)

    def load_param_from_file(self, path: str) -> None:
        import struct
        with open(path, "rb") as f:
            magic = f.read(17)
            assert magic == b"TVM_MODEL_PARAMS\0", "bad .param magic"
            (count,) = struct.unpack("<Q", f.read(8))
            params = {}
            for _ in range(count):
                key = bytearray()
                while True:
                    c = f.read(1)
                    if c == b"\0":
                        break
                    key += c
                (n,) = struct.unpack("<Q", f.read(8))
                params[key.decode()] = np.frombuffer(f.read(4 * n), dtype="<f4")
        for i, n in enumerate(self.names):
            if n in params:
                arr = params[n]
                self.storage[i][: arr.size] = arr

    def find(self, name: str) -> int:
        return self.names.index(name)

    def set_input(self, name: str, value) -> None:
        i = self.find(name)
        v = np.asarray(value).reshape(-1)
        if v.size < self.storage[i].size:
            raise IndexError("OutOfRange: input shorter than the storage entry")
        self.storage[i][:] = v[: self.storage[i].size].astype(self.storage[i].dtype)

    def execute(self, upto: int | None = None) -> None:
        ks = self.model["kernels"]
        for k in ks[: len(ks) if upto is None else upto]:
            run_kernel(k["name"], [self.storage[a] for a in k["args"]], self.acc64)

    def get_output(self, name: str = "output") -> np.ndarray:
        return self.storage[self.find(name)].copy()

    def get_data(self, idx: int) -> np.ndarray:
        return self.storage[idx].copy()
