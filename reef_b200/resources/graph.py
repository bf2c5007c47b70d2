"""Schedule-graph builder that emits REEF model resources.

A REEF model directory holds ``<model>.json`` (storage table, kernel list with
launch parameters and positional storage indices, I/O index list, shared-memory
table), ``<model>.param`` (named fp32 blobs) and ``<model>.profile.json``
(per-kernel latency tables).  The json schema is the one parsed by the
reference loader (reference: src/reef/executor/model.cpp:13-55) and the
``.param`` byte format is the one its export script writes (reference:
script/tvm_generate_model.py:66-76, parsed at src/reef/executor/model.cpp:82-121).

The reference obtained the kernel list from a TVM build; here every kernel is a
hand-written sm_100a kernel looked up by *name*, so the name carries the fused
op family exactly as TVM spelt it (``fused_nn_conv2d_add_nn_relu`` ...) followed
by ``__`` and a list of ``<key><int>`` shape tokens, e.g.
``fused_nn_conv2d_add_nn_relu__ci64_hi56_wi56_co256_kh1_kw1_sh1_sw1_ph0_pw0``.
Positional argument order per family follows the reference kernels
(reference: resource/resnet152/resnet152.cu:2,315,340,365,771,775,4390,4472).

Data layout contract (ours, since the resources are ours): model input ``data``
is NCHW fp32 as in the reference; every intermediate activation is channels-last
(NHWC) fp32; convolution weights are stored OHWI = [Cout][kh][kw][Cin]; dense
weights are [N][K] row-major as in the reference.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field

import numpy as np

PARAM_MAGIC = b"TVM_MODEL_PARAMS\0"


def kname(op: str, **attrs: int) -> str:
    """Kernel name = op family + '__' + '_'.join(key+int)."""
    if not attrs:
        return op
    return op + "__" + "_".join(f"{k}{int(v)}" for k, v in attrs.items())


_TUNED = None


def tuned_plan(name: str) -> dict:
    """Measured launch plan of a tensor-core kernel name ({} when the shape was never tuned): ``tp`` = pixel-tile
    cap, ``ts`` = K splits, as written by ``python -m reef_b200.tune`` into ``tuned_plans.json`` beside this file.
    The generators append them to the kernel name, so the plan is part of the schedule a ``<model>.json`` records."""
    global _TUNED
    if _TUNED is None:
        import json
        import os
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tuned_plans.json")
        _TUNED = json.load(open(path))["plans"] if os.path.exists(path) else {}
    if os_environ_untuned():
        return {}
    hit = _TUNED.get(name)
    return dict(tp=int(hit[0]), ts=int(hit[1])) if hit else {}


def os_environ_untuned() -> bool:
    import os
    return os.environ.get("REEF_UNTUNED", "") not in ("", "0")


def parse_kname(name: str):
    """Inverse of :func:`kname` -> (op, {key: int})."""
    if "__" not in name:
        return name, {}
    op, tail = name.split("__", 1)
    attrs = {}
    for tok in tail.split("_"):
        i = 0
        while i < len(tok) and not (tok[i].isdigit()):
            i += 1
        attrs[tok[:i]] = int(tok[i:])
    return op, attrs


@dataclass
class Tensor:
    """Handle to a storage entry plus the logical NHWC view the builder tracks."""
    idx: int
    h: int = 1
    w: int = 1
    c: int = 1           # logical channels of this view
    cs: int = 0          # channel stride of the underlying buffer (0 -> == c)
    coff: int = 0        # channel offset inside the underlying buffer

    @property
    def cstride(self):
        return self.cs or self.c


@dataclass
class Graph:
    name: str
    storage: list = field(default_factory=list)
    kernels: list = field(default_factory=list)
    params: dict = field(default_factory=dict)
    io_args: list = field(default_factory=list)
    n_params: int = 0

    # ---- storage -------------------------------------------------------
    def add_storage(self, name: str, size: int, stype: str = "float32") -> int:
        self.storage.append({"name": name, "stype": stype, "size": int(size)})
        return len(self.storage) - 1

    def input(self, name: str, size: int, stype: str = "float32") -> int:
        idx = self.add_storage(name, size, stype)
        self.io_args.append(idx)
        return idx

    def param(self, array) -> int:
        a = np.ascontiguousarray(array, dtype=np.float32).reshape(-1)
        name = f"p{self.n_params}"
        self.n_params += 1
        idx = self.add_storage(name, a.size)
        self.params[name] = a
        self.io_args.append(idx)
        return idx

    def temp(self, size: int, name: str = "null") -> int:
        return self.add_storage(name, size)

    # ---- kernels -------------------------------------------------------
    def kernel(self, name: str, args: list) -> None:
        self.kernels.append({"name": name, "launch_params": None, "args": [int(a) for a in args]})

    # ---- emit ----------------------------------------------------------
    def finalize(self, plan_fn) -> dict:
        """Fill launch_params / shared_memory from the kernel registry.

        ``plan_fn(name) -> (dims[6], dyn_smem_bytes)`` is the C-ABI query
        ``reef_kernel_plan`` so that the json and the registry cannot disagree.
        """
        shared = {}
        for k in self.kernels:
            dims, smem = plan_fn(k["name"])
            k["launch_params"] = [int(d) for d in dims]
            shared[k["name"]] = int(smem)
        return {
            "storage": self.storage,
            "kernels": self.kernels,
            "args": self.io_args,
            "shared_memory": shared,
        }

    def write(self, out_dir: str, plan_fn, profile: dict | None = None) -> str:
        os.makedirs(out_dir, exist_ok=True)
        j = self.finalize(plan_fn)
        base = os.path.join(out_dir, self.name)
        with open(base + ".json", "w") as f:
            json.dump(j, f, indent=1)
        write_param_file(base + ".param", self.params)
        if profile is None:
            profile = default_profile(j)
        with open(base + ".profile.json", "w") as f:
            json.dump(profile, f)
        return base


def default_profile(model_json: dict) -> dict:
    """Placeholder latency tables (1 us) until the profiler has measured the kernels.

    Schema: reference src/reef/executor/model.cpp:57-82 — ``model_latency`` (us)
    and per kernel name ``total_latency`` plus ``latency[j]`` = duration of one
    persistent wave at occupancy j+1.
    """
    names = []
    for k in model_json["kernels"]:
        if k["name"] not in names:
            names.append(k["name"])
    return {
        "model_latency": len(model_json["kernels"]),
        "kernel_latency": {n: {"total_latency": 1, "latency": [1] * 8} for n in names},
    }


def write_param_file(path: str, params: dict) -> None:
    """magic(17 B incl. NUL) | u64 count | count x (key NUL u64 n, n x f32 LE)."""
    with open(path, "wb") as f:
        f.write(PARAM_MAGIC)
        f.write(struct.pack("<Q", len(params)))
        for key, arr in params.items():
            a = np.ascontiguousarray(arr, dtype="<f4").reshape(-1)
            f.write(key.encode() + b"\0")
            f.write(struct.pack("<Q", a.size))
            f.write(a.tobytes())


def read_param_file(path: str) -> dict:
    out = {}
    with open(path, "rb") as f:
        magic = f.read(len(PARAM_MAGIC))
        if magic != PARAM_MAGIC:
            raise ValueError("bad .param magic")
        (count,) = struct.unpack("<Q", f.read(8))
        for _ in range(count):
            key = bytearray()
            while True:
                c = f.read(1)
                if not c:
                    raise ValueError("truncated .param key")
                if c == b"\0":
                    break
                key += c
            (n,) = struct.unpack("<Q", f.read(8))
            buf = f.read(4 * n)
            if len(buf) != 4 * n:
                raise ValueError("truncated .param array")
            out[key.decode()] = np.frombuffer(buf, dtype="<f4").copy()
    return out
