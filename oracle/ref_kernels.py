"""Runs the reference's OWN generated kernels on the CPU (oracle/_ref/libref_<model>.so: the sources of
resource/<model>/<model>.cu compiled unchanged, executed by the fiber emulator in refkernels/).

TEST INFRASTRUCTURE ONLY.  The libraries exist where the reference tree was present when ``make -C oracle ref`` ran;
``available()`` says whether they do.  Launch geometry comes from the reference's shipped ``<model>.json`` (copies
under tests/golden/ref), exactly as the reference executor takes it (reference: src/reef/executor/executor_base.cpp:211-223).
"""
from __future__ import annotations

import ctypes as C
import json
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF_JSON = os.path.join(os.path.dirname(_HERE), "tests", "golden", "ref")
_LIBS = {}
_PARAMS = {}


def lib_path(model: str) -> str:
    return os.path.join(_HERE, "_ref", f"libref_{model}.so")


def available(model: str = "resnet152") -> bool:
    return os.path.exists(lib_path(model))


def _lib(model):
    if model not in _LIBS:
        lib = C.CDLL(lib_path(model), mode=os.RTLD_LOCAL)
        lib.reef_ref_launch.restype = C.c_int
        _LIBS[model] = lib
    return _LIBS[model]


def launch_params(model: str, kernel: str):
    if model not in _PARAMS:
        j = json.load(open(os.path.join(_REF_JSON, model + ".json")))
        _PARAMS[model] = {k["name"]: k["launch_params"] for k in j["kernels"]}
    return _PARAMS[model][kernel]


def launch(model: str, kernel: str, bufs: list) -> None:
    """Run one reference kernel on numpy buffers (positional like the reference's json "args")."""
    dims = (C.c_int * 6)(*launch_params(model, kernel))
    args = (C.c_void_p * len(bufs))(*[b.ctypes.data for b in bufs])
    rc = _lib(model).reef_ref_launch(kernel.encode(), dims, args, C.c_int(len(bufs)))
    if rc != 0:
        raise RuntimeError(f"reef_ref_launch({kernel}) failed with {rc}")
