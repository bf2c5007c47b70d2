"""In-tree build of the two shared libraries.

``libreef_cuda.so``  C-ABI device layer + every CUDA kernel, nvcc for sm_100a only.
``libreef_host.so``  C++ host side (loader, executors, scheduler) + its C entry points, linked
                     against libreef_cuda.so through the C-ABI header only.

A content hash of sources and flags is stored beside each library so that an up-to-date
library (for instance one that travelled to a GPU machine with the source tree) is not rebuilt.
"""
from __future__ import annotations

import glob
import hashlib
import os
import shutil
import subprocess

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared", "-cudart", "static",
]
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-pthread", "-Wall"]
# REEF_DEBUG_AIDS=1 in the environment builds the development flavour: phase-trace stamps in the tensor-core kernel,
# reef_trace_* entry points (include/reef_debug_aids.h), REEF_PAD_* / REEF_PDL environment knobs, padding-loop statistics
if os.environ.get("REEF_DEBUG_AIDS", "") not in ("", "0"):
    NVCC_FLAGS.append("-DREEF_DEBUG_AIDS")
    CXX_FLAGS.append("-DREEF_DEBUG_AIDS")


def _nvcc() -> str:
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _cxx() -> str:
    for c in ("/usr/bin/g++", shutil.which("g++") or "g++"):
        if os.path.exists(c):
            return c
    return "g++"


def _digest(files, flags) -> str:
    """Hash of the sources and the command, with paths taken relative to the repository so that a tree that was
    built in one place and copied to another (same sources, same compiler flags) is not rebuilt there."""
    root = os.path.dirname(PKG)
    rel = lambda s: s.replace(root, ".")
    h = hashlib.sha256()
    for f in sorted(files, key=rel):
        h.update(rel(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(rel(x) for x in flags).encode())
    return h.hexdigest()


def _build(out: str, cmd: list, deps: list, verbose: bool) -> bool:
    stamp = out + ".stamp"
    dig = _digest(deps, cmd)
    if os.path.exists(out) and os.path.exists(stamp) and open(stamp).read().strip() == dig:
        return False
    if verbose:
        print("[reef_b200.build]", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    with open(stamp, "w") as f:
        f.write(dig)
    return True


def build_cuda(verbose: bool = False, extra_flags=()) -> str:
    out = os.path.join(PKG, "libreef_cuda.so")
    srcs = sorted(glob.glob(os.path.join(CSRC, "abi", "*.cu")) + glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
    deps = srcs + glob.glob(os.path.join(CSRC, "kernels", "*.cuh")) + glob.glob(os.path.join(CSRC, "kernels", "*.h")) \
        + glob.glob(os.path.join(INCLUDE, "*.h"))
    cmd = [_nvcc()] + NVCC_FLAGS + list(extra_flags) + ["-I", INCLUDE, "-o", out] + srcs
    _build(out, cmd, deps, verbose)
    return out


def build_host(verbose: bool = False) -> str:
    out = os.path.join(PKG, "libreef_host.so")
    srcs = sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    deps = srcs + glob.glob(os.path.join(CSRC, "host", "*.h")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    cmd = [_cxx()] + CXX_FLAGS + ["-I", INCLUDE, "-o", out] + srcs + \
        ["-L", PKG, "-lreef_cuda", "-Wl,-rpath,$ORIGIN"]
    _build(out, cmd, deps, verbose)
    return out


def build_all(verbose: bool = False):
    return build_cuda(verbose), build_host(verbose)


if __name__ == "__main__":
    print(build_all(verbose=True))
