"""reef_b200 — the REEF executor kernel path, B200-native.

The product is two native libraries built in-tree (``libreef_cuda.so``: C-ABI device layer and
sm_100a kernels; ``libreef_host.so``: C++ loader, executors and scheduler).  This package holds the
build recipe, thin ctypes bindings that mirror the reference's C++ class surface, and the
generator of model resources (``<model>.json`` / ``.param`` / ``.profile.json``).
There is no CPU fallback: everything that computes fails loudly without the CUDA library and a GPU.
"""
from . import build  # noqa: F401
