import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
os.environ.setdefault("REEF_QUIET", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU machine)")


@pytest.fixture(scope="session")
def libs():
    """Both native libraries, built in-tree (no-op when up to date)."""
    from reef_b200 import build
    return build.build_all()


@pytest.fixture(scope="session")
def resource_root(libs):
    d = os.environ.get("REEF_RESOURCE_DIR", "/tmp/reef_b200_resources")
    os.makedirs(d, exist_ok=True)
    return d


@pytest.fixture(scope="session")
def gen(resource_root):
    from reef_b200 import resources

    def _gen(model, **kw):
        d = resources.generate(model, resource_root, **kw)
        name = os.path.basename(d)
        return os.path.join(d, name)   # base path: + ".json" / ".param" / ".profile.json"
    return _gen


def rel_err(y, ref):
    """max_i |y_i - ref_i| / max(max_j |ref_j|, 1e-30) — the parity metric of every test."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


def seeded_input(n, seed=7):
    return np.random.default_rng(seed).normal(0.0, 1.0, n).astype(np.float32)
