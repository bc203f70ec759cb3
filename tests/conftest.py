import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "go-nngpu_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def built_lib():
    """Builds (if stale) and loads the C-ABI library; no compute call is made."""
    import build as gonn_build  # go-nngpu_b200/build.py
    gonn_build.build()
    import gonngpu
    return gonngpu


@pytest.fixture(scope="session")
def gpu(built_lib):
    """The binding, after checking a device is really there: GPU tests must
    fail loudly, not skip, when the CUDA path is unusable."""
    g = built_lib
    assert g.lib().gonngpu_device_count() >= 1, "no CUDA device visible: GPU tests cannot run"
    assert g.lib().gonngpu_set_device(0) == 0, "device 0 is not a usable sm_100 GPU"
    return g


@pytest.fixture(scope="session")
def golden():
    import json
    import numpy as np
    gdir = os.path.join(ROOT, "tests", "golden")
    with open(os.path.join(gdir, "reference_kats.json")) as f:
        ref = json.load(f)
    kats = dict(np.load(os.path.join(gdir, "oracle_kats.npz")))
    return ref, kats
