import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle_clib():
    """The plain-C oracle, built on demand (test infrastructure)."""
    import ctypes
    import subprocess

    odir = os.path.join(ROOT, "oracle")
    so = os.path.join(odir, "_build", "libdkv_oracle.so")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(os.path.join(odir, "ref_attention.c")):
        subprocess.run(["make", "-C", odir], check=True, capture_output=True)
    return ctypes.CDLL(so)
