import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); never skipped silently on a GPU box")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def lib_built():
    """Make sure libb200fp4.so exists (built ahead of time; nvcc needs no GPU)."""
    import importlib.util

    path = os.path.join(ROOT, "cutedsl-fully-opensourced_b200", "build.py")
    spec = importlib.util.spec_from_file_location("_b200_build", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if not os.path.exists(mod.LIB_PATH):
        mod.build()
    return mod.LIB_PATH


@pytest.fixture(scope="session")
def b200(lib_built):
    import cutedsl_fully_opensourced_b200 as pkg

    return pkg


def golden(name):
    import numpy as np

    return np.load(os.path.join(GOLDEN, name))
