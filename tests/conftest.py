import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device; run with -m gpu")


def _have_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    # Like the reference's device tests (tests/infra/gpu_tests.rs:6-17), GPU tests are skipped,
    # not mocked, on a machine without a device.  On a GPU box nothing is skipped: a missing
    # library or a failing kernel is a test failure.
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device on this machine")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def nne():
    """The package under test (its directory name has a hyphen, so import it by string)."""
    return importlib.import_module("neural-network-engine_b200")


@pytest.fixture(scope="session")
def ctx(nne):
    return nne.default_context(0)
