"""pytest configuration: markers, import path, shared fixtures."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu")
    config.addinivalue_line("markers", "ref: needs the compiled reference under oracle/_ref")


def _has_gpu():
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped (not failed) on a machine without a device, the
    way the reference skips ISA-specific tests (tests/conftest.py:295-326)."""
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def port():
    import oracle

    return oracle.port()


@pytest.fixture(scope="session")
def ref():
    import oracle

    if not oracle.ref_available():
        pytest.skip("compiled reference (oracle/_ref) not available on this machine")
    return oracle.ref()


@pytest.fixture(scope="session")
def torch_mod():
    import torch

    return torch
