"""Shared fixtures.  Tests marked ``gpu`` need a B200; everything else runs on a CPU
box (multi-process cases use localhost sockets)."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """Build libflagcx.so once per session if it is missing."""
    from flagcx_b200 import capi
    if not os.path.exists(capi.LIB_PATH):
        from flagcx_b200.build import build_core
        build_core()
    return capi.LIB_PATH


def has_cuda() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False
