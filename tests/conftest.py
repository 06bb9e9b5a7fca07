import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def built_kernels():
    """Every kernel of the tuning space, compiled (or adopted from the in-tree cache)."""
    from fray_b200.jit_kernels.flashattn_cute import prebuild
    return sorted(prebuild())
