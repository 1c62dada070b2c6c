import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import binding
    binding.build()
    return binding


@pytest.fixture(scope="session")
def vdnn():
    """The product package with its CUDA library loaded (built on demand where nvcc exists)."""
    import vdnn_implementation_b200 as v
    if not os.path.exists(v.lib_path()):
        from vdnn_implementation_b200 import build
        build.build()
    v.lib()
    return v
