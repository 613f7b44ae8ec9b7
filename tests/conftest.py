import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import binding
    binding.lib()
    return binding


@pytest.fixture(scope="session")
def built():
    """Builds the native libraries in-tree if they are stale."""
    from jitllm_b200 import build
    build.build_all()
    return True


@pytest.fixture(scope="session")
def dev(built):
    import jitllm_b200 as jl
    d = jl.Device(0)
    yield d
    d.close()
