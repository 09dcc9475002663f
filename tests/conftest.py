import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def orc():
    o = entry.load_oracle()
    o.build()
    return o


@pytest.fixture(scope="session")
def synth(pkg):
    from strix_rs_b200 import synth as s
    return s


@pytest.fixture(scope="session")
def accel(pkg):
    """One accelerator on cuda:0 for the whole GPU session. Loading fails loudly if the
    CUDA library is missing: there is no fallback path to fall back to."""
    a = pkg.CudaWeightAccel(0)
    yield a
    a.close()
