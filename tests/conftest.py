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


@pytest.fixture(autouse=True)
def no_cuda_error_left_behind(request):
    """After every GPU test the CUDA runtime must hold no pending error: a runtime call that failed inside the library
    (even one whose return code was handled) stays 'the last error' until someone asks, and the next library that
    checks after a launch of its own would report it as its own."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import ctypes
    try:
        rt = ctypes.CDLL("libcudart.so.12")
    except OSError:
        return
    rt.cudaGetLastError.restype = ctypes.c_int
    rt.cudaGetErrorString.restype = ctypes.c_char_p
    rt.cudaGetErrorString.argtypes = [ctypes.c_int]
    err = rt.cudaGetLastError()          # (also clears it, so that only the test that left it fails; 600 = "not ready",
                                         # the answer of a stream or event query, is no failure)
    assert err in (0, 600), "a CUDA error was left pending: %s" % rt.cudaGetErrorString(err).decode()
