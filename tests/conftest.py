import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    # build the native library and the oracle once, before collection imports them
    # loaded by path: importing the package needs the library this builds
    import importlib.util
    spec = importlib.util.spec_from_file_location("accy_b200_build", os.path.join(ROOT, "accy_b200", "build.py"))
    native_build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(native_build)
    native_build.build()
    from oracle import build as oracle_build
    oracle_build.build()


@pytest.fixture(scope="session")
def cpu_session():
    """compile-only session: planner, emitter and NVRTC (sm_100a) run, no device is touched"""
    from accy_b200 import tensor
    s = tensor.Session(device=-1)
    yield s
    s.deinit()


@pytest.fixture(scope="session")
def gpu_session():
    from accy_b200 import tensor
    s = tensor.Session(device=0)
    yield s
    s.deinit()
