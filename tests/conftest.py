import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def gpu():
    """(engine, stream) on CUDA device 0 through the library's C API."""
    from onednn_b200 import api
    assert api.engine.get_count(api.engine.kind.gpu) > 0, "no CUDA device visible"
    eng = api.engine(api.engine.kind.gpu, 0)
    strm = api.stream(eng)
    yield eng, strm


@pytest.fixture(scope="session")
def host_engine():
    """Device-less engine for host-logic tests (descriptor / attribute /
    primitive-descriptor creation and queries; nothing executes)."""
    os.environ["DNNL_B200_NO_DEVICE"] = "1"
    from onednn_b200 import api
    if api.engine.get_count(api.engine.kind.gpu) > 0:
        return api.engine(api.engine.kind.gpu, 0)
    return api.engine(api.engine.kind.gpu, 0)
