import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def port():
    from oracle import build, pyoracle
    build.build_port()
    return pyoracle.port()


@pytest.fixture(scope="session")
def reference():
    """The reference's own compiled CPU code, or a skip when oracle/_ref was not built."""
    from oracle import build, pyoracle
    try:
        build.build_reference()
    except Exception:  # the reference tree may be absent; a prebuilt library may still be there
        pass
    ref = pyoracle.reference()
    if ref is None:
        pytest.skip("oracle/_ref/libcct_ref.so not available")
    return ref


@pytest.fixture(scope="session")
def ctx():
    from caffecontroll_b200 import Context
    c = Context(0)
    yield c
    c.close()
