import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def port():
    import oracle
    if not os.path.exists(oracle.PORT_SO):
        oracle.build(ref=False)
    return oracle.port()


@pytest.fixture(scope="session")
def ref():
    import oracle
    if not oracle.have_ref():
        if oracle.reference_root() is not None:
            oracle.build(ref=True)
        else:
            pytest.skip("the compiled reference (oracle/_ref) is not available on this machine")
    return oracle.ref()
