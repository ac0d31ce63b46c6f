import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """The product library and the C restatement must exist before any test runs."""
    import acrotensor_b200 as ab
    from oracle import oracle
    if not os.path.exists(ab.LIB_PATH):
        ab.build()
    if not oracle.have("port"):
        oracle.build()
