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
    from oracle import g4_oracle
    return g4_oracle.load("port")


@pytest.fixture(scope="session")
def ref():
    """The reference's own host code; skipped where it has not been built."""
    from oracle import g4_oracle
    if not g4_oracle.available("reference"):
        pytest.skip("oracle/_ref/libg4ref.so not built (needs a reference checkout)")
    return g4_oracle.load("reference")
