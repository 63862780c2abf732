import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def ref_oracle():
    """The reference's own CPU sources compiled under oracle/_ref (present only where the reference tree was)."""
    from oracle.oracle import Oracle, have_reference
    if not have_reference():
        pytest.skip("oracle/_ref not built (no reference tree on this machine)")
    return Oracle(reference=True)
