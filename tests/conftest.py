import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import Oracle
    return Oracle(threads=1)


@pytest.fixture(scope="session")
def refcheck():
    from oracle import RefCheck
    if not RefCheck.available():
        pytest.skip("oracle/_ref was not built (the cutorch tree is not mounted here)")
    return RefCheck()


@pytest.fixture(scope="session")
def state():
    """A THCState on cuda:0.  The product has no CPU path: a missing library is an error."""
    from cutorch_b200 import thc
    s = thc.State()
    yield s
    s.shutdown()
