import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.pgoracle import Oracle

    return Oracle(mt=False)


@pytest.fixture(scope="session")
def oracle_mt():
    from oracle.pgoracle import Oracle

    return Oracle(mt=True)


@pytest.fixture(scope="session")
def gpu():
    """The thread's GPU context.  Fails (never skips) if the CUDA library cannot be used."""
    import peregrine_b200 as pg

    return pg.init_gpu(0)
