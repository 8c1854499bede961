import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.binding import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def lib():
    """The C-ABI library on a machine with a GPU.  Fails loudly if it is missing."""
    from bpd_substrate_b200 import capi
    l = capi.load()
    l.bpdq_clear_status()
    return l
