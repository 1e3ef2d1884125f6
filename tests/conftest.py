import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (runs the sm_100a kernels through the C ABI)')


@pytest.fixture(scope='session')
def fwp():
    """The product package; importing it loads libfwp.so (no fallback)."""
    import recurrent_fwp_b200
    return recurrent_fwp_b200
