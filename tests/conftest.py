import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(autouse=True)
def _fresh_grid():
    """Each test starts without an installed parallel grid."""
    from easyllm_b200.parallel import grid
    grid.set_grid(None)
    yield
    grid.set_grid(None)
