import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def pytest_collection_modifyitems(config, items):
    # Fail loudly rather than silently skip: a GPU-marked test on a box without a GPU is
    # deselected by `-m "not gpu"`; if it is selected anyway it must error, not pass.
    pass
