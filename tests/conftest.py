"""Shared pytest configuration: the ``gpu`` marker and import paths."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "spline_kv_golden.npz")
    data = np.load(path)
    cases = {}
    for key in data.files:
        case, name = key.split("/")
        cases.setdefault(case, {})[name] = data[key]
    return cases
