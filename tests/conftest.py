import os
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    from cases import load_golden
    return load_golden()


@pytest.fixture(scope="session")
def golden_bwd():
    from cases import BACKWARD_GOLDEN, load_golden
    return load_golden(os.path.join(ROOT, "tests", "golden", BACKWARD_GOLDEN))
