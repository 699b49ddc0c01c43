import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


def reference_dir():
    """The reference checkout when one is reachable (TPUC_REFERENCE_DIR, or a directory named ``reference`` beside
    this repository), else None: tests that read its fixtures as text skip without it."""
    cand = os.environ.get("TPUC_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    return cand if os.path.isdir(os.path.join(cand, "lib", "Dialect", "TPU")) else None
