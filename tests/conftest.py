"""Shared pytest configuration: markers, seeding and paths.

GPU tests are marked ``gpu`` and are skipped nowhere: run ``-m "not gpu"`` on a machine
without a B200 and ``-m gpu`` on one.
"""

import os
import random
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


@pytest.fixture(autouse=True)
def _seed_everything():
    # same seed the reference's test-suite uses (tests/conftest.py:37-56 there)
    torch.manual_seed(32)
    np.random.seed(32)
    random.seed(32)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(32)
    yield


def tolerance(dtype):
    """Absolute tolerances of the reference's tests (tests/conftest.py:27-34 there)."""
    return {torch.float32: 1e-5, torch.float16: 1e-3, torch.bfloat16: 7e-3}[dtype]
