import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(autouse=True)
def _seeded():
    """Every test draws the same random numbers every time."""
    import random

    import torch
    random.seed(1234)
    torch.manual_seed(1234)
    yield
