import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def golden_quant():
    return np.load(os.path.join(GOLDEN, "quant_cases.npz"))


@pytest.fixture(scope="session")
def golden_forward():
    return np.load(os.path.join(GOLDEN, "forward_cases.npz"))


@pytest.fixture(scope="session")
def golden_toy():
    return np.load(os.path.join(GOLDEN, "toy_forward.npz"))


@pytest.fixture(scope="session")
def golden_patch():
    import json
    with open(os.path.join(GOLDEN, "patch_cases.json")) as f:
        return json.load(f)
