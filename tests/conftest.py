import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "ml-recurrent-drafter_b200"), os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


@pytest.fixture(scope="session")
def g_unit():
    return load_golden("reference_unit_tests")


@pytest.fixture(scope="session")
def g_pack():
    return load_golden("pack_cases")


@pytest.fixture(scope="session")
def g_acc():
    return load_golden("acceptance_cases")


@pytest.fixture(scope="session")
def g_model():
    return load_golden("model_cases")


@pytest.fixture(scope="session")
def g_variants():
    return load_golden("drafter_variants")
