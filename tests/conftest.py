"""Shared fixtures.  GPU tests are marked ``gpu``; everything else runs on a CPU-only box."""
import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def accb():
    """The product package (its directory name is not a Python identifier)."""
    return importlib.import_module("accelerate-cuda_b200")


@pytest.fixture(scope="session")
def workloads(accb):
    return importlib.import_module("accelerate-cuda_b200.workloads")


@pytest.fixture(scope="session")
def P(accb):
    return importlib.import_module("accelerate-cuda_b200.programs")


@pytest.fixture(scope="session")
def oracle():
    return importlib.import_module("oracle")


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    return torch


@pytest.fixture(scope="session")
def ctx(accb, torch_cuda):
    c = accb.Context(0)
    yield c
    c.sync()


@pytest.fixture
def rng():
    return np.random.default_rng(0xB200)
