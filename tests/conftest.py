"""Shared fixtures.  Tests marked ``gpu`` need a CUDA device and call the
kernels through the C ABI; everything else runs on the CPU."""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on the GPU box)")


@pytest.fixture
def rng():
    return np.random.RandomState(1)


@pytest.fixture(scope="session")
def golden_tables():
    return np.load(os.path.join(GOLDEN, "tables.npz"), allow_pickle=False)


@pytest.fixture(scope="session")
def golden_kernels():
    return np.load(os.path.join(GOLDEN, "kernels.npz"), allow_pickle=False)


@pytest.fixture(scope="session")
def ctx():
    from nengo_ocl_b200.runtime import create_some_context

    return create_some_context()


@pytest.fixture
def queue(ctx):
    from nengo_ocl_b200.runtime import CommandQueue

    return CommandQueue(ctx)
