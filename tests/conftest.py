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


# Whole-model parity tests record what they measured (elements compared, elements that are
# not bit-identical, elements outside rtol 1e-5 / atol 1e-6, spikes that moved) so that the
# numbers appear in the test log instead of only a pass mark.
PARITY_ROWS = []


@pytest.fixture
def parity_report():
    def add(name, **fields):
        PARITY_ROWS.append((name, fields))

    return add


def pytest_terminal_summary(terminalreporter):
    if not PARITY_ROWS:
        return
    terminalreporter.section("whole-model parity against the CPU oracle (measured)")
    for name, f in PARITY_ROWS:
        terminalreporter.write_line("%-44s %s" % (name, "  ".join("%s=%s" % kv for kv in f.items())))


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
