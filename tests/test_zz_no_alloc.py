"""The entry point that allocates nothing (``nb2_probes_wide_noalloc``: arrival
counters in a device array of the library) against ``nb2_probes_wide`` with
caller-provided counters, on two calls in a row."""

import ctypes

import numpy as np
import pytest

from nengo_ocl_b200 import _capi
from nengo_ocl_b200.curaggedarray import CUDARaggedArray as CLRA
from nengo_ocl_b200.raggedarray import RaggedArray as RA
from nengo_ocl_b200.runtime import to_device

pytestmark = pytest.mark.gpu


def _setup(queue, sig, n_pre, periods):
    X = CLRA(queue, sig)
    Y = CLRA(queue, RA([np.zeros((n_pre, int(s))) for s in sig.sizes], dtype=np.float32))
    periods = np.asarray(periods, np.float32)
    state = dict(X=X, Y=Y, periods=to_device(queue, periods), countdowns=to_device(queue, periods - 1),
                 pos=to_device(queue, np.zeros(len(periods), np.int32)))
    state["tables"] = (state["countdowns"].ptr, state["pos"].ptr, state["periods"].ptr, X.cl_starts.ptr,
                       X.cl_shape0s.ptr, X.cl_shape1s.ptr, X.cl_stride0s.ptr, X.cl_stride1s.ptr, X.cl_buf.ptr,
                       Y.cl_starts.ptr, Y.cl_buf.ptr)
    return state


def test_no_alloc_entry_point_matches_on_two_calls(queue, rng):
    sig = RA([rng.normal(size=(20000, 1)), rng.normal(size=(3, 1)), rng.normal(size=(9000, 1))], dtype=np.float32)
    periods, n_pre, chunks = [1, 2, 1], 4, 5
    a = _setup(queue, sig, n_pre, periods)   # caller-provided counters
    b = _setup(queue, sig, n_pre, periods)   # counters inside the library
    arrive = to_device(queue, np.zeros(3, np.int32))
    for call in range(2):
        new = rng.normal(size=(3, 1)).astype(np.float32)
        a["X"][1] = new
        b["X"][1] = new
        _capi.call("nb2_probes_wide", queue.stream, 3, chunks, *a["tables"], arrive.ptr)
        _capi.call("nb2_probes_wide_noalloc", queue.stream, 3, chunks, *b["tables"])
        queue.finish()
        assert np.array_equal(a["Y"].cl_buf.get(), b["Y"].cl_buf.get())
        assert np.array_equal(a["pos"].get(), b["pos"].get())
        assert np.array_equal(a["countdowns"].get(), b["countdowns"].get())
    assert a["pos"].get().tolist() == [2, 1, 2]
    assert np.any(a["Y"].cl_buf.get() != 0)
    assert np.array_equal(arrive.get(), np.zeros(3, np.int32))


def test_no_alloc_entry_point_rejects_oversize(queue):
    n = 4097  # NB2_PROBES_STATIC_MAX + 1
    null = ctypes.c_void_p(0)
    status = _capi.lib().nb2_probes_wide_noalloc(queue.stream, n, 1, *([null] * 11))
    assert status < 0
    assert b"static arrival counters" in _capi.lib().nb2_last_error()
