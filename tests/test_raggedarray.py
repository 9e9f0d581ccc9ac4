"""Host ragged array semantics (cases of the reference's
nengo_ocl/tests/test_clraggedarray.py:28-117 that need no device, plus the
``align`` rule of nengo_ocl/raggedarray.py:46-55)."""

import numpy as np
import pytest

from nengo_ocl_b200 import raggedarray as ra
from nengo_ocl_b200.raggedarray import RaggedArray as RA


def test_shape_zeros():
    A = RA([[]], dtype=np.float32)
    assert A[0].shape == (0, 1)


def test_layout_and_views(rng):
    arrays = [rng.normal(size=s).astype(np.float32) for s in [(3, 4), (5,), (), (2, 1)]]
    A = RA(arrays)
    assert A.starts.tolist() == [0, 12, 17, 18]
    assert A.shape0s.tolist() == [3, 5, 1, 2]
    assert A.shape1s.tolist() == [4, 1, 1, 1]
    assert A.stride0s.tolist() == [4, 1, 1, 1]
    assert A.stride1s.tolist() == [1, 1, 1, 1]
    assert A.buf.dtype == np.float32 and A.buf.size == 20
    assert A.nbytes == 80
    for i, a in enumerate(arrays):
        assert np.array_equal(A[i], np.asarray(a).reshape(A[i].shape))
    # item access is a view into buf
    A[0][1, 2] = 7
    assert A.buf[6] == 7
    A[1] = 3
    assert (A.buf[12:17] == 3).all()
    with pytest.raises(NotImplementedError):
        A[[0, 1]] = 1
    with pytest.raises((ValueError, AttributeError)):
        A.starts[0] = 5  # index arrays are read-only


def test_list_index_shares_buffer(rng):
    A = RA([rng.normal(size=(n, 2)) for n in (3, 4, 5)], dtype=np.float32)
    B = A[[2, 0]]
    assert len(B) == 2 and B.buf is A.buf
    assert B.starts.tolist() == [14, 0]
    assert np.array_equal(B[0], A[2])
    C = A[1:]
    assert C.starts.tolist() == [6, 14]


def test_align_rule():
    sizes = [3, 20, 9, 5, 16]
    A = RA([np.ones(n) for n in sizes], dtype=np.float32, align=True)
    # start of item i is rounded up to 16 if its size >= 16, to 4 if >= 8, else 1
    assert A.starts.tolist() == [0, 16, 36, 45, 64]
    B = RA([np.ones(n) for n in sizes], dtype=np.float32)
    assert B.starts.tolist() == [0, 3, 23, 32, 37]


def test_add_views_and_discontiguous_set(rng):
    A = RA([rng.normal(size=(6, 8)), rng.normal(size=(4,))], dtype=np.float32)
    A0 = np.array(A[0])
    A.add_views([A.starts[0]], [2], [4], [24], [2], names=["v"])
    assert len(A) == 3 and A.names[-1] == "v"
    v = rng.uniform(-1, 1, size=(2, 4)).astype(np.float32)
    A[-1] = v
    expect = A0.copy()
    expect[::3, ::2] = v
    assert np.array_equal(A[0], expect)
    assert np.array_equal(A[2], v)


def test_allclose_checks_indices(rng):
    A = RA([rng.normal(size=(3, 3)), rng.normal(size=(2,))], dtype=np.float32)
    B = RA([A[0].copy(), A[1].copy()], dtype=np.float32)
    assert ra.allclose(A, B)
    B[1][0, 0] += 1
    assert not ra.allclose(A, B)
    C = RA([A[0].copy().reshape(9, 1), A[1].copy()], dtype=np.float32)
    assert not ra.allclose(A, C)


def test_int32_dtype_and_dtype_restriction():
    A = RA([[1, 2], [3]], dtype=np.int32)
    assert A.buf.dtype == np.int32
    with pytest.raises(AssertionError):
        RA([np.ones(3)], dtype=np.float64)
