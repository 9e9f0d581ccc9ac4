"""Device ragged array: the cases of the reference's
nengo_ocl/tests/test_clraggedarray.py:33-117 against the CUDA store."""

import numpy as np
import pytest

from nengo_ocl_b200 import raggedarray as ra
from nengo_ocl_b200.curaggedarray import CUDARaggedArray as CLRA
from nengo_ocl_b200.raggedarray import RaggedArray as RA

pytestmark = pytest.mark.gpu


def make_random_ra(n, d, low=20, high=40, rng=None):
    shapes = zip(*(rng.randint(low=low, high=high + 1, size=n).tolist() for dd in range(d)))
    return RA([rng.normal(size=shape).astype(np.float32) for shape in shapes])


def test_unit(queue, rng):
    val = np.float32(rng.randn())
    clA = CLRA(queue, RA([val]))
    assert np.allclose(val, clA[0])


def test_roundtrip(queue, rng):
    A = RA([rng.normal(size=3).astype(np.float32) for _ in range(3)])
    assert ra.allclose(A, CLRA(queue, A).to_host())
    A = make_random_ra(int(rng.randint(5, 10)), 1, low=3000, high=4000, rng=rng)
    assert ra.allclose(A, CLRA(queue, A).to_host())
    A = make_random_ra(int(rng.randint(5, 10)), 2, rng=rng)
    clA = CLRA(queue, A)
    assert ra.allclose(A, clA.to_host())
    assert np.array_equal(A.buf, clA.to_host().buf)  # bit-exact round trip


def test_getitem_and_getitems(queue, rng):
    A = make_random_ra(10, 2, rng=rng)
    clA = CLRA(queue, A)
    assert np.array_equal(A[3], clA[3])
    s = [1, 3, 7, 8]
    sub = clA[s]
    assert sub.cl_buf is clA.cl_buf  # a device view, no copy
    assert ra.allclose(A[s], sub.to_host())
    assert not clA[3].flags.writeable


def test_setitem(queue, rng):
    A = make_random_ra(3, 2, rng=rng)
    clA = CLRA(queue, A)
    v = rng.uniform(0, 1, size=A[0].shape)
    A[0] = v.astype(A.dtype)
    clA[0] = v.astype(clA.dtype)
    A[1] = 3
    clA[1] = 3
    assert ra.allclose(A, clA.to_host())
    with pytest.raises(NotImplementedError):
        clA[[0, 1]] = 1


def test_discontiguous_setitem(queue, rng):
    A = make_random_ra(3, 2, rng=rng)
    A0 = np.array(A[0])
    a = A0[::3, ::2]
    v = rng.uniform(-1, 1, size=a.shape)
    assert a.size > 0
    A.add_views([A.starts[0]], [a.shape[0]], [a.shape[1]], [a.strides[0] / a.itemsize],
                [a.strides[1] / a.itemsize])
    clA = CLRA(queue, A)
    a[...] = v
    A[-1] = v
    assert np.allclose(A[0], A0)
    clA[-1] = v
    assert ra.allclose(A, clA.to_host())
    assert np.allclose(clA[-1], v)


def test_empty_item_and_int32(queue):
    A = RA([[], [1.0, 2.0]], dtype=np.float32)
    clA = CLRA(queue, A)
    assert clA[0].shape == (0, 1)
    assert np.array_equal(clA[1].ravel(), [1, 2])
    I = CLRA(queue, RA([[1, 2, 3], [4]], dtype=np.int32))
    assert I.dtype == np.int32 and I.ctype == "int"
    assert np.array_equal(I[0].ravel(), [1, 2, 3])
