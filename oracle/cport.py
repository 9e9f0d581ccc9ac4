"""Loader of the compiled half of the CPU oracle (``oracle/cport.c``).

TEST INFRASTRUCTURE ONLY (see ``oracle/kernels.py``).  The C file is compiled
with ``gcc -O2 -ffp-contract=off -fopenmp`` into ``oracle/_cport.so`` (an
ignored build product) the first time it is needed and whenever the source is
newer than the library.
"""

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "cport.c")
LIB = os.path.join(HERE, "_cport.so")

_lib = None
_F = ctypes.POINTER(ctypes.c_float)


def build(force=False):
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        tmp = LIB + ".%d.tmp" % os.getpid()
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-shared", "-fPIC",
                        "-o", tmp, SRC, "-lm"], check=True)
        os.replace(tmp, LIB)
    return LIB


def lib():
    global _lib
    if _lib is None:
        handle = ctypes.CDLL(build())
        handle.nb2o_block_rows.argtypes = [_F, ctypes.c_long, ctypes.c_long, ctypes.c_int, ctypes.c_int, _F,
                                           ctypes.c_long, _F, ctypes.c_long, ctypes.c_double]
        handle.nb2o_block_rows.restype = None
        handle.nb2o_lif.argtypes = [ctypes.c_int, ctypes.c_double, _F, _F, _F, _F, ctypes.c_float, ctypes.c_float,
                                    ctypes.c_float]
        handle.nb2o_lif.restype = None
        handle.nb2o_pes_step.argtypes = ([ctypes.c_int] * 4 + [ctypes.c_double] + [_F] * 13
                                         + [ctypes.c_float] * 8)
        handle.nb2o_pes_step.restype = None
        handle.nb2o_set_threads.argtypes = [ctypes.c_int]
        handle.nb2o_set_threads.restype = ctypes.c_int
        _lib = handle
    return _lib


def set_threads(n=0):
    """Use ``n`` OpenMP threads in the compiled kernels (0: leave as is); returns the count in use."""
    return int(lib().nb2o_set_threads(int(n)))


def _ptr(a):
    return ctypes.cast(a.__array_interface__["data"][0], _F)


def block_rows(total, A, x, alpha=1.0):
    """``total += block-order A . x`` in place.  ``total``: float32 vector (any
    stride), ``A``: 2-D float32 view (any strides), ``x``: float32 vector."""
    assert total.dtype == A.dtype == x.dtype == np.float32
    M, N = A.shape
    assert total.shape == (M,) and x.shape == (N,)
    isz = 4
    lib().nb2o_block_rows(_ptr(A), A.strides[0] // isz, A.strides[1] // isz, M, N, _ptr(x), x.strides[0] // isz,
                          _ptr(total), total.strides[0] // isz, float(alpha))


def block_rows_args(total, A, x, alpha=1.0):
    """Argument tuple of ``block_rows`` for arrays that stay where they are (a simulator's
    signals): build once, run every step with ``block_rows_run``."""
    assert total.dtype == A.dtype == x.dtype == np.float32
    M, N = A.shape
    assert total.shape == (M,) and x.shape == (N,)
    assert not np.shares_memory(total, A) and not np.shares_memory(total, x)
    lib()
    return (_ptr(A), A.strides[0] // 4, A.strides[1] // 4, M, N, _ptr(x), x.strides[0] // 4, _ptr(total),
            total.strides[0] // 4, float(alpha), (total, A, x))  # (the arrays are kept alive)


def block_rows_run(args):
    _lib.nb2o_block_rows(*args[:10])


def lif(dt, J, V, W, S, tau, ref, amp):
    """One LIF step in place on contiguous float32 vectors."""
    for a in (J, V, W, S):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    lib().nb2o_lif(J.size, float(dt), _ptr(J), _ptr(V), _ptr(W), _ptr(S), float(tau), float(ref), float(amp))


def pes_step(n_ens, n, d, dc, dt, arrays, scalars):
    """One step of a batch of PES ensembles, operator by operator (see cport.c).
    ``arrays``: the 13 float32 arrays in the order of the C signature."""
    for a in arrays:
        assert a.dtype == np.float32 and a.flags.c_contiguous
    lib().nb2o_pes_step(n_ens, n, d, dc, float(dt), *[_ptr(a) for a in arrays], *[float(s) for s in scalars])
