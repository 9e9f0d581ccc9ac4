"""Device context, queue and flat device arrays over the C ABI.

Stands in for the slice of PyOpenCL the reference uses: ``cl.Context`` /
``cl.CommandQueue`` (nengo_ocl/simulator.py:209-219), ``pyopencl.array.Array``
and ``to_device`` (nengo_ocl/clraggedarray.py:12-19).  The queue exposes the
attributes plan code reads: ``.context``, ``.device.max_work_group_size``,
``.device.global_mem_size``, ``.device.local_mem_size`` and ``.finish()``.
"""

import ctypes
import weakref

import numpy as np

from nengo_ocl_b200 import _capi


class Device:
    """Static device properties used by the index planners.

    ``max_work_group_size`` is 1024 (what NVIDIA's OpenCL reports), so block
    tables that depend on it (nengo_ocl/clra_gemv.py:719-721,
    clra_nonlinearities.py:18-19) come out identical to the reference's.
    """

    max_work_group_size = 1024
    local_mem_size = 48 * 1024

    def __init__(self, ordinal):
        self.ordinal = ordinal
        sm = ctypes.c_int()
        mt = ctypes.c_int()
        gm = ctypes.c_size_t()
        sh = ctypes.c_size_t()
        major = ctypes.c_int()
        minor = ctypes.c_int()
        _capi.call("nb2_device_info", ordinal, ctypes.byref(sm), ctypes.byref(mt), ctypes.byref(gm),
                   ctypes.byref(sh), ctypes.byref(major), ctypes.byref(minor))
        self.sm_count = sm.value
        self.global_mem_size = gm.value
        self.shared_mem_optin = sh.value
        self.compute_capability = (major.value, minor.value)
        self.name = "cuda:%d" % ordinal


class Context:
    """One CUDA device made current for the calling process."""

    def __init__(self, ordinal=0):
        n = ctypes.c_int()
        _capi.call("nb2_device_count", ctypes.byref(n))
        if not 0 <= ordinal < n.value:
            raise RuntimeError("CUDA device %d not available (%d devices)" % (ordinal, n.value))
        _capi.call("nb2_set_device", ordinal)
        self.ordinal = ordinal
        self.devices = [Device(ordinal)]


_default_context = None


def create_some_context(ordinal=None):
    """Default context: the device given, else LOCAL_RANK, else device 0."""
    global _default_context
    import os

    if ordinal is None:
        ordinal = int(os.environ.get("LOCAL_RANK", "0"))
    if _default_context is None or _default_context.ordinal != ordinal:
        _default_context = Context(ordinal)
    return _default_context


def _free_stream(handle):
    try:
        _capi.lib().nb2_stream_destroy(handle)
    except Exception:  # interpreter shutdown
        pass


class CommandQueue:
    """An in-order CUDA stream."""

    def __init__(self, context=None, profiling=False):
        self.context = context if context is not None else create_some_context()
        self.device = self.context.devices[0]
        self.profiling = bool(profiling)
        s = ctypes.c_void_p()
        _capi.call("nb2_stream_create", ctypes.byref(s))
        self.stream = s.value
        self._finalizer = weakref.finalize(self, _free_stream, self.stream)

    def finish(self):
        _capi.call("nb2_stream_sync", self.stream)


def _free_device(ptr):
    try:
        _capi.lib().nb2_free(ptr)
    except Exception:
        pass


class DeviceArray:
    """A flat, owned (or borrowed) block of device memory with a dtype.

    Mirrors the small part of ``pyopencl.array.Array`` the reference relies on:
    ``data`` (here: the device address as int), ``shape``, ``dtype``, ``size``,
    ``nbytes``, ``ctype``, ``get()``, ``set()``, ``fill()``.
    """

    def __init__(self, queue, shape, dtype, data=None, offset=0, base=None):
        self.queue = queue
        self.shape = tuple(int(s) for s in (shape if np.iterable(shape) else (shape,)))
        self.dtype = np.dtype(dtype)
        self.size = int(np.prod(self.shape)) if self.shape else 1
        self.nbytes = self.size * self.dtype.itemsize
        self.offset = int(offset)
        if data is None:
            p = ctypes.c_void_p()
            _capi.call("nb2_malloc", ctypes.byref(p), self.nbytes)
            self.base_data = p.value
            self._finalizer = weakref.finalize(self, _free_device, self.base_data)
            self._base = None
        else:
            self.base_data = int(data)
            self._base = base  # keeps the owner alive
        self.data = self.base_data + self.offset

    def __len__(self):
        return self.shape[0] if self.shape else 1

    @property
    def ctype(self):
        return {"float32": "float", "int32": "int"}[self.dtype.name]

    @property
    def start(self):
        return self.offset // self.dtype.itemsize

    @property
    def ptr(self):
        return ctypes.c_void_p(self.data)

    def get(self):
        out = np.empty(self.shape, dtype=self.dtype)
        if self.nbytes:
            _capi.call("nb2_memcpy_d2h", out.ctypes.data_as(ctypes.c_void_p), self.ptr, self.nbytes,
                       self.queue.stream, 1)
        return out

    def set(self, array):
        array = np.ascontiguousarray(array, dtype=self.dtype)
        assert array.size == self.size
        if self.nbytes:
            _capi.call("nb2_memcpy_h2d", self.ptr, array.ctypes.data_as(ctypes.c_void_p), self.nbytes,
                       self.queue.stream, 1)

    def fill(self, value):
        if np.all(np.asarray(value) == 0):
            _capi.call("nb2_memset", self.ptr, 0, self.nbytes, self.queue.stream)
            self.queue.finish()
        else:
            self.set(np.full(self.shape, value, dtype=self.dtype))

    def read_region(self, elem_start, n_elems):
        """Blocking copy of ``n_elems`` elements starting at ``elem_start``."""
        out = np.empty(int(n_elems), dtype=self.dtype)
        if n_elems:
            isz = self.dtype.itemsize
            _capi.call("nb2_memcpy_d2h", out.ctypes.data_as(ctypes.c_void_p),
                       ctypes.c_void_p(self.data + int(elem_start) * isz), int(n_elems) * isz,
                       self.queue.stream, 1)
        return out

    def write_region(self, elem_start, array):
        array = np.ascontiguousarray(array, dtype=self.dtype)
        if array.size:
            isz = self.dtype.itemsize
            _capi.call("nb2_memcpy_h2d", ctypes.c_void_p(self.data + int(elem_start) * isz),
                       array.ctypes.data_as(ctypes.c_void_p), array.size * isz, self.queue.stream, 1)


Array = DeviceArray


def to_device(queue, array):
    """Upload a host ndarray (float32 / int32) and return a DeviceArray."""
    array = np.ascontiguousarray(array)
    out = DeviceArray(queue, array.shape, array.dtype)
    out.set(array)
    return out


def zeros(queue, shape, dtype):
    out = DeviceArray(queue, shape, dtype)
    _capi.call("nb2_memset", out.ptr, 0, out.nbytes, queue.stream)
    queue.finish()
    return out
