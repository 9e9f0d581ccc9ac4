"""Device ragged array: one HBM buffer + int32 index arrays, CUDA-backed.

Same Python semantics as the reference's ``CLRaggedArray``
(nengo_ocl/clraggedarray.py:65-311):

* constructed from a host ``RaggedArray`` (one upload of the flat buffer);
* ``starts/shape0s/shape1s/stride0s/stride1s`` host copies (read-only) with
  device twins ``cl_starts`` ... (uploaded lazily here: the reference uploads
  and synchronises on every assignment, lines 128-196);
* ``clra[int]`` -> read-only host ndarray, copying only the bounding region of
  the (possibly strided) item; ``clra[list]`` -> a new device view sharing the
  buffer; ``clra[int] = value`` -> contiguous write, or read-modify-write of
  the bounding region for a discontiguous view (lines 256-299);
* ``to_host()`` -> host ``RaggedArray`` of the whole buffer.
"""

from io import StringIO

import numpy as np

from nengo_ocl_b200.raggedarray import RaggedArray
from nengo_ocl_b200.runtime import DeviceArray, to_device
from nengo_ocl_b200.utils import equal_strides, is_iterable


def to_host(queue, darray, dtype, start, shape, elemstrides):
    """Copy one strided 2-D item off the device (bounding region only)."""
    if min(elemstrides) < 0:
        raise NotImplementedError()
    m, n = int(shape[0]), int(shape[1])
    sm, sn = int(elemstrides[0]), int(elemstrides[1])
    if m * n == 0:
        return np.zeros((m, n), dtype=dtype)
    span = (m - 1) * sm + (n - 1) * sn + 1
    region = darray.read_region(int(start), span)
    isz = np.dtype(dtype).itemsize
    return np.ndarray(shape=(m, n), dtype=dtype, buffer=region.data, offset=0,
                      strides=(isz * sm, isz * sn))


class _LazyIndex:
    """Descriptor pair: host int32 array + lazily uploaded device twin."""

    def __init__(self, name):
        self.name = name

    def __set_name__(self, owner, attr):
        self.attr = attr

    def __get__(self, obj, objtype=None):
        if obj is None:
            return self
        return obj.__dict__["_" + self.name]

    def __set__(self, obj, values):
        arr = np.array(values, dtype=np.int32)
        arr.setflags(write=False)
        obj.__dict__["_" + self.name] = arr
        obj.__dict__.pop("_cl_" + self.name, None)
        obj.__dict__["_sizes"] = None


class CUDARaggedArray:
    """A linear device buffer partitioned into variable-size 2-D sections."""

    starts = _LazyIndex("starts")
    shape0s = _LazyIndex("shape0s")
    shape1s = _LazyIndex("shape1s")
    stride0s = _LazyIndex("stride0s")
    stride1s = _LazyIndex("stride1s")

    def __init__(self, queue, np_raggedarray):
        self.queue = queue
        self.starts = np_raggedarray.starts
        self.shape0s = np_raggedarray.shape0s
        self.shape1s = np_raggedarray.shape1s
        self.stride0s = np_raggedarray.stride0s
        self.stride1s = np_raggedarray.stride1s
        self.buf = np_raggedarray.buf
        self.names = np_raggedarray.names

    @classmethod
    def from_arrays(cls, queue, arrays, names=None, dtype=None, align=False):
        return cls(queue, RaggedArray(arrays, names=names, dtype=dtype, align=align))

    @classmethod
    def from_buffer(cls, queue, cl_buf, starts, shape0s, shape1s, stride0s, stride1s, names=None):
        self = cls.__new__(cls)
        self.queue = queue
        self.starts = starts
        self.shape0s = shape0s
        self.shape1s = shape1s
        self.stride0s = stride0s
        self.stride1s = stride1s
        self.cl_buf = cl_buf
        self.names = names
        return self

    def _device_index(self, name):
        key = "_cl_" + name
        if key not in self.__dict__:
            self.__dict__[key] = to_device(self.queue, self.__dict__["_" + name])
        return self.__dict__[key]

    cl_starts = property(lambda self: self._device_index("starts"))
    cl_shape0s = property(lambda self: self._device_index("shape0s"))
    cl_shape1s = property(lambda self: self._device_index("shape1s"))
    cl_stride0s = property(lambda self: self._device_index("stride0s"))
    cl_stride1s = property(lambda self: self._device_index("stride1s"))

    @property
    def ctype(self):
        return self.cl_buf.ctype

    @property
    def dtype(self):
        return self.cl_buf.dtype

    @property
    def names(self):
        return self._names

    @names.setter
    def names(self, names):
        if names is None:
            names = [""] * len(self.starts)
        self._names = tuple(names)

    @property
    def sizes(self):
        if self.__dict__.get("_sizes") is None:
            self.__dict__["_sizes"] = self.shape0s * self.shape1s
        return self.__dict__["_sizes"]

    @property
    def nbytes(self):
        return int(self.sizes.sum()) * self.dtype.itemsize

    @property
    def buf(self):
        buf = self.cl_buf.get()
        buf.setflags(write=False)
        return buf

    @buf.setter
    def buf(self, buf):
        buf = np.asarray(buf)
        assert buf.dtype in (np.float32, np.int32)
        self.cl_buf = to_device(self.queue, buf)

    def __len__(self):
        return len(self.starts)

    def __str__(self):
        out = StringIO()
        width = max([0] + [len(n) for n in self.names])
        for i, name in enumerate(self.names):
            print(name.rjust(width), self[i], file=out)
        return out.getvalue()

    def __getitem__(self, item):
        """One item -> host ndarray (read-only); several items -> device view."""
        if is_iterable(item) or isinstance(item, slice):
            return self.getitem_device(item)
        item = int(item)
        buf = to_host(self.queue, self.cl_buf, self.dtype, self.starts[item],
                      (self.shape0s[item], self.shape1s[item]),
                      (self.stride0s[item], self.stride1s[item]))
        buf.setflags(write=False)
        return buf

    def getitem_device(self, item):
        if isinstance(item, slice):
            item = np.arange(len(self))[item]
        if is_iterable(item):
            item = np.asarray([int(i) for i in item], dtype=np.intp)
            return CUDARaggedArray.from_buffer(
                self.queue, self.cl_buf, self.starts[item], self.shape0s[item], self.shape1s[item],
                self.stride0s[item], self.stride1s[item], names=[self.names[i] for i in item])
        item = int(item)
        isz = self.dtype.itemsize
        arr = DeviceArray(self.queue, (self.shape0s[item], self.shape1s[item]), self.dtype,
                          data=self.cl_buf.base_data,
                          offset=self.cl_buf.offset + int(self.starts[item]) * isz, base=self.cl_buf)
        arr.strides = (int(self.stride0s[item]) * isz, int(self.stride1s[item]) * isz)
        return arr

    def __setitem__(self, item, new_value):
        if isinstance(item, slice) or is_iterable(item):
            raise NotImplementedError("assigning to several items at once is not supported")
        item = int(item)
        m, n = int(self.shape0s[item]), int(self.shape1s[item])
        sm, sn = int(self.stride0s[item]), int(self.stride1s[item])
        start = int(self.starts[item])
        if m * n == 0:
            return
        if (sm, sn) in [(1, m), (n, 1)] or equal_strides((sm, sn), (n, 1), (m, n)):
            # contiguous: one write
            if isinstance(new_value, np.ndarray):
                array = np.asarray(new_value, order="C", dtype=self.dtype)
                assert array.size == m * n
            else:
                array = np.zeros((m, n), dtype=self.dtype)
                array[...] = new_value
            if (sm, sn) == (1, m) and m > 1 and n > 1:
                array = np.ascontiguousarray(array.reshape(m, n).T)
            self.cl_buf.write_region(start, array.ravel())
        else:
            # discontiguous: read the bounding region, patch it, write it back
            span = (m - 1) * sm + (n - 1) * sn + 1
            region = self.cl_buf.read_region(start, span)
            isz = self.dtype.itemsize
            view = np.ndarray(shape=(m, n), dtype=self.dtype, buffer=region.data, offset=0,
                              strides=(isz * sm, isz * sn))
            view[...] = new_value
            self.cl_buf.write_region(start, region)

    def to_host(self):
        """Copy the whole object to a host RaggedArray."""
        return RaggedArray.from_buffer(self.buf, self.starts, self.shape0s, self.shape1s,
                                       self.stride0s, self.stride1s, names=self.names)


# The reference's name, so planning code written against it imports unchanged.
CLRaggedArray = CUDARaggedArray
