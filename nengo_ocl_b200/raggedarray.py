"""Host ragged array: a list of <=2-D arrays packed into one flat buffer.

Same semantics as the reference's ``nengo_ocl/raggedarray.py:31-236``:

* one flat ``buf`` (float32 or int32) plus five read-only int32 index arrays
  ``starts / shape0s / shape1s / stride0s / stride1s`` (element units);
* items are row-major by default (``stride0 = shape1``, ``stride1 = 1``);
* ``align=True`` pads item starts to 16 / 4 / 1 elements depending on the
  item size (reference lines 46-55);
* ``ra[int]`` is a strided ndarray *view* into ``buf``; ``ra[list]`` is a new
  ragged array sharing ``buf``; ``add_views`` appends extra items that alias
  existing storage (used for signal views, reference lines 224-236).
"""

from io import StringIO

import numpy as np

from nengo_ocl_b200.utils import is_iterable, round_up

_DTYPES = (np.dtype(np.float32), np.dtype(np.int32))


def _index_array(values):
    arr = np.array(values, dtype=np.int32)
    arr.setflags(write=False)
    return arr


def allclose(a, b, atol=1e-3, rtol=1e-3):
    """Index arrays equal and buffers close (reference raggedarray.py:15-28)."""
    for name in ("starts", "shape0s", "shape1s", "stride0s", "stride1s"):
        if not np.array_equal(getattr(a, name), getattr(b, name)):
            return False
    return bool(np.allclose(a.buf, b.buf, atol=atol, rtol=rtol))


class RaggedArray:
    """A linear buffer partitioned into variable-size 2-D sections."""

    def __init__(self, arrays, names=None, dtype=None, align=False):
        arrays = [np.asarray(a) for a in arrays]
        assert len(arrays) > 0
        assert all(a.ndim <= 2 for a in arrays)

        dtype = arrays[0].dtype if dtype is None else dtype
        dtype = np.dtype(dtype)
        assert dtype in _DTYPES

        sizes = [a.size for a in arrays]
        starts = [0]
        for prev_size, size in zip(sizes[:-1], sizes[1:]):
            end = starts[-1] + prev_size
            if align:
                quantum = 16 if size >= 16 else 4 if size >= 8 else 1
                end = round_up(end, quantum)
            starts.append(end)

        self.starts = starts
        self.shape0s = [a.shape[0] if a.ndim > 0 else 1 for a in arrays]
        self.shape1s = [a.shape[1] if a.ndim > 1 else 1 for a in arrays]
        self.stride0s = [a.shape[1] if a.ndim == 2 else 1 for a in arrays]
        self.stride1s = [1] * len(arrays)

        buf = np.zeros(starts[-1] + sizes[-1], dtype=dtype)
        for a, s in zip(arrays, starts):
            buf[s : s + a.size] = a.ravel()
        self.buf = buf
        self.names = names

    @classmethod
    def from_buffer(cls, buf, starts, shape0s, shape1s, stride0s, stride1s, names=None):
        self = cls.__new__(cls)
        self.starts = starts
        self.shape0s = shape0s
        self.shape1s = shape1s
        self.stride0s = stride0s
        self.stride1s = stride1s
        self.buf = buf
        self.names = names
        return self

    # ---- metadata ---------------------------------------------------------
    @property
    def dtype(self):
        return self.buf.dtype

    @property
    def names(self):
        return self._names

    @names.setter
    def names(self, names):
        if names is None:
            names = [""] * len(self._starts)
        self._names = tuple(names)
        assert len(self._names) == self._starts.size

    @property
    def starts(self):
        return self._starts

    @starts.setter
    def starts(self, values):
        self._starts = _index_array(values)
        assert np.all(self._starts >= 0)

    @property
    def shape0s(self):
        return self._shape0s

    @shape0s.setter
    def shape0s(self, values):
        self._shape0s = _index_array(values)
        self._sizes = None
        assert np.all(self._shape0s >= 0)
        assert self._shape0s.size == self._starts.size

    @property
    def shape1s(self):
        return self._shape1s

    @shape1s.setter
    def shape1s(self, values):
        self._shape1s = _index_array(values)
        self._sizes = None
        assert np.all(self._shape1s > 0)
        assert self._shape1s.size == self._starts.size

    @property
    def stride0s(self):
        return self._stride0s

    @stride0s.setter
    def stride0s(self, values):
        self._stride0s = _index_array(values)
        assert np.all(self._stride0s != 0)

    @property
    def stride1s(self):
        return self._stride1s

    @stride1s.setter
    def stride1s(self, values):
        self._stride1s = _index_array(values)
        assert np.all(self._stride1s != 0)

    @property
    def sizes(self):
        if getattr(self, "_sizes", None) is None:
            self._sizes = self._shape0s * self._shape1s
        return self._sizes

    @property
    def nbytes(self):
        return int(self.sizes.sum()) * self.dtype.itemsize

    @property
    def buf(self):
        return self._buf

    @buf.setter
    def buf(self, buf):
        buf = np.asarray(buf)
        assert buf.dtype in _DTYPES
        self._buf = buf

    # ---- container protocol ----------------------------------------------
    def __len__(self):
        return len(self._starts)

    def __str__(self):
        out = StringIO()
        width = max(len(n) for n in self.names)
        for i, name in enumerate(self.names):
            print(name.rjust(width), self[i], file=out)
        return out.getvalue()

    def __getitem__(self, item):
        if isinstance(item, slice):
            item = np.arange(len(self))[item]

        if is_iterable(item):
            item = [int(i) for i in item]
            sub = self.__class__.__new__(self.__class__)
            sub.starts = self._starts[item]
            sub.shape0s = self._shape0s[item]
            sub.shape1s = self._shape1s[item]
            sub.stride0s = self._stride0s[item]
            sub.stride1s = self._stride1s[item]
            sub.buf = self._buf
            sub.names = [self._names[i] for i in item]
            return sub

        item = int(item)
        isz = self.dtype.itemsize
        return np.ndarray(
            shape=(self._shape0s[item], self._shape1s[item]),
            dtype=self.dtype,
            buffer=self._buf.data,
            offset=isz * int(self._starts[item]),
            strides=(isz * int(self._stride0s[item]), isz * int(self._stride1s[item])),
        )

    def __setitem__(self, item, value):
        try:
            item = int(item)
        except TypeError as e:
            raise NotImplementedError("`item` must be castable to int") from e
        self[item][...] = value

    def add_views(self, starts, shape0s, shape1s, stride0s, stride1s, names=None):
        """Append items that alias existing storage (no new data)."""
        assert all(
            s + n0 * n1 <= self._buf.size for s, n0, n1 in zip(starts, shape0s, shape1s)
        )
        old_names = self._names
        self.starts = list(self._starts) + list(starts)
        self.shape0s = list(self._shape0s) + list(shape0s)
        self.shape1s = list(self._shape1s) + list(shape1s)
        self.stride0s = list(self._stride0s) + [int(s) for s in stride0s]
        self.stride1s = list(self._stride1s) + [int(s) for s in stride1s]
        self.names = old_names + (tuple(names) if names else ("",) * len(starts))
