"""Test infrastructure: a host-memory stand-in for the C library, so that the planning code of
the simulator (operator grouping, fusion, index tables, graph shape) can be exercised without a
GPU.  "Device" allocations are host buffers, copies are memmoves, launches are recorded and do
nothing.  Nothing outside tests/ uses this module."""

import ctypes

from nengo_ocl_b200 import _capi


class FakeLibrary:
    def __init__(self):
        self.calls = []      # (entry point, argument count) of every launch-like call
        self._keep = []
        self._next = 1000

    def _handle(self):
        self._next += 1
        return self._next

    def _invoke(self, name, args):
        if name in ("nb2_malloc", "nb2_host_alloc"):
            buf = ctypes.create_string_buffer(max(int(args[1]), 8) + 256)
            self._keep.append(buf)
            args[0]._obj.value = (ctypes.addressof(buf) + 255) & ~255
        elif name in ("nb2_memcpy_h2d", "nb2_memcpy_d2h", "nb2_memcpy_d2d"):
            ctypes.memmove(args[0], args[1], int(args[2]))
        elif name == "nb2_memset":
            ctypes.memset(args[0], int(args[1]), int(args[2]))
        elif name == "nb2_device_count":
            args[0]._obj.value = 1
        elif name == "nb2_device_info":
            for a, v in zip(args[1:], (148, 1024, 232448, 180 << 30, 10, 0)):
                a._obj.value = v
        elif name in ("nb2_stream_create", "nb2_event_create", "nb2_step_loop_create"):
            args[0]._obj.value = self._handle()
        elif name == "nb2_graph_end":
            args[1]._obj.value = self._handle()
        elif name == "nb2_step_loop_info":
            for a in args[1:]:
                a._obj.value = 1
        elif name == "nb2_step_loop_status":
            args[2]._obj.value = 0
        else:
            self.calls.append((name, len(args)))
        return 0

    def __getattr__(self, name):
        if name == "nb2_last_error":
            return lambda: b"fake library"
        if not name.startswith("nb2_"):
            raise AttributeError(name)
        return lambda *args: self._invoke(name, args)


def install(monkeypatch):
    """Route ``_capi.lib()`` / ``_capi.call`` to a fresh FakeLibrary for the duration of a test."""
    fake = FakeLibrary()
    monkeypatch.setattr(_capi, "_lib", fake)
    monkeypatch.setattr(_capi, "lib", lambda: fake)
    return fake
