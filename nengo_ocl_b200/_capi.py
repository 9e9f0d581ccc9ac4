"""ctypes binding of libnengo_b200.so (declared in include/nengo_b200.h).

The library is the only compute path: there is no CPU fallback.  Importing
this module never touches the GPU; ``lib()`` loads the shared library on first
use and raises ``RuntimeError`` if it has not been built
(``python -m nengo_ocl_b200.csrc.build``).
"""

import ctypes
import os
import re
from ctypes import POINTER, Structure, c_char_p, c_double, c_float, c_int, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnengo_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "nengo_b200.h")

NB2_ERR_TIMEOUT = -4
GEMV_CTA, GEMV_CTA_BULK, GEMV_WARP, GEMV_PIPE = 0, 1, 2, 3
GEMV_ABUF, GEMV_XBUF, GEMV_RMAX = 8192, 2048, 1024
NEURON_LIF, NEURON_LIF_RATE, NEURON_RELU, NEURON_SPIKING_RELU, NEURON_SIGMOID = range(5)


class NB2Error(RuntimeError):
    """A C-ABI call returned a negative status."""


class nb2_var(Structure):
    _fields_ = [("starts", c_void_p), ("buf", c_void_p), ("value", c_float)]


class nb2_neuron_args(Structure):
    _fields_ = [(n, nb2_var) for n in "J V W S N tau ref amp tau_n inc_n".split()] + [
        ("dt", c_double),
        ("upsample", c_int),
        ("adaptive", c_int),
        ("fastlif", c_int),
    ]


_P = c_void_p  # every device / host pointer crosses the boundary as void*

_SIGNATURES = {
    "nb2_abi_version": [],
    "nb2_set_programmatic_launch": [c_int],
    "nb2_device_count": [POINTER(c_int)],
    "nb2_set_device": [c_int],
    "nb2_device_info": [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_size_t), POINTER(c_size_t),
                        POINTER(c_int), POINTER(c_int)],
    "nb2_malloc": [POINTER(c_void_p), c_size_t],
    "nb2_free": [_P],
    "nb2_host_alloc": [POINTER(c_void_p), c_size_t],
    "nb2_host_free": [_P],
    "nb2_memcpy_h2d": [_P, _P, c_size_t, _P, c_int],
    "nb2_memcpy_d2h": [_P, _P, c_size_t, _P, c_int],
    "nb2_memcpy_d2d": [_P, _P, c_size_t, _P],
    "nb2_memset": [_P, c_int, c_size_t, _P],
    "nb2_stream_create": [POINTER(c_void_p)],
    "nb2_stream_destroy": [_P],
    "nb2_stream_sync": [_P],
    "nb2_device_sync": [],
    "nb2_event_create": [POINTER(c_void_p)],
    "nb2_event_destroy": [_P],
    "nb2_event_record": [_P, _P],
    "nb2_stream_wait_event": [_P, _P],
    "nb2_event_sync": [_P],
    "nb2_event_elapsed_ms": [_P, _P, POINTER(c_float)],
    "nb2_graph_begin": [_P],
    "nb2_graph_end": [_P, POINTER(c_void_p)],
    "nb2_graph_abort": [_P],
    "nb2_graph_launch": [_P, _P, c_int],
    "nb2_graph_destroy": [_P],
    "nb2_ipc_get_handle": [_P, _P],
    "nb2_ipc_open_handle": [_P, POINTER(c_void_p)],
    "nb2_ipc_close_handle": [_P],
    "nb2_gemv_ragged": [_P, c_int, _P, c_int, c_int, _P, _P, c_int, _P, _P, _P, _P, c_double, c_double,
                        c_double, _P, _P, _P, _P],
    "nb2_gemv_block": [_P, _P, c_int, c_int, _P, _P, c_int, _P, c_int, _P, _P, _P, _P, c_double, c_double,
                       c_double],
    "nb2_gemv_pipelined": [_P, _P, c_int, _P, c_int, _P, _P, _P, _P, c_double, c_double, c_double, _P, _P, _P,
                           _P],
    "nb2_timeupdate": [_P, _P, _P, c_double],
    "nb2_reset": [_P, c_int, _P, _P, _P, _P],
    "nb2_copy": [_P, c_int, c_int] + [_P] * 10,
    "nb2_slicedcopy": [_P, c_int, c_int] + [_P] * 12,
    "nb2_elementwise_inc": [_P, c_int, c_int, c_int] + [_P] * 17,
    "nb2_linearfilter": [_P, c_int, c_int, c_int] + [_P] * 23,
    "nb2_learning_delta": [_P, c_int, c_int, c_int] + [_P] * 21,
    "nb2_probes": [_P, c_int, c_int] + [_P] * 11,
    "nb2_probes_wide": [_P, c_int, c_int] + [_P] * 12,
    "nb2_probes_wide_noalloc": [_P, c_int, c_int] + [_P] * 11,
    "nb2_presentinput": [_P, c_int, c_int, _P, c_double] + [_P] * 9,
    "nb2_neurons": [_P, c_int, c_int, c_int, _P, POINTER(nb2_neuron_args)],
    "nb2_spmv_csr": [_P, _P, _P, _P, c_int, c_int, _P, _P, c_int],
    "nb2_spmv_ell": [_P, _P, _P, _P, c_int, c_int, c_int, _P, _P, c_int],
    "nb2_ensemble_stream": [_P, _P, c_int, _P, c_int, _P, _P, _P, _P, c_double, _P, _P],
    "nb2_exchange_wait": [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_double],
    "nb2_exchange_push": [_P, _P, _P, _P, _P, c_int, c_int, c_int],
    "nb2_gather_sum": [_P, c_int, c_int, _P, _P, _P],
    "nb2_whitenoise": [_P, c_int, c_int] + [_P] * 10 + [c_double],
    "nb2_conv2d": [_P, _P, _P, _P] + [c_int] * 15,
    "nb2_pool2d": [_P, _P, _P] + [c_int] * 9,
    "nb2_ensemble_step": [_P, c_int, _P, c_int, _P, _P, _P, _P, _P, c_double],
    "nb2_direct": [_P, c_int, _P, c_int, c_int, _P, c_int, _P, _P, _P, _P, _P, _P],
    "nb2_step_loop_create": [POINTER(c_void_p)],
    "nb2_step_loop_destroy": [_P],
    "nb2_step_loop_finalize": [_P, c_int],
    "nb2_step_loop_run": [_P, _P, c_int],
    "nb2_step_loop_info": [_P, POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int)],
    "nb2_step_loop_status": [_P, _P, POINTER(c_int)],
    "nb2_step_loop_wait_selftest": [_P, _P],
    "nb2_step_loop_clear_status": [_P, _P],
}
# a phase of the step loop takes (loop, barrier) + the arguments of the launch entry point without the stream
for _name in ("timeupdate", "gather_sum", "direct", "ensemble_step", "gemv_block", "probes", "linearfilter",
              "presentinput"):
    _SIGNATURES["nb2_step_loop_add_" + _name] = [_P, c_int] + _SIGNATURES["nb2_" + _name][1:]
del _name

_lib = None


def declared_symbols():
    """Names of every function declared in include/nengo_b200.h."""
    with open(HEADER_PATH) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nb2_[a-z0-9_]+)\s*\(", text)))


class ExchangeDesc(ctypes.Structure):
    """``nb2_exchange_desc``"""

    _fields_ = [("peer_staging", c_void_p), ("peer_flags", c_void_p), ("ctl", c_void_p), ("cta_runs", c_void_p),
                ("x_base", c_int), ("x_lo", c_int), ("x_hi", c_int),
                ("rank", c_int), ("world", c_int), ("seg", c_int)]


def header_constants(prefix):
    """Integer ``#define``s of the C header whose names start with ``prefix``."""
    with open(HEADER_PATH) as f:
        text = f.read()
    return {k: int(v) for k, v in re.findall(r"#define\s+(%s[A-Z0-9_]*)\s+(\d+)\b" % prefix, text)}


def lib():
    """Load the shared library (once) and attach argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libnengo_b200.so is not built; run `python -m nengo_ocl_b200.csrc.build`. "
            "There is no CPU fallback for the device path."
        )
    handle = ctypes.CDLL(LIB_PATH)
    handle.nb2_last_error.restype = c_char_p
    handle.nb2_last_error.argtypes = []
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(handle, name, None)
        if fn is None:
            continue
        fn.argtypes = argtypes
        fn.restype = c_int
    _lib = handle
    return _lib


def check(status):
    if status < 0:
        msg = lib().nb2_last_error()
        raise NB2Error("nb2 call failed (%d): %s" % (status, msg.decode() if msg else "?"))
    return status


def call(name, *args):
    """Call ``name`` through the C ABI and raise on a negative status."""
    return check(getattr(lib(), name)(*args))


def phase(name, *args):
    """``(loop, barrier) -> None`` that appends the launch ``nb2_<name>(stream, *args)`` as a
    phase of a persistent step loop (``nb2_step_loop_add_<name>``, csrc/nb2_step_loop.cu)."""

    def add(loop, barrier):
        call("nb2_step_loop_add_" + name, loop, int(bool(barrier)), *args)

    return add
