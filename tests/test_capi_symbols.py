"""The C-ABI library loads without a GPU and exports what the header declares."""

import ctypes

from nengo_ocl_b200 import _capi


def test_library_exports_every_declared_symbol():
    lib = _capi.lib()
    names = _capi.declared_symbols()
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_every_declared_symbol_has_a_python_signature():
    names = set(_capi.declared_symbols()) - {"nb2_last_error"}
    assert names <= set(_capi._SIGNATURES), sorted(names - set(_capi._SIGNATURES))


def test_abi_version_and_error_string():
    lib = _capi.lib()
    assert lib.nb2_abi_version() == 1
    assert isinstance(lib.nb2_last_error(), bytes)


def test_argument_errors_are_reported_not_raised_in_c():
    # a NULL output pointer is rejected with NB2_ERR_ARG before any CUDA call
    lib = _capi.lib()
    status = lib.nb2_malloc(None, 16)
    assert status == -2
    assert b"dptr" in lib.nb2_last_error()


def test_neuron_args_struct_layout():
    # 10 x {ptr, ptr, float(+pad)} + double + 2 ints
    assert ctypes.sizeof(_capi.nb2_var) == 24
    # 10 variables, double dt, int upsample / adaptive / fastlif, padded to the 8-byte alignment
    assert ctypes.sizeof(_capi.nb2_neuron_args) == 10 * 24 + 24
    assert _capi.nb2_neuron_args.fastlif.offset == 10 * 24 + 16
