"""The C-ABI library loads and exports every function include/elman_b200.h declares
(no compute calls: this runs without a GPU)."""
import ctypes

import pytest

from elman_b200 import _lib


def test_library_loads_and_reports_version():
    lib = _lib.load()
    assert lib.elman_b200_version() >= 100
    assert lib.elman_b200_last_error() is not None


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.load()
    declared = _lib.header_function_names()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    for name in _lib.SIGNATURES:
        assert name in declared, f"{name} bound in Python but not declared in the header"


def test_workspace_queries_are_pure_host_functions():
    lib = _lib.load()
    T, B, d = 512, 32, 1280
    bf = lib.elman_e1_forward_workspace(_lib.ELMAN_BF16, T, B, d)
    f32 = lib.elman_e1_forward_workspace(_lib.ELMAN_F32, T, B, d)
    assert bf >= T * B * d * 2 and f32 >= T * B * d * 4
    assert bf % 256 == 0 and f32 % 256 == 0
    assert lib.elman_e1_backward_workspace(_lib.ELMAN_BF16, T, B, d) >= (T + 1) * B * d * 2
    assert lib.elman_e0_forward_workspace(_lib.ELMAN_F32, 4, 2, 8) > 0
    assert lib.elman_e5_backward_workspace(_lib.ELMAN_BF16, 16, 4, 64, 8) > 0


def test_options_round_trip_and_unknown_name_is_an_error():
    _lib.set_option("spin_limit", 12345)
    assert _lib.get_option("spin_limit") == 12345
    _lib.set_option("spin_limit", 4000000)
    with pytest.raises(_lib.ElmanB200Error):
        _lib.set_option("no_such_option", 1)
    assert _lib.get_option("no_such_option") == -1


def test_argument_errors_are_reported_without_a_gpu():
    lib = _lib.load()
    rc = lib.elman_projection(7, 4, 4, 4, None, 4, None, 4, None, None, 4, 0, None)
    assert rc != 0
    assert b"dtype" in lib.elman_b200_last_error()
    rc = lib.elman_e1_forward(_lib.ELMAN_F32, 1, -1, 2, 2, *([None] * 9), None, 0, None)
    assert rc != 0
