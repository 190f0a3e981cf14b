"""ctypes binding of libelman_b200.so (the C ABI declared in include/elman_b200.h).

There is no fallback: if the library is missing, loading raises with the build
command, and every compute call raises when the C side reports an error.
"""
from __future__ import annotations

import ctypes
import os
import re
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libelman_b200.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "elman_b200.h")

ELMAN_OK = 0
ELMAN_F32 = 0
ELMAN_BF16 = 1

_c = ctypes
_P = _c.c_void_p
_I = _c.c_int
_Z = _c.c_size_t
_L = _c.c_long
_F = _c.c_float

# name -> (restype, argtypes); must list every function the header declares
SIGNATURES = {
    "elman_b200_version": (_I, []),
    "elman_b200_last_error": (_c.c_char_p, []),
    "elman_b200_device_status": (_I, [_c.POINTER(_I), _I]),
    "elman_b200_set_option": (_I, [_c.c_char_p, _L]),
    "elman_b200_get_option": (_L, [_c.c_char_p]),
    "elman_b200_wait_probe": (_I, [_L, _P, _P]),
    "elman_b200_last_timing": (_I, [_I, _c.POINTER(_c.c_float)]),
    "elman_b200_recurrence_trace": (_I, [_c.POINTER(_c.c_longlong), _I]),
    "elman_b200_launch_count": (_L, []),
    "elman_b200_tc_launch_count": (_L, []),
    "elman_e1_forward_workspace": (_Z, [_I, _I, _I, _I]),
    "elman_e1_forward": (_I, [_I, _I, _I, _I, _I] + [_P] * 6 + [_P] * 3 + [_P, _Z, _P]),
    "elman_e1_forward_static_scratch_bytes": (_Z, []),
    "elman_e1_forward_static": (_I, [_I, _I, _I, _I, _I] + [_P] * 6 + [_P] * 3 + [_P]),
    "elman_e1_backward_workspace": (_Z, [_I, _I, _I, _I]),
    "elman_e1_backward": (_I, [_I, _I, _I, _I] + [_P] * 7 + [_P] * 5 + [_P, _Z, _P]),
    "elman_e1_forward_flags": (_I, [_I, _I, _I, _I, _I, _I] + [_P] * 6 + [_P] * 3 + [_P, _Z, _P]),
    "elman_e1_backward_carry": (_I, [_I, _I, _I, _I, _I] + [_P] * 8 + [_P] * 6 + [_P, _Z, _P]),
    "elman_b200_recurrence_blocks": (_I, [_I, _I, _I, _I, _I]),
    "elman_gemm": (_I, [_I, _I, _I, _I, _I, _P, _P, _P, _P, _I, _P]),
    "elman_column_sum_workspace": (_Z, [_I]),
    "elman_column_sum": (_I, [_I, _L, _I, _P, _P, _P, _Z, _P]),
    "elman_e1_recurrence_workspace": (_Z, [_I, _I]),
    "elman_e1_recurrence_forward": (_I, [_I] * 6 + [_P] * 4 + [_P] * 3 + [_P, _Z, _P]),
    "elman_e1_recurrence_backward": (_I, [_I] * 5 + [_P] * 7 + [_P] * 3 + [_P, _Z, _P]),
    "elman_e0_forward_workspace": (_Z, [_I, _I, _I, _I]),
    "elman_e0_forward": (_I, [_I, _I, _I, _I, _I] + [_P] * 7 + [_P] * 4 + [_P, _Z, _P]),
    "elman_e0_backward_workspace": (_Z, [_I, _I, _I, _I]),
    "elman_e0_backward": (_I, [_I, _I, _I, _I] + [_P] * 8 + [_P] * 6 + [_P, _Z, _P]),
    "elman_e5_forward_workspace": (_Z, [_I, _I, _I, _I, _I]),
    "elman_e5_forward": (_I, [_I, _I, _I, _I, _I, _I] + [_P] * 9 + [_P] * 3 + [_P, _Z, _P]),
    "elman_e5_backward_workspace": (_Z, [_I, _I, _I, _I, _I]),
    "elman_e5_backward": (_I, [_I, _I, _I, _I, _I] + [_P] * 10 + [_P] * 8 + [_P, _Z, _P]),
    "elman_e5_backward_carry": (_I, [_I, _I, _I, _I, _I] + [_P] * 11 + [_P] * 9 + [_P, _Z, _P]),
    "elman_b200_lowrank_blocks": (_I, [_I, _I, _I, _I, _I]),
    "elman_add_rmsnorm_backward_workspace": (_Z, [_I]),
    "elman_add_rmsnorm_forward": (_I, [_I, _L, _I, _P, _P, _P, _c.c_float, _P, _P, _P, _P]),
    "elman_add_rmsnorm_backward": (_I, [_I, _L, _I] + [_P] * 8 + [_P, _Z, _P]),
    "elman_in_proj_workspace": (_Z, [_I, _L, _I]),
    "elman_in_proj_split_silu": (_I, [_I, _L, _I, _I] + [_P] * 5 + [_P, _Z, _P]),
    "elman_silu_backward_concat": (_I, [_I, _L, _I, _P, _P, _P, _P, _P]),
    "elman_e1_hx_forward_workspace": (_Z, [_I, _I, _I, _I]),
    "elman_e1_hx_forward": (_I, [_I, _I, _I, _I, _I] + [_P] * 7 + [_P] * 4 + [_P, _Z, _P]),
    "elman_e1_hx_backward_workspace": (_Z, [_I, _I, _I, _I]),
    "elman_e1_hx_backward": (_I, [_I, _I, _I, _I] + [_P] * 8 + [_P] * 6 + [_P, _Z, _P]),
    "elman_spectral_norm_forward": (_I, [_I, _I, _P, _P, _P, _P, _P, _F, _F, _I, _P]),
    "elman_spectral_norm_backward": (_I, [_I, _I, _P, _P, _P, _P, _P, _P, _I, _F, _F, _P]),
    "elman_e4_forward_workspace": (_Z, [_I, _I, _I, _I, _I]),
    "elman_e4_forward": (_I, [_I, _I, _I, _I, _I, _I] + [_P] * 7 + [_P] * 3 + [_P, _Z, _P]),
    "elman_e4_backward_workspace": (_Z, [_I, _I, _I, _I, _I]),
    "elman_e4_backward": (_I, [_I, _I, _I, _I, _I] + [_P] * 8 + [_P] * 6 + [_P, _Z, _P]),
    "elman_e33_forward_workspace": (_Z, [_I, _I, _I, _I]),
    "elman_e33_forward": (_I, [_I, _I, _I, _I, _I] + [_P] * 5 + [_P] * 3 + [_P, _Z, _P]),
    "elman_e33_backward_workspace": (_Z, [_I, _I, _I, _I]),
    "elman_e33_backward": (_I, [_I, _I, _I, _I] + [_P] * 6 + [_P] * 4 + [_P, _Z, _P]),
    "elman_adamw_step": (_I, [_I, _L, _P, _P, _P, _P] + [_c.c_float] * 5 + [_P, _P, _P]),
    "elman_projection": (_I, [_I, _I, _I, _I, _P, _I, _P, _I, _P, _P, _I, _I, _P]),
}

_lib = None
_lock = threading.Lock()


class ElmanB200Error(RuntimeError):
    """An entry point of libelman_b200 returned a non-zero status."""


def header_function_names():
    """Function names declared in include/elman_b200.h (parsed from the header text)."""
    with open(HEADER_PATH) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(elman_[a-z0-9_]+)\s*\(", text)))


def load():
    """Load the shared library (once) and attach the signatures."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing. Build it with `python -m elman_b200.build` "
                "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback.")
        try:
            import torch  # noqa: F401  (makes the CUDA runtime PyTorch ships resolvable)
        except Exception:  # pragma: no cover
            pass
        lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc != ELMAN_OK:
        msg = load().elman_b200_last_error().decode(errors="replace")
        raise ElmanB200Error(f"{what} failed (code {rc}): {msg}")


def set_option(name: str, value: int) -> None:
    check(load().elman_b200_set_option(name.encode(), int(value)), f"set_option({name})")


def get_option(name: str) -> int:
    return int(load().elman_b200_get_option(name.encode()))


def device_status(clear: bool = False):
    """(code, detail) of the current device's bounded-wait status word."""
    detail = ctypes.c_int(0)
    rc = load().elman_b200_device_status(ctypes.byref(detail), 1 if clear else 0)
    return rc, detail.value


def launch_count() -> int:
    return int(load().elman_b200_launch_count())


def tc_launch_count() -> int:
    return int(load().elman_b200_tc_launch_count())


def last_timing_ms(phase: int) -> float:
    """Elapsed ms of a timed phase of the most recent call (option time_kernels)."""
    ms = ctypes.c_float(0.0)
    check(load().elman_b200_last_timing(int(phase), ctypes.byref(ms)), "last_timing")
    return float(ms.value)
