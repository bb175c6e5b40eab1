"""ctypes binding of libpaged_attention_b200_test_aids.so (include/paged_attention_b200_test_aids.h).

Test and measurement aids only (a self-test of the bounded wait, a read-only streaming probe);
nothing on the product path imports this module.  Used by the tests and by bench.py's
roofline report.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

from . import _cabi

_LIB_NAME = "libpaged_attention_b200_test_aids.so"
_lib = None

EXPORTED_SYMBOLS = ("pa_aid_selftest_wait_timeout", "pa_aid_measure_read_bandwidth", "pa_aid_time_launches",
                    "pa_aid_last_error")


def library_path() -> Path:
    return Path(__file__).resolve().parent / _LIB_NAME


def load_library() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise RuntimeError(f"{path} is missing: build it with `python -m flash_attention_factory_b200.build`")
    lib = ctypes.CDLL(str(path))
    lib.pa_aid_selftest_wait_timeout.argtypes = [ctypes.c_uint32, ctypes.POINTER(ctypes.c_int32)]
    lib.pa_aid_selftest_wait_timeout.restype = ctypes.c_int
    lib.pa_aid_measure_read_bandwidth.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p,
                                                  ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32,
                                                  ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)]
    lib.pa_aid_measure_read_bandwidth.restype = ctypes.c_int
    lib.pa_aid_time_launches.argtypes = [ctypes.c_void_p, ctypes.POINTER(_cabi.PaParams), ctypes.c_uint32,
                                         ctypes.c_uint32, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)]
    lib.pa_aid_time_launches.restype = ctypes.c_int
    lib.pa_aid_last_error.argtypes = []
    lib.pa_aid_last_error.restype = ctypes.c_char_p
    _lib = lib
    return lib


def _check(rc: int) -> None:
    if rc != _cabi.PA_OK:
        raise RuntimeError(load_library().pa_aid_last_error().decode())


def selftest_wait_timeout(limit_us: int) -> int:
    """Runs the bounded-wait self-test; returns the device status word its kernel recorded."""
    word = ctypes.c_int32(-1)
    _check(load_library().pa_aid_selftest_wait_timeout(limit_us, ctypes.byref(word)))
    return int(word.value)


def measure_read_bandwidth(ptr: int, nbytes: int, iters: int = 10, stream: int = 0,
                           ptr2: int = 0, nbytes2: int = 0, method: int = 0) -> float:
    """GB/s of a kernel that only reads `nbytes` at `ptr` (+ `nbytes2` at `ptr2`), blocking.
    method 0: 16-byte loads; method 1: bulk copies into a shared-memory ring."""
    rate = ctypes.c_float(0.0)
    _check(load_library().pa_aid_measure_read_bandwidth(ctypes.c_void_p(ptr), nbytes, ctypes.c_void_p(ptr2 or None),
                                                        nbytes2, method, iters, ctypes.c_void_p(stream),
                                                        ctypes.byref(rate)))
    return float(rate.value)


def time_launches(entry: str, params_list, calls: int, stream: int = 0) -> float:
    """Mean microseconds per call of `calls` back-to-back asynchronous calls of the product entry
    point `entry`, issued from C, call i with params_list[i % len(params_list)]."""
    product = _cabi.load_library()
    fn = ctypes.cast(getattr(product, entry), ctypes.c_void_p)
    arr = (_cabi.PaParams * len(params_list))()
    for i, p in enumerate(params_list):
        ctypes.memmove(ctypes.byref(arr[i]), ctypes.byref(p), ctypes.sizeof(_cabi.PaParams))
    us = ctypes.c_float(0.0)
    _check(load_library().pa_aid_time_launches(fn, arr, len(params_list), calls, ctypes.c_void_p(stream),
                                               ctypes.byref(us)))
    return float(us.value)
