"""CUDA-event timing of the dominant kernel through the library's own profiling hook
(``ckv_profile_enable`` / ``ckv_profile_read``), the counterpart of the reference's
``sink_cache(..., BENCHMARK=True)`` event timing (cascading_cache.py:986-1026)."""
from __future__ import annotations

import ctypes

from . import _lib


def time_dominant_kernel(run_step, n_steps: int = 20):
    """Run ``run_step(i)`` ``n_steps`` times with the hook on; return (ms per launch, launches, kernel name)."""
    lib = _lib.load()
    lib.ckv_profile_enable(1)
    try:
        for i in range(n_steps):
            run_step(i)
        total, n, name = ctypes.c_double(0), ctypes.c_int32(0), ctypes.c_char_p()
        _lib.check(lib.ckv_profile_read(ctypes.byref(total), ctypes.byref(n), ctypes.byref(name)),
                   "ckv_profile_read")
    finally:
        lib.ckv_profile_enable(0)
    launches = max(n.value, 1)
    return total.value / launches, n.value, (name.value or b"").decode()


def kernel_breakdown():
    """Per-kernel totals of the collection the last ``time_dominant_kernel`` read: a list of
    ``(kernel name, ms per launch, launches)``, largest total first."""
    lib = _lib.load()
    out, i = [], 0
    while True:
        name, ms, n = ctypes.c_char_p(), ctypes.c_double(0), ctypes.c_int32(0)
        if lib.ckv_profile_kernel(i, ctypes.byref(name), ctypes.byref(ms), ctypes.byref(n)) != 0:
            return out
        out.append(((name.value or b"").decode(), ms.value / max(n.value, 1), n.value))
        i += 1


def last_launch_count() -> int:
    return int(_lib.load().ckv_last_launch_count())
