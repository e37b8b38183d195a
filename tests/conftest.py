import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


def pytest_sessionfinish(session, exitstatus):
    """Under the debug build of the library (``CKV_B200_LIB`` naming the ``-DCKV_BOUNDS`` build) every kernel
    records the first out-of-range slot index or counter it met instead of using it.  A whole test session run
    that way must end with nothing recorded:
    ``CKV_B200_LIB=.../libckv_b200_bounds.so python -m pytest tests -m gpu --deselect tests/test_debug_paths_gpu.py``
    (the deselected file corrupts a counter on purpose, in a child process of its own)."""
    if not os.environ.get("CKV_B200_LIB"):
        return
    import ctypes
    try:
        import torch
        if not torch.cuda.is_available():
            return
        from cascading_kv_cache_b200 import _lib
        lib = _lib.load()
    except Exception:
        return
    status = ctypes.c_int32(0)
    if lib.ckv_bounds_status(ctypes.byref(status)) != 0:
        return                                            # not the debug build
    line = f"[bounds build] recorded status at session end: {status.value} (0 = every index stayed in range)"
    print("\n" + line)
    if status.value != 0:
        session.exitstatus = 1
