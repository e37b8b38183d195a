"""Error-reporting paths that a healthy run never takes, exercised without faulting or stalling anything:

* the bounded waits of the decode and prefill kernels give up on a barrier phase that nothing completes
  (a self-test launch of one thread with a short limit) and raise the status word;
* the debug build of the library (``-DCKV_BOUNDS``) runs a normal stream clean, and reports -- instead of
  using -- a ring start index that was corrupted from the host.  The corrupted value is chosen so that even
  an unchecked kernel would stay inside the cache tensors (a slot of the next cascade).
"""
import ctypes
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bounded_waits_give_up_and_report():
    from cascading_kv_cache_b200 import _lib
    lib = _lib.load()
    ws = torch.zeros(64, dtype=torch.int32, device="cuda:0")
    stream = _lib.current_stream_ptr(ws.device)
    status = ctypes.c_int32(0)
    _lib.check(lib.ckv_selftest_bounded_wait(1, ws.data_ptr(), stream), "selftest")
    _lib.check(lib.ckv_read_status(ws.data_ptr(), ctypes.byref(status)), "read_status")
    assert status.value == 1                              # decode kernels: code 1
    _lib.check(lib.ckv_selftest_bounded_wait(2, ws.data_ptr(), stream), "selftest")
    _lib.check(lib.ckv_read_status(ws.data_ptr(), ctypes.byref(status)), "read_status")
    assert status.value & 0xff == 2 and status.value >> 8 > 0   # prefill kernels: 2 | source line << 8
    assert lib.ckv_selftest_bounded_wait(3, ws.data_ptr(), stream) == -1
    # the context is as usable as before
    torch.cuda.synchronize()
    assert int((ws[1:] == 0).all())
    rc = lib.ckv_bounds_status(ctypes.byref(status))
    assert rc == -2 and b"CKV_BOUNDS" in lib.ckv_last_error()      # the ordinary build has no bounds checks


BOUNDS_SCRIPT = textwrap.dedent('''
    import ctypes, sys, torch
    sys.path.insert(0, %r)
    from cascading_kv_cache_b200 import CascadingKVCache, cascade_attention
    W, C, NS, B, KVH, H, D = 64, 4, 4, 2, 2, 8, 128
    cache = CascadingKVCache(W, NS, B, KVH, D, W * C, device="cuda:0", dtype=torch.bfloat16, layers=1, verbose=False)
    lib = cache._lib
    status = ctypes.c_int32(-1)
    g = torch.Generator().manual_seed(0)
    mk = lambda h, n: torch.randn(B, h, n, D, generator=g).bfloat16().cuda()
    for n in (200, 150, 1, 1, 1):                      # chunk update, decode update: past the cache size
        cascade_attention(mk(H, n), mk(KVH, n), mk(KVH, n), cache, 0)
    cache.update(mk(KVH, 300), mk(KVH, 300), 0)         # parallel chunk update alone
    cache.force_serial_update = True
    cache.update(mk(KVH, 7), mk(KVH, 7), 0)             # one-warp-per-lane walk
    assert lib.ckv_bounds_status(ctypes.byref(status)) == 0 and status.value == 0, status.value
    assert cache.kernel_status() == 0
    # a ring start index outside its window, written from the host behind the library's back
    cache._start_indices[0][0] = W + 3
    cascade_attention(mk(H, 1), mk(KVH, 1), mk(KVH, 1), cache, 0)
    assert lib.ckv_bounds_status(ctypes.byref(status)) == 0
    assert status.value & 0xff == 4 and status.value >> 8 > 0, status.value
    for serial in (True, False):                          # the walk, then the parallel chunk update
        cache._start_indices[0][0] = W + 3                  # (advancing the counters had wrapped it back in range)
        cache.force_serial_update = serial
        cache.update(mk(KVH, 5), mk(KVH, 5), 0)
        assert lib.ckv_bounds_status(ctypes.byref(status)) == 0 and status.value & 0xff == 4, (serial, status.value)
    assert lib.ckv_bounds_status(ctypes.byref(status)) == 0 and status.value == 0      # reading clears it
    torch.cuda.synchronize()
    print("BOUNDS-OK")
''')


def test_bounds_build_runs_clean_and_reports_a_corrupted_counter():
    from cascading_kv_cache_b200.build import BOUNDS_LIB_PATH
    if not os.path.exists(BOUNDS_LIB_PATH):
        pytest.fail(f"{BOUNDS_LIB_PATH} is missing: build it with `python -m cascading_kv_cache_b200.build --bounds`")
    env = dict(os.environ, CKV_B200_LIB=BOUNDS_LIB_PATH)
    r = subprocess.run([sys.executable, "-c", BOUNDS_SCRIPT % ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "BOUNDS-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
