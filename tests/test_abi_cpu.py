"""CPU-side checks of the shipped package: the C-ABI library loads and exports every declared
symbol, and the host mirror validates its arguments.  No compute calls."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from cascading_kv_cache_b200 import _lib
    from cascading_kv_cache_b200.build import build
    build()
    header = open(os.path.join(ROOT, "include", "cascade_kv_b200.h")).read()
    declared = set(re.findall(r"\b(ckv_[a-z_0-9]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS)
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert _lib.load().ckv_abi_version() == 1


def test_struct_layout_matches_header():
    from cascading_kv_cache_b200 import _lib
    assert ctypes.sizeof(_lib.CkvConfig) == 12 * 4 + 8
    assert ctypes.sizeof(_lib.CkvLayerState) == 15 * 8


def test_argument_errors_do_not_need_a_gpu():
    from cascading_kv_cache_b200 import _lib
    lib = _lib.load()
    cfg = _lib.CkvConfig(batch=1, kv_heads=3, q_heads=4, head_dim=8, num_sinks=1, window=4, cascades=2, dtype=0)
    assert lib.ckv_attention_workspace_bytes(ctypes.byref(cfg), 4) == 0  # q_heads not a multiple of kv_heads
    st = _lib.CkvLayerState()
    rc = lib.ckv_cascade_update(ctypes.byref(cfg), ctypes.byref(st), None, None, 0, 0, 0, None, 0, 0, 0, 1, None, 0, None)
    assert rc == -1 and b"multiple" in lib.ckv_last_error()
    cfg.q_heads = 6
    assert lib.ckv_attention_workspace_bytes(ctypes.byref(cfg), 4) > 0
    rc = lib.ckv_cascade_update(ctypes.byref(cfg), ctypes.byref(st), None, None, 0, 0, 0, None, 0, 0, 0, 1, None, 0, None)
    assert rc == -1 and b"null" in lib.ckv_last_error()


def test_workspace_is_sized_for_the_path_the_flags_select():
    """Decode at Llama-3.1-8B heads, 16 sequences, 8 x 8192 slots: the tuned path needs its split-K
    partials and one 16-bit logit row per query head, the generic path fp32 logit rows and rotated keys."""
    from cascading_kv_cache_b200 import _lib
    lib = _lib.load()
    cfg = _lib.CkvConfig(batch=16, kv_heads=8, q_heads=32, head_dim=128, num_sinks=64, window=8192, cascades=8,
                         dtype=_lib.CKV_BF16, eager_fill=1, head_reduction=1, homogeneous_heads=0, admission=1,
                         beta=0.9999)
    ref = ctypes.byref(cfg)
    tuned = lib.ckv_attention_workspace_bytes_for(ref, 1, _lib.CKV_ATTN_UPDATE)
    generic = lib.ckv_attention_workspace_bytes_for(ref, 1, _lib.CKV_ATTN_UPDATE | _lib.CKV_ATTN_FORCE_GENERIC)
    assert 0 < tuned < 128 << 20 < generic
    assert lib.ckv_attention_workspace_bytes_for(ref, 1, 0) == tuned          # only the generic flag matters
    assert lib.ckv_attention_workspace_bytes(ref, 1) == max(tuned, generic)
    # fp32 has no tuned path: both answers are the generic one
    cfg.dtype = _lib.CKV_F32
    assert lib.ckv_attention_workspace_bytes_for(ref, 1, 0) == \
        lib.ckv_attention_workspace_bytes_for(ref, 1, _lib.CKV_ATTN_FORCE_GENERIC) > 0
    cfg.q_heads = 33
    assert lib.ckv_attention_workspace_bytes_for(ref, 1, 0) == 0


def test_cache_refuses_cpu_device_and_bad_configs():
    from cascading_kv_cache_b200 import CascadingKVCache, cascade_every_n
    with pytest.raises(RuntimeError):
        CascadingKVCache(8, 4, 1, 2, 16, 32, device="cpu", dtype=torch.float32, layers=1)
    with pytest.raises(ValueError):
        CascadingKVCache(7, 4, 1, 2, 16, 32, device="cuda", dtype=torch.float32, layers=1)
    with pytest.raises(ValueError):
        CascadingKVCache(8, 4, 1, 2, 16, [32], device="cuda", dtype=torch.float32, layers=1)
    with pytest.raises(ValueError):
        CascadingKVCache(8, 4, 1, 2, 16, 32, device="cuda", dtype=torch.float32, layers=1, cascade_func="nope")
    assert cascade_every_n("pow2", 4) == [1, 2, 4, 8]


def test_host_counters_follow_the_update_state_machine():
    """ckv_advance_counters_host (what get_seq_length reads instead of the device) against the oracle's
    counters on streams fed in ragged calls, with and without eager fill, several admission schedules."""
    import numpy as np
    from cascading_kv_cache_b200 import _lib
    from oracle.cascade_oracle import OracleCascadingKVCache, cascade_every_n
    lib = _lib.load()
    rng = np.random.default_rng(3)
    for (W, C, NS, func, eager) in [(4, 4, 2, "pow2", False), (8, 3, 3, "pow2", True), (4, 4, 0, "pow3", False),
                                    (8, 4, 1, "iplus1", True), (16, 2, 5, "1-then-2", False)]:
        ref = OracleCascadingKVCache(W, NS, 1, 1, 4, W * C, dtype=torch.float32, cascade_func=func, layers=1,
                                     eager_fill=eager)
        cfg = _lib.CkvConfig(batch=1, kv_heads=1, q_heads=1, head_dim=4, num_sinks=NS, window=W, cascades=C, dtype=0,
                             eager_fill=int(eager))
        arr = ctypes.c_int64 * C
        stored, start, sinks = arr(), arr(), ctypes.c_int64(0)
        every = arr(*cascade_every_n(func, C))
        seen = 0
        for _ in range(12):
            n = int(rng.integers(1, 40))
            x = torch.randn(1, 1, n, 4)
            ref.update(x, x, 0)
            assert lib.ckv_advance_counters_host(ctypes.byref(cfg), every, seen, n, stored, start,
                                                 ctypes.byref(sinks)) == 0
            seen += n
            assert list(stored) == ref.stored_tokens[0][0, 0].tolist()
            assert list(start) == ref.start_indices[0][0, 0].tolist()
            assert sinks.value == int(ref.stored_sinks[0][0, 0])


def test_attention_refuses_null_sink_buffers():
    from cascading_kv_cache_b200 import _lib
    lib = _lib.load()
    cfg = _lib.CkvConfig(batch=1, kv_heads=1, q_heads=1, head_dim=8, num_sinks=2, window=4, cascades=2, dtype=0)
    one = ctypes.c_void_p(16)       # any non-null value: the call must stop at the argument checks
    st = _lib.CkvLayerState(**{n: one for n, _ in _lib.CkvLayerState._fields_})
    st.sink_keys = None
    rc = lib.ckv_attention(ctypes.byref(cfg), ctypes.byref(st), one, 0, 0, 0, one, one, 0, 0, 0, 1, one, 100, None, None,
                           one, 0, 0, 0, None, 0, 0, None)
    assert rc == -1 and b"sink" in lib.ckv_last_error()
    cfg.num_sinks = 0
    rc = lib.ckv_attention(ctypes.byref(cfg), ctypes.byref(st), one, 0, 0, 0, one, one, 0, 0, 0, 1, one, 100, None, None,
                           one, 0, 0, 0, None, 0, 0, None)
    assert rc == -2 and b"sink" in lib.ckv_last_error()
    assert lib.ckv_dense_attention_workspace_bytes(1, 2, 16) > 0
    status = ctypes.c_int32(0)
    assert lib.ckv_static_status(None) == -1


def test_layer_operator_argument_errors_do_not_need_a_gpu():
    """``ckv_add_rmsnorm`` / ``ckv_silu_mul`` refuse what they cannot serve before any CUDA call."""
    from cascading_kv_cache_b200 import _lib
    lib = _lib.load()
    p = ctypes.c_void_p(4096)          # an aligned, never dereferenced address: every case below is refused first
    assert lib.ckv_add_rmsnorm(None, None, p, p, None, 4, 64, 1e-5, _lib.CKV_BF16, None) == -1
    assert b"required" in lib.ckv_last_error()
    assert lib.ckv_add_rmsnorm(p, None, p, p, None, 4, 60, 1e-5, _lib.CKV_BF16, None) == -1
    assert b"multiple of 8" in lib.ckv_last_error()
    assert lib.ckv_add_rmsnorm(p, None, p, p, None, 4, 64, 1e-5, _lib.CKV_F32, None) != 0
    assert b"16-bit" in lib.ckv_last_error()
    assert lib.ckv_add_rmsnorm(ctypes.c_void_p(4100), None, p, p, None, 4, 64, 1e-5, _lib.CKV_BF16, None) == -1
    assert b"aligned" in lib.ckv_last_error()
    assert lib.ckv_add_rmsnorm(p, None, p, p, None, 0, 64, 1e-5, _lib.CKV_BF16, None) == 0      # no rows: nothing to do
    assert lib.ckv_silu_mul(p, None, p, 4, 64, 64, 64, _lib.CKV_BF16, None) == -1
    assert lib.ckv_silu_mul(p, p, p, 4, 64, 32, 64, _lib.CKV_BF16, None) == -1                 # row stride shorter than a row
    assert lib.ckv_silu_mul(p, p, p, 4, 64, 64, 64, _lib.CKV_F32, None) != 0
    assert lib.ckv_silu_mul(p, p, p, 0, 64, 64, 64, _lib.CKV_BF16, None) == 0
