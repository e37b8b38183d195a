"""ctypes binding of libckv_b200.so (the C ABI declared in include/cascade_kv_b200.h).

There is no CPU or PyTorch fallback: if the shared library is missing or a call
fails, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
import os

import torch

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# CKV_B200_LIB points at another build of the library (A/B timing of kernel variants)
LIB_PATH = os.environ.get("CKV_B200_LIB") or os.path.join(PKG_DIR, "libckv_b200.so")

CKV_F32, CKV_F16, CKV_BF16 = 0, 1, 2
CKV_REDUCE = {"mean": 0, "max": 1, "median": 2}
CKV_ADMIT = {"stride": 0, "ema": 1}
CKV_ATTN_UPDATE = 1
CKV_ATTN_FORCE_GENERIC = 2
CKV_DENSE_SCORES_FLASH, CKV_DENSE_SCORES_EAGER = 0, 1
DTYPE_CODE = {torch.float32: CKV_F32, torch.float16: CKV_F16, torch.bfloat16: CKV_BF16}

EXPORTS = ("ckv_abi_version", "ckv_last_error", "ckv_cascade_update", "ckv_update_workspace_bytes",
           "ckv_attention_workspace_bytes", "ckv_attention_workspace_bytes_for",
           "ckv_attention", "ckv_last_launch_count", "ckv_profile_enable", "ckv_profile_read", "ckv_profile_kernel", "ckv_read_status",
           "ckv_static_scratch_bytes", "ckv_attention_static", "ckv_static_status", "ckv_advance_counters_host",
           "ckv_dense_attention_workspace_bytes", "ckv_dense_attention", "ckv_bounds_status", "ckv_selftest_bounded_wait",
           "ckv_add_rmsnorm", "ckv_silu_mul")


class CkvConfig(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int32), ("kv_heads", ctypes.c_int32), ("q_heads", ctypes.c_int32),
                ("head_dim", ctypes.c_int32), ("num_sinks", ctypes.c_int32), ("window", ctypes.c_int32),
                ("cascades", ctypes.c_int32), ("dtype", ctypes.c_int32), ("eager_fill", ctypes.c_int32),
                ("head_reduction", ctypes.c_int32), ("homogeneous_heads", ctypes.c_int32),
                ("admission", ctypes.c_int32), ("beta", ctypes.c_double)]


class CkvLayerState(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "key_cache", "value_cache", "score_cache", "sink_keys", "sink_values", "mask", "sink_mask", "pos", "og_pos",
        "sink_pos", "stored_tokens", "start_indices", "stored_sinks", "seen_tokens", "every_n")]


_lib = None


def load():
    """Load libckv_b200.so; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m cascading_kv_cache_b200.build` "
            "(needs nvcc); there is no fallback path")
    lib = ctypes.CDLL(LIB_PATH)
    i32, i64, vp, sz = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t
    cfgp, stp = ctypes.POINTER(CkvConfig), ctypes.POINTER(CkvLayerState)
    lib.ckv_abi_version.restype = ctypes.c_int
    lib.ckv_last_error.restype = ctypes.c_char_p
    lib.ckv_cascade_update.restype = ctypes.c_int
    lib.ckv_cascade_update.argtypes = [cfgp, stp, vp, vp, i64, i64, i64, vp, i64, i64, i64, i32, vp, sz, vp]
    lib.ckv_advance_counters_host.restype = ctypes.c_int
    lib.ckv_advance_counters_host.argtypes = [cfgp, ctypes.POINTER(i64), i64, i64, ctypes.POINTER(i64),
                                              ctypes.POINTER(i64), ctypes.POINTER(i64)]
    lib.ckv_update_workspace_bytes.restype = sz
    lib.ckv_update_workspace_bytes.argtypes = [cfgp, i32]
    lib.ckv_attention_workspace_bytes.restype = sz
    lib.ckv_attention_workspace_bytes.argtypes = [cfgp, i32]
    lib.ckv_attention_workspace_bytes_for.restype = sz
    lib.ckv_attention_workspace_bytes_for.argtypes = [cfgp, i32, i32]
    lib.ckv_attention.restype = ctypes.c_int
    lib.ckv_attention.argtypes = [cfgp, stp, vp, i64, i64, i64, vp, vp, i64, i64, i64, i32, vp, i64, vp, vp,
                                  vp, i64, i64, i64, vp, sz, i32, vp]
    lib.ckv_static_scratch_bytes.restype = sz
    lib.ckv_attention_static.restype = ctypes.c_int
    lib.ckv_attention_static.argtypes = [cfgp, stp, vp, i64, i64, i64, vp, vp, i64, i64, i64, i32, vp, i64, vp, vp,
                                         vp, i64, i64, i64, i32, vp]
    lib.ckv_dense_attention_workspace_bytes.restype = sz
    lib.ckv_dense_attention_workspace_bytes.argtypes = [i32, i32, i32]
    lib.ckv_add_rmsnorm.restype = ctypes.c_int
    lib.ckv_add_rmsnorm.argtypes = [vp, vp, vp, vp, vp, i64, i32, ctypes.c_double, i32, vp]
    lib.ckv_silu_mul.restype = ctypes.c_int
    lib.ckv_silu_mul.argtypes = [vp, vp, vp, i64, i32, i64, i64, i32, vp]
    lib.ckv_dense_attention.restype = ctypes.c_int
    lib.ckv_dense_attention.argtypes = [vp, i64, i64, i64, vp, i64, i64, i64, vp, i64, i64, i64, vp,
                                        i32, i32, i32, i32, i32, i32, i32, ctypes.c_double, ctypes.c_double, i32,
                                        vp, vp, vp, i64, i64, i64, vp, vp, sz, vp]
    lib.ckv_selftest_bounded_wait.restype = ctypes.c_int
    lib.ckv_selftest_bounded_wait.argtypes = [i32, vp, vp]
    lib.ckv_bounds_status.restype = ctypes.c_int
    lib.ckv_bounds_status.argtypes = [ctypes.POINTER(i32)]
    lib.ckv_static_status.restype = ctypes.c_int
    lib.ckv_static_status.argtypes = [ctypes.POINTER(i32)]
    lib.ckv_last_launch_count.restype = ctypes.c_int
    lib.ckv_profile_enable.restype = ctypes.c_int
    lib.ckv_profile_enable.argtypes = [ctypes.c_int]
    lib.ckv_profile_read.restype = ctypes.c_int
    lib.ckv_profile_read.argtypes = [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(i32),
                                     ctypes.POINTER(ctypes.c_char_p)]
    lib.ckv_profile_kernel.restype = ctypes.c_int
    lib.ckv_profile_kernel.argtypes = [i32, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_double),
                                       ctypes.POINTER(i32)]
    lib.ckv_read_status.restype = ctypes.c_int
    lib.ckv_read_status.argtypes = [vp, ctypes.POINTER(i32)]
    if lib.ckv_abi_version() != 1:
        raise RuntimeError("libckv_b200.so has an unexpected ABI version")
    _lib = lib
    return lib


def check(rc: int, what: str):
    if rc != 0:
        msg = load().ckv_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def current_stream_ptr(device) -> int:
    """The current CUDA stream of ``device`` as an integer handle (no Stream object is built when torch
    exposes the raw accessor)."""
    if _raw_stream is not None:
        index = getattr(device, "index", device)
        if isinstance(index, int):
            return _raw_stream(index)
    return torch.cuda.current_stream(device).cuda_stream
