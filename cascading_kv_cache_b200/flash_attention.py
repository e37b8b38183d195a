"""Functional attention with per-column scores over dense, already rotated tensors.

Mirrors ``attention = _attention.apply`` of the reference
(cascade/models/flash_attention.py:540-652, :713): same positional arguments, same returned pair.
The work is done by ``ckv_dense_attention`` of libckv_b200.so; there is no backward pass (the
reference's Triton backward kernels are outside the serving hot path).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib


def _rows(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: Optional[torch.Tensor],
                    sm_scale: float, beta: float, score_mode: int = _lib.CKV_DENSE_SCORES_FLASH,
                    ema_w_cache: Optional[torch.Tensor] = None, ema_w_new: Optional[torch.Tensor] = None,
                    want_scores: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """One ``ckv_dense_attention`` call.  ``q [B,H,N_CTX,D]``, ``k, v [B,h,N_KV,D]`` with ``h`` dividing
    ``H``; ``mask [>= N_KV-N_CTX]`` bool, True = masked.  Returns ``(o [B,H,N_CTX,D], scores [B,H,N_KV])``."""
    if q.device.type != "cuda":
        raise RuntimeError("attention runs on a CUDA device only (there is no CPU path)")
    if q.dtype not in _lib.DTYPE_CODE or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError(f"unsupported dtypes {q.dtype}, {k.dtype}, {v.dtype}")
    B, H, N_CTX, D = q.shape
    h, N_KV = k.size(1), k.size(2)
    if k.shape != v.shape or k.size(0) != B or k.size(3) != D or H % h != 0 or N_KV < N_CTX:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)} k {tuple(k.shape)} v {tuple(v.shape)}")
    n_cached = N_KV - N_CTX
    q, k, v = _rows(q), _rows(k), _rows(v)
    mask_ptr = None
    if n_cached > 0:
        if mask is None or mask.numel() < n_cached:
            raise ValueError(f"mask must cover the {n_cached} cached columns")
        m8 = mask.reshape(-1)[:n_cached].to(device=q.device, dtype=torch.bool).contiguous().view(torch.uint8)
        mask_ptr = m8.data_ptr()
    lib = _lib.load()
    out = torch.empty(B, H, N_CTX, D, device=q.device, dtype=q.dtype)
    scores = torch.empty(B, H, N_KV, device=q.device, dtype=q.dtype) if want_scores else None
    nbytes = lib.ckv_dense_attention_workspace_bytes(B, H, N_CTX)
    ws = torch.empty(nbytes, device=q.device, dtype=torch.uint8)
    with torch.cuda.device(q.device):
        rc = lib.ckv_dense_attention(
            q.data_ptr(), q.stride(0), q.stride(1), q.stride(2),
            k.data_ptr(), k.stride(0), k.stride(1), k.stride(2),
            v.data_ptr(), v.stride(0), v.stride(1), v.stride(2),
            mask_ptr, B, H, h, N_CTX, N_KV, D, _lib.DTYPE_CODE[q.dtype], float(sm_scale), float(beta), score_mode,
            None if ema_w_cache is None else ema_w_cache.data_ptr(),
            None if ema_w_new is None else ema_w_new.data_ptr(),
            out.data_ptr(), out.stride(0), out.stride(1), out.stride(2),
            None if scores is None else scores.data_ptr(), ws.data_ptr(), nbytes,
            _lib.current_stream_ptr(q.device))
    _lib.check(rc, "ckv_dense_attention")
    return out, scores


def attention(q, k, v, causal, sm_scale, mask, beta):
    """``attention(q, k, v, causal, sm_scale, mask, beta) -> (o, scores)`` as in the reference.

    The key axis is ``[cached columns | N_CTX new columns]``: the first ``N_KV - N_CTX`` columns are
    visible where ``mask`` is False, the last ``N_CTX`` are causal.  As in the reference kernel the
    ``causal`` argument does not change that layout (flash_attention.py:54-61 applies it
    unconditionally).  ``scores[b, h, col] = sum_q p[q, col] * (1 - beta) * beta**(N_CTX - 1 - q)``
    with exactly normalised probabilities (the reference approximates the normaliser while it
    streams, :92-100, and accepts a rank correlation of 0.95 against this definition in its tests).
    """
    del causal
    return dense_attention(q, k, v, mask, sm_scale, beta, _lib.CKV_DENSE_SCORES_FLASH)
