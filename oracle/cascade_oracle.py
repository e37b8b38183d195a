"""TEST INFRASTRUCTURE ONLY -- CPU oracle for the cascading KV cache hot path.

This module restates, on the CPU, the reference path that the CUDA kernels
replace.  Only tests/, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import it; the shipped package never does.

* ``OracleCascadingKVCache`` mirrors the tensor layout of the reference cache
  object (cascade/models/cascading_cache.py:1031-1348: ``init_cache`` :1187-1276,
  ``get_vals`` :1278-1295, ``update`` :1297-1348) and drives the C state machine
  in ``cascade_update_oracle.c`` (a restatement of the Triton kernel
  :145-774).
* ``rope_tables`` / ``apply_rope`` follow ``LlamaRotaryEmbedding.forward``
  (cascade/models/llama/modeling_llama.py:199-220), ``Qwen2RotaryEmbedding``
  (cascade/models/qwen2/modeling_qwen2.py:140-173) and
  ``apply_rotary_pos_emb_one`` (cascade/models/cascade_attention.py:31-35).
* ``cascade_attention_step`` follows ``CascadeAttention.forward_cascade``
  (cascade_attention.py:82-200, positions and RoPE), ``cascade_attn_eager``
  (:250-340, the three-segment softmax, EMA scores and score-cache decay) and
  ``calc_scores`` (:231-248, head reduction).

Parity status: pinned.  The update is checked against ``CascadingKVCacheSlow``
(stride rule) and against state dumps of the reference's own ``CascadingKVCache``
whose Triton kernel's source was executed on the CPU (score-driven rule, every
dtype); attention against the reference's own ``forward_cascade`` /
``cascade_attn_eager`` run on CPU over that cache (default positions and
``do_og_pos``).  The vectors and the scripts that produced them are under
tests/golden/.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from typing import List, Optional, Sequence, Union

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcascade_oracle.so")
_SRC_PATH = os.path.join(_HERE, "cascade_update_oracle.c")
_lib = None

_DT_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def build_oracle_lib(force: bool = False) -> str:
    """Compile the C restatement with gcc into oracle/libcascade_oracle.so."""
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(_SRC_PATH)):
        return _LIB_PATH
    subprocess.check_call(
        ["gcc", "-O2", "-fPIC", "-shared", "-o", _LIB_PATH, _SRC_PATH])
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build_oracle_lib()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.cascade_update_oracle.restype = ctypes.c_int
    return _lib


def cascade_every_n(cascade_func: str, cascades: int) -> List[int]:
    """Admission strides per cascade (cascading_cache.py:1201-1244)."""
    c = cascades
    n = c // 4
    if cascade_func == "pow2":
        return [2 ** i for i in range(c)]
    if cascade_func == "pow2-1":
        return [1] * (c - 1) + [2 ** i for i in range(c - 1, c)]
    if cascade_func == "pow2-1-4":
        return [1] * (3 * n) + [2 ** i for i in range(3 * n, c)]
    if cascade_func == "pow2-2-4":
        return [1] * (2 * n) + [2 ** i for i in range(2 * n, c)]
    if cascade_func == "pow2-3-4":
        return [1] * n + [2 ** i for i in range(n, c)]
    if cascade_func == "1-then-2":
        return [1] + [2] * (c - 1)
    if cascade_func == "pow3":
        return [3 ** i for i in range(c)]
    if cascade_func == "pow4":
        return [4 ** i for i in range(c)]
    if cascade_func == "iplus1":
        return [i + 1 for i in range(c)]
    raise ValueError(f"unknown cascade func: {cascade_func}")


class OracleCascadingKVCache:
    """CPU cache with the reference's state tensors (one layer list each)."""

    def __init__(self, window_length=8, num_sink_tokens=4, max_batch_size=1, heads=16, dim=128,
                 max_seq_len=32, dtype=torch.float16, cascade_func="pow2", head_reduction="mean",
                 layers=1, eager_fill=True, beta=0.9999999):
        if max_seq_len % window_length != 0:
            raise ValueError("window length must evenly divide max seq len")
        self.window_length = window_length
        self.num_sink_tokens = num_sink_tokens
        self.max_batch_size = max_batch_size
        self.heads = heads
        self.dim = dim
        self.max_seq_len = max_seq_len
        self.dtype = dtype
        self.cascade_func = cascade_func
        self.head_reduction = head_reduction
        self.layers = layers
        self.eager_fill = eager_fill
        self.cascades = max_seq_len // window_length
        self.beta = beta
        self.every_n = torch.tensor(cascade_every_n(cascade_func, self.cascades), dtype=torch.long)
        self.reset()

    def reset(self):
        L, B, H, D = self.layers, self.max_batch_size, self.heads, self.dim
        S, NS, C, dt = self.max_seq_len, self.num_sink_tokens, self.cascades, self.dtype
        z = torch.zeros
        self.seen_tokens_by_layer = [0 for _ in range(L)]
        self.key_cache = [z(B, H, S, D, dtype=dt) for _ in range(L)]
        self.value_cache = [z(B, H, S, D, dtype=dt) for _ in range(L)]
        self.score_cache = [z(B, H, S, dtype=dt) for _ in range(L)]
        self.sink_keys = [z(B, H, NS, D, dtype=dt) for _ in range(L)]
        self.sink_values = [z(B, H, NS, D, dtype=dt) for _ in range(L)]
        self.mask = [torch.ones(B, H, S, dtype=torch.bool) for _ in range(L)]
        self.sink_mask = [torch.ones(B, H, NS, dtype=torch.bool) for _ in range(L)]
        self.pos = [z(B, H, S, dtype=torch.long) for _ in range(L)]
        self.og_pos = [z(B, H, S, dtype=torch.long) for _ in range(L)]
        self.sink_pos = [z(B, H, NS, dtype=torch.long) for _ in range(L)]
        self.stored_tokens = [z(B, H, C, dtype=torch.long) for _ in range(L)]
        self.start_indices = [z(B, H, C, dtype=torch.long) for _ in range(L)]
        self.stored_sinks = [z(B, H, dtype=torch.long) for _ in range(L)]

    def get_vals(self, layer_idx: int):
        """cascading_cache.py:1278-1295"""
        shift = self.num_sink_tokens if self.seen_tokens_by_layer[layer_idx] > self.num_sink_tokens else 0
        l = layer_idx
        return (self.sink_keys[l], self.sink_values[l], self.sink_pos[l][:1, 0], self.sink_mask[l],
                self.key_cache[l], self.value_cache[l], self.pos[l][:1, 0] + shift, self.mask[l],
                self.og_pos[l])

    def update(self, key_states, value_states, layer_idx, score_states=None):
        """cascading_cache.py:1297-1348 with the kernel replaced by the C restatement."""
        l = layer_idx
        B, H, K, D = key_states.shape
        assert (B, H, D) == (self.max_batch_size, self.heads, self.dim)
        dt = self.dtype
        k = key_states.to(dt).contiguous()
        v = value_states.to(dt).contiguous()
        if score_states is None:
            score_states = torch.zeros(B, H, K, dtype=dt)
        s = score_states.to(dt)
        assert s.size(0) == B and s.size(1) >= H and s.size(2) == K
        mask_u8 = self.mask[l].view(torch.uint8)
        smask_u8 = self.sink_mask[l].view(torch.uint8)
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        i64 = ctypes.c_int64
        rc = _load().cascade_update_oracle(
            p(k), p(v), p(s), i64(s.stride(0)), i64(s.stride(1)), i64(s.stride(2)),
            p(self.sink_keys[l]), p(self.sink_values[l]),
            p(self.key_cache[l]), p(self.value_cache[l]), p(self.score_cache[l]),
            p(smask_u8), p(mask_u8),
            p(self.sink_pos[l]), p(self.pos[l]), p(self.og_pos[l]),
            p(self.stored_sinks[l]), p(self.stored_tokens[l]), p(self.start_indices[l]),
            p(self.every_n),
            i64(B), i64(H), i64(K), i64(D), i64(self.num_sink_tokens), i64(self.window_length),
            i64(self.cascades), i64(self.seen_tokens_by_layer[l]), i64(self.max_seq_len),
            ctypes.c_int(1 if self.eager_fill else 0), ctypes.c_int(_DT_CODE[dt]))
        if rc != 0:
            raise RuntimeError(f"cascade_update_oracle failed with code {rc}")
        self.seen_tokens_by_layer[l] += K
        return self.get_vals(l)


# --------------------------------------------------------------------------- RoPE

def rope_inv_freq(dim: int, theta: float) -> torch.Tensor:
    """inv_freq of the default rope type: 1 / theta^(2i/dim), fp32."""
    return 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))


def rope_cos_sin(pos: torch.Tensor, dim: int, theta: float, dtype: torch.dtype):
    """cos/sin rows for integer positions: fp32 angle, fp32 cos/sin, cast to ``dtype``.

    modeling_llama.py:199-220 computes ``inv_freq @ pos`` in fp32 (a one-term
    product), concatenates ``(freqs, freqs)`` and casts cos/sin to the activation
    dtype; the Qwen2 table (modeling_qwen2.py:155-173) is ``outer(t, inv_freq)``
    with the same arithmetic, looked up by position.
    """
    freqs = pos.reshape(-1).float()[:, None] * rope_inv_freq(dim, theta)[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x):
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """x [B,h,len,D] rotated at ``pos`` [len] in x's dtype (cascade_attention.py:31-35)."""
    cos, sin = rope_cos_sin(pos, x.size(-1), theta, x.dtype)
    return (x * cos[None, None]) + (rotate_half(x) * sin[None, None])


def apply_rope_per_lane(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """x [B,h,len,D] rotated at ``pos`` [B,h,len]: every lane at its own positions (the
    ``do_og_pos`` branch, cascade_attention.py:161-164)."""
    B, h, n, D = x.shape
    cos, sin = rope_cos_sin(pos.reshape(-1), D, theta, x.dtype)
    cos, sin = cos.view(B, h, n, D), sin.view(B, h, n, D)
    return (x * cos) + (rotate_half(x) * sin)


# ---------------------------------------------------------------------- attention

def _reduce_heads(x: torch.Tensor, how: str, dim: int, keepdim: bool = False) -> torch.Tensor:
    if how == "mean":
        return torch.mean(x, dim=dim, keepdim=keepdim)
    if how == "max":
        return torch.amax(x, dim=dim, keepdim=keepdim)
    if how == "median":
        return torch.median(x, dim=dim, keepdim=keepdim).values
    raise ValueError(how)


def cascade_attention_step(q, k, v, cache: OracleCascadingKVCache, layer_idx: int = 0, theta: float = 500000.0,
                           head_reduction: Optional[str] = None, homogeneous_heads: bool = False,
                           do_update: bool = True, do_og_pos: bool = False):
    """One attention call over the cascading cache plus the cache update.

    q [B,H,K,D]; k,v [B,KVH,K,D] (un-rotated), all in the cache dtype.  Returns
    ``out`` [B,H,K,D].  Follows forward_cascade (cascade_attention.py:103-181) and
    cascade_attn_eager (:250-340) operation by operation, including the points
    where the reference rounds to the activation dtype.
    """
    B, H, K, D = q.shape
    KVH = k.size(1)
    G = H // KVH
    dt = q.dtype
    how = head_reduction or cache.head_reduction
    beta = cache.beta

    first_it = cache.seen_tokens_by_layer[layer_idx] == 0
    sink_k, sink_v, sink_pos, sink_mask, ck, cv, key_pos, key_mask, og_pos = cache.get_vals(layer_idx)
    max_pos = 0
    if not first_it:
        # :141-148: with do_og_pos the keys keep the stream index they arrived with
        top = og_pos.amax().item() if do_og_pos else key_pos.amax().item()
        max_pos = int(max(sink_pos.amax().item() if sink_pos.numel() else 0, top)) + 1
    query_pos = torch.arange(K, dtype=torch.long) + max_pos

    q_r = apply_rope(q, query_pos, theta)
    k_r = apply_rope(k, query_pos, theta)
    sk_r = apply_rope(sink_k, sink_pos.reshape(-1), theta)
    ck_r = apply_rope_per_lane(ck, og_pos, theta) if do_og_pos else apply_rope(ck, key_pos.reshape(-1), theta)

    rep = lambda t: t.repeat_interleave(G, dim=1) if G > 1 else t
    scale = 1.0 / math.sqrt(D)
    rs = np.sqrt(scale)
    val = torch.finfo(dt).min

    causal = torch.full((K, K), True, dtype=torch.bool).triu(1)
    qs = q_r * rs
    qattn = torch.einsum("bhqd,bhkd->bhqk", qs, rep(k_r) * rs)
    qattn = qattn + (causal * val).to(dt)
    sattn = torch.einsum("bhqd,bhkd->bhqk", qs, rep(sk_r) * rs)
    sattn = sattn + (val * sink_mask[:1, :1, None, :]).to(dt)
    cattn = torch.einsum("bhqd,bhkd->bhqk", qs, rep(ck_r) * rs)
    cattn = cattn + (val * key_mask[:1, :1, None, :]).to(dt)

    attn = torch.cat((sattn, cattn, qattn), dim=-1).softmax(dim=-1)
    NS, S = sink_k.size(2), ck.size(2)
    out = attn[..., :NS] @ rep(sink_v)
    out = out + attn[..., NS:NS + S] @ rep(cv)
    out = out + attn[..., NS + S:] @ rep(v)

    # EMA weights for cached slots: (1-beta) * beta^(K-1-q)   (:315-320)
    exps = (1 - beta) * beta ** torch.arange(K).flip(dims=(0,))
    ema = (attn[..., NS:NS + S] * exps[None, None, :, None]).sum(dim=2).to(dt)
    # new-token scores: sum_{q>=i} attn[q,i] * (1-beta) * beta^(q-i), all in the cache dtype (:269-282,:322-323)
    rows = []
    for i in range(K):
        e = (1 - beta) * beta ** torch.arange(K - i, dtype=dt)
        rows.append(torch.cat((torch.zeros(i, dtype=dt), e)))
    ema_mask = torch.stack(rows).T
    new_scores = (attn[..., NS + S:] * ema_mask[None, None].to(dt)).sum(dim=2)

    # head reduction (:231-248)
    if homogeneous_heads:
        ema_r = _reduce_heads(ema, how, dim=1, keepdim=True)
        new_r = _reduce_heads(new_scores, how, dim=1, keepdim=True).repeat(1, KVH, 1)
    else:
        ema_r = _reduce_heads(ema.view(B, KVH, G, S), how, dim=2)
        new_r = _reduce_heads(new_scores.view(B, KVH, G, K), how, dim=2)

    if do_update:
        # :329-330  two roundings to the cache dtype: beta^K * cache, then + ema
        cache.score_cache[layer_idx] = beta ** K * cache.score_cache[layer_idx] + ema_r
        cache.update(k, v, layer_idx, score_states=new_r)
    return out
