"""Patched attention forward over the cascading cache, backed by libckv_b200.so.

Mirrors cascade/models/cascade_attention.py of the reference:
``CascadeAttention.forward`` / ``forward_cascade`` (:39-200), ``LlamaCascadeAttention``
and ``Qwen2CascadeAttention`` (:343-367).  The reference's two attention bodies
(``cascade_attn_eager`` :250-340 for one token, ``cascade_attn_flash`` :202-229 for
chunks) are both served by one call, ``cascade_attention``, which computes the
eager path's definition of outputs and EMA scores for any chunk length.

What moved into the kernels (and therefore no longer appears here): query/key
position computation from the cache counters (:114-150), RoPE of q, new k, sink k
and of every cached key (:157-166), ``repeat_kv`` (:176-180), the masks, the joint
softmax, the EMA score extraction and head reduction, the score-cache decay and
``cache.update`` -- none of which synchronises with the host.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
from torch import nn

from . import _lib
from .cascading_cache import CascadingKVCache


def _rows(t: torch.Tensor, dtype, device) -> torch.Tensor:
    if t.dtype != dtype or t.device != device:
        t = t.to(device=device, dtype=dtype)
    esz = t.element_size()
    ok = t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all((t.stride(i) * esz) % 16 == 0 for i in range(3))
    return t if ok else t.contiguous()


def cascade_attention(
    query_states: torch.Tensor,
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    cache: CascadingKVCache,
    layer_idx: int = 0,
    rope_theta: float = 500000.0,
    homogeneous_heads: bool = False,
    head_reduction: Optional[str] = None,
    update: bool = True,
    out: Optional[torch.Tensor] = None,
    force_generic: bool = False,
) -> torch.Tensor:
    """Attention of ``K`` new tokens over sinks + cascade cache + themselves, then (``update``)
    the EMA score update and the cache update, all on the current CUDA stream.

    ``query_states`` ``[B, H, K, D]``, ``key_states``/``value_states`` ``[B, KVH, K, D]``: un-rotated,
    any batch/head/token strides (the transposed views the projections produce are fine).
    Returns ``[B, H, K, D]``.  Under ``cache.admission == "stride"`` no scores are computed and the
    update admits by the stride rule alone.
    """
    B, H, K, D = query_states.shape
    KVH = key_states.size(1)
    if (B, KVH, D) != (cache.max_batch_size, cache.heads, cache.dim) or key_states.shape != value_states.shape \
            or key_states.shape != (B, KVH, K, D):
        raise ValueError(f"shape mismatch: q {tuple(query_states.shape)} k {tuple(key_states.shape)} "
                         f"v {tuple(value_states.shape)} cache ({cache.max_batch_size}, {cache.heads}, K, {cache.dim})")
    dev, dt = cache.device, cache.dtype
    q = _rows(query_states, dt, dev)
    k = _rows(key_states, dt, dev)
    v = _rows(value_states, dt, dev)
    if k.stride() != v.stride():
        k, v = k.contiguous(), v.contiguous()
    if out is None:
        out = torch.empty(B, H, K, D, device=dev, dtype=dt)
    lib = cache._lib
    cfg = cache.ckv_config(layer_idx, q_heads=H, homogeneous_heads=homogeneous_heads, head_reduction=head_reduction)
    st = cache.ckv_state(layer_idx)
    flags = (_lib.CKV_ATTN_UPDATE if update else 0) | (_lib.CKV_ATTN_FORCE_GENERIC if force_generic else 0)
    # sized for the path this call takes: the generic path's logit rows are only allocated once it is asked for
    nbytes = lib.ckv_attention_workspace_bytes_for(ctypes.byref(cfg), K, flags)
    cache.workspace(nbytes)
    ws_ptr = cache.workspace_ptr()
    rope = cache.rope_table(rope_theta, cache.num_sink_tokens + cache.max_seq_len[layer_idx] + K + 1)
    if cache.admission == "ema" and update:
        w_cache, w_new = cache.ema_weights(K)
        w_cache_ptr, w_new_ptr = w_cache.data_ptr(), w_new.data_ptr()
    else:
        w_cache_ptr, w_new_ptr = None, None
    rc = lib.ckv_attention(
        ctypes.byref(cfg), ctypes.byref(st),
        q.data_ptr(), q.stride(0), q.stride(1), q.stride(2),
        k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), k.stride(2),
        K, rope.data_ptr(), rope.size(0), w_cache_ptr, w_new_ptr,
        out.data_ptr(), out.stride(0), out.stride(1), out.stride(2),
        ws_ptr, nbytes, flags, _lib.current_stream_ptr(dev))
    _lib.check(rc, "ckv_attention")
    if update:
        cache.note_tokens_seen(layer_idx, K)
    return out


class CascadeAttention(nn.Module):
    """Drop-in for the reference mixin: subclasses also inherit a HF attention module that owns
    ``q_proj/k_proj/v_proj/o_proj``, ``config`` and ``layer_idx``."""

    rope_theta_default = 10000.0

    def forward(
        self,
        hidden_states: torch.Tensor,
        attention_mask: Optional[torch.Tensor] = None,
        position_ids: Optional[torch.LongTensor] = None,
        past_key_value=None,
        output_attentions: bool = False,
        use_cache: bool = False,
        cache_position: Optional[torch.LongTensor] = None,
        position_embeddings: Optional[torch.Tensor] = None,
        past_key_values=None,
        **kwargs,
    ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[Tuple[torch.Tensor]]]:
        cache = past_key_value if past_key_value is not None else past_key_values
        if isinstance(cache, CascadingKVCache):
            return self.forward_cascade(
                hidden_states=hidden_states, past_key_value=cache,
                homogeneous_heads=getattr(self.config, "_homogeneous_heads", False),
                do_og_pos=getattr(self.config, "_do_og_pos", False))
        raise ValueError("unknown custom attention")

    def _head_counts(self):
        cfg = self.config
        n_heads = getattr(self, "num_heads", None) or cfg.num_attention_heads
        n_kv = getattr(self, "num_key_value_heads", None) or cfg.num_key_value_heads
        head_dim = getattr(self, "head_dim", None) or cfg.hidden_size // n_heads
        return n_heads, n_kv, head_dim

    def qkv(self, x, size, kv_size):
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        q = q.view(*size).transpose(1, 2)
        k = k.view(*kv_size).transpose(1, 2)
        v = v.view(*kv_size).transpose(1, 2)
        return q, k, v

    def rope_theta(self) -> float:
        cfg = self.config
        theta = getattr(cfg, "rope_theta", None)
        if theta is None:
            params = getattr(cfg, "rope_parameters", None) or {}
            theta = params.get("rope_theta", self.rope_theta_default)
        return float(theta)

    def forward_cascade(
        self,
        hidden_states: torch.Tensor,
        attention_mask=None,
        position_ids=None,
        past_key_value: Optional[CascadingKVCache] = None,
        output_attentions: bool = False,
        use_cache: bool = False,
        cache_position=None,
        use_flash: bool = True,
        homogeneous_heads: bool = True,
        do_og_pos: bool = False,
        use_selfextend: bool = False,
        position_embeddings=None,
    ):
        if do_og_pos or use_selfextend:
            raise NotImplementedError("do_og_pos / use_selfextend position modes are not implemented")
        bsz, q_len, _ = hidden_states.size()
        n_heads, n_kv, head_dim = self._head_counts()
        q, k, v = self.qkv(hidden_states, (bsz, q_len, n_heads, head_dim), (bsz, q_len, n_kv, head_dim))
        out = torch.empty(bsz, q_len, n_heads, head_dim, device=hidden_states.device, dtype=past_key_value.dtype)
        cascade_attention(q, k, v, past_key_value, self.layer_idx, rope_theta=self.rope_theta(),
                          homogeneous_heads=homogeneous_heads,
                          head_reduction=getattr(self.config, "_head_reduction", None),
                          out=out.transpose(1, 2))
        out = out.view(bsz, q_len, n_heads * head_dim).to(hidden_states.dtype)
        return self.o_proj(out), None, past_key_value

    @staticmethod
    def rope_reference(x, pos, theta):
        """RoPE of ``x [B,h,len,D]`` at ``pos [len]`` with the reference's arithmetic, in torch
        (used by tests and by callers that want rotated keys outside the kernels)."""
        D = x.size(-1)
        inv_freq = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.int64, device=x.device).float() / D))
        freqs = pos.reshape(-1).float()[:, None] * inv_freq[None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        cos, sin = emb.cos().to(x.dtype), emb.sin().to(x.dtype)
        x1, x2 = x[..., : D // 2], x[..., D // 2:]
        return (x * cos) + (torch.cat((-x2, x1), dim=-1) * sin), cos, sin

    def rope(self, x, pos, cos=None, sin=None):
        out, cos, sin = self.rope_reference(x, pos, self.rope_theta())
        return out, cos, sin


def _hf_llama_attention():
    from transformers.models.llama.modeling_llama import LlamaAttention
    return LlamaAttention


def _hf_qwen2_attention():
    from transformers.models.qwen2.modeling_qwen2 import Qwen2Attention
    return Qwen2Attention


class LlamaCascadeAttention(CascadeAttention, _hf_llama_attention()):
    rope_theta_default = 500000.0


class Qwen2CascadeAttention(CascadeAttention, _hf_qwen2_attention()):
    rope_theta_default = 1000000.0
