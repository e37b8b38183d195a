"""Patched attention forward over the cascading cache, backed by libckv_b200.so.

Mirrors cascade/models/cascade_attention.py of the reference: ``CascadeAttention.forward`` /
``forward_cascade`` (:39-200), ``cascade_attn_flash`` (:202-229), ``calc_scores`` (:231-248),
``cascade_attn_eager`` (:250-340), ``LlamaCascadeAttention`` / ``Qwen2CascadeAttention`` (:343-367)
and ``sample_monkeypatch`` (:370-592).

Two ways through ``forward_cascade``:

* the fused call ``cascade_attention`` (one ``ckv_attention`` launch sequence): query/key positions
  from the cache counters (:114-150), RoPE of q, new k, sink k and of every cached key (:157-166),
  ``repeat_kv`` (:176-180), the masks, the joint softmax, the EMA score extraction and head
  reduction, the score-cache decay and ``cache.update`` all happen in the kernels, none of it
  synchronising with the host.  This is what the default position mode takes.
* the materialised composition of the reference (``get_vals`` -> ``rope`` -> ``repeat_kv`` ->
  ``cascade_attn_eager`` / ``cascade_attn_flash`` -> ``calc_scores`` -> ``cache.update``), whose
  attention is the dense operator ``ckv_dense_attention``.  It serves ``do_og_pos`` (cached keys
  rotated at their per-lane original positions), callers that invoke the two attention methods
  directly with the reference's fifteen arguments, and any call on a cache whose ad-hoc attribute
  ``force_materialized`` is set (the counterpart of the reference's ``force_eager`` switch).
"""
from __future__ import annotations

import ctypes
import math
import types
from typing import Optional, Tuple

import numpy as np
import torch
from torch import nn

from . import _lib
from .cascading_cache import CascadingKVCache
from .flash_attention import attention, dense_attention


def _rows(t: torch.Tensor, dtype, device):
    """The tensor as the ABI wants it (last dimension contiguous, rows 16-byte aligned) and its strides."""
    if t.dtype != dtype or t.device != device:
        t = t.to(device=device, dtype=dtype)
    st = t.stride()
    # every outer stride a multiple of 16 bytes <=> their bitwise OR is (element sizes are powers of two)
    if st[3] == 1 and not (((st[0] | st[1] | st[2]) * t.element_size()) & 15) and not (t.data_ptr() & 15):
        return t, st
    t = t.contiguous()
    return t, t.stride()


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
    q, qs = _rows(query_states, dt, dev)
    k, ks = _rows(key_states, dt, dev)
    v, vs = _rows(value_states, dt, dev)
    if ks != vs:
        k, v = k.contiguous(), v.contiguous()
        ks = k.stride()
    if out is None:
        out = torch.empty(B, H, K, D, device=dev, dtype=dt)
    os_ = out.stride()
    lib = cache._lib
    cfg = cache.ckv_config(layer_idx, q_heads=H, homogeneous_heads=homogeneous_heads, head_reduction=head_reduction)
    st = cache.ckv_state(layer_idx)
    flags = (_lib.CKV_ATTN_UPDATE if update else 0) | (_lib.CKV_ATTN_FORCE_GENERIC if force_generic else 0)
    # sized for the path this call takes: the generic path's logit rows are only allocated once it is asked for
    nbytes = cache.attention_workspace_bytes(cfg, K, flags)
    cache.workspace(nbytes)
    ws_ptr = cache.workspace_ptr()
    rope = cache.rope_table(rope_theta, cache.num_sink_tokens + cache.max_seq_len[layer_idx] + K + 1)
    if cache.admission == "ema" and update:
        w_cache, w_new = cache.ema_weights(K)
        w_cache_ptr, w_new_ptr = w_cache.data_ptr(), w_new.data_ptr()
    else:
        w_cache_ptr, w_new_ptr = None, None
    with cache.device_guard():
        rc = lib.ckv_attention(
            cfg.ref, st.ref,
            q.data_ptr(), qs[0], qs[1], qs[2],
            k.data_ptr(), v.data_ptr(), ks[0], ks[1], ks[2],
            K, rope.data_ptr(), rope.size(0), w_cache_ptr, w_new_ptr,
            out.data_ptr(), os_[0], os_[1], os_[2],
            ws_ptr, nbytes, flags, _lib.current_stream_ptr(dev))
    _lib.check(rc, "ckv_attention")
    if update:
        cache.note_tokens_seen(layer_idx, K)
    return out


def rotate_half(x):
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb_one(x, cos, sin, position_ids=None, unsqueeze_dim=1):
    """cascade_attention.py:31-35 of the reference."""
    cos = cos.unsqueeze(unsqueeze_dim)
    sin = sin.unsqueeze(unsqueeze_dim)
    return (x * cos) + (rotate_half(x) * sin)


def repeat_kv(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    batch, kvh, slen, head_dim = hidden_states.shape
    if n_rep == 1:
        return hidden_states
    hidden_states = hidden_states[:, :, None, :, :].expand(batch, kvh, n_rep, slen, head_dim)
    return hidden_states.reshape(batch, kvh * n_rep, slen, head_dim)


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
            force_eager = getattr(cache, "force_eager", False)
            use_flash = False if force_eager else hidden_states.size(1) > 1
            return self.forward_cascade(
                hidden_states=hidden_states, attention_mask=attention_mask, position_ids=position_ids,
                past_key_value=cache, output_attentions=output_attentions, use_cache=use_cache,
                cache_position=cache_position, use_flash=use_flash, position_embeddings=position_embeddings,
                homogeneous_heads=getattr(self.config, "_homogeneous_heads", False),
                do_og_pos=getattr(self.config, "_do_og_pos", False))
        raise ValueError("unknown custom attention")

    # ------------------------------------------------------------------ module geometry
    def _head_counts(self):
        cfg = self.config
        n_heads = getattr(self, "num_heads", None) or cfg.num_attention_heads
        n_kv = getattr(self, "num_key_value_heads", None) or cfg.num_key_value_heads
        head_dim = getattr(self, "head_dim", None) or cfg.hidden_size // n_heads
        return n_heads, n_kv, head_dim

    def qkv(self, x, size, kv_size):
        w = getattr(self, "_qkv_weight", None)
        if w is not None and w.device == x.device and w.dtype == x.dtype:
            # one projection for q | k | v (thin_model.fuse_projections); the three results are strided views of
            # its output, which the attention call reads in place
            qkv = nn.functional.linear(x, w, getattr(self, "_qkv_bias", None))
            nq, nkv = size[2] * size[3], kv_size[2] * kv_size[3]
            q = qkv[..., :nq].view(*size).transpose(1, 2)
            k = qkv[..., nq:nq + nkv].view(*kv_size).transpose(1, 2)
            v = qkv[..., nq + nkv:].view(*kv_size).transpose(1, 2)
            return q, k, v
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

    # ------------------------------------------------------------------------- forward
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
        """cascade_attention.py:82-200 of the reference.  ``use_flash`` names the reference's two
        attention bodies; on the fused path both are the same kernels (the eager definition of outputs
        and scores for any chunk length), on the materialised path it picks the method called."""
        cache = past_key_value
        bsz, q_len, _ = hidden_states.size()
        n_heads, n_kv, head_dim = self._head_counts()
        if not hasattr(self, "last_q_size"):
            self.last_q_size = None
        query_states, key_states, value_states = self.qkv(
            hidden_states, (bsz, q_len, n_heads, head_dim), (bsz, q_len, n_kv, head_dim))
        if hasattr(cache, "plot_attn"):
            raise NotImplementedError("plot_attn (a dump of the full attention matrix per layer) is not provided")

        if use_selfextend:
            # The reference's branch (:126-139) slices og_pos with cache.window_length, which its cache
            # turns into a per-layer list in the constructor (cascading_cache.py:1055-1057): the mode
            # raises a TypeError there and nothing in the reference enables it.
            raise NotImplementedError("use_selfextend is not provided (the reference's own branch cannot run)")

        if not do_og_pos and not getattr(cache, "force_materialized", False):
            out = torch.empty(bsz, q_len, n_heads, head_dim, device=hidden_states.device, dtype=cache.dtype)
            cascade_attention(query_states, key_states, value_states, cache, self.layer_idx,
                              rope_theta=self.rope_theta(), homogeneous_heads=homogeneous_heads,
                              head_reduction=getattr(self.config, "_head_reduction", None),
                              out=out.transpose(1, 2))
            self.last_attn_called = "flash" if use_flash else "eager"
            self.last_q_size = q_len
            out = out.view(bsz, q_len, n_heads * head_dim)
            if out.dtype != self.o_proj.weight.dtype:
                out = out.to(self.o_proj.weight.dtype)
            return self.o_proj(out), None, cache

        # ---- materialised composition (per-lane key positions), reference :103-200 --------------------
        dt = cache.dtype
        query_states, key_states, value_states = (t.to(dt) for t in (query_states, key_states, value_states))
        first_it = cache.seen_tokens_host(self.layer_idx) == 0
        sink_key_states, sink_value_states, sink_pos, sink_mask, k_states, v_states, key_pos, key_mask, og_pos = \
            cache.get_vals(self.layer_idx)
        max_pos = 0
        if first_it:
            self.last_attn_called = None
        if not first_it:
            if do_og_pos:
                max_pos = torch.cat((sink_pos.amax().view(1), og_pos.amax().view(1)), dim=-1).amax() + 1
            else:
                max_pos = torch.cat((sink_pos.amax().view(1), key_pos.amax().view(1)), dim=-1).amax() + 1
        query_pos = torch.arange(0, q_len, device=query_states.device, dtype=torch.long).view(1, -1) + max_pos

        query_states, cos_q, sin_q = self.rope(query_states, query_pos)
        key_states_pos, _, _ = self.rope(key_states, query_pos, cos=cos_q, sin=sin_q)
        sink_key_states, _, _ = self.rope(sink_key_states, sink_pos)
        if do_og_pos:
            b, h, s, d = k_states.size()
            k_states, _, _ = self.rope(k_states.reshape(b * h, 1, s, d), og_pos.reshape(b * h, -1))
            k_states = k_states.view(b, h, s, d)
        else:
            k_states, _, _ = self.rope(k_states, key_pos)

        G = n_heads // n_kv
        key_states_pos = repeat_kv(key_states_pos, G)
        sink_key_states = repeat_kv(sink_key_states, G)
        sink_value_states = repeat_kv(sink_value_states, G)
        k_states = repeat_kv(k_states, G)
        v_states = repeat_kv(v_states, G)
        scale = 1 / math.sqrt(query_states.size(-1))
        func_args = (query_states, key_states, value_states, key_states_pos, v_states, sink_key_states,
                     sink_value_states, k_states, sink_mask, key_mask, first_it, cache, scale, q_len,
                     homogeneous_heads)
        if not use_flash:
            out, cache = self.cascade_attn_eager(*func_args)
        else:
            out, cache = self.cascade_attn_flash(*func_args)
        out = out.transpose(1, 2).contiguous().view(bsz, q_len, -1)
        if out.dtype != self.o_proj.weight.dtype:
            out = out.to(self.o_proj.weight.dtype)
        return self.o_proj(out), None, cache

    # ------------------------------------------------------ the reference's two attention bodies
    def cascade_attn_flash(self, query_states, key_states, value_states, key_states_pos, v_states,
                           sink_key_states, sink_value_states, k_states, sink_mask, key_mask, first_it,
                           past_key_value, scale, q_len, homogeneous_heads):
        """cascade_attention.py:202-229: the functional ``attention`` over ``cat(sinks, cache, new)``,
        then ``calc_scores``, the score-cache decay and ``cache.update``.  ``query_states``,
        ``key_states_pos``, ``sink_key_states`` and ``k_states`` are rotated; ``key_states`` /
        ``value_states`` are the un-rotated new tokens that enter the cache.

        One deliberate difference: the cached-slot scores are taken from columns ``NS .. NS+S`` of the
        kernel's score row.  The reference slices ``[:n_keys]`` from column 0 (:220, :241), which
        attributes the sink columns' scores to the first ``NS`` slots and shifts the rest; its eager
        body (:319) aligns them as done here."""
        self.last_attn_called = "flash"
        self.last_q_size = query_states.size(2)
        G = query_states.size(1) // value_states.size(1)
        mask = torch.cat((sink_mask[0, 0], key_mask[0, 0]))
        out, scores = attention(
            query_states,
            torch.cat((sink_key_states, k_states, key_states_pos), dim=2),
            torch.cat((sink_value_states, v_states, repeat_kv(value_states, G)), dim=2),
            True, scale, mask, past_key_value.beta)
        sk = sink_key_states.size(2)
        ema_scores, scores = self.calc_scores(scores[:, :, sk:], homogeneous_heads, k_states.size(2), q_len)
        beta = past_key_value.beta
        past_key_value.score_cache[self.layer_idx] = \
            beta ** out.size(2) * past_key_value.score_cache[self.layer_idx] + ema_scores
        _ = past_key_value.update(key_states, value_states, self.layer_idx, score_states=scores)
        return out, past_key_value

    def calc_scores(self, scores, homogeneous_heads, n_keys, q_len):
        """cascade_attention.py:231-248: head reduction of the per-head column scores."""
        _, kvh, _ = self._head_counts()
        func = {
            "mean": torch.mean,
            "max": torch.amax,
            "median": lambda x, **kwargs: torch.median(x, **kwargs).values,
        }[self.config._head_reduction]
        if homogeneous_heads:
            ema_scores = func(scores[:, :, :n_keys], dim=1, keepdim=True)
            scores = func(scores[:, :, -q_len:], dim=1, keepdim=True).repeat(1, kvh, 1)
        else:
            b, h, s = scores.size()
            ema_scores = func(scores[:, :, :n_keys].view(b, kvh, h // kvh, -1), dim=2)
            scores = func(scores[:, :, -q_len:].view(b, kvh, h // kvh, -1), dim=2)
        return ema_scores, scores

    def cascade_attn_eager(self, query_states, key_states, value_states, key_states_pos, v_states,
                           sink_key_states, sink_value_states, k_states, sink_mask, key_mask, first_it,
                           past_key_value, scale, q_len, homogeneous_heads):
        """cascade_attention.py:250-340 with the three einsums, the joint softmax, the three
        probability-value products and the two score sums done by one ``ckv_dense_attention`` call in
        its eager mode (operands scaled by sqrt(scale) each and logits / probabilities rounded to the
        tensor dtype, as the reference's torch ops round them)."""
        self.last_attn_called = "eager"
        self.last_q_size = query_states.size(2)
        cache = past_key_value
        G = query_states.size(1) // value_states.size(1)
        rs = np.sqrt(scale)
        mask = torch.cat((sink_mask[0, 0], key_mask[0, 0]))
        keys = torch.cat((sink_key_states, k_states, key_states_pos), dim=2) * rs
        vals = torch.cat((sink_value_states, v_states, repeat_kv(value_states, G)), dim=2)
        w_cache, w_new = cache.ema_weights(q_len)
        out, scores = dense_attention(query_states * rs, keys, vals, mask, 1.0, cache.beta,
                                      _lib.CKV_DENSE_SCORES_EAGER, w_cache, w_new)
        sk = sink_key_states.size(2)
        ema_scores, scores = self.calc_scores(scores[:, :, sk:], homogeneous_heads, k_states.size(2), q_len)
        beta = cache.beta
        cache.score_cache[self.layer_idx] = beta ** scores.size(2) * cache.score_cache[self.layer_idx] + ema_scores
        scores = scores.repeat(1, query_states.size(1), 1)
        _ = cache.update(key_states, value_states, self.layer_idx, score_states=scores)
        return out, cache

    # ----------------------------------------------------------------------------- RoPE
    @staticmethod
    def rope_reference(x, pos, theta):
        """RoPE of ``x [B,h,len,D]`` at ``pos`` (``[len]``, ``[1,len]`` or one row per leading index of
        ``x``) with the reference's arithmetic: fp32 angle, fp32 cos/sin, cast to ``x``'s dtype
        (cascade/models/llama/modeling_llama.py:199-220).  Returns ``(x', cos, sin)``, cos/sin ``[n,len,D]``."""
        D = x.size(-1)
        pos = pos.reshape(1, -1) if pos.dim() < 2 else pos
        inv_freq = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.int64, device=x.device).float() / D))
        freqs = pos.float()[:, :, None] * inv_freq[None, None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        cos, sin = emb.cos().to(x.dtype), emb.sin().to(x.dtype)
        return apply_rotary_pos_emb_one(x, cos, sin), cos, sin

    def rope(self, x, pos, cos=None, sin=None):
        """``rope(x, pos, cos, sin) -> (x', cos, sin)`` (cascade_attention.py:343-367); given cos / sin
        are reused as the reference reuses layer 0's."""
        if cos is None or sin is None:
            return self.rope_reference(x, pos, self.rope_theta())
        return apply_rotary_pos_emb_one(x, cos, sin), cos, sin


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


# --------------------------------------------------------------------------- generation loop
@torch.no_grad()
def _sample_monkeypatch(self, input_ids: torch.LongTensor, past_key_values: CascadingKVCache,
                        max_new_tokens: int = 128, do_sample: bool = False, eos_token_id: Optional[int] = None,
                        pad_token_id: int = 0, streamer=None, logits_processor=None, **model_kwargs):
    """The reference's strided-prefill generation loop (cascade_attention.py:370-592) for a model whose
    forward is ``model(input_ids, past_key_values=cache).logits``.

    First iteration: the prompt is fed in chunks of ``config._cascade_stride`` tokens, every chunk
    going through the cascading cache on every layer (:473-496; ``last_it`` is raised on each layer's
    attention for the final chunk, :484-487).  After that one token per iteration; greedy
    ``argmax`` unless ``do_sample`` (:534-538).  Sequences that emitted ``eos_token_id`` keep producing
    ``pad_token_id`` (:541-542).  Returns ``input_ids`` extended by the generated tokens, as the
    reference does without ``return_dict_in_generate``."""
    stride = self.config._cascade_stride
    layers = getattr(getattr(self, "model", self), "layers", [])
    unfinished = torch.ones(input_ids.size(0), dtype=torch.long, device=input_ids.device)
    first_it = True
    for _ in range(max_new_tokens):
        if first_it:
            for lyr in layers:
                lyr.self_attn.last_it = False
            n = input_ids.size(1)
            for i in range(0, n, stride):
                if i + stride >= n:
                    for lyr in layers:
                        lyr.self_attn.last_it = True
                outputs = self(input_ids[:, i:i + stride], past_key_values=past_key_values, **model_kwargs)
            first_it = False
        else:
            outputs = self(input_ids[:, -1:], past_key_values=past_key_values, **model_kwargs)
        next_token_logits = outputs.logits[:, -1, :].clone()
        del outputs
        scores = logits_processor(input_ids, next_token_logits) if logits_processor is not None else next_token_logits
        if do_sample:
            next_tokens = torch.multinomial(nn.functional.softmax(scores, dim=-1), num_samples=1).squeeze(1)
        else:
            next_tokens = torch.argmax(scores, dim=-1)
        if eos_token_id is not None:
            next_tokens = next_tokens * unfinished + pad_token_id * (1 - unfinished)
        input_ids = torch.cat([input_ids, next_tokens[:, None]], dim=-1)
        if streamer is not None:
            streamer.put(next_tokens.cpu())
        if eos_token_id is not None:
            unfinished = unfinished & (next_tokens != eos_token_id).long()
            if int(unfinished.max()) == 0:
                break
    if streamer is not None:
        streamer.end()
    return input_ids


def sample_monkeypatch(model) -> nn.Module:
    """``sample_monkeypatch(model)`` of the reference (:590-592): bind the strided-prefill loop as the
    model's ``_sample``."""
    model._sample = types.MethodType(_sample_monkeypatch, model)
    return model
