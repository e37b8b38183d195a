"""A thin decoder stack around the patched attention: what the end-to-end configuration needs.

The reference runs its attention inside forked Hugging Face models
(cascade/models/llama/modeling_llama.py:701-782 decoder layer, :939-1058 model, :1164-1256 causal LM;
cascade/models/qwen2/modeling_qwen2.py likewise), which cannot be constructed under the installed
transformers.  This module is the same computation with nothing else around it: token embedding,
``L x [RMSNorm -> cascade attention -> residual -> RMSNorm -> SwiGLU MLP -> residual]``, final RMSNorm,
``lm_head``.  The attention is ``LlamaCascadeAttention`` / ``Qwen2CascadeAttention`` (hand-written kernels
behind the C ABI); the dense layers are plain ``torch.nn.Linear`` (library GEMMs); RMSNorm follows
modeling_llama.py:113-127 (fp32 variance, weight applied after the cast back) and is fused with the residual
add before it, the SwiGLU gate is one kernel too (``ckv_add_rmsnorm`` / ``ckv_silu_mul`` on 16-bit CUDA
tensors, the same torch operations as the reference elsewhere).

Configuration: a Hugging Face ``LlamaConfig`` / ``Qwen2Config`` carrying the reference's private fields
(cascade/main/llama_eval.py:143-152): ``_sinks, _cascades, _window, _cascade_func, _head_reduction,
_cascade_stride, _homogeneous_heads, _do_og_pos``, plus ``_batch_size``.  ``get_cache(model)`` builds the
cache from them as the reference's helper does (cascade/models/test.py:21-39).
"""
from __future__ import annotations

import types
from typing import Optional

import torch
from torch import nn

from . import _lib
from .cascade_attention import LlamaCascadeAttention, Qwen2CascadeAttention, sample_monkeypatch
from .cascading_cache import CascadingKVCache


def _fusable(x: torch.Tensor) -> bool:
    """The element-wise kernels of the library take contiguous 16-bit CUDA rows of a multiple of 8 elements."""
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.size(-1) % 8 == 0 and x.is_contiguous()


def add_rmsnorm(x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float):
    """``s = x + residual`` (``s = x`` without a residual) and ``weight * rmsnorm(s)``: the residual add of a
    decoder layer and the norm that follows it (modeling_llama.py:113-127, :745-770), one kernel on 16-bit CUDA
    tensors (``ckv_add_rmsnorm``), the reference's own sequence of torch operations otherwise.
    Returns ``(normed, s)``."""
    if _fusable(x) and (residual is None or (_fusable(residual) and residual.shape == x.shape)) \
            and weight.dtype == x.dtype and weight.is_contiguous():
        lib = _lib.load()
        normed = torch.empty_like(x)
        s = x if residual is None else torch.empty_like(x)
        hidden = x.size(-1)
        with torch.cuda.device(x.device):
            rc = lib.ckv_add_rmsnorm(x.data_ptr(), None if residual is None else residual.data_ptr(), weight.data_ptr(),
                                     normed.data_ptr(), None if residual is None else s.data_ptr(), x.numel() // hidden,
                                     hidden, float(eps), _lib.DTYPE_CODE[x.dtype], _lib.current_stream_ptr(x.device))
        _lib.check(rc, "ckv_add_rmsnorm")
        return normed, s
    s = x if residual is None else residual + x
    h = s.to(torch.float32)
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return weight * h.to(s.dtype), s


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` (modeling_llama.py:282-313), one kernel on 16-bit CUDA tensors (``ckv_silu_mul``)."""
    if _fusable(gate) and _fusable(up) and gate.shape == up.shape and gate.dtype == up.dtype:
        cols = gate.size(-1)
        return _silu_mul_rows(gate, up, gate.numel() // cols, cols, cols, cols, gate.shape)
    return nn.functional.silu(gate) * up


def _silu_mul_rows(gate, up, rows, cols, ld_gate, ld_up, shape):
    lib = _lib.load()
    out = torch.empty(shape, device=gate.device, dtype=gate.dtype)
    with torch.cuda.device(gate.device):
        rc = lib.ckv_silu_mul(gate.data_ptr(), up.data_ptr(), out.data_ptr(), rows, cols, ld_gate, ld_up,
                              _lib.DTYPE_CODE[gate.dtype], _lib.current_stream_ptr(gate.device))
    _lib.check(rc, "ckv_silu_mul")
    return out


class RMSNorm(nn.Module):
    """modeling_llama.py:113-127 of the reference."""

    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, hidden_states, residual: Optional[torch.Tensor] = None):
        """Without ``residual``: the norm of ``hidden_states``.  With it: ``(norm(hidden_states + residual),
        hidden_states + residual)`` -- the add that precedes every norm of the stack but the first."""
        normed, s = add_rmsnorm(hidden_states, residual, self.weight, self.variance_epsilon)
        return normed if residual is None else (normed, s)


class SwiGLU(nn.Module):
    """LlamaMLP / Qwen2MLP: ``down(silu(gate(x)) * up(x))`` (modeling_llama.py:282-313)."""

    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__()
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)

    def forward(self, x):
        w = getattr(self, "_gate_up_weight", None)
        if w is not None and w.device == x.device and w.dtype == x.dtype:
            # one projection for gate | up (fuse_projections); the gate kernel reads the two halves in place
            n = w.size(0) // 2
            gu = nn.functional.linear(x, w).view(-1, 2 * n)
            if _fusable(gu) and n % 8 == 0:
                h = _silu_mul_rows(gu[:, :n], gu[:, n:], gu.size(0), n, 2 * n, 2 * n, (*x.shape[:-1], n))
            else:
                h = (nn.functional.silu(gu[:, :n]) * gu[:, n:]).view(*x.shape[:-1], n)
            return self.down_proj(h)
        return self.down_proj(silu_mul(self.gate_proj(x), self.up_proj(x)))


class DecoderLayer(nn.Module):
    """modeling_llama.py:701-782: pre-norm attention and MLP with residuals.  The layer hands its MLP output and
    the running residual to the next layer separately, so that every residual add is done by the norm that
    consumes its result (same values, same rounding points, one kernel instead of two)."""

    def __init__(self, config, layer_idx: int, attention_cls):
        super().__init__()
        self.self_attn = attention_cls(config, layer_idx)
        self.mlp = SwiGLU(config.hidden_size, config.intermediate_size)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, hidden_states, residual, past_key_values):
        if residual is None:
            residual, hidden_states = hidden_states, self.input_layernorm(hidden_states)
        else:
            hidden_states, residual = self.input_layernorm(hidden_states, residual)
        hidden_states, _, _ = self.self_attn(hidden_states, past_key_values=past_key_values, use_cache=True)
        hidden_states, residual = self.post_attention_layernorm(hidden_states, residual)
        return self.mlp(hidden_states), residual


class CascadeModel(nn.Module):
    def __init__(self, config, attention_cls):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([DecoderLayer(config, i, attention_cls) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, input_ids, past_key_values):
        hidden_states, residual = self.embed_tokens(input_ids), None
        for layer in self.layers:
            hidden_states, residual = layer(hidden_states, residual, past_key_values)
        if residual is None:
            return self.norm(hidden_states)
        return self.norm(hidden_states, residual)[0]


class CascadeForCausalLM(nn.Module):
    """``model(input_ids, past_key_values=cache)`` -> object with ``.logits`` and ``.past_key_values``
    (modeling_llama.py:1164-1256).  ``num_logits_to_keep`` > 0 applies ``lm_head`` to the last positions only:
    a 4096-token prefill chunk needs one row of logits, not 4096 x vocab."""

    def __init__(self, config, family: str = "llama"):
        super().__init__()
        if family not in ("llama", "qwen2"):
            raise ValueError(f"unknown model family {family}")
        self.config = config
        self.family = family
        self.model = CascadeModel(config, LlamaCascadeAttention if family == "llama" else Qwen2CascadeAttention)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        sample_monkeypatch(self)

    def forward(self, input_ids, past_key_values: CascadingKVCache, num_logits_to_keep: int = 0, **_):
        hidden_states = self.model(input_ids, past_key_values)
        if num_logits_to_keep > 0:
            hidden_states = hidden_states[:, -num_logits_to_keep:]
        return types.SimpleNamespace(logits=self.lm_head(hidden_states), past_key_values=past_key_values)

    @torch.no_grad()
    def generate(self, input_ids, past_key_values: CascadingKVCache, max_new_tokens: int = 128,
                 do_sample: bool = False, **kwargs):
        """The reference's generation path: ``_sample`` bound by ``sample_monkeypatch`` -- the prompt in strides of
        ``config._cascade_stride`` through the cascading cache, then one token at a time."""
        return self._sample(input_ids, past_key_values, max_new_tokens=max_new_tokens, do_sample=do_sample,
                            num_logits_to_keep=1, **kwargs)

    @torch.no_grad()
    def fuse_projections(self):
        """q | k | v and gate | up of every layer as one weight each, so that a layer runs four projections instead
        of seven.  The separate parameters stay (same names, same values in ``state_dict``): they become views of
        the fused storage.  Call it once the model sits on its device in its dtype; a later ``.to()`` drops the
        sharing and the layers fall back to the separate projections."""
        for lyr in self.model.layers:
            a, m = lyr.self_attn, lyr.mlp
            parts = [a.q_proj, a.k_proj, a.v_proj]
            with_bias = [p.bias is not None for p in parts]
            if any(with_bias) and not all(with_bias):
                raise ValueError("fuse_projections: q / k / v projections must all have a bias or none")
            w = torch.cat([p.weight for p in parts], dim=0)
            off = 0
            for p in parts:
                n = p.weight.size(0)
                p.weight.data = w[off:off + n]
                off += n
            a._qkv_weight = w
            if all(with_bias):
                bias = torch.cat([p.bias for p in parts], dim=0)
                off = 0
                for p in parts:
                    n = p.bias.size(0)
                    p.bias.data = bias[off:off + n]
                    off += n
                a._qkv_bias = bias
            wg = torch.cat([m.gate_proj.weight, m.up_proj.weight], dim=0)
            n = m.gate_proj.weight.size(0)
            m.gate_proj.weight.data, m.up_proj.weight.data = wg[:n], wg[n:]
            m._gate_up_weight = wg
        return self

    @torch.no_grad()
    def init_weights(self, seed: int, std: float = 0.02):
        """Random N(0, std) matrices and embeddings from ``seed`` (norm weights stay 1, biases 0), drawn on the
        parameters' device in their order of registration."""
        dev = self.lm_head.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) * std)
            elif name.endswith("bias"):
                p.zero_()
        return self


def cascade_config(family: str = "llama", hidden_size: int = 4096, intermediate_size: int = 14336,
                   num_hidden_layers: int = 32, num_attention_heads: int = 32, num_key_value_heads: int = 8,
                   vocab_size: int = 128256, rope_theta: float = 500000.0, rms_norm_eps: float = 1e-5,
                   sinks: int = 64, cascades: int = 4, window: int = 32768, cascade_func: str = "pow2",
                   head_reduction: str = "max", cascade_stride: int = 4096, homogeneous_heads: bool = False,
                   do_og_pos: bool = False, batch_size: int = 1):
    """A Hugging Face config with the reference's private cascade fields; defaults = Llama-3.1-8B shapes with a
    plain RoPE base (no frequency scaling)."""
    if family == "llama":
        from transformers import LlamaConfig
        cfg = LlamaConfig(hidden_size=hidden_size, intermediate_size=intermediate_size,
                          num_hidden_layers=num_hidden_layers, num_attention_heads=num_attention_heads,
                          num_key_value_heads=num_key_value_heads, head_dim=hidden_size // num_attention_heads,
                          vocab_size=vocab_size, rope_theta=rope_theta, rms_norm_eps=rms_norm_eps)
    else:
        from transformers import Qwen2Config
        cfg = Qwen2Config(hidden_size=hidden_size, intermediate_size=intermediate_size,
                          num_hidden_layers=num_hidden_layers, num_attention_heads=num_attention_heads,
                          num_key_value_heads=num_key_value_heads, vocab_size=vocab_size, rope_theta=rope_theta,
                          rms_norm_eps=rms_norm_eps)
    cfg._method = "sink"
    cfg._sinks, cfg._cascades, cfg._window, cfg._cascade_func = sinks, cascades, window, cascade_func
    cfg._head_reduction, cfg._cascade_stride = head_reduction, cascade_stride
    cfg._homogeneous_heads, cfg._do_og_pos, cfg._batch_size = homogeneous_heads, do_og_pos, batch_size
    return cfg


def get_cache(model: CascadeForCausalLM, dtype: Optional[torch.dtype] = None, eager_fill: bool = True,
              admission: str = "ema") -> CascadingKVCache:
    """The cache for ``model`` from its config's cascade fields (cascade/models/test.py:21-39)."""
    cfg = model.config
    param = model.lm_head.weight
    return CascadingKVCache(
        cfg._window // cfg._cascades, num_sink_tokens=cfg._sinks, max_batch_size=cfg._batch_size,
        heads=cfg.num_key_value_heads, dim=cfg.hidden_size // cfg.num_attention_heads, max_seq_len=cfg._window,
        dtype=dtype or param.dtype, device=param.device, cascade_func=cfg._cascade_func,
        head_reduction=cfg._head_reduction, layers=cfg.num_hidden_layers, eager_fill=eager_fill, verbose=False,
        admission=admission)
