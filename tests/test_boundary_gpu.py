"""The Python surface callers of the reference import, on the GPU: the patched attention classes under
the installed transformers, the two attention methods with the reference's arguments, ``calc_scores``,
``force_eager``, ``do_og_pos``, and the functional ``attention`` -- each against the CPU oracle or
against the reference-generated golden vectors."""
import types

import numpy as np
import pytest
import torch

from oracle.cascade_oracle import OracleCascadingKVCache, cascade_attention_step
from tests.test_attention_gpu import close_enough
from tests.test_oracle import ATTN, run_attention_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tiny_attention(family, dtype, head_reduction="max", homogeneous=False, do_og_pos=False):
    """LlamaCascadeAttention / Qwen2CascadeAttention of a tiny config built under the installed transformers:
    hidden 512, 4 query / 2 KV heads, head_dim 128 (Qwen2: q/k/v bias, theta 1e6)."""
    from cascading_kv_cache_b200 import LlamaCascadeAttention, Qwen2CascadeAttention
    if family == "llama":
        from transformers import LlamaConfig
        cfg = LlamaConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                          intermediate_size=64, num_hidden_layers=1, vocab_size=64, rope_theta=500000.0)
        cls = LlamaCascadeAttention
    else:
        from transformers import Qwen2Config
        cfg = Qwen2Config(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, intermediate_size=64,
                          num_hidden_layers=1, vocab_size=64, rope_theta=1000000.0)
        cls = Qwen2CascadeAttention
    cfg._head_reduction, cfg._homogeneous_heads, cfg._do_og_pos = head_reduction, homogeneous, do_og_pos
    torch.manual_seed(5)
    m = cls(cfg, 0)
    for p in m.parameters():                       # projections that keep activations near N(0,1)
        torch.nn.init.normal_(p, std=0.05 if p.dim() > 1 else 0.3)
    return m.to(device=DEV, dtype=dtype).eval(), cfg


def _oracle_forward(m, x, ref, theta, red, homog, og, dtype):
    """The same module's projections on the CPU around the oracle's attention."""
    cpu = lambda lin: (lin.weight.detach().cpu(), None if lin.bias is None else lin.bias.detach().cpu())
    lin = lambda name, t: torch.nn.functional.linear(t, *cpu(getattr(m, name)))
    B, n, _ = x.shape
    q = lin("q_proj", x).view(B, n, 4, 128).transpose(1, 2)
    k = lin("k_proj", x).view(B, n, 2, 128).transpose(1, 2)
    v = lin("v_proj", x).view(B, n, 2, 128).transpose(1, 2)
    o = cascade_attention_step(q, k, v, ref, 0, theta, red, homog, do_og_pos=og)
    return lin("o_proj", o.transpose(1, 2).reshape(B, n, 512))


CLASS_CASES = [
    # family, dtype, reduction, homogeneous, do_og_pos, force_eager, chunk lengths
    ("llama", torch.bfloat16, "max", False, False, False, [40, 40, 40, 1, 1, 1]),
    ("qwen2", torch.bfloat16, "mean", False, False, False, [64, 17, 1, 1, 50, 1]),
    ("llama", torch.float32, "mean", True, False, False, [24, 24, 24, 1, 1]),
    ("qwen2", torch.float32, "max", False, True, True, [24, 24, 24, 1, 1]),
    ("llama", torch.bfloat16, "max", False, True, True, [30, 30, 1, 1]),
    ("llama", torch.float32, "median", False, False, True, [24, 24, 1, 1]),
]


@pytest.mark.parametrize("case", CLASS_CASES, ids=lambda c: f"{c[0]}-{str(c[1])[6:]}-{c[2]}-h{int(c[3])}-og{int(c[4])}-e{int(c[5])}")
def test_patched_attention_classes_against_oracle(case):
    """``forward(hidden_states, past_key_values=cache)`` of the two patched classes over chunks and single
    tokens (reference contract: cascade_attention.py:39-71, :82-200, :343-367)."""
    from cascading_kv_cache_b200 import CascadingKVCache
    family, dtype, red, homog, og, force_eager, steps = case
    m, cfg = _tiny_attention(family, dtype, red, homog, og)
    theta = 500000.0 if family == "llama" else 1000000.0
    assert m.rope_theta() == theta
    W, C, NS, B = 16, 4, 4, 2
    cache = CascadingKVCache(W, NS, B, 2, 128, W * C, device=DEV, dtype=dtype, head_reduction=red, layers=1,
                             eager_fill=True, verbose=False)
    ref = OracleCascadingKVCache(W, NS, B, 2, 128, W * C, dtype=dtype, head_reduction=red, layers=1, eager_fill=True)
    cache.beta = ref.beta = 0.999
    if force_eager:
        cache.force_eager = True
    g = torch.Generator().manual_seed(8)
    is16 = dtype != torch.float32
    with torch.no_grad():
        for n in steps:
            x = torch.randn(B, n, 512, generator=g).to(dtype)
            out, attn_w, returned = m(x.to(DEV), past_key_values=cache)
            assert attn_w is None and returned is cache and out.shape == (B, n, 512)
            want = _oracle_forward(m, x, ref, theta, red, homog, og, dtype)
            # the projections run as bf16 GEMMs on either side and already differ in their last place,
            # hence the lower element-wise share
            ok, err = close_enough(out.float().cpu(), want.float(), is16, elementwise_min=0.85)
            assert ok, (n, err)
            assert m.last_attn_called == ("eager" if (force_eager or n == 1) else "flash")
    assert cache.kernel_status() == 0
    valid = ~ref.mask[0]
    assert torch.equal(cache.mask[0].cpu(), ref.mask[0])
    assert torch.equal(cache.pos[0].cpu()[valid], ref.pos[0][valid])
    assert cache.get_seq_length(0) == int(ref.stored_sinks[0][0, 0]) + int(ref.stored_tokens[0][0, 0].sum())
    if not is16:
        agree = (cache.og_pos[0].cpu()[valid] == ref.og_pos[0][valid]).float().mean().item()
        assert agree >= 0.999, agree


class _SlicingAttention:
    """A CascadeAttention whose projections slice the hidden state, as the golden vectors were made."""

    @staticmethod
    def make(H, KVH, D, theta, red, homog, og):
        from cascading_kv_cache_b200 import CascadeAttention

        class Shim(CascadeAttention):
            pass

        m = Shim()
        m.num_heads, m.num_key_value_heads, m.num_key_value_groups, m.head_dim, m.layer_idx = H, KVH, H // KVH, D, 0
        m.config = types.SimpleNamespace(_head_reduction=red, _homogeneous_heads=homog, _do_og_pos=og,
                                         rope_theta=theta, num_attention_heads=H, num_key_value_heads=KVH,
                                         hidden_size=H * D)
        hq, hk = H * D, KVH * D
        m.q_proj = lambda x: x[..., :hq]
        m.k_proj = lambda x: x[..., hq:hq + hk]
        m.v_proj = lambda x: x[..., hq + hk:]
        m.o_proj = types.SimpleNamespace(weight=torch.empty(0))
        return m


def _golden_through_the_class(name, mode):
    """Drive ``forward_cascade`` with the golden hidden states; ``mode``: fused / eager / flash."""
    from cascading_kv_cache_b200 import CascadingKVCache
    st = ATTN[name]
    B, H, KVH, D, NS, W, C, chunk, n_chunks, n_dec = (int(x) for x in st["cfg"])
    theta, red, homog, og = float(st["theta"]), str(st["reduction"]), bool(st["homogeneous"]), bool(st["do_og_pos"])
    m = _SlicingAttention.make(H, KVH, D, theta, red, homog, og)

    def make_cache(W, NS, B, KVH, D, S, dtype, red, eager_fill, beta):
        c = CascadingKVCache(W, NS, B, KVH, D, S, device=DEV, dtype=dtype, head_reduction=red, layers=1,
                             eager_fill=eager_fill, verbose=False)
        c.beta = beta
        m.o_proj = type("Id", (), {"weight": torch.empty(0, dtype=dtype), "__call__": lambda self, x: x})()
        if mode != "fused":
            c.force_materialized = True
        return c

    def step(q, k, v, cache, theta, red, homog, rule, do_og_pos=False):
        # undo run_attention_case's split: forward_cascade projects by slicing the same hidden state
        B, _, n, _ = q.shape
        x = torch.cat((q.transpose(1, 2).reshape(B, n, -1), k.transpose(1, 2).reshape(B, n, -1),
                       v.transpose(1, 2).reshape(B, n, -1)), dim=-1).to(DEV)
        o, _, _ = m.forward_cascade(hidden_states=x, past_key_value=cache, use_flash=(mode == "flash"),
                                    homogeneous_heads=homog, do_og_pos=do_og_pos)
        return o.view(B, n, H, D).transpose(1, 2)

    out, cache = run_attention_case(st, step, make_cache)
    return st, out, cache


@pytest.mark.parametrize("name", ["ema_f32_max", "ema_f32_mean_h", "ema_f32_median", "ema_bf16_max",
                                  "ogpos_f32_max", "ogpos_bf16_mean_h"])
@pytest.mark.parametrize("mode", ["fused", "eager", "flash"])
def test_reference_golden_outputs_through_forward_cascade(name, mode):
    """The reference's own forward_cascade outputs (golden vectors) through this package's
    ``forward_cascade``: the fused call, and the materialised composition with ``cascade_attn_eager`` and
    with ``cascade_attn_flash`` (+ ``calc_scores``, the score decay and ``cache.update``)."""
    if name.startswith("ogpos") and mode == "fused":
        pytest.skip("do_og_pos always takes the materialised composition")
    st, out, cache = _golden_through_the_class(name, mode)
    is16 = "bfloat16" in str(st["dtype"])
    share = 0.93 if mode != "fused" else 0.97     # the dense operator sums P.V in another order
    ok, err = close_enough(out, torch.from_numpy(st["out"]), is16, share)
    # the flash body scores new tokens with the flash weights, so a stream may admit other tokens than the
    # eager-made golden stream did: its outputs are only held to the golden ones while the cache still fills
    if mode == "flash":
        B, H, KVH, D, NS, W, C, chunk, n_chunks, n_dec = (int(x) for x in st["cfg"])
        fill = min(out.size(1), NS + W)       # cascade 0 has not evicted yet
        ok, err = close_enough(out[:, :fill], torch.from_numpy(st["out"])[:, :fill], is16, share)
    assert ok, err
    valid = ~st["masked"].astype(bool)
    assert np.array_equal(~cache.mask[0][0, 0].cpu().numpy(), valid)
    assert np.array_equal((cache.pos[0][0, 0].cpu().numpy() + cache.num_sink_tokens)[valid], st["pos"][valid])
    if not is16 and mode != "flash":
        assert np.allclose(cache.key_cache[0].cpu().numpy()[:, :, valid], st["key_cache"][:, :, valid])
        assert np.allclose(cache.score_cache[0].cpu().numpy()[:, :, valid], st["score_cache"][:, :, valid],
                           rtol=2e-3, atol=1e-7)


def test_selfextend_and_plot_attn_are_refused():
    from cascading_kv_cache_b200 import CascadingKVCache
    m = _SlicingAttention.make(4, 2, 128, 5e5, "max", False, False)
    cache = CascadingKVCache(16, 4, 1, 2, 128, 64, device=DEV, dtype=torch.bfloat16, layers=1, verbose=False)
    x = torch.zeros(1, 3, 8 * 128, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        m.forward_cascade(hidden_states=x, past_key_value=cache, use_selfextend=True)
    cache.plot_attn = True
    with pytest.raises(NotImplementedError):
        m.forward_cascade(hidden_states=x, past_key_value=cache)
    with pytest.raises(ValueError):
        m.forward(x, past_key_values=object())


FLASH_SHAPES = [(1, 2, 128, 128, 64), (1, 2, 256, 256, 64), (1, 1, 128, 128 + 128, 64), (1, 2, 512, 2560, 64),
                (1, 2, 500, 2048 + 500, 64), (1, 2, 500, 2048 + 64 + 500, 64), (2, 4, 192, 1024 + 192, 128)]


@pytest.mark.parametrize("shape", FLASH_SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_functional_attention_forward(shape, dtype):
    """``attention(q, k, v, causal, sm_scale, mask, beta) -> (o, scores)``: the forward half of the
    reference's own test (cascade/models/test.py:177-269: inputs N(0, 0.5), sm_scale 0.5, a random mask over
    the cached columns, ``atol=1e-2``) plus the column scores against their definition."""
    from cascading_kv_cache_b200 import attention
    Z, H, N_CTX, N_KV, D = shape
    torch.manual_seed(20)
    q = torch.empty((Z, H, N_CTX, D), dtype=dtype, device=DEV).normal_(mean=0.0, std=0.5)
    k = torch.empty((Z, H, N_KV, D), dtype=dtype, device=DEV).normal_(mean=0.0, std=0.5)
    v = torch.empty((Z, H, N_KV, D), dtype=dtype, device=DEV).normal_(mean=0.0, std=0.5)
    if N_CTX == N_KV:
        M = torch.full((1, N_KV), 1, dtype=torch.bool, device=DEV)
        M_eager = M.repeat(N_CTX, 1).triu(1)
    else:
        M = torch.rand((1, N_KV - N_CTX), device=DEV) > 0.5
        M2 = torch.full((N_CTX, N_CTX), 1, dtype=torch.bool, device=DEV).triu(1)
        M_eager = torch.cat((M.repeat(N_CTX, 1), M2), dim=-1)
    sm_scale, beta = 0.5, 0.999
    p = torch.matmul(q.float(), k.float().transpose(2, 3)) * sm_scale
    p[:, :, M_eager == 1] = float("-inf")
    p = torch.softmax(p, dim=-1)
    ref_out = torch.matmul(p, v.float())
    out, scores = attention(q, k, v, True, sm_scale, M.squeeze(0), beta)
    assert out.shape == q.shape and scores.shape == (Z, H, N_KV) and out.dtype == dtype
    assert torch.allclose(ref_out, out.float(), atol=1e-2, rtol=0), (ref_out - out.float()).abs().max().item()
    w = (1 - beta) * beta ** torch.arange(N_CTX, device=DEV).flip(dims=(0,)).float()
    ref_scores = (p * w[None, None, :, None]).sum(dim=2)
    assert torch.allclose(ref_scores, scores.float(), rtol=2e-2, atol=1e-6), \
        (ref_scores - scores.float()).abs().max().item()
    # beta = 1 switches the scores off, as in the reference's forward test
    _, zero = attention(q, k, v, True, sm_scale, M.squeeze(0), 1.0)
    assert float(zero.abs().max()) == 0.0


def test_calc_scores_reductions():
    """calc_scores (cascade_attention.py:231-248): per KV group and over all heads, mean / max / median."""
    m = _SlicingAttention.make(6, 2, 16, 1e4, "mean", False, False)
    g = torch.Generator().manual_seed(3)
    scores = torch.rand(2, 6, 40, generator=g)
    for red, f in (("mean", lambda x, d: x.mean(d)), ("max", lambda x, d: x.amax(d)),
                   ("median", lambda x, d: x.median(d).values)):
        m.config._head_reduction = red
        ema, new = m.calc_scores(scores, False, 30, 10)
        assert torch.equal(ema, f(scores[:, :, :30].view(2, 2, 3, 30), 2)) and ema.shape == (2, 2, 30)
        assert torch.equal(new, f(scores[:, :, -10:].view(2, 2, 3, 10), 2))
        ema, new = m.calc_scores(scores, True, 30, 10)
        assert torch.equal(ema, f(scores[:, :, :30], 1).unsqueeze(1)) and new.shape == (2, 2, 10)
        assert torch.equal(new[:, 0], new[:, 1])


def test_wrong_device_is_refused_on_the_host():
    """A cache on one GPU while another is current: the mirror makes the cache's device current; a raw
    ABI call with the wrong device current is refused with CKV_E_ARG instead of faulting."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import ctypes
    from cascading_kv_cache_b200 import CascadingKVCache, cascade_attention, _lib
    cache = CascadingKVCache(16, 4, 1, 2, 128, 64, device="cuda:1", dtype=torch.bfloat16, layers=1, verbose=False)
    x = torch.randn(1, 2, 8, 128, device="cuda:1", dtype=torch.bfloat16)
    with torch.cuda.device(0):
        out = cascade_attention(x, x, x, cache, 0)          # guarded by the mirror
        assert out.device.index == 1 and cache.kernel_status() == 0
        cfg, st = cache.ckv_config(0), cache.ckv_state(0)
        rc = cache._lib.ckv_cascade_update(ctypes.byref(cfg), ctypes.byref(st), x.data_ptr(), x.data_ptr(),
                                           x.stride(0), x.stride(1), x.stride(2), None, 0, 0, 0, 8, None, 0, None)
        assert rc == -1 and b"device" in cache._lib.ckv_last_error()
