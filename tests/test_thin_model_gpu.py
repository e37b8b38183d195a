"""The thin decoder stack and the strided-prefill generation loop (the end-to-end configuration) on the GPU.

* chunked == one-shot: with one cascade and a sequence that fits the window, feeding the prompt in strides
  through the cascading cache gives the logits of a single dense pass (the reference's own check,
  cascade/models/test.py:123-170: ``atol=1e-1``, equal argmax), for the Llama and the Qwen2 variant;
* the whole stack against a torch-CPU replica of itself whose attention is the CPU oracle;
* ``generate``: the greedy tokens of the GPU model equal those of the CPU replica.
"""
import pytest
import torch

from oracle.cascade_oracle import OracleCascadingKVCache, cascade_attention_step

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tiny(family, dtype, cascades=1, window=1024, sinks=4, stride=128, layers=2, head_reduction="max"):
    from cascading_kv_cache_b200.thin_model import CascadeForCausalLM, cascade_config
    cfg = cascade_config(family, hidden_size=256, intermediate_size=512, num_hidden_layers=layers,
                         num_attention_heads=2, num_key_value_heads=1, vocab_size=512,
                         rope_theta=500000.0 if family == "llama" else 1000000.0, sinks=sinks, cascades=cascades,
                         window=window, cascade_stride=stride, head_reduction=head_reduction)
    model = CascadeForCausalLM(cfg, family).to(device=DEV, dtype=dtype).eval()
    model.init_weights(seed=4, std=0.05)
    if family == "qwen2":       # exercise the q/k/v biases
        with torch.no_grad():
            for lyr in model.model.layers:
                for name in ("q_proj", "k_proj", "v_proj"):
                    getattr(lyr.self_attn, name).bias.normal_(std=0.1)
    return model, cfg


@pytest.mark.parametrize("family", ["llama", "qwen2"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_chunked_prefill_equals_one_dense_pass(family, dtype):
    from cascading_kv_cache_b200.thin_model import get_cache
    model, cfg = _tiny(family, dtype)
    cache = get_cache(model, eager_fill=False)
    g = torch.Generator().manual_seed(1)
    inputs = torch.randint(0, cfg.vocab_size, (1, 1024 - (128 - 92)), generator=g).to(DEV)
    with torch.no_grad():
        chunked = []
        for i in range(0, inputs.size(1), cfg._cascade_stride):
            chunked.append(model(inputs[:, i:i + cfg._cascade_stride], past_key_values=cache).logits.float())
        cache.reset(verbose=False)
        dense = model(inputs, past_key_values=cache).logits.float()
    for c, d in zip(chunked, torch.split(dense, cfg._cascade_stride, dim=1)):
        assert torch.allclose(c, d, atol=1e-1, rtol=0), (c - d).abs().max().item()
        # 16-bit logits of a random model tie now and then: equal argmax wherever the top two are apart
        top2 = d.topk(2, dim=-1).values
        clear = (top2[..., 0] - top2[..., 1]) > (2e-2 if dtype == torch.bfloat16 else 1e-4)
        assert bool((c.argmax(-1) == d.argmax(-1))[clear].all())
    assert cache.kernel_status() == 0


def _cpu_replica_forward(model, ids, ref, theta, num_logits_to_keep=0):
    """The same weights on the CPU: embedding, RMSNorm, projections, the ORACLE's attention per layer, SwiGLU."""
    sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    cfg = model.config
    H, KVH = cfg.num_attention_heads, cfg.num_key_value_heads
    D = cfg.hidden_size // H
    lin = lambda x, name: torch.nn.functional.linear(x, sd[name + ".weight"], sd.get(name + ".bias"))

    def norm(x, w):
        dt = x.dtype
        x = x.float()
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps)
        return w * x.to(dt)

    x = torch.nn.functional.embedding(ids.cpu(), sd["model.embed_tokens.weight"])
    B, n = ids.shape
    for l in range(cfg.num_hidden_layers):
        pre = f"model.layers.{l}."
        h = norm(x, sd[pre + "input_layernorm.weight"])
        q = lin(h, pre + "self_attn.q_proj").view(B, n, H, D).transpose(1, 2)
        k = lin(h, pre + "self_attn.k_proj").view(B, n, KVH, D).transpose(1, 2)
        v = lin(h, pre + "self_attn.v_proj").view(B, n, KVH, D).transpose(1, 2)
        o = cascade_attention_step(q, k, v, ref, l, theta, cfg._head_reduction, cfg._homogeneous_heads)
        x = x + lin(o.transpose(1, 2).reshape(B, n, H * D), pre + "self_attn.o_proj")
        h = norm(x, sd[pre + "post_attention_layernorm.weight"])
        x = x + lin(torch.nn.functional.silu(lin(h, pre + "mlp.gate_proj")) * lin(h, pre + "mlp.up_proj"),
                    pre + "mlp.down_proj")
    x = norm(x, sd["model.norm.weight"])
    if num_logits_to_keep:
        x = x[:, -num_logits_to_keep:]
    return lin(x, "lm_head")


def _oracle_cache_for(cfg, dtype, eager_fill=True):
    ref = OracleCascadingKVCache(cfg._window // cfg._cascades, cfg._sinks, cfg._batch_size, cfg.num_key_value_heads,
                                 cfg.hidden_size // cfg.num_attention_heads, cfg._window, dtype=dtype,
                                 cascade_func=cfg._cascade_func, head_reduction=cfg._head_reduction,
                                 layers=cfg.num_hidden_layers, eager_fill=eager_fill)
    return ref


@pytest.mark.parametrize("family,dtype", [("llama", torch.float32), ("qwen2", torch.float32), ("llama", torch.bfloat16)],
                         ids=["llama-fp32", "qwen2-fp32", "llama-bf16"])
def test_stack_and_generation_against_cpu_replica(family, dtype):
    """Four cascades of 32 slots, a 150-token prompt in strides of 48 (the cache overflows and admits by EMA
    score on every layer), then 12 greedy tokens."""
    from cascading_kv_cache_b200.thin_model import get_cache
    model, cfg = _tiny(family, dtype, cascades=4, window=128, sinks=4, stride=48, layers=3)
    theta = 500000.0 if family == "llama" else 1000000.0
    cache, ref = get_cache(model), _oracle_cache_for(cfg, dtype)
    cache.beta = ref.beta = 0.999
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab_size, (1, 150), generator=g)
    tol = 2e-3 if dtype == torch.float32 else 1.5e-1
    with torch.no_grad():
        for i in range(0, 150, 48):
            got = model(prompt[:, i:i + 48].to(DEV), past_key_values=cache).logits.float().cpu()
            want = _cpu_replica_forward(model, prompt[:, i:i + 48], ref, theta).float()
            assert (got - want).abs().max().item() <= tol, (i, (got - want).abs().max().item())
    assert cache.kernel_status() == 0
    for l in range(cfg.num_hidden_layers):
        valid = ~ref.mask[l]
        assert torch.equal(cache.pos[l].cpu()[valid], ref.pos[l][valid])
        if dtype == torch.float32:
            agree = (cache.og_pos[l].cpu()[valid] == ref.og_pos[l][valid]).float().mean().item()
            assert agree >= 0.999, (l, agree)
    assert cache.get_seq_length() == cfg._sinks + cfg._window
    if dtype != torch.float32:
        return
    # generation: the same greedy continuation as the CPU replica
    cache.reset(verbose=False)
    ref.reset()
    cache.beta = ref.beta = 0.999
    out = model.generate(prompt.to(DEV), cache, max_new_tokens=12)
    assert out.shape == (1, 162) and torch.equal(out[:, :150].cpu(), prompt)
    ids = prompt.clone()
    with torch.no_grad():
        for i in range(0, 150, 48):
            logits = _cpu_replica_forward(model, ids[:, i:i + 48], ref, theta, 1)
        for _ in range(12):
            nxt = logits[:, -1].argmax(-1)
            ids = torch.cat([ids, nxt[:, None]], dim=-1)
            logits = _cpu_replica_forward(model, ids[:, -1:], ref, theta, 1)
    assert torch.equal(out.cpu(), ids), (out.cpu()[0, 150:].tolist(), ids[0, 150:].tolist())
    for lyr in model.model.layers:
        assert lyr.self_attn.last_it is True        # raised for the prompt's final stride, as the reference does


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("shape", [(2, 7, 4096), (5, 256), (1, 1, 14336)])
def test_fused_layer_operators_against_torch(dtype, shape):
    """``ckv_add_rmsnorm`` and ``ckv_silu_mul`` against the sequence of torch operations they replace
    (modeling_llama.py:113-127, :282-313 of the reference): the residual sum is the same bits, the normalised
    rows agree except where the block's summation order moves the variance by an fp32 ulp, the gate is the same
    arithmetic."""
    from cascading_kv_cache_b200.thin_model import add_rmsnorm, silu_mul
    g = torch.Generator().manual_seed(shape[-1])
    x = (torch.randn(shape, generator=g) * 1.5).to(dtype).to(DEV)
    r = torch.randn(shape, generator=g).to(dtype).to(DEV)
    w = (1 + 0.1 * torch.randn(shape[-1], generator=g)).to(dtype).to(DEV)
    eps = 1e-5

    def torch_norm(s):
        h = s.float()
        h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
        return w * h.to(dtype)

    for residual in (r, None):
        normed, s = add_rmsnorm(x, residual, w, eps)
        want_s = x if residual is None else residual + x
        assert torch.equal(s, want_s)
        want = torch_norm(want_s)
        assert torch.allclose(normed.float(), want.float(), rtol=2 ** -7 if dtype == torch.bfloat16 else 2 ** -10, atol=1e-6)
        assert (normed == want).float().mean().item() >= 0.99
    got = silu_mul(x, r)
    want = torch.nn.functional.silu(x) * r
    assert torch.allclose(got.float(), want.float(), rtol=2 ** -7 if dtype == torch.bfloat16 else 2 ** -10, atol=1e-6)
    assert (got == want).float().mean().item() >= 0.999


@pytest.mark.parametrize("family", ["llama", "qwen2"])
def test_fused_projections_give_the_same_model(family):
    """``fuse_projections``: q|k|v and gate|up as one weight each.  The parameters keep their names and values, the
    logits of a chunked prefill + decode agree with the separate projections (the library GEMM may pick another
    kernel for the wider weight: 16-bit tolerance), and the caches hold the same tokens."""
    from cascading_kv_cache_b200.thin_model import get_cache
    model, cfg = _tiny(family, torch.bfloat16, cascades=4, window=128, sinks=4, stride=48, layers=2)
    before = {k: v.clone() for k, v in model.state_dict().items()}
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size, (1, 150), generator=g).to(DEV)

    def run():
        cache = get_cache(model)
        cache.beta = 0.999
        outs = []
        with torch.no_grad():
            for i in range(0, 150, 48):
                outs.append(model(ids[:, i:i + 48], past_key_values=cache).logits.float())
            for t in range(3):
                outs.append(model(ids[:, t:t + 1], past_key_values=cache).logits.float())
        assert cache.kernel_status() == 0
        return outs, [cache.og_pos[l].clone() for l in range(cfg.num_hidden_layers)]

    want, want_pos = run()
    model.fuse_projections()
    after = model.state_dict()
    assert set(after) == set(before) and all(torch.equal(after[k], before[k]) for k in before)
    lyr = model.model.layers[0]
    assert lyr.self_attn.q_proj.weight.data_ptr() == lyr.self_attn._qkv_weight.data_ptr()       # views, not copies
    got, got_pos = run()
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=1e-1, rtol=0), (a - b).abs().max().item()
    agree = sum((p == q).float().mean().item() for p, q in zip(got_pos, want_pos)) / len(want_pos)
    assert agree >= 0.99, agree
