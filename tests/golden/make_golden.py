"""Generate the golden vectors under tests/golden/ by running the REFERENCE on CPU.

Run in a container where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own modules unmodified:

* ``CascadingKVCacheSlow`` (+ its four helper functions, attached the same way
  the reference's tests do, cascade/models/test.py:525-528) for the stride-rule
  cache state vectors, and
* ``CascadeAttention.forward_cascade`` / ``cascade_attn_eager`` / ``calc_scores``
  with ``LlamaCascadeAttention.rope`` and the forked ``LlamaRotaryEmbedding``
  for the attention vectors.

The attention vectors drive the reference attention code with a cache behind it:
``CascadingKVCacheSlow`` through a thin adapter for the stride rule, and the
reference's own ``CascadingKVCache`` for the score-driven rule (see next paragraph),
so every number in the vectors comes from reference code.

The score-driven branch of the update has no CPU implementation in the reference: it exists only
as the Triton kernel ``_update_kv_cache``.  ``gen_update_score_vectors`` therefore runs the
reference's own ``CascadingKVCache`` class on CPU tensors with that kernel's SOURCE executed by
``triton_source_shim`` (a torch stand-in for ``triton.language`` with the arithmetic of the Triton
version the reference pins), and first checks the stand-in the way the reference checks its kernel:
against ``CascadingKVCacheSlow`` on stride-rule streams (cascade/models/test.py:499-651).

Outputs are small ``.npz`` files; the tests never need the reference checkout.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def load_reference(ref_root):
    sys.path.insert(0, ref_root)
    import cascade.models.cascading_cache as cc
    import cascade.models.cascade_attention as ca
    import cascade.models.llama.modeling_llama as ml
    return cc, ca, ml


class KernelSourceLauncher:
    """Stands where the reference's ``_update_kv_cache`` JITFunction stood: ``launcher[grid](*args)`` runs
    the kernel's source once per program through the stand-in ``tl``."""

    def __init__(self, cc):
        import triton_source_shim as tss
        self.tss = tss
        self.ns, self.tl = tss.compile_kernels(
            {"_update_sink_cache": cc._update_sink_cache, "_update_positional_idx": cc._update_positional_idx,
             "_update_kv_cache_inner": cc._update_kv_cache_inner, "_update_kv_cache": cc._update_kv_cache},
            {"IDTYPE": tss.TL.int64})

    def __getitem__(self, grid):
        def run(*args, **launch_options):      # num_warps / num_stages mean nothing on a CPU
            self.tss.launch(self.ns["_update_kv_cache"], self.tl, grid, *args)
        return run


def make_reference_cache_class(cc):
    """The reference's CascadingKVCache, constructible on a CPU: its Triton kernel is replaced by the
    execution of the kernel's source, and three things of the environment are neutralised --
    ``Cache.__init__`` of the installed transformers (wants layer objects), its read-only
    ``max_batch_size`` property, and ``torch.cuda.current_device/set_device`` (no GPU here)."""
    import transformers.cache_utils as cu
    cu.Cache.__init__ = lambda self, *a, **k: None
    torch.cuda.current_device = lambda: 0
    torch.cuda.set_device = lambda d: None
    cc._update_kv_cache = KernelSourceLauncher(cc)

    class ReferenceCache(cc.CascadingKVCache):
        max_batch_size = None
        max_cache_len = None

    return ReferenceCache


def make_slow(cc, W, NS, B, H, D, S, dtype=torch.float32):
    slow = cc.CascadingKVCacheSlow(window_length=W, num_sink_tokens=NS, max_batch_size=B, heads=H, dim=D,
                                   n_layers=1, max_seq_len=S, device="cpu", dtype=dtype)
    slow.add_sinks = cc.add_sinks
    slow.append_to_cache = cc.append_to_cache
    slow.evict_from_cache = cc.evict_from_cache
    slow.overwrite_cache = cc.overwrite_cache
    return slow


def slow_state(slow, out):
    (sk, sv, spos, smask, k, v, pos, mask) = out
    return dict(
        sink_keys=sk.float().numpy().copy(), sink_values=sv.float().numpy().copy(),
        sink_pos=spos.numpy().copy(), sink_valid=(smask.reshape(-1) == 0).numpy().copy(),
        key_cache=k.float().numpy().copy(), value_cache=v.float().numpy().copy(),
        pos=pos.reshape(-1).numpy().copy(), valid=(mask.reshape(-1) == 0).numpy().copy(),
        stored_tokens=slow.stored_tokens.numpy().copy(), start_indices=slow.start_indices.numpy().copy(),
        stored_sinks=np.int64(slow.stored_sinks))


def gen_update_vectors(cc):
    """Stride-rule cache states from CascadingKVCacheSlow, fed one token at a time."""
    cases = {}
    # known-answer stream: token value == its 1-based index
    W, C, NS, N, H, D = 4, 4, 2, 60, 1, 1
    slow = make_slow(cc, W, NS, 1, H, D, W * C)
    k = (torch.arange(N, dtype=torch.float32) + 1).view(1, 1, N, 1)
    for i in range(N):
        out = slow.update(k[:, :, i:i + 1].clone(), k[:, :, i:i + 1].clone())
    st = slow_state(slow, out)
    st.update(cfg=np.array([W, C, NS, N, 1, H, D]), k=k.numpy(), v=k.numpy())
    cases["count60"] = st

    g = torch.Generator().manual_seed(1234)
    cfgs = [(2, 1, 1, 37), (2, 3, 0, 90), (4, 2, 3, 75), (4, 4, 4, 300), (8, 3, 2, 260), (8, 4, 1, 700),
            (16, 2, 5, 150), (3, 3, 2, 200), (5, 4, 0, 333), (4, 1, 2, 50), (8, 4, 4, 5), (8, 4, 4, 3),
            (32, 4, 8, 1500)]
    for n, (W, C, NS, N) in enumerate(cfgs):
        B, H, D = 2, 3, 4
        slow = make_slow(cc, W, NS, B, H, D, W * C)
        k = torch.randn(B, H, N, D, generator=g)
        v = torch.randn(B, H, N, D, generator=g)
        for i in range(N):
            out = slow.update(k[:, :, i:i + 1].clone(), v[:, :, i:i + 1].clone())
        st = slow_state(slow, out)
        st.update(cfg=np.array([W, C, NS, N, B, H, D]), k=k.numpy(), v=v.numpy())
        cases[f"rand{n}"] = st
    flat = {}
    for name, st in cases.items():
        for key, val in st.items():
            flat[f"{name}/{key}"] = val
    np.savez_compressed(os.path.join(HERE, "update_stride_slow.npz"), **flat)
    print("update vectors:", len(cases), "cases")


def reference_cache_state(c, l=0):
    return dict(key_cache=c.key_cache[l].float().numpy().copy(), value_cache=c.value_cache[l].float().numpy().copy(),
                score_cache=c.score_cache[l].float().numpy().copy(), og_pos=c.og_pos[l].numpy().copy(),
                pos=c.pos[l].numpy().copy(), mask=c.mask[l].numpy().copy(),
                sink_keys=c.sink_keys[l].float().numpy().copy(), sink_values=c.sink_values[l].float().numpy().copy(),
                sink_pos=c.sink_pos[l].numpy().copy(), sink_mask=c.sink_mask[l].numpy().copy(),
                stored_tokens=c.stored_tokens[l].numpy().copy(), start_indices=c.start_indices[l].numpy().copy(),
                stored_sinks=c.stored_sinks[l].numpy().copy(), seen=np.int64(c.seen_tokens_by_layer[l].item()))


def check_shim_like_the_reference_checks_its_kernel(cc, RefCache):
    """cascade/models/test.py:499-651 on the CPU: the kernel (here: its source under the stand-in) against
    CascadingKVCacheSlow, stride rule, token by token and in chunks."""
    g = torch.Generator().manual_seed(99)
    for (W, C, NS, N, chunk) in [(4, 4, 2, 90, 1), (8, 3, 3, 150, 7), (4, 2, 0, 40, 5), (16, 2, 5, 100, 16)]:
        B, H, D = 1, 2, 4
        S = W * C
        slow = make_slow(cc, W, NS, B, H, D, S)
        fast = RefCache(window_length=W, num_sink_tokens=NS, max_batch_size=B, heads=H, dim=D, max_seq_len=S,
                        device="cpu", dtype=torch.float32, layers=1, eager_fill=False, verbose=False)
        k = torch.randn(B, H, N, D, generator=g)
        v = torch.randn(B, H, N, D, generator=g)
        for i in range(N):
            out = slow.update(k[:, :, i:i + 1].clone(), v[:, :, i:i + 1].clone())
        for i in range(0, N, chunk):
            vals = fast.update(k[:, :, i:i + chunk], v[:, :, i:i + chunk], 0)
        (sk, sv, spos, smask, ck, cv, pos, mask) = out
        valid = (mask.reshape(-1) == 0)
        fvalid = ~vals[7][0, 0]
        assert torch.equal(valid, fvalid), (W, C, NS)
        assert torch.equal(ck[:, :, valid], vals[4][:, :, fvalid]) and torch.equal(cv[:, :, valid], vals[5][:, :, fvalid])
        assert torch.equal(pos.reshape(-1)[valid], vals[6].reshape(-1)[fvalid]), (W, C, NS)
        assert torch.equal(sk, vals[0]) and torch.equal(spos.reshape(-1), vals[2].reshape(-1))
    print("kernel source under the stand-in == CascadingKVCacheSlow on 4 stride-rule streams")


def gen_update_score_vectors(cc, RefCache):
    """Score-driven streams through the reference's CascadingKVCache (kernel source on the CPU): incoming
    scores drawn from a few levels so that ties are frequent, every dtype, eager fill on and off, calls of
    one token and of many."""
    cases = {}
    specs = [
        # W, C, NS, B, H, D, dtype, cascade_func, eager_fill, chunk lengths, score levels
        (4, 4, 2, 1, 2, 4, torch.float32, "pow2", False, [1] * 70, 4),
        (4, 4, 2, 1, 2, 4, torch.float32, "pow2", True, [7] * 12, 4),
        (8, 3, 3, 2, 2, 4, torch.bfloat16, "pow2", True, [16, 1, 1, 30, 5, 64, 1, 2], 3),
        (8, 3, 3, 2, 2, 4, torch.float16, "pow2", False, [16, 1, 1, 30, 5, 64, 1, 2], 3),
        (16, 2, 5, 1, 3, 8, torch.bfloat16, "pow2", False, [40, 40, 40, 1, 1, 1], 0),
        (4, 4, 0, 1, 2, 4, torch.float32, "pow3", False, [9] * 12, 5),
        (8, 4, 4, 1, 2, 4, torch.float32, "pow2-1", True, [33] * 5, 2),
        (8, 4, 1, 1, 2, 4, torch.bfloat16, "iplus1", False, [13] * 11, 6),
        (4, 3, 2, 1, 2, 4, torch.float16, "1-then-2", True, [3] * 30, 2),
        (8, 4, 2, 1, 2, 4, torch.float32, "pow4", False, [50, 50, 50], 0),
        (2, 4, 1, 1, 1, 2, torch.float32, "pow2", False, [1] * 60, 2),
        (32, 2, 4, 1, 2, 4, torch.bfloat16, "pow2", True, [100, 1, 1, 1, 60], 4),
    ]
    for n, (W, C, NS, B, H, D, dtype, func, eager, chunks, levels) in enumerate(specs):
        S = W * C
        g = torch.Generator().manual_seed(4000 + n)
        c = RefCache(window_length=W, num_sink_tokens=NS, max_batch_size=B, heads=H, dim=D, max_seq_len=S,
                     device="cpu", dtype=dtype, cascade_func=func, layers=1, eager_fill=eager, verbose=False)
        N = sum(chunks)
        k = torch.randn(B, H, N, D, generator=g).to(dtype)
        v = torch.randn(B, H, N, D, generator=g).to(dtype)
        if levels > 0:      # a few distinct values: admissions are decided by ties and near-ties
            s = (torch.randint(0, levels, (B, H, N), generator=g).float() / levels).to(dtype)
        else:               # continuous scores
            s = torch.rand(B, H, N, generator=g).to(dtype)
        t0 = 0
        for m in chunks:
            c.update(k[:, :, t0:t0 + m], v[:, :, t0:t0 + m], 0, score_states=s[:, :, t0:t0 + m])
            t0 += m
        st = reference_cache_state(c)
        st.update(cfg=np.array([W, C, NS, B, H, D]), dtype=np.array(str(dtype)), cascade_func=np.array(func),
                  eager_fill=np.array(eager), chunks=np.array(chunks), k=k.float().numpy(), v=v.float().numpy(),
                  s=s.float().numpy())
        cases[f"score{n}"] = st
        print(f"score{n}: W{W} C{C} NS{NS} {dtype} {func} eager={eager} tokens={N} valid={int((~c.mask[0]).sum())}")
    flat = {}
    for name, st in cases.items():
        for key, val in st.items():
            flat[f"{name}/{key}"] = val
    np.savez_compressed(os.path.join(HERE, "update_scores_kernel_source.npz"), **flat)
    print("score-driven update vectors:", len(cases), "cases")


class SlowAdapter:
    """Exposes the reference CascadingKVCacheSlow through the interface that
    forward_cascade/cascade_attn_eager use (get_vals, update, score_cache, beta,
    seen_tokens_by_layer).  Scores are ignored: this is the stride rule."""

    def __init__(self, cc, W, NS, B, KVH, D, S, dtype, beta):
        self.slow = make_slow(cc, W, NS, B, KVH, D, S, dtype)
        self.num_sink_tokens = NS
        self.window_length = W
        self.beta = beta
        self.seen_tokens_by_layer = torch.zeros(1, dtype=torch.long)
        self.score_cache = [torch.zeros(B, KVH, S, dtype=dtype)]
        self.dtype = dtype
        self.S = S

    def get_vals(self, layer_idx):
        s = self.slow
        shift = self.num_sink_tokens if int(self.seen_tokens_by_layer[0]) > self.num_sink_tokens else 0
        return (s.sink_keys, s.sink_values, s.sink_pos, (s.sink_mask != 0).view(1, 1, -1),
                s.key_cache, s.value_cache, s.pos + shift, (s.mask != 0).view(1, 1, -1),
                torch.zeros(1, 1, self.S, dtype=torch.long))

    def update(self, key_states, value_states, layer_idx, score_states=None):
        for i in range(key_states.size(2)):
            self.slow.update(key_states[:, :, i:i + 1].clone(), value_states[:, :, i:i + 1].clone())
        self.seen_tokens_by_layer[0] += key_states.size(2)
        return self.get_vals(layer_idx)


def make_ref_attention(ca, ml, H, KVH, D, theta, head_reduction, homogeneous):
    """The reference CascadeAttention with slicing stand-ins for the q/k/v/o projections."""

    class Shim(ca.CascadeAttention):
        rope = ca.LlamaCascadeAttention.rope

    m = Shim()
    m.num_heads, m.num_key_value_heads, m.num_key_value_groups, m.head_dim = H, KVH, H // KVH, D
    m.layer_idx = 0
    m.config = types.SimpleNamespace(_head_reduction=head_reduction, _homogeneous_heads=homogeneous,
                                     _do_og_pos=False)
    rot = ml.LlamaRotaryEmbedding.__new__(ml.LlamaRotaryEmbedding)
    torch.nn.Module.__init__(rot)
    rot.rope_type = "default"
    rot.attention_scaling = 1.0
    rot.register_buffer("inv_freq",
                        1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.int64).float() / D)), persistent=False)
    m.rotary_emb = rot
    hq, hk = H * D, KVH * D
    m.q_proj = lambda x: x[..., :hq]
    m.k_proj = lambda x: x[..., hq:hq + hk]
    m.v_proj = lambda x: x[..., hq + hk:]
    m.o_proj = lambda x: x
    return m


def gen_attention_vectors(cc, ca, ml, RefCache):
    cases = {}
    specs = [
        # name, B,H,KVH,D, NS,W,C, chunk, n_chunks, n_decode, dtype, rule, reduction, homogeneous, eager_fill, beta, theta
        ("stride_f32", 1, 8, 2, 32, 4, 16, 4, 16, 12, 6, torch.float32, "stride", "max", False, False, 0.9999, 5e5),
        ("stride_bf16", 2, 4, 2, 64, 2, 8, 2, 8, 6, 4, torch.bfloat16, "stride", "mean", False, False, 0.9999, 5e5),
        ("ema_f32_max", 2, 8, 2, 32, 4, 16, 4, 16, 14, 8, torch.float32, "ema", "max", False, True, 0.999, 5e5),
        ("ema_f32_mean_h", 1, 6, 2, 16, 3, 8, 3, 5, 20, 8, torch.float32, "ema", "mean", True, True, 0.99, 1e6),
        ("ema_f32_median", 1, 8, 2, 16, 2, 8, 4, 8, 12, 5, torch.float32, "ema", "median", False, False, 0.99, 1e4),
        ("ema_bf16_max", 1, 8, 2, 64, 4, 16, 2, 16, 6, 6, torch.bfloat16, "ema", "max", False, True, 0.9999, 5e5),
        # do_og_pos: cached keys are rotated at the stream index they arrived with, per lane (:141-148, :161-164)
        ("ogpos_f32_max", 2, 8, 2, 32, 4, 16, 4, 16, 14, 8, torch.float32, "ema", "max", False, True, 0.999, 5e5),
        ("ogpos_bf16_mean_h", 1, 4, 2, 64, 2, 8, 3, 8, 10, 6, torch.bfloat16, "ema", "mean", True, False, 0.99, 5e5),
    ]
    for (name, B, H, KVH, D, NS, W, C, chunk, n_chunks, n_dec, dtype, rule, red, homog, eager_fill, beta,
         theta) in specs:
        S = W * C
        g = torch.Generator().manual_seed(sum(ord(c) for c in name))
        attn = make_ref_attention(ca, ml, H, KVH, D, theta, red, homog)
        if rule == "stride":
            cache = SlowAdapter(cc, W, NS, B, KVH, D, S, dtype, beta)
        else:
            # the reference's own cache object, its update kernel's source executed on the CPU
            cache = RefCache(window_length=W, num_sink_tokens=NS, max_batch_size=B, heads=KVH, dim=D, max_seq_len=S,
                             device="cpu", dtype=dtype, head_reduction=red, layers=1, eager_fill=eager_fill,
                             verbose=False)
            cache.beta = beta
        T = chunk * n_chunks + n_dec
        hidden = torch.randn(B, T, (H + 2 * KVH) * D, generator=g).to(dtype)
        outs = []
        steps = [(i * chunk, chunk) for i in range(n_chunks)] + [(chunk * n_chunks + i, 1) for i in range(n_dec)]
        with torch.no_grad():
            for (t0, n) in steps:
                o, _, _ = attn.forward_cascade(hidden_states=hidden[:, t0:t0 + n], past_key_value=cache,
                                               use_flash=False, homogeneous_heads=homog,
                                               do_og_pos=name.startswith("ogpos"))
                outs.append(o.float())
        out = torch.cat(outs, dim=1)  # [B,T,H*D]
        vals = cache.get_vals(0)
        st = dict(cfg=np.array([B, H, KVH, D, NS, W, C, chunk, n_chunks, n_dec]),
                  dtype=np.array(str(dtype)), rule=np.array(rule), reduction=np.array(red),
                  homogeneous=np.array(homog), eager_fill=np.array(eager_fill), beta=np.array(beta),
                  theta=np.array(theta), do_og_pos=np.array(name.startswith("ogpos")),
                  hidden=hidden.float().numpy(), out=out.numpy(),
                  key_cache=vals[4].float().numpy().copy(), value_cache=vals[5].float().numpy().copy(),
                  pos=vals[6].reshape(-1).numpy().copy(), masked=vals[7].reshape(-1, S)[0].numpy().copy(),
                  score_cache=cache.score_cache[0].float().numpy().copy())
        cases[name] = st
        print(name, "out abs mean", float(out.abs().mean()))
    flat = {}
    for name, st in cases.items():
        for key, val in st.items():
            flat[f"{name}/{key}"] = val
    np.savez_compressed(os.path.join(HERE, "attention_eager_ref.npz"), **flat)
    print("attention vectors:", len(cases), "cases")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference/checkout")
    ref_root = sys.argv[1]
    sys.path.insert(0, HERE)
    torch.set_num_threads(1)  # fixed summation order
    cc, ca, ml = load_reference(ref_root)
    gen_update_vectors(cc)
    RefCache = make_reference_cache_class(cc)
    check_shim_like_the_reference_checks_its_kernel(cc, RefCache)
    gen_update_score_vectors(cc, RefCache)
    gen_attention_vectors(cc, ca, ml, RefCache)
