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

The reference's ``CascadingKVCache`` itself cannot be constructed on a CPU (its
update is a Triton kernel), so the attention vectors drive the reference
attention code through an adapter object: backed by ``CascadingKVCacheSlow`` for
the stride rule (every number then comes from reference code) and by the C
restatement in oracle/ for the score-driven rule (the attention arithmetic and
the scores are the reference's; only the slot bookkeeping is the restatement).

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


class OracleAdapter:
    """Same interface, slot bookkeeping by oracle/ (needed for the score-driven rule)."""

    def __init__(self, W, NS, B, KVH, D, S, dtype, beta, eager_fill, cascade_func="pow2"):
        from oracle.cascade_oracle import OracleCascadingKVCache
        self.c = OracleCascadingKVCache(window_length=W, num_sink_tokens=NS, max_batch_size=B, heads=KVH, dim=D,
                                        max_seq_len=S, dtype=dtype, cascade_func=cascade_func, layers=1,
                                        eager_fill=eager_fill, beta=beta)
        self.num_sink_tokens = NS
        self.window_length = W
        self.beta = beta
        self.seen_tokens_by_layer = torch.zeros(1, dtype=torch.long)

    @property
    def score_cache(self):
        return self.c.score_cache

    def get_vals(self, layer_idx):
        return self.c.get_vals(layer_idx)

    def update(self, key_states, value_states, layer_idx, score_states=None):
        self.c.update(key_states, value_states, layer_idx, score_states=score_states)
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


def gen_attention_vectors(cc, ca, ml):
    cases = {}
    specs = [
        # name, B,H,KVH,D, NS,W,C, chunk, n_chunks, n_decode, dtype, rule, reduction, homogeneous, eager_fill, beta, theta
        ("stride_f32", 1, 8, 2, 32, 4, 16, 4, 16, 12, 6, torch.float32, "stride", "max", False, False, 0.9999, 5e5),
        ("stride_bf16", 2, 4, 2, 64, 2, 8, 2, 8, 6, 4, torch.bfloat16, "stride", "mean", False, False, 0.9999, 5e5),
        ("ema_f32_max", 2, 8, 2, 32, 4, 16, 4, 16, 14, 8, torch.float32, "ema", "max", False, True, 0.999, 5e5),
        ("ema_f32_mean_h", 1, 6, 2, 16, 3, 8, 3, 5, 20, 8, torch.float32, "ema", "mean", True, True, 0.99, 1e6),
        ("ema_f32_median", 1, 8, 2, 16, 2, 8, 4, 8, 12, 5, torch.float32, "ema", "median", False, False, 0.99, 1e4),
        ("ema_bf16_max", 1, 8, 2, 64, 4, 16, 2, 16, 6, 6, torch.bfloat16, "ema", "max", False, True, 0.9999, 5e5),
    ]
    for (name, B, H, KVH, D, NS, W, C, chunk, n_chunks, n_dec, dtype, rule, red, homog, eager_fill, beta,
         theta) in specs:
        S = W * C
        g = torch.Generator().manual_seed(sum(ord(c) for c in name))
        attn = make_ref_attention(ca, ml, H, KVH, D, theta, red, homog)
        if rule == "stride":
            cache = SlowAdapter(cc, W, NS, B, KVH, D, S, dtype, beta)
        else:
            cache = OracleAdapter(W, NS, B, KVH, D, S, dtype, beta, eager_fill)
        T = chunk * n_chunks + n_dec
        hidden = torch.randn(B, T, (H + 2 * KVH) * D, generator=g).to(dtype)
        outs = []
        steps = [(i * chunk, chunk) for i in range(n_chunks)] + [(chunk * n_chunks + i, 1) for i in range(n_dec)]
        with torch.no_grad():
            for (t0, n) in steps:
                o, _, _ = attn.forward_cascade(hidden_states=hidden[:, t0:t0 + n], past_key_value=cache,
                                               use_flash=False, homogeneous_heads=homog, do_og_pos=False)
                outs.append(o.float())
        out = torch.cat(outs, dim=1)  # [B,T,H*D]
        vals = cache.get_vals(0)
        st = dict(cfg=np.array([B, H, KVH, D, NS, W, C, chunk, n_chunks, n_dec]),
                  dtype=np.array(str(dtype)), rule=np.array(rule), reduction=np.array(red),
                  homogeneous=np.array(homog), eager_fill=np.array(eager_fill), beta=np.array(beta),
                  theta=np.array(theta),
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
    ref_root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    torch.set_num_threads(1)  # fixed summation order
    cc, ca, ml = load_reference(ref_root)
    gen_update_vectors(cc)
    gen_attention_vectors(cc, ca, ml)
