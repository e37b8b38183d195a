"""Seeded synthetic workloads with the shapes of the benchmark configurations.

``populate_steady_state`` fills a cache object (the CUDA ``CascadingKVCache`` or any object with
the same tensor lists, e.g. the CPU oracle's) as if a long stream had already passed through it:
every slot valid, ring start indices at seeded offsets, positions from the update's own formula
(reference cascading_cache.py:112-142), original positions increasing with rank, N(0,1) keys and
values and uniform prior scores.
"""
from __future__ import annotations

import torch


def steady_state_layout(W: int, C: int, NS: int, seed: int):
    """Lane-invariant part of a full cache: start indices, positions, original positions, seen."""
    g = torch.Generator().manual_seed(seed)
    S = W * C
    start = torch.randint(0, W, (C,), generator=g, dtype=torch.long)
    stored = torch.full((C,), W, dtype=torch.long)
    j = torch.arange(W, dtype=torch.long)
    pos = torch.empty(S, dtype=torch.long)
    ub = S
    for i in range(C):
        pos[i * W:(i + 1) * W] = ((j + W - start[i]) % W) + ub - W
        ub -= W
    seen = NS + 10 * S
    og = NS + 1 + pos * 10  # strictly increasing with rank, all below `seen`
    return start, stored, pos, og, seen


def populate_steady_state(cache, layer: int = 0, seed: int = 1, beta: float = 0.9999, first_sequence: int = 0,
                          first_kv_head: int = 0, global_kv_heads: int = 0):
    """Fill ``cache`` in place (works for CUDA and CPU tensor lists alike).

    Every lane (sequence, KV head) draws its keys, values and prior scores from its own generator, seeded by
    ``seed`` and the lane's GLOBAL index.  A rank that owns sequences ``first_sequence ...`` or KV heads
    ``first_kv_head ...`` of a larger job (``global_kv_heads`` heads per sequence) therefore holds exactly the
    slice of the data that a single-GPU run holds for those lanes."""
    l = layer
    W = cache.window_length[l] if isinstance(cache.window_length, (list, tuple)) else cache.window_length
    S = cache.max_seq_len[l] if isinstance(cache.max_seq_len, (list, tuple)) else cache.max_seq_len
    C, NS = S // W, cache.num_sink_tokens
    start, stored, pos, og, seen = steady_state_layout(W, C, NS, seed)
    kc = cache.key_cache[l]
    dev, dt = kc.device, kc.dtype
    g = torch.Generator(device=dev)
    kvh_global = global_kv_heads or kc.size(1)
    sc = cache.score_cache[l]
    # lane by lane: bounds the fp32 temporaries and makes the data independent of how lanes are sharded
    for b in range(kc.size(0)):
        for h in range(kc.size(1)):
            g.manual_seed(seed * 1000003 + (first_sequence + b) * kvh_global + first_kv_head + h)
            for t in (cache.key_cache[l], cache.value_cache[l], cache.sink_keys[l], cache.sink_values[l]):
                t[b, h].copy_(torch.randn(t[b, h].shape, generator=g, device=dev, dtype=torch.float32))
            sc[b, h].copy_(torch.rand(sc[b, h].shape, generator=g, device=dev, dtype=torch.float32) * (1 - beta))

    def base(name):
        return getattr(cache, "_" + name)[l] if hasattr(cache, "_" + name) else None

    def fill(name, row):
        t = base(name)
        if t is not None:  # lane-invariant storage of the CUDA cache
            t.copy_(row.to(t.device))
        else:              # per-lane storage (CPU oracle)
            getattr(cache, name)[l][:] = row.to(dev)

    fill("stored_tokens", stored)
    fill("start_indices", start)
    fill("pos", pos)
    fill("sink_pos", torch.arange(NS, dtype=torch.long))
    fill("mask", torch.zeros(S, dtype=torch.bool))
    fill("sink_mask", torch.zeros(NS, dtype=torch.bool))
    t = base("stored_sinks")
    if t is not None:
        t.fill_(NS)
    else:
        cache.stored_sinks[l].fill_(NS)
    cache.og_pos[l][:] = og.to(dev)
    if isinstance(cache.seen_tokens_by_layer, torch.Tensor):
        cache.seen_tokens_by_layer[l] = seen
        cache._seen_host[l] = seen
        cache.invalidate_host_counters(l)   # the counters were written directly
    else:
        cache.seen_tokens_by_layer[l] = seen
    cache.beta = beta
    return seen


def decode_algorithmic_bytes(B, H, KVH, D, NS, S, esz=2, score_esz=2, ema=True):
    """Bytes one decode step must move: K and V read once, score cache read+written once (EMA rule),
    q / out / new k,v once."""
    kv = 2 * B * KVH * (S + NS) * D * esz
    sc = 2 * B * KVH * S * score_esz if ema else 0
    io = B * (2 * H + 2 * KVH) * D * esz
    return kv + sc + io


def prefill_algorithmic_flops(B, H, D, K, n_valid_keys):
    """QK^T and PV flops of one chunk: 4*B*H*D*[K*n_valid + K(K+1)/2]."""
    return 4 * B * H * D * (K * n_valid_keys + K * (K + 1) // 2)
