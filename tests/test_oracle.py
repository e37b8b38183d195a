"""The CPU oracle against the reference-generated golden vectors (no GPU)."""
import os

import numpy as np
import pytest
import torch

from oracle.cascade_oracle import OracleCascadingKVCache, cascade_attention_step, cascade_every_n

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _cases(npz):
    names = sorted({k.split("/")[0] for k in npz.files})
    return {n: {k.split("/", 1)[1]: npz[k] for k in npz.files if k.startswith(n + "/")} for n in names}


UPDATE = _cases(np.load(os.path.join(GOLD, "update_stride_slow.npz")))
ATTN = _cases(np.load(os.path.join(GOLD, "attention_eager_ref.npz")))
SCORED = _cases(np.load(os.path.join(GOLD, "update_scores_kernel_source.npz")))


def check_against_slow(cache, st, NS):
    """Compare an oracle-layout cache with a CascadingKVCacheSlow state dump."""
    B, H = cache.max_batch_size, cache.heads
    shift = NS if cache.seen_tokens_by_layer[0] > NS else 0
    for b in range(B):
        for h in range(H):
            valid = ~cache.mask[0][b, h].numpy()
            assert np.array_equal(valid, st["valid"])
            assert np.array_equal(cache.key_cache[0][b, h].float().numpy()[valid], st["key_cache"][b, h][valid])
            assert np.array_equal(cache.value_cache[0][b, h].float().numpy()[valid], st["value_cache"][b, h][valid])
            assert np.array_equal((cache.pos[0][b, h].numpy() + shift)[valid], st["pos"][valid])
            assert np.array_equal(cache.stored_tokens[0][b, h].numpy(), st["stored_tokens"])
            assert np.array_equal(cache.start_indices[0][b, h].numpy(), st["start_indices"])
            assert int(cache.stored_sinks[0][b, h]) == int(st["stored_sinks"])
            sv = ~cache.sink_mask[0][b, h].numpy()
            assert np.array_equal(sv, st["sink_valid"])
            assert np.array_equal(cache.sink_keys[0][b, h].float().numpy()[sv], st["sink_keys"][b, h][sv])
            assert np.array_equal(cache.sink_values[0][b, h].float().numpy()[sv], st["sink_values"][b, h][sv])
            assert np.array_equal(cache.sink_pos[0][b, h].numpy()[sv], st["sink_pos"].reshape(-1)[sv])
            # every valid slot records the 1-based index of the token it holds
            og = cache.og_pos[0][b, h].numpy()[valid]
            assert np.array_equal(cache.key_cache[0][b, h].float().numpy()[valid], st["k"][b, h][og - 1])


@pytest.mark.parametrize("name", sorted(UPDATE))
@pytest.mark.parametrize("mode", ["token", "one_call", "ragged"])
def test_update_oracle_matches_reference_slow_cache(name, mode):
    st = UPDATE[name]
    W, C, NS, N, B, H, D = (int(x) for x in st["cfg"])
    cache = OracleCascadingKVCache(window_length=W, num_sink_tokens=NS, max_batch_size=B, heads=H, dim=D,
                                   max_seq_len=W * C, dtype=torch.float32, layers=1, eager_fill=False)
    k, v = torch.from_numpy(st["k"]), torch.from_numpy(st["v"])
    if mode == "token":
        cuts = list(range(N + 1))
    elif mode == "one_call":
        cuts = [0, N]
    else:
        rng = np.random.default_rng(N)
        cuts = sorted({0, N, *rng.integers(0, N + 1, size=6).tolist()})
    for a, b in zip(cuts[:-1], cuts[1:]):
        cache.update(k[:, :, a:b], v[:, :, a:b], 0)
    check_against_slow(cache, st, NS)


_DT = {"torch.float32": torch.float32, "torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16}


def check_against_reference_cache(cache, st):
    """Compare an oracle-layout cache, bit for bit, with a state dump of the reference's own
    CascadingKVCache (whose update kernel's source produced the dump)."""
    valid = ~st["mask"].astype(bool)
    assert np.array_equal(~cache.mask[0].numpy(), valid)
    assert np.array_equal(~cache.sink_mask[0].numpy(), ~st["sink_mask"].astype(bool))
    for name in ("stored_tokens", "start_indices", "stored_sinks"):
        assert np.array_equal(getattr(cache, name)[0].numpy(), st[name]), name
    assert cache.seen_tokens_by_layer[0] == int(st["seen"])
    # what a masked slot holds is undefined in both; everything else must be the same bits
    for name in ("key_cache", "value_cache"):
        assert np.array_equal(getattr(cache, name)[0].float().numpy()[valid], st[name][valid]), name
    assert np.array_equal(cache.score_cache[0].float().numpy()[valid], st["score_cache"][valid])
    assert np.array_equal(cache.og_pos[0].numpy()[valid], st["og_pos"][valid])
    assert np.array_equal(cache.pos[0].numpy()[valid], st["pos"][valid])
    sv = ~st["sink_mask"].astype(bool)
    assert np.array_equal(cache.sink_keys[0].float().numpy()[sv], st["sink_keys"][sv])
    assert np.array_equal(cache.sink_values[0].float().numpy()[sv], st["sink_values"][sv])
    assert np.array_equal(cache.sink_pos[0].numpy()[sv], st["sink_pos"][sv])


def run_scored_case(st, make_cache, mode):
    W, C, NS, B, H, D = (int(x) for x in st["cfg"])
    dtype = _DT[str(st["dtype"])]
    cache = make_cache(W, NS, B, H, D, W * C, dtype, str(st["cascade_func"]), bool(st["eager_fill"]))
    k, v, s = (torch.from_numpy(st[n]).to(dtype) for n in ("k", "v", "s"))
    chunks = [int(x) for x in st["chunks"]] if mode == "same_calls" else [1] * k.size(2)
    t0 = 0
    for m in chunks:
        cache.update(k[:, :, t0:t0 + m], v[:, :, t0:t0 + m], 0, score_states=s[:, :, t0:t0 + m])
        t0 += m
    return cache


@pytest.mark.parametrize("name", sorted(SCORED))
@pytest.mark.parametrize("mode", ["same_calls", "token"])
def test_update_oracle_matches_reference_kernel_source_on_scored_streams(name, mode):
    """The score-driven branch (an evictee competes with the newest slot of the next cascade,
    cascading_cache.py:667-726) pinned to the reference's own kernel: streams with frequent score ties,
    all dtypes, eager fill on and off, calls of one and of many tokens."""
    st = SCORED[name]
    make = lambda W, NS, B, H, D, S, dtype, func, eager: OracleCascadingKVCache(
        window_length=W, num_sink_tokens=NS, max_batch_size=B, heads=H, dim=D, max_seq_len=S, dtype=dtype,
        cascade_func=func, layers=1, eager_fill=eager)
    cache = run_scored_case(st, make, mode)
    check_against_reference_cache(cache, st)


def test_known_answer_stream():
    """60 tokens whose value is their index, W=4 C=4 NS=2, stride rule (reference CascadingKVCacheSlow output)."""
    st = UPDATE["count60"]
    cache = OracleCascadingKVCache(window_length=4, num_sink_tokens=2, max_batch_size=1, heads=1, dim=1,
                                   max_seq_len=16, dtype=torch.float32, layers=1, eager_fill=False)
    k = torch.from_numpy(st["k"])
    cache.update(k, k, 0)
    assert cache.key_cache[0].reshape(-1).tolist() == [59, 60, 57, 58, 52, 54, 56, 50, 38, 42, 46, 48, 34, 14, 22, 30]
    assert (cache.pos[0].reshape(-1) + 2).tolist() == [16, 17, 14, 15, 11, 12, 13, 10, 6, 7, 8, 9, 5, 2, 3, 4]
    assert cache.stored_tokens[0].reshape(-1).tolist() == [4, 4, 4, 4]
    assert cache.start_indices[0].reshape(-1).tolist() == [2, 3, 0, 1]
    assert cache.sink_keys[0].reshape(-1).tolist() == [1, 2]
    assert cache.og_pos[0].reshape(-1).tolist() == cache.key_cache[0].reshape(-1).long().tolist()


def test_eager_fill_equals_sliding_window_until_full():
    """While the cache first fills, every cascade accepts every token (cascading_cache.py:440-445;
    reference test_eager_add_same_as_one_cascade): after NS + S tokens the cache holds the last S tokens."""
    W, C, NS, D = 8, 4, 3, 2
    S = W * C
    k = (torch.arange(NS + S, dtype=torch.float32) + 1).view(1, 1, -1, 1).repeat(1, 2, 1, D)
    multi = OracleCascadingKVCache(W, NS, 1, 2, D, S, torch.float32, layers=1, eager_fill=True)
    single = OracleCascadingKVCache(S, NS, 1, 2, D, S, torch.float32, layers=1, eager_fill=True)
    multi.update(k, k, 0)
    single.update(k, k, 0)
    a = sorted(multi.key_cache[0][0, 0, :, 0].tolist())
    assert a == sorted(single.key_cache[0][0, 0, :, 0].tolist()) == list(range(NS + 1, NS + S + 1))
    assert not multi.mask[0].any()


def test_cascade_functions():
    assert cascade_every_n("pow2", 4) == [1, 2, 4, 8]
    assert cascade_every_n("pow2-1", 4) == [1, 1, 1, 8]
    assert cascade_every_n("pow2-1-4", 8) == [1, 1, 1, 1, 1, 1, 64, 128]
    assert cascade_every_n("pow2-2-4", 4) == [1, 1, 4, 8]
    assert cascade_every_n("pow2-3-4", 4) == [1, 2, 4, 8]
    assert cascade_every_n("1-then-2", 3) == [1, 2, 2]
    assert cascade_every_n("pow3", 3) == [1, 3, 9]
    assert cascade_every_n("pow4", 3) == [1, 4, 16]
    assert cascade_every_n("iplus1", 3) == [1, 2, 3]
    with pytest.raises(ValueError):
        cascade_every_n("nope", 3)


def run_attention_case(st, step_fn, make_cache):
    B, H, KVH, D, NS, W, C, chunk, n_chunks, n_dec = (int(x) for x in st["cfg"])
    dtype = _DT[str(st["dtype"])]
    rule, red = str(st["rule"]), str(st["reduction"])
    homog, eager_fill = bool(st["homogeneous"]), bool(st["eager_fill"])
    beta, theta = float(st["beta"]), float(st["theta"])
    cache = make_cache(W, NS, B, KVH, D, W * C, dtype, red, eager_fill, beta)
    hidden = torch.from_numpy(st["hidden"]).to(dtype)
    og = bool(st["do_og_pos"])
    hq, hk = H * D, KVH * D
    outs = []
    steps = [(i * chunk, chunk) for i in range(n_chunks)] + [(chunk * n_chunks + i, 1) for i in range(n_dec)]
    for (t0, n) in steps:
        x = hidden[:, t0:t0 + n]
        q = x[..., :hq].view(B, n, H, D).transpose(1, 2)
        k = x[..., hq:hq + hk].view(B, n, KVH, D).transpose(1, 2)
        v = x[..., hq + hk:].view(B, n, KVH, D).transpose(1, 2)
        o = step_fn(q, k, v, cache, theta, red, homog, rule, **({"do_og_pos": True} if og else {}))
        outs.append(o.transpose(1, 2).reshape(B, n, H * D).float().cpu())
    return torch.cat(outs, dim=1), cache


def _oracle_step(q, k, v, cache, theta, red, homog, rule, do_og_pos=False):
    if rule == "stride":
        out = cascade_attention_step(q, k, v, cache, 0, theta, red, homog, do_update=False, do_og_pos=do_og_pos)
        cache.update(k, v, 0)
        return out
    return cascade_attention_step(q, k, v, cache, 0, theta, red, homog, do_og_pos=do_og_pos)


def _oracle_cache(W, NS, B, KVH, D, S, dtype, red, eager_fill, beta):
    return OracleCascadingKVCache(W, NS, B, KVH, D, S, dtype, head_reduction=red, layers=1,
                                  eager_fill=eager_fill, beta=beta)


@pytest.mark.parametrize("name", sorted(ATTN))
def test_attention_oracle_matches_reference_eager(name):
    st = ATTN[name]
    torch.set_num_threads(1)
    out, cache = run_attention_case(st, _oracle_step, _oracle_cache)
    ref = torch.from_numpy(st["out"])
    is_bf16 = "bfloat16" in str(st["dtype"])
    # same torch ops in the same order as the reference: only thread-count / BLAS blocking may differ
    tol = 2e-2 if is_bf16 else 2e-5
    assert (out - ref).abs().max().item() <= tol
    valid = ~cache.mask[0][0, 0].numpy()
    assert np.array_equal(valid, ~st["masked"].astype(bool))
    shift = cache.num_sink_tokens
    assert np.array_equal((cache.pos[0][0, 0].numpy() + shift)[valid], st["pos"][valid])
    if not is_bf16:
        assert np.allclose(cache.key_cache[0].numpy()[:, :, valid], st["key_cache"][:, :, valid])
        if str(st["rule"]) == "ema":
            assert np.allclose(cache.score_cache[0].numpy()[:, :, valid], st["score_cache"][:, :, valid],
                               rtol=1e-4, atol=1e-7)
