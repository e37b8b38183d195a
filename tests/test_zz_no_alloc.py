"""The allocation-free entry point, ckv_attention_static, against ckv_attention.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test.

Who needs it: hosts that cannot hand the library a scratch buffer -- a serving process that fixed
its device-memory budget at start-up, or a plugin that must not touch its host's allocator.  The
entry point takes its scratch from an 8 MiB array inside the library's device image and must give
the same results as the ordinary entry point.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

B, H, KVH, D, NS, W, C = 2, 8, 2, 128, 4, 64, 4
THETA = 500000.0


def _call(cache, q, k, v, static):
    """Marshal one attention+update call through the C ABI by hand (static or ordinary entry point)."""
    from cascading_kv_cache_b200 import _lib
    lib = cache._lib
    K = q.size(2)
    out = torch.empty(B, H, K, D, device=q.device, dtype=q.dtype)
    cfg = cache.ckv_config(0, q_heads=H)
    st = cache.ckv_state(0)
    rope = cache.rope_table(THETA, NS + W * C + K + 1)
    w_cache, w_new = cache.ema_weights(K)
    common = [ctypes.byref(cfg), ctypes.byref(st), q.data_ptr(), q.stride(0), q.stride(1), q.stride(2),
              k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), k.stride(2), K, rope.data_ptr(), rope.size(0),
              w_cache.data_ptr(), w_new.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)]
    stream = _lib.current_stream_ptr(q.device)
    if static:
        rc = lib.ckv_attention_static(*common, _lib.CKV_ATTN_UPDATE, stream)
        _lib.check(rc, "ckv_attention_static")
    else:
        nbytes = lib.ckv_attention_workspace_bytes(ctypes.byref(cfg), K)
        cache.workspace(nbytes)
        rc = lib.ckv_attention(*common, cache.workspace_ptr(), nbytes, _lib.CKV_ATTN_UPDATE, stream)
        _lib.check(rc, "ckv_attention")
    cache.note_tokens_seen(0, K)
    return out


def test_static_scratch_matches_ordinary_entry_point_on_consecutive_calls():
    from cascading_kv_cache_b200 import CascadingKVCache
    dev = torch.device("cuda:0")
    make = lambda: CascadingKVCache(W, NS, B, KVH, D, W * C, device=dev, dtype=torch.bfloat16, head_reduction="max",
                                    layers=1, eager_fill=True)
    ordinary, static = make(), make()
    ordinary.beta = static.beta = 0.999
    g = torch.Generator().manual_seed(7)
    # a prefill chunk (scratch: rotated keys, row statistics, column scores), then two decode calls in
    # a row (scratch: logits, split partials, block counters, cos/sin image) -- the second call finds
    # the array as the first one left it
    for n in (300, 1, 1, 1):
        q = torch.randn(B, H, n, D, generator=g).bfloat16().to(dev)
        k = torch.randn(B, KVH, n, D, generator=g).bfloat16().to(dev)
        v = torch.randn(B, KVH, n, D, generator=g).bfloat16().to(dev)
        want = _call(ordinary, q, k, v, static=False).float()
        got = _call(static, q, k, v, static=True).float()
        err = (got - want).abs()
        rel = err.norm().item() / want.norm().item()
        assert err.max().item() <= 2e-2 and rel <= 1e-2, (n, err.max().item(), rel)
    torch.cuda.synchronize()
    # no bounded wait inside a kernel gave up: the status word of the built-in array, read without a
    # workspace pointer
    status = ctypes.c_int32(-1)
    assert static._lib.ckv_static_status(ctypes.byref(status)) == 0 and status.value == 0
    assert torch.equal(static.pos[0], ordinary.pos[0])
    assert torch.equal(static.stored_tokens[0], ordinary.stored_tokens[0])
    assert torch.equal(static.start_indices[0], ordinary.start_indices[0])
    agree = (static.og_pos[0] == ordinary.og_pos[0]).float().mean().item()
    assert agree >= 0.999, agree
    assert torch.allclose(static.score_cache[0].float(), ordinary.score_cache[0].float(), rtol=2e-2, atol=1e-8)


def test_static_scratch_refuses_what_does_not_fit():
    from cascading_kv_cache_b200 import CascadingKVCache, _lib
    dev = torch.device("cuda:0")
    big = CascadingKVCache(4096, NS, 4, 8, D, 32768, device=dev, dtype=torch.bfloat16, layers=1)
    lib = big._lib
    cfg = big.ckv_config(0, q_heads=32)
    assert lib.ckv_attention_workspace_bytes(ctypes.byref(cfg), 1) > lib.ckv_static_scratch_bytes() == 8 << 20
    st = big.ckv_state(0)
    x = torch.zeros(4, 32, 1, D, device=dev, dtype=torch.bfloat16)
    kv = torch.zeros(4, 8, 1, D, device=dev, dtype=torch.bfloat16)
    rope = big.rope_table(THETA, NS + 32768 + 2)
    rc = lib.ckv_attention_static(ctypes.byref(cfg), ctypes.byref(st), x.data_ptr(), x.stride(0), x.stride(1),
                                  x.stride(2), kv.data_ptr(), kv.data_ptr(), kv.stride(0), kv.stride(1), kv.stride(2),
                                  1, rope.data_ptr(), rope.size(0), None, None, x.data_ptr(), x.stride(0), x.stride(1),
                                  x.stride(2), 0, _lib.current_stream_ptr(dev))
    assert rc == -3
    assert b"built-in array" in lib.ckv_last_error()
