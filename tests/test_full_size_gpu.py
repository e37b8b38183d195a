"""The benchmark configurations at their full sizes (reference shapes of Llama-3.1-8B / Qwen2-7B heads).

The CPU oracle cannot hold a whole batch of these, so each case combines
  * the oracle on ONE sequence of the batch, started from a copy of the GPU cache's state,
  * the tuned kernels against the generic CUDA-core path (itself checked against the oracle at
    small sizes) on the whole batch, and
  * size-independent properties of the cache state: positions of the valid slots are a
    permutation of the ranks, original positions increase with rank inside a lane, counters
    follow the score-free state machine, a call without update changes nothing.
"""
import pytest
import torch

from oracle.cascade_oracle import OracleCascadingKVCache, cascade_attention_step
from tests.test_attention_gpu import close_enough, slot_report

pytestmark = pytest.mark.gpu

C2 = dict(B=16, H=32, KVH=8, D=128, NS=64, W=8192, C=8, theta=5e5, beta=0.9999, rule="ema", red="max", seed=1)
C4 = dict(B=32, H=28, KVH=4, D=128, NS=4, W=2048, C=8, theta=1e6, beta=0.9999, rule="stride", red="max", seed=3)
C3 = dict(B=1, H=32, KVH=8, D=128, NS=4, W=8192, C=4, K=4096, theta=5e5, beta=0.9999, rule="ema", red="max", seed=2)


def _gpu_cache(w, batch=None):
    from cascading_kv_cache_b200 import CascadingKVCache
    from cascading_kv_cache_b200.synthetic import populate_steady_state
    B = batch or w["B"]
    c = CascadingKVCache(w["W"], w["NS"], B, w["KVH"], w["D"], w["W"] * w["C"], device="cuda:0", dtype=torch.bfloat16,
                         head_reduction=w["red"], layers=1, eager_fill=True, admission=w["rule"])
    populate_steady_state(c, 0, seed=w["seed"], beta=w["beta"])
    return c


def _oracle_from_gpu(cache, w, b):
    """CPU oracle holding sequence ``b`` of the GPU cache, bit for bit."""
    S = w["W"] * w["C"]
    ref = OracleCascadingKVCache(w["W"], w["NS"], 1, w["KVH"], w["D"], S, dtype=torch.bfloat16, head_reduction=w["red"],
                                 layers=1, eager_fill=True, beta=w["beta"])
    for name in ("key_cache", "value_cache", "score_cache", "sink_keys", "sink_values", "og_pos"):
        getattr(ref, name)[0].copy_(getattr(cache, name)[0][b:b + 1].cpu())
    for name in ("stored_tokens", "start_indices", "pos", "sink_pos", "mask", "sink_mask"):
        getattr(ref, name)[0][:] = getattr(cache, "_" + name)[0].cpu()
    ref.stored_sinks[0][:] = cache._stored_sinks[0].cpu()
    ref.seen_tokens_by_layer[0] = cache.seen_tokens_host(0)
    ref.beta = cache.beta
    return ref


def _oracle_from_gpu_head(cache, w, h):
    """CPU oracle holding KV head ``h`` (with its group of query heads) of a batch-1 GPU cache, bit for bit."""
    S = w["W"] * w["C"]
    ref = OracleCascadingKVCache(w["W"], w["NS"], 1, 1, w["D"], S, dtype=torch.bfloat16, head_reduction=w["red"],
                                 layers=1, eager_fill=True, beta=w["beta"])
    for name in ("key_cache", "value_cache", "score_cache", "sink_keys", "sink_values", "og_pos"):
        getattr(ref, name)[0].copy_(getattr(cache, name)[0][:1, h:h + 1].cpu())
    for name in ("stored_tokens", "start_indices", "pos", "sink_pos", "mask", "sink_mask"):
        getattr(ref, name)[0][:] = getattr(cache, "_" + name)[0].cpu()
    ref.stored_sinks[0][:] = cache._stored_sinks[0].cpu()
    ref.seen_tokens_by_layer[0] = cache.seen_tokens_host(0)
    ref.beta = cache.beta
    return ref


def _state_properties(cache, w):
    """Invariants of any reachable cache state (cascading_cache.py:729-774 for the positions)."""
    S = w["W"] * w["C"]
    mask = cache._mask[0].cpu()
    pos = cache._pos[0].cpu()
    stored = cache._stored_tokens[0].cpu()
    total = int(stored.sum())
    assert int((~mask).sum()) == total
    assert sorted(pos[~mask].tolist()) == list(range(total))          # a permutation of the ranks
    # newer tokens have higher ranks: inside every lane the original positions increase with the rank
    order = torch.argsort(pos[~mask])
    og = cache.og_pos[0].reshape(-1, S)[:, ~mask][:, order].cpu()
    assert bool((og[:, 1:] > og[:, :-1]).all())
    assert cache.kernel_status() == 0


def _decode_case(w, steps=2):
    from cascading_kv_cache_b200 import cascade_attention
    tuned, generic = _gpu_cache(w), _gpu_cache(w)
    ref = _oracle_from_gpu(tuned, w, 0)
    seen0 = tuned.seen_tokens_host(0)
    g = torch.Generator().manual_seed(100 + w["seed"])
    agree = []
    for s in range(steps):
        q = torch.randn(w["B"], w["H"], 1, w["D"], generator=g).bfloat16()
        k = torch.randn(w["B"], w["KVH"], 1, w["D"], generator=g).bfloat16()
        v = torch.randn(w["B"], w["KVH"], 1, w["D"], generator=g).bfloat16()
        # a call without update leaves the state alone, and repeating it gives the same answer up to the
        # last bit (the stream kernel merges its warps' partial sums with shared-memory float atomics,
        # whose order is not fixed; a fixed-order merge cost 8 % of the kernel's time)
        if s == 0:
            before = tuned.og_pos[0].clone(), tuned.score_cache[0].clone(), tuned._pos[0].clone()
            o1 = cascade_attention(q.cuda(), k.cuda(), v.cuda(), tuned, 0, rope_theta=w["theta"], update=False).float()
            o2 = cascade_attention(q.cuda(), k.cuda(), v.cuda(), tuned, 0, rope_theta=w["theta"], update=False).float()
            assert tuned.seen_tokens_host(0) == seen0
            assert (o1 - o2).abs().max().item() <= 2.0 ** -8 * o1.abs().max().item()
            for x, y in zip(before, (tuned.og_pos[0], tuned.score_cache[0], tuned._pos[0])):
                assert torch.equal(x, y)
        got = cascade_attention(q.cuda(), k.cuda(), v.cuda(), tuned, 0, rope_theta=w["theta"]).float().cpu()
        alt = cascade_attention(q.cuda(), k.cuda(), v.cuda(), generic, 0, rope_theta=w["theta"],
                                force_generic=True).float().cpu()
        if w["rule"] == "stride":
            want = cascade_attention_step(q[:1], k[:1], v[:1], ref, 0, w["theta"], w["red"], False, do_update=False)
            ref.update(k[:1], v[:1], 0)
        else:
            want = cascade_attention_step(q[:1], k[:1], v[:1], ref, 0, w["theta"], w["red"], False)
        ok, err = close_enough(got[:1], want.float(), True)
        assert ok, ("sequence 0 against the oracle", err)
        ok, err = close_enough(got, alt, True)
        assert ok, ("whole batch, tuned against generic", err)
        valid = ~ref.mask[0][0, 0]
        assert torch.equal(tuned._pos[0].cpu()[valid], ref.pos[0][0, 0][valid])
        assert torch.equal(tuned._stored_tokens[0].cpu(), ref.stored_tokens[0][0, 0])
        assert torch.equal(tuned._start_indices[0].cpu(), ref.start_indices[0][0, 0])
        agree.append((tuned.og_pos[0][:1].cpu()[:, :, valid] == ref.og_pos[0][:, :, valid]).float().mean().item())
        agree.append((tuned.og_pos[0] == generic.og_pos[0]).float().mean().item())
        # the admitted token is the newest entry of the first cascade in every lane
        newest = int(torch.argmax(tuned._pos[0][: w["W"]]).item())
        assert bool((tuned.og_pos[0][:, :, newest] == seen0 + s + 1).all())
    assert min(agree) >= (1.0 if w["rule"] == "stride" else 0.999), agree
    _state_properties(tuned, w)


def test_c2_llama8b_decode_full_size():
    _decode_case(C2)


def test_c4_qwen2_decode_full_size():
    _decode_case(C4)


def test_c3_chunked_prefill_full_size():
    """4096-token chunks over the full 4 x 8192 cache, all eight KV heads: tcgen05 path against the CUDA-core
    path (one head against the CPU oracle in the test above), then the state invariants."""
    from cascading_kv_cache_b200 import cascade_attention
    w = C3
    tuned, generic = _gpu_cache(w), _gpu_cache(w)
    g = torch.Generator().manual_seed(102)
    for _ in range(2):
        q = torch.randn(w["B"], w["H"], w["K"], w["D"], generator=g).bfloat16().cuda()
        k = torch.randn(w["B"], w["KVH"], w["K"], w["D"], generator=g).bfloat16().cuda()
        v = torch.randn(w["B"], w["KVH"], w["K"], w["D"], generator=g).bfloat16().cuda()
        got = cascade_attention(q, k, v, tuned, 0, rope_theta=w["theta"]).float().cpu()
        alt = cascade_attention(q, k, v, generic, 0, rope_theta=w["theta"], force_generic=True).float().cpu()
        ok, err = close_enough(got, alt, True)
        assert ok, err
        for name in ("_pos", "_mask", "_stored_tokens", "_start_indices"):
            assert torch.equal(getattr(tuned, name)[0], getattr(generic, name)[0]), name
        agree = (tuned.og_pos[0] == generic.og_pos[0]).float().mean().item()
        assert agree >= 0.999, agree
        # keep the two caches on the same trajectory: a legitimate tie flip must not carry over
        for name in ("key_cache", "value_cache", "score_cache", "og_pos"):
            getattr(generic, name)[0].copy_(getattr(tuned, name)[0])
    _state_properties(tuned, w)


@pytest.mark.parametrize("rule", ["ema", "stride"])
def test_c3_chunked_prefill_full_size_against_the_oracle(rule):
    """4096-token chunks over the full 4 x 8192 cache at the Llama-3.1-8B head shapes, FREE-RUNNING for four
    chunks, KV head 0 with its four query heads against the CPU oracle (started from a copy of the GPU
    cache): outputs within 2e-2 / 1e-2 every chunk; positions and counters equal; under the stride rule the
    slots bit for bit, under the EMA rule the same token in at least 99.9 % of the slots after every chunk,
    divergent slots reported with their two competing scores."""
    from cascading_kv_cache_b200 import cascade_attention
    w = dict(C3, rule=rule)
    G = w["H"] // w["KVH"]
    tuned = _gpu_cache(w)
    ref = _oracle_from_gpu_head(tuned, w, 0)
    g = torch.Generator().manual_seed(104)
    for chunk in range(4):
        q = torch.randn(w["B"], w["H"], w["K"], w["D"], generator=g).bfloat16()
        k = torch.randn(w["B"], w["KVH"], w["K"], w["D"], generator=g).bfloat16()
        v = torch.randn(w["B"], w["KVH"], w["K"], w["D"], generator=g).bfloat16()
        got = cascade_attention(q.cuda(), k.cuda(), v.cuda(), tuned, 0, rope_theta=w["theta"]).float().cpu()
        if rule == "stride":
            want = cascade_attention_step(q[:, :G], k[:, :1], v[:, :1], ref, 0, w["theta"], w["red"], False,
                                          do_update=False)
            ref.update(k[:, :1], v[:, :1], 0)
        else:
            want = cascade_attention_step(q[:, :G], k[:, :1], v[:, :1], ref, 0, w["theta"], w["red"], False)
        ok, err = close_enough(got[:, :G], want.float(), True)
        assert ok, (chunk, err)
        assert torch.equal(tuned._pos[0].cpu(), ref.pos[0][0, 0])
        assert torch.equal(tuned._stored_tokens[0].cpu(), ref.stored_tokens[0][0, 0])
        assert torch.equal(tuned._start_indices[0].cpu(), ref.start_indices[0][0, 0])
        og_gpu, og_ref = tuned.og_pos[0][:1, :1].cpu(), ref.og_pos[0]
        valid = ~ref.mask[0]
        if rule == "stride":
            assert torch.equal(og_gpu, og_ref)
            assert torch.equal(tuned.key_cache[0][:1, :1].cpu(), ref.key_cache[0])
            assert torch.equal(tuned.value_cache[0][:1, :1].cpu(), ref.value_cache[0])
        else:
            report = slot_report(og_gpu, og_ref, tuned.score_cache[0][:1, :1].float().cpu(),
                                 ref.score_cache[0].float(), valid)
            assert report["divergent"] <= 1e-3 * report["of"], (chunk, report)
            same = (og_gpu == og_ref) & valid
            bits = (tuned.score_cache[0][:1, :1].cpu()[same] == ref.score_cache[0][same]).float().mean().item()
            assert bits >= 0.99, (chunk, bits)
    _state_properties(tuned, w)


def test_c1_fp32_stride_stream_in_full():
    """The reference's own CPU-runnable configuration in full: fp32, B1 H32/KVH8 D128, 4 sinks, 4 x 512 slots,
    stride rule without eager fill, 16384 tokens in chunks of 512 and then 64 single steps.  Outputs against
    the oracle step by step; at the end slots, positions, counters and original positions bit for bit."""
    from cascading_kv_cache_b200 import CascadingKVCache, cascade_attention
    B, H, KVH, D, NS, W, C, theta = 1, 32, 8, 128, 4, 512, 4, 5e5
    cache = CascadingKVCache(W, NS, B, KVH, D, W * C, device="cuda:0", dtype=torch.float32, layers=1,
                             eager_fill=False, admission="stride")
    ref = OracleCascadingKVCache(W, NS, B, KVH, D, W * C, dtype=torch.float32, layers=1, eager_fill=False)
    g = torch.Generator().manual_seed(0)
    worst = 0.0
    for n in [512] * 32 + [1] * 64:
        q = torch.randn(B, H, n, D, generator=g)
        k = torch.randn(B, KVH, n, D, generator=g)
        v = torch.randn(B, KVH, n, D, generator=g)
        want = cascade_attention_step(q, k, v, ref, 0, theta, None, False, do_update=False)
        ref.update(k, v, 0)
        got = cascade_attention(q.cuda(), k.cuda(), v.cuda(), cache, 0, rope_theta=theta).cpu()
        worst = max(worst, (got - want).abs().max().item())
    assert worst <= 2e-4, worst
    valid = ~ref.mask[0]
    assert torch.equal(cache.mask[0].cpu(), ref.mask[0])
    for name in ("pos", "og_pos"):
        assert torch.equal(getattr(cache, name)[0].cpu()[valid], getattr(ref, name)[0][valid]), name
    for name in ("key_cache", "value_cache"):
        assert torch.equal(getattr(cache, name)[0].cpu()[valid], getattr(ref, name)[0][valid]), name
    for name in ("stored_tokens", "start_indices", "sink_keys", "sink_values", "sink_pos"):
        assert torch.equal(getattr(cache, name)[0].cpu(), getattr(ref, name)[0]), name
    assert cache.seen_tokens_host(0) == 16384 + 64 and cache.kernel_status() == 0


def test_c3_shapes_stride_rule_single_pass_full_size():
    """The c3 shapes under the stride rule: the single-pass tcgen05 kernel (key tiles split over two CTAs per
    query tile, partials merged by their maxima and sums) against the CUDA-core path; the cache bit for bit."""
    from cascading_kv_cache_b200 import cascade_attention
    w = dict(C3, rule="stride")
    tuned, generic = _gpu_cache(w), _gpu_cache(w)
    g = torch.Generator().manual_seed(103)
    for _ in range(2):
        q = torch.randn(w["B"], w["H"], w["K"], w["D"], generator=g).bfloat16().cuda()
        k = torch.randn(w["B"], w["KVH"], w["K"], w["D"], generator=g).bfloat16().cuda()
        v = torch.randn(w["B"], w["KVH"], w["K"], w["D"], generator=g).bfloat16().cuda()
        got = cascade_attention(q, k, v, tuned, 0, rope_theta=w["theta"]).float().cpu()
        alt = cascade_attention(q, k, v, generic, 0, rope_theta=w["theta"], force_generic=True).float().cpu()
        ok, err = close_enough(got, alt, True)
        assert ok, err
        for name in ("_pos", "_mask", "_stored_tokens", "_start_indices"):
            assert torch.equal(getattr(tuned, name)[0], getattr(generic, name)[0]), name
        for name in ("og_pos", "key_cache", "value_cache"):
            assert torch.equal(getattr(tuned, name)[0], getattr(generic, name)[0]), name
    _state_properties(tuned, w)
