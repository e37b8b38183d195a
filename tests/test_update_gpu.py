"""Cache update through the C ABI on the GPU against the CPU oracle: bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle.cascade_oracle import OracleCascadingKVCache
from tests.test_oracle import UPDATE

pytestmark = pytest.mark.gpu


def assert_same_state(cache, ref, layer=0):
    l = layer
    valid = ~ref.mask[l]
    assert torch.equal(cache.mask[l].cpu(), ref.mask[l])
    assert torch.equal(cache.sink_mask[l].cpu(), ref.sink_mask[l])
    assert torch.equal(cache.stored_tokens[l].cpu(), ref.stored_tokens[l])
    assert torch.equal(cache.start_indices[l].cpu(), ref.start_indices[l])
    assert torch.equal(cache.stored_sinks[l].cpu(), ref.stored_sinks[l])
    assert torch.equal(cache.pos[l].cpu()[valid], ref.pos[l][valid])
    assert torch.equal(cache.og_pos[l].cpu()[valid], ref.og_pos[l][valid])
    svalid = ~ref.sink_mask[l]
    assert torch.equal(cache.sink_pos[l].cpu()[svalid], ref.sink_pos[l][svalid])
    # raw bits, so that -0.0 / NaN payloads would also be caught
    bits = lambda t: t.cpu().contiguous().view(torch.int16 if t.element_size() == 2 else torch.int32)
    assert torch.equal(bits(cache.key_cache[l])[valid], bits(ref.key_cache[l])[valid])
    assert torch.equal(bits(cache.value_cache[l])[valid], bits(ref.value_cache[l])[valid])
    assert torch.equal(bits(cache.score_cache[l])[valid], bits(ref.score_cache[l])[valid])
    assert torch.equal(bits(cache.sink_keys[l])[svalid], bits(ref.sink_keys[l])[svalid])
    assert torch.equal(bits(cache.sink_values[l])[svalid], bits(ref.sink_values[l])[svalid])
    assert cache.seen_tokens_by_layer[l].item() == ref.seen_tokens_by_layer[l] == cache.seen_tokens_host(l)


def make_pair(W, C, NS, B, H, D, dtype, eager_fill, cascade_func="pow2"):
    from cascading_kv_cache_b200 import CascadingKVCache
    cache = CascadingKVCache(W, NS, B, H, D, W * C, device="cuda:0", dtype=dtype, cascade_func=cascade_func,
                             layers=1, eager_fill=eager_fill)
    ref = OracleCascadingKVCache(W, NS, B, H, D, W * C, dtype=dtype, cascade_func=cascade_func, layers=1,
                                 eager_fill=eager_fill)
    return cache, ref


@pytest.mark.parametrize("name", sorted(UPDATE))
def test_golden_stride_streams(name):
    """The reference CascadingKVCacheSlow vectors, fed in ragged chunks."""
    st = UPDATE[name]
    W, C, NS, N, B, H, D = (int(x) for x in st["cfg"])
    D4 = 4  # rows must be multiples of 16 bytes: widen D=1 fixtures by repetition
    k = torch.from_numpy(st["k"]).float()
    v = torch.from_numpy(st["v"]).float()
    if D < D4:
        k, v = k.repeat(1, 1, 1, D4), v.repeat(1, 1, 1, D4)
        D = D4
    cache, ref = make_pair(W, C, NS, B, H, D, torch.float32, False)
    cache.force_serial_update = N % 2 == 1      # alternate between the two update kernels
    rng = np.random.default_rng(N)
    cuts = sorted({0, N, *rng.integers(0, N + 1, size=5).tolist()})
    for a, b in zip(cuts[:-1], cuts[1:]):
        cache.update(k[:, :, a:b].cuda(), v[:, :, a:b].cuda(), 0)
        ref.update(k[:, :, a:b], v[:, :, a:b], 0)
        assert_same_state(cache, ref)
    # and against the reference's own dump
    valid = st["valid"]
    got_k = cache.key_cache[0].cpu().numpy()
    assert np.array_equal(got_k[:, :, valid, :st["key_cache"].shape[-1]], st["key_cache"][:, :, valid])
    shift = NS if N > NS else 0
    assert np.array_equal((cache.pos[0][0, 0].cpu().numpy() + shift)[valid], st["pos"][valid])


CASES = [
    # W, C, NS, B, H, D, dtype, eager_fill, func, n_tokens, chunk
    (4, 4, 2, 1, 2, 8, torch.float32, False, "pow2", 300, 1),
    (4, 4, 2, 2, 2, 8, torch.float32, True, "pow2", 300, 7),
    (8, 4, 4, 2, 3, 16, torch.bfloat16, True, "pow2", 700, 64),
    (8, 4, 4, 2, 3, 16, torch.float16, False, "iplus1", 500, 33),
    (16, 3, 1, 1, 2, 128, torch.bfloat16, True, "pow3", 900, 100),
    (16, 4, 64, 1, 4, 128, torch.float16, False, "pow2", 1000, 1000),
    (32, 4, 4, 2, 2, 64, torch.bfloat16, False, "1-then-2", 1200, 31),
    (8, 8, 3, 1, 2, 32, torch.bfloat16, True, "pow2-1-4", 1500, 50),
    (8, 4, 0, 1, 2, 32, torch.float32, True, "pow4", 400, 9),
    (512, 4, 4, 1, 8, 128, torch.float32, False, "pow2", 5000, 512),
    (64, 4, 4, 1, 2, 128, torch.bfloat16, True, "pow2", 9000, 4500),
    (256, 4, 64, 2, 2, 128, torch.bfloat16, True, "pow2", 6000, 2048),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"W{c[0]}C{c[1]}NS{c[2]}-{str(c[6])[6:]}-{c[8]}-k{c[10]}")
@pytest.mark.parametrize("rule", ["stride", "ema"])
@pytest.mark.parametrize("path", ["parallel", "serial"])
def test_update_matches_oracle(case, rule, path):
    """Random streams; under 'ema' every token arrives with a random score and the score cache is
    perturbed between calls as the attention would, so the score-driven branch is exercised."""
    W, C, NS, B, H, D, dtype, eager_fill, func, N, chunk = case
    g = torch.Generator().manual_seed(W * 1000 + C * 100 + NS + N)
    cache, ref = make_pair(W, C, NS, B, H, D, dtype, eager_fill, func)
    cache.force_serial_update = path == "serial"
    done = 0
    while done < N:
        n = min(chunk, N - done)
        k = torch.randn(B, H, n, D, generator=g).to(dtype)
        v = torch.randn(B, H, n, D, generator=g).to(dtype)
        s = None
        if rule == "ema":
            # few distinct values so that ties (>=) are frequent
            s = (torch.randint(0, 6, (B, H + 1, n), generator=g).float() / 8).to(dtype)
            bump = (torch.randint(0, 3, (B, H, W * C), generator=g).float() / 8).to(dtype)
            ref.score_cache[0] = (ref.score_cache[0] + bump).to(dtype)
            cache.score_cache[0] = (cache.score_cache[0] + bump.cuda()).to(dtype)
        # strided input views, as the projections produce them
        kk = k.transpose(1, 2).contiguous().cuda().transpose(1, 2)
        vv = v.transpose(1, 2).contiguous().cuda().transpose(1, 2)
        cache.update(kk, vv, 0, score_states=None if s is None else s.cuda())
        ref.update(k, v, 0, score_states=s)
        done += n
        if done % (chunk * 4) == 0 or done == N:
            assert_same_state(cache, ref)
    assert_same_state(cache, ref)


def test_reset_and_reuse():
    cache, ref = make_pair(8, 2, 2, 1, 2, 8, torch.float32, True)
    k = torch.randn(1, 2, 50, 8)
    cache.update(k.cuda(), k.cuda(), 0)
    cache.reset()
    assert cache.mask[0].all() and cache.get_seq_length(0) == 0 and cache.seen_tokens_host(0) == 0
    cache.update(k.cuda(), k.cuda(), 0)
    ref.update(k, k, 0)
    assert_same_state(cache, ref)
    assert cache.get_seq_length(0) == 2 + 16


def test_update_rejects_bad_shapes():
    cache, _ = make_pair(8, 2, 2, 1, 2, 8, torch.float32, True)
    with pytest.raises(ValueError):
        cache.update(torch.zeros(1, 3, 4, 8).cuda(), torch.zeros(1, 3, 4, 8).cuda(), 0)
    with pytest.raises(ValueError):
        cache.update(torch.zeros(1, 2, 4, 8).cuda(), torch.zeros(1, 2, 4, 8).cuda(), 0,
                     score_states=torch.zeros(1, 1, 4).cuda())
    # empty chunk is a no-op
    cache.update(torch.zeros(1, 2, 0, 8).cuda(), torch.zeros(1, 2, 0, 8).cuda(), 0)
    assert cache.seen_tokens_host(0) == 0


@pytest.mark.parametrize("seed", range(16))
def test_random_configurations_and_ragged_chunks(seed):
    """Randomly drawn window / cascade / sink counts, cascade functions, dtypes and chunk lengths (from one
    token to several thousand, so that the fused, the per-cascade and the split launches all run), EMA scores
    with frequent ties: the whole state bit for bit against the oracle after every call."""
    rng = np.random.default_rng(1000 + seed)
    W = int(rng.choice([4, 8, 16, 32, 64, 128]))
    C = int(rng.integers(1, 7))
    NS = int(rng.integers(0, 7))
    B, H = int(rng.integers(1, 3)), int(rng.integers(1, 4))
    D = int(rng.choice([8, 32, 128]))
    dtype = [torch.float32, torch.float16, torch.bfloat16][int(rng.integers(0, 3))]
    eager_fill = bool(rng.integers(0, 2))
    func = str(rng.choice(["pow2", "pow2-1", "pow2-1-4", "pow2-2-4", "pow2-3-4", "1-then-2", "pow3", "pow4", "iplus1"]))
    rule = "ema" if seed % 2 else "stride"
    g = torch.Generator().manual_seed(seed)
    cache, ref = make_pair(W, C, NS, B, H, D, dtype, eager_fill, func)
    total = 0
    while total < 6000:
        n = int(rng.choice([1, 2, int(rng.integers(3, 64)), int(rng.integers(64, 1024)), int(rng.integers(1024, 4600))]))
        k = torch.randn(B, H, n, D, generator=g).to(dtype)
        v = torch.randn(B, H, n, D, generator=g).to(dtype)
        s = None
        if rule == "ema":
            s = (torch.randint(0, 5, (B, H, n), generator=g).float() / 8).to(dtype)
            bump = (torch.randint(0, 3, (B, H, W * C), generator=g).float() / 8).to(dtype)
            ref.score_cache[0] = (ref.score_cache[0] + bump).to(dtype)
            cache.score_cache[0] = (cache.score_cache[0] + bump.cuda()).to(dtype)
        cache.update(k.cuda(), v.cuda(), 0, score_states=None if s is None else s.cuda())
        ref.update(k, v, 0, score_states=s)
        total += n
        assert_same_state(cache, ref)


def _widen(t, D, Dw):
    """Rows must be multiples of 16 bytes on the GPU: repeat the fixture's few columns."""
    return t if D == Dw else t.repeat(1, 1, 1, Dw // D)


def _scored_inputs(st):
    from tests.test_oracle import _DT
    W, C, NS, B, H, D = (int(x) for x in st["cfg"])
    dtype = _DT[str(st["dtype"])]
    Dw = max(D, 16 // torch.empty(0, dtype=dtype).element_size())
    k, v, s = (torch.from_numpy(st[n]).to(dtype) for n in ("k", "v", "s"))
    return (W, C, NS, B, H, D, Dw, dtype), _widen(k, D, Dw).cuda(), _widen(v, D, Dw).cuda(), s.cuda()


def _assert_matches_reference_dump(state, st, D):
    """``state``: name -> tensor in the reference's [B,H,...] layout; ``st``: dump of the reference's cache."""
    valid = ~st["mask"].astype(bool)
    assert np.array_equal(~state["mask"].cpu().numpy().astype(bool), valid)
    for name in ("stored_tokens", "start_indices", "stored_sinks"):
        assert np.array_equal(state[name].cpu().numpy(), st[name]), name
    for name in ("key_cache", "value_cache"):
        assert np.array_equal(state[name].float().cpu().numpy()[..., :D][valid], st[name][valid]), name
    assert np.array_equal(state["score_cache"].float().cpu().numpy()[valid], st["score_cache"][valid])
    assert np.array_equal(state["og_pos"].cpu().numpy()[valid], st["og_pos"][valid])
    assert np.array_equal(state["pos"].cpu().numpy()[valid], st["pos"][valid])
    sv = ~st["sink_mask"].astype(bool)
    assert np.array_equal(state["sink_keys"].float().cpu().numpy()[..., :D][sv], st["sink_keys"][sv])
    assert np.array_equal(state["sink_pos"].cpu().numpy()[sv], st["sink_pos"][sv])


from tests.test_oracle import SCORED  # noqa: E402


@pytest.mark.parametrize("name", sorted(SCORED))
@pytest.mark.parametrize("serial", [False, True], ids=["parallel", "serial"])
def test_scored_streams_against_the_reference_kernel_source(name, serial):
    """ckv_cascade_update on streams with incoming scores (frequent ties) against state dumps of the
    reference's own CascadingKVCache, produced by executing its Triton kernel's source on a CPU."""
    from cascading_kv_cache_b200 import CascadingKVCache
    st = SCORED[name]
    (W, C, NS, B, H, D, Dw, dtype), k, v, s = _scored_inputs(st)
    cache = CascadingKVCache(W, NS, B, H, Dw, W * C, device="cuda:0", dtype=dtype, cascade_func=str(st["cascade_func"]),
                             layers=1, eager_fill=bool(st["eager_fill"]), verbose=False)
    cache.force_serial_update = serial
    t0 = 0
    for m in (int(x) for x in st["chunks"]):
        cache.update(k[:, :, t0:t0 + m], v[:, :, t0:t0 + m], 0, score_states=s[:, :, t0:t0 + m])
        t0 += m
    state = {n: getattr(cache, n)[0] for n in ("mask", "stored_tokens", "start_indices", "stored_sinks", "key_cache",
                                                "value_cache", "score_cache", "og_pos", "pos", "sink_keys", "sink_pos")}
    _assert_matches_reference_dump(state, st, D)
    assert cache.get_seq_length(0) == int(st["stored_sinks"][0, 0]) + int(st["stored_tokens"][0, 0].sum())
    assert cache.seen_tokens_host(0) == int(st["seen"])


@pytest.mark.parametrize("name", ["score2", "score6", "score11"])
@pytest.mark.parametrize("per_lane", [False, True], ids=["shared_rows", "per_lane_rows"])
def test_functional_sink_cache(name, per_lane):
    """sink_cache(...) with the reference's 23 positional arguments (cascading_cache.py:962-987): on tensors
    in the reference's own per-lane layout, and on the stride-0 views of this package's cache."""
    from cascading_kv_cache_b200 import CascadingKVCache, cascade_every_n, sink_cache
    st = SCORED[name]
    (W, C, NS, B, H, D, Dw, dtype), k, v, s = _scored_inputs(st)
    S, dev = W * C, "cuda:0"
    if per_lane:   # allocate as the reference's init_cache does (cascading_cache.py:1249-1276)
        z = lambda *shape, dt=torch.long: torch.zeros(*shape, device=dev, dtype=dt)
        t = dict(sink_keys=z(B, H, NS, Dw, dt=dtype), sink_values=z(B, H, NS, Dw, dt=dtype),
                 sink_mask=torch.ones(B, H, NS, device=dev, dtype=torch.bool), sink_pos=z(B, H, NS),
                 key_cache=z(B, H, S, Dw, dt=dtype), value_cache=z(B, H, S, Dw, dt=dtype),
                 score_cache=z(B, H, S, dt=dtype), mask=torch.ones(B, H, S, device=dev, dtype=torch.bool),
                 pos=z(B, H, S), og_pos=z(B, H, S), stored_tokens=z(B, H, C), start_indices=z(B, H, C),
                 stored_sinks=z(B, H))
        every = torch.tensor(cascade_every_n(str(st["cascade_func"]), C), device=dev)
        seen = z(1)
    else:
        cache = CascadingKVCache(W, NS, B, H, Dw, S, device=dev, dtype=dtype, cascade_func=str(st["cascade_func"]),
                                 layers=1, eager_fill=bool(st["eager_fill"]), verbose=False)
        t = {n: getattr(cache, n)[0] for n in ("sink_keys", "sink_values", "sink_mask", "sink_pos", "key_cache",
                                                "value_cache", "score_cache", "mask", "pos", "og_pos",
                                                "stored_tokens", "start_indices", "stored_sinks")}
        every, seen = cache.do_cache_every_n[0], cache.seen_tokens_by_layer
    do_cache = torch.ones(C, device=dev, dtype=torch.bool)
    t0 = 0
    for m in (int(x) for x in st["chunks"]):
        rk, rv = sink_cache(k[:, :, t0:t0 + m], v[:, :, t0:t0 + m], s[:, :, t0:t0 + m], t["sink_keys"],
                            t["sink_values"], t["sink_mask"], t["sink_pos"], t["key_cache"], t["value_cache"],
                            t["score_cache"], t["mask"], t["pos"], t["og_pos"], do_cache, every, t["stored_tokens"],
                            t["start_indices"], t["stored_sinks"], NS, W, seen[0], S, bool(st["eager_fill"]))
        assert rk.data_ptr() == k[:, :, t0:t0 + m].data_ptr()
        seen[0] += m            # the caller advances the token counter, as the reference's update() does
        t0 += m
    _assert_matches_reference_dump(t, st, D)
