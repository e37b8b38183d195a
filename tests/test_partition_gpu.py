"""The multi-GPU path is a partition of independent lanes with no data-path collective: a rank that owns
sequences ``[b0, b1)`` (or KV heads ``[h0, h1)`` of a single sequence) must compute exactly what a single
GPU computes for those lanes.  Here the ranks of a world of 2 and 4 run one after the other on one device,
each on the shard ``shard_lanes`` gives it, and their results are laid beside the unpartitioned run's.

Chunked prefill works lane by lane (one CTA per query tile, lane and head pair), so its outputs and the
cache it leaves are bit-identical under any partition.  The decode kernels split the flat key stream of all
lanes over the SMs, so the grouping of a lane's partial sums changes with the number of lanes on the GPU:
outputs agree within the last bits of the 16-bit result and the caches hold the same tokens.
(Under ``homogeneous_heads`` the scores are reduced over all heads of a sequence, which is why the partition
by KV head is only offered without it; the benchmark's configurations reduce per KV group.)
"""
import pytest
import torch

from cascading_kv_cache_b200.dist_utils import shard_lanes

pytestmark = pytest.mark.gpu
D, THETA = 128, 5e5


def _cache(B, KVH, NS, W, C, rule, red="max"):
    from cascading_kv_cache_b200 import CascadingKVCache
    return CascadingKVCache(W, NS, B, KVH, D, W * C, device="cuda:0", dtype=torch.bfloat16, head_reduction=red,
                            layers=1, eager_fill=True, admission=rule, verbose=False)


def _inputs(B, H, KVH, n, steps, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda h: torch.randn(B, h, n, D, generator=g).bfloat16().cuda()
    return [(mk(H), mk(KVH), mk(KVH)) for _ in range(steps)]


def _slice(x, sh, group):
    (b0, b1), (h0, h1) = sh["batch"], sh["kv_heads"]
    return x[b0:b1, h0 * group:h1 * group].contiguous()


def _state(cache):
    return {name: getattr(cache, name)[0].clone() for name in ("key_cache", "value_cache", "score_cache", "og_pos",
                                                                 "sink_keys", "sink_values")}


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("rule", ["ema", "stride"])
def test_decode_partitioned_by_sequence(world, rule):
    """c2 / c4 style: the batch is split over the ranks; every rank populates its lanes from their global seeds."""
    from cascading_kv_cache_b200 import cascade_attention
    from cascading_kv_cache_b200.synthetic import populate_steady_state
    B, H, KVH, NS, W, C, steps = 4, 8, 2, 4, 256, 4, 6
    G = H // KVH
    steps_in = _inputs(B, H, KVH, 1, steps, seed=21)

    whole = _cache(B, KVH, NS, W, C, rule)
    populate_steady_state(whole, 0, seed=9, beta=0.999)
    outs = [cascade_attention(q, k, v, whole, 0, rope_theta=THETA) for q, k, v in steps_in]
    want = _state(whole)

    for rank in range(world):
        sh = shard_lanes(B, KVH, world, rank)
        (b0, b1), (h0, h1) = sh["batch"], sh["kv_heads"]
        mine = _cache(b1 - b0, h1 - h0, NS, W, C, rule)
        populate_steady_state(mine, 0, seed=9, beta=0.999, first_sequence=b0, first_kv_head=h0, global_kv_heads=KVH)
        for (q, k, v), full in zip(steps_in, outs):
            got = cascade_attention(_slice(q, sh, G), _slice(k, sh, 1), _slice(v, sh, 1), mine, 0, rope_theta=THETA)
            ref = _slice(full, sh, G)
            assert torch.allclose(got.float(), ref.float(), atol=2e-2, rtol=2e-2), (rank, (got.float() - ref.float()).abs().max())
        assert mine.kernel_status() == 0
        got_state = _state(mine)
        same_tokens = (got_state["og_pos"] == want["og_pos"][b0:b1, h0:h1]).float().mean().item()
        assert same_tokens >= 0.999, (rank, same_tokens)
        if same_tokens == 1.0:
            assert torch.equal(got_state["key_cache"], want["key_cache"][b0:b1, h0:h1])
            assert torch.equal(got_state["value_cache"], want["value_cache"][b0:b1, h0:h1])
        assert torch.equal(mine.pos[0], whole.pos[0][b0:b1, h0:h1])


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("rule", ["ema", "stride"])
def test_chunked_prefill_partitioned_by_kv_head(world, rule):
    """c3 style: one sequence, its KV heads (with their query heads) split over the ranks.  Bit-identical."""
    from cascading_kv_cache_b200 import cascade_attention
    B, H, KVH, NS, W, C, chunk, n_chunks = 1, 16, 4, 4, 128, 4, 200, 4
    G = H // KVH
    steps_in = _inputs(B, H, KVH, chunk, n_chunks, seed=22)

    whole = _cache(B, KVH, NS, W, C, rule, red="mean")
    outs = [cascade_attention(q, k, v, whole, 0, rope_theta=THETA) for q, k, v in steps_in]
    want = _state(whole)

    for rank in range(world):
        sh = shard_lanes(B, KVH, world, rank)
        (b0, b1), (h0, h1) = sh["batch"], sh["kv_heads"]
        mine = _cache(1, h1 - h0, NS, W, C, rule, red="mean")
        for (q, k, v), full in zip(steps_in, outs):
            got = cascade_attention(_slice(q, sh, G), _slice(k, sh, 1), _slice(v, sh, 1), mine, 0, rope_theta=THETA)
            assert torch.equal(got, _slice(full, sh, G)), rank
        assert mine.kernel_status() == 0
        for name, t in _state(mine).items():
            assert torch.equal(t, want[name][:, h0:h1]), (rank, name)
        assert mine.get_seq_length(0) == whole.get_seq_length(0)
