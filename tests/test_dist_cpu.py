"""World-size-2 checks of the multi-GPU host logic on CPU ranks (gloo)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cascading_kv_cache_b200.dist_utils import gather_token_ids, max_over_ranks, shard_lanes


def test_shard_lanes():
    assert shard_lanes(16, 8, 1, 0) == {"batch": (0, 16), "kv_heads": (0, 8)}
    assert shard_lanes(16, 8, 8, 3) == {"batch": (6, 8), "kv_heads": (0, 8)}
    assert shard_lanes(32, 4, 4, 3) == {"batch": (24, 32), "kv_heads": (0, 4)}
    assert shard_lanes(1, 8, 8, 5) == {"batch": (0, 1), "kv_heads": (5, 6)}
    assert shard_lanes(1, 8, 2, 1) == {"batch": (0, 1), "kv_heads": (4, 8)}
    covered = sorted(b for r in range(4) for b in range(*shard_lanes(16, 8, 4, r)["batch"]))
    assert covered == list(range(16))
    with pytest.raises(ValueError):
        shard_lanes(3, 8, 2, 0)
    with pytest.raises(ValueError):
        shard_lanes(16, 8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        times = max_over_ranks([1.0 + rank, 5.0 - rank])
        ids = gather_token_ids(torch.arange(4) + 10 * rank)
        dist.barrier()
        q.put((rank, times, ids.tolist()))
    finally:
        dist.destroy_process_group()


def test_max_over_ranks_and_gather_two_ranks():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, times, ids in results:
        assert times == [2.0, 5.0]
        assert ids == [[0, 1, 2, 3], [10, 11, 12, 13]]


def test_single_process_is_identity():
    assert max_over_ranks([3.0, 1.0]) == [3.0, 1.0]
    assert gather_token_ids(torch.arange(3)).tolist() == [[0, 1, 2]]


def _shard_worker(rank, world, port, q):
    """Each rank fills ITS share of a partitioned workload; rank 0 also fills the whole and compares."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.cascade_oracle import OracleCascadingKVCache
        from cascading_kv_cache_b200.synthetic import populate_steady_state
        B, KVH, W, C, NS, D = 4, 2, 16, 2, 2, 8
        ok = True
        # by batch (decode configurations), then by KV head (batch 1: chunked prefill)
        for (gb, split) in ((B, "batch"), (1, "kv_heads")):
            sh = shard_lanes(gb, KVH, world, rank)
            (b0, b1), (h0, h1) = sh["batch"], sh["kv_heads"]
            mine = OracleCascadingKVCache(W, NS, b1 - b0, h1 - h0, D, W * C, dtype=torch.bfloat16, layers=1)
            populate_steady_state(mine, 0, seed=9, first_sequence=b0, first_kv_head=h0, global_kv_heads=KVH)
            parts = [None] * world
            dist.all_gather_object(parts, (mine.key_cache[0], mine.score_cache[0], mine.og_pos[0]))
            if rank == 0:
                whole = OracleCascadingKVCache(W, NS, gb, KVH, D, W * C, dtype=torch.bfloat16, layers=1)
                populate_steady_state(whole, 0, seed=9)
                dim = 0 if split == "batch" else 1
                for i, name in enumerate(("key_cache", "score_cache", "og_pos")):
                    ok = ok and torch.equal(torch.cat([p[i] for p in parts], dim=dim), getattr(whole, name)[0])
        dist.barrier()
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_partitioned_workload_holds_the_single_gpu_data_two_ranks():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_shard_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok in results)
