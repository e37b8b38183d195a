"""Host-side helpers for running the hot path on several GPUs of one node.

Lanes (batch, kv head) are independent, so the path needs no data-path collective: every rank owns
a slice of the batch (or, for batch 1, a slice of the KV heads with their query-head groups) and
``torch.distributed`` is used only for the barrier around the timed region and the max-over-ranks
of the measured times.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch
import torch.distributed as dist


def shard_lanes(batch: int, kv_heads: int, world_size: int, rank: int) -> Dict[str, Tuple[int, int]]:
    """Slice of the (batch, kv head) lane grid owned by ``rank``.

    Shard the batch when it has at least ``world_size`` sequences, otherwise shard the KV heads
    (each with its group of query heads).  Returns half-open ranges ``{"batch": (b0, b1),
    "kv_heads": (h0, h1)}``.  Raises when neither dimension divides evenly.
    """
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if batch % world_size == 0:
        per = batch // world_size
        return {"batch": (rank * per, (rank + 1) * per), "kv_heads": (0, kv_heads)}
    if batch == 1 and kv_heads % world_size == 0:
        per = kv_heads // world_size
        return {"batch": (0, 1), "kv_heads": (rank * per, (rank + 1) * per)}
    raise ValueError(f"cannot shard batch {batch} x kv_heads {kv_heads} over {world_size} ranks evenly")


def max_over_ranks(values: List[float], device=None) -> List[float]:
    """Element-wise maximum of ``values`` over all ranks (identity without a process group)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(values)
    t = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def gather_token_ids(ids: torch.Tensor) -> torch.Tensor:
    """All-gather of per-rank generated ids ``[n]`` into ``[world, n]`` (the only collective an
    end-to-end generation run needs)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return ids.unsqueeze(0)
    out = [torch.empty_like(ids) for _ in range(dist.get_world_size())]
    dist.all_gather(out, ids)
    return torch.stack(out)
