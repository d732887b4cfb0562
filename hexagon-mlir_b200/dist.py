"""Multi-GPU partitioning: one process per GPU, independent shards, one all-gather of outputs.

The reference has no multi-device path; its only parallelism is rows spread over SPMD programs
(``row = pid + j * num_programs``, test/python/triton/test_softmax.py:52-62).  Here the same
independence is used across GPUs: contiguous row blocks (softmax, LayerNorm, matmul M dimension),
(batch, head) pairs (attention) or sequences (decoder).  No kernel reads a peer's memory; the only
exchange is an all-gather of output shards through torch.distributed (NCCL over NVLink on GPUs,
gloo on CPU for tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous block partition of ``n`` units: returns (start, count) for ``rank``.

    The first ``n % world_size`` ranks get one extra unit, so counts differ by at most one and
    every unit is owned exactly once (also when n < world_size: trailing ranks get count 0).
    """
    if world_size <= 0 or not 0 <= rank < world_size or n < 0:
        raise ValueError("bad partition request")
    base, extra = divmod(n, world_size)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def shard_rows(t: torch.Tensor, world_size: int, rank: int) -> torch.Tensor:
    """The rank's block of dimension 0 (a view)."""
    s, c = shard_range(t.shape[0], world_size, rank)
    return t[s:s + c]


def all_gather_rows(local: torch.Tensor, total_rows: int, group=None) -> torch.Tensor:
    """Gathers dimension-0 shards made by ``shard_range`` into the full tensor on every rank.

    Ragged shards (total_rows not divisible by the world size) are padded to the largest shard for
    the collective and trimmed afterwards.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    counts = [shard_range(total_rows, world, r)[1] for r in range(world)]
    if local.shape[0] != counts[rank]:
        raise ValueError(f"rank {rank}: shard has {local.shape[0]} rows, partition says {counts[rank]}")
    mx = max(counts)
    if mx == 0:
        return local.new_empty((0,) + tuple(local.shape[1:]))
    if all(c == mx for c in counts):
        out = local.new_empty((world * mx,) + tuple(local.shape[1:]))
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = local.new_zeros((mx,) + tuple(local.shape[1:]))
    padded[: local.shape[0]] = local
    buf = local.new_empty((world * mx,) + tuple(local.shape[1:]))
    dist.all_gather_into_tensor(buf, padded, group=group)
    return torch.cat([buf[r * mx: r * mx + counts[r]] for r in range(world)], dim=0)
