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


# ------------------------------------------------------------------ the five configurations, partitioned
# name -> (unit, operands cut along their leading units, operands every rank holds whole).
# Attention tensors [Z, H, N, D] are cut in (batch, head) pairs, i.e. along dimension 0 of their
# [Z*H, N, D] view; everything else is cut along dimension 0 as stored.
PARTITIONS = {
    "softmax": ("row", ("x",), ()),
    "layernorm": ("row", ("x",), ("weight", "bias")),
    "gemm": ("row of A", ("a",), ("b",)),
    "attention": ("(batch, head) pair", ("q", "k", "v"), ()),
    "decoder": ("sequence", ("x",), ("weights",)),
}


def units_view(name: str, t: torch.Tensor) -> torch.Tensor:
    """The tensor with its partition units along dimension 0."""
    if name == "attention":
        if t.dim() != 4:
            raise ValueError("attention operands are [Z, H, N, D]")
        return t.reshape(t.shape[0] * t.shape[1], t.shape[2], t.shape[3])
    return t


def partition(name: str, inputs: dict, world_size: int, rank: int) -> dict:
    """The operands rank ``rank`` works on: its block of every cut operand (a view, no copy),
    the replicated operands untouched.  ``inputs`` maps operand names of PARTITIONS[name] to tensors."""
    _, cut, whole = PARTITIONS[name]
    missing = [k for k in cut + whole if k not in inputs]
    if missing:
        raise KeyError(f"{name}: missing operands {missing}")
    out = {k: inputs[k] for k in whole}
    for k in cut:
        out[k] = shard_rows(units_view(name, inputs[k]), world_size, rank)
    return out


def units_of(name: str, inputs: dict) -> int:
    """Number of independent units (rows, (batch, head) pairs, sequences) in the whole problem."""
    return units_view(name, inputs[PARTITIONS[name][1][0]]).shape[0]


def run_partitioned(name: str, inputs: dict, compute, world_size: int, rank: int, group=None, gather: bool = True):
    """Shard -> compute -> gather for one configuration.

    ``compute(**local_operands)`` returns the rank's block of the output with the units along
    dimension 0 (for attention: [pairs, N, D]).  With ``gather`` the blocks of all ranks are
    all-gathered and every rank returns the whole output; otherwise the local block is returned.
    The benchmark's multi-GPU leg and the two-rank CPU test both go through this function.
    """
    local = partition(name, inputs, world_size, rank)
    y_local = compute(**local)
    total = units_of(name, inputs)
    want = shard_range(total, world_size, rank)[1]
    if y_local.shape[0] != want:
        raise ValueError(f"{name}: compute returned {y_local.shape[0]} units, the partition gives rank {rank} {want}")
    if not gather:
        return y_local
    y = all_gather_rows(y_local, total, group=group)
    if name == "attention":
        q = inputs["q"]
        y = y.reshape(q.shape[0], q.shape[1], y.shape[1], y.shape[2])
    return y


def sample_units(total: int, world_size: int, per_rank: int = 2) -> list:
    """Unit indices for a spot check of a gathered output: the first and last unit of every rank's
    block (plus evenly spaced ones up to ``per_rank``), so that a misplaced or missing shard of any
    rank shows up."""
    picks = set()
    for r in range(world_size):
        s, c = shard_range(total, world_size, r)
        if c == 0:
            continue
        n = min(per_rank, c)
        for i in range(n):
            picks.add(s + (i * (c - 1)) // max(n - 1, 1))
    return sorted(picks)
