"""Multi-GPU plumbing: one process per GPU, independent shards, no collective on the timed path.

Every (batch, head) attention problem and every batch element of the encoder is independent, so ranks
own disjoint contiguous batch slices (or head slices when the batch does not divide).  The only
collectives are the timing reduction (max over ranks) and an all-gather of finished outputs for
verification.
"""
from __future__ import annotations

import os
from typing import Tuple

import torch
import torch.distributed as dist


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) slice of `n` items owned by `rank`; the first n % world ranks get one extra."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def attention_shard(batch: int, heads: int, rank: int, world: int):
    """Which (batch slice, head slice) a rank owns: batch is split when it divides evenly (shards stay
    rectangular for the (B,H,S,D) operator API), otherwise heads are split, otherwise batch unevenly."""
    if batch % world == 0:
        return shard_range(batch, rank, world), (0, heads)
    if heads % world == 0:
        return (0, batch), shard_range(heads, rank, world)
    return shard_range(batch, rank, world), (0, heads)


def init_from_env(backend: str | None = None):
    """Initialises the default process group from torchrun's environment; returns (rank, world, local_rank).
    Without WORLD_SIZE > 1 nothing is initialised."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
        dist.init_process_group(backend=backend)
    return rank, world, local


def max_over_ranks(value: float, device=None) -> float:
    """Largest value over all ranks (device-timed milliseconds are reduced with this)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device=None) -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def gather_shards(local: torch.Tensor, total: int, dim: int = 0) -> torch.Tensor:
    """All-gathers unevenly sized shards along `dim` into the full tensor (verification only; never on the
    timed path).  Shards are padded to the largest shard for the collective and trimmed afterwards."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    sizes = [shard_range(total, r, world) for r in range(world)]
    biggest = max(hi - lo for lo, hi in sizes)
    pad_shape = list(local.shape)
    pad_shape[dim] = biggest
    padded = local.new_zeros(pad_shape)
    padded.narrow(dim, 0, local.shape[dim]).copy_(local)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous())
    return torch.cat([p.narrow(dim, 0, hi - lo) for p, (lo, hi) in zip(parts, sizes)], dim=dim)
