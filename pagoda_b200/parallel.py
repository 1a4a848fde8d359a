"""Multi-GPU plumbing (one process per GPU, torch.distributed): how rows and columns are split, and
the one exchange step of the vocabulary-sharded mode.  Works on the gloo backend with CPU tensors
too, which is how the host-side logic is tested without GPUs."""
from __future__ import annotations

import torch
import torch.distributed as dist


def row_shard(rows: int, world: int, rank: int):
    """Batch-sharded mode: rank r samples rows [lo, hi); rows are independent, nothing is exchanged."""
    return rows * rank // world, rows * (rank + 1) // world


def column_shard(vocab: int, world: int, rank: int):
    """Vocabulary-sharded mode: rank r holds columns [lo, hi) of every row."""
    if vocab % world:
        raise ValueError(f"vocabulary {vocab} is not divisible by {world} ranks")
    per = vocab // world
    return rank * per, (rank + 1) * per


def all_gather_records(local: torch.Tensor, group=None) -> torch.Tensor:
    """[rows, record_bytes] uint8 per rank -> [world, rows, record_bytes] on every rank (NCCL
    all-gather over NVLink on GPUs).  The merge kernel reads shard r at index r."""
    world = dist.get_world_size(group)
    local = local.contiguous()
    out = torch.empty((world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local, group=group)
    return out.view((world,) + tuple(local.shape))


def max_over_ranks(value: float, device, group=None) -> float:
    """Timing rule: a multi-GPU step takes as long as its slowest rank."""
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
