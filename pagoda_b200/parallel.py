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


class _DeviceView:
    """A raw device address as something torch.as_tensor understands."""

    def __init__(self, addr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (addr, False), "version": 2}


class PeerExchange:
    """Buffers of the peer-store exchange of the vocabulary-sharded mode: on every rank a gather buffer
    [2, world, rows, record_bytes] and a flag array [2, world], double-buffered by step parity, allocated by
    the sampler library and mapped on every other rank through CUDA IPC for that rank's device, so that a
    rank's emitting kernel can store its records and raise its flag directly in its peers' memory over
    NVLink.  One process per GPU."""

    def __init__(self, sampler, rows: int, record_bytes: int, device, group=None):
        self.sampler = sampler
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows, self.record_bytes = rows, record_bytes
        self.buf_bytes = self.world * rows * record_bytes          # one parity
        self.flag_off = (2 * self.buf_bytes + 255) // 256 * 256      # flags behind both gather buffers
        total = self.flag_off + 2 * self.world * 4
        self.base, handle = sampler.peer_alloc(total)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, handle, group=group)
        self.peer_base = [self.base if r == self.rank else sampler.peer_open(everyone[r]) for r in range(self.world)]
        self.device = device
        self._buf = self._flags = None
        self.epoch = 0
        dist.barrier(group=group)   # every rank has mapped every buffer before anyone stores

    @property
    def buf(self):
        """This rank's gather buffers as a uint8 tensor [2, world, rows, record_bytes] (a view, made on first use)."""
        if self._buf is None:
            self._buf = torch.as_tensor(_DeviceView(self.base, (2, self.world, self.rows, self.record_bytes), "|u1"),
                                        device=self.device)
        return self._buf

    @property
    def flags(self):
        """This rank's flag arrays as an int32 tensor [2, world]."""
        if self._flags is None:
            self._flags = torch.as_tensor(_DeviceView(self.base + self.flag_off, (2, self.world), "<i4"), device=self.device)
        return self._flags

    def next_step(self):
        """-> (epoch, parity, gather-buffer addresses per rank, flag-array addresses per rank) of the next step."""
        self.epoch += 1
        par = self.epoch & 1
        return (self.epoch, par, [b + par * self.buf_bytes for b in self.peer_base],
                [b + self.flag_off + par * self.world * 4 for b in self.peer_base])

    def close(self, group=None):
        """Unmap the peers' buffers, then (after everyone has) free this rank's."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self._buf = self._flags = None
        for r, b in enumerate(self.peer_base):
            if r != self.rank:
                self.sampler.peer_close(b)
        dist.barrier(group=group)
        self.sampler.peer_free(self.base)


def max_over_ranks(value: float, device, group=None) -> float:
    """Timing rule: a multi-GPU step takes as long as its slowest rank."""
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
