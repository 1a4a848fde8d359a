"""Host-side multi-rank plumbing on CPU: two gloo ranks split rows and columns, exchange records the
way the vocabulary-sharded mode does, and agree on the slowest rank's time."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from pagoda_b200.parallel import all_gather_records, column_shard, max_over_ranks, row_shard
    rows, vocab, rec = 10, 1024, 528
    lo, hi = row_shard(rows, world, rank)
    clo, chi = column_shard(vocab, world, rank)
    local = torch.full((rows, rec), rank + 1, dtype=torch.uint8)
    local[:, 0] = torch.arange(rows, dtype=torch.uint8)
    allrec = all_gather_records(local)
    ok = allrec.shape == (world, rows, rec)
    for r in range(world):
        ok = ok and bool((allrec[r, :, 1:] == r + 1).all()) and bool((allrec[r, :, 0] == torch.arange(rows, dtype=torch.uint8)).all())
    slow = max_over_ranks(1.0 + rank, torch.device("cpu"))

    # the peer-store exchange's bookkeeping, with a stand-in for the sampler library: every rank ends up with
    # every rank's buffer address, and the addresses of a step follow its parity
    from pagoda_b200.parallel import PeerExchange

    class FakeSampler:
        opened, closed, freed = [], [], []

        def peer_alloc(self, nbytes):
            self.nbytes = nbytes
            return 0x10000000 * (rank + 1), (rank + 1).to_bytes(8, "little") + bytes(56)

        def peer_open(self, handle):
            r = int.from_bytes(handle[:8], "little")
            self.opened.append(r)
            return 0x10000000 * r + 0x1000000          # a peer's buffer appears at some other local address

        def peer_close(self, addr):
            self.closed.append(addr)

        def peer_free(self, addr):
            self.freed.append(addr)

    fs = FakeSampler()
    px = PeerExchange(fs, rows, rec, torch.device("cpu"))
    steps = [px.next_step() for _ in range(3)]
    want_base = [0x10000000 * (r + 1) + (0 if r == rank else 0x1000000) for r in range(world)]
    one = world * rows * rec
    ok = ok and fs.nbytes >= 2 * one + 2 * world * 4 and fs.opened == [r + 1 for r in range(world) if r != rank]
    for epoch, par, recs, flags in steps:
        ok = ok and par == (epoch & 1) and recs == [b + par * one for b in want_base]
        ok = ok and flags == [b + px.flag_off + par * world * 4 for b in want_base]
    ok = ok and [s_[0] for s_ in steps] == [1, 2, 3]
    px.close()
    ok = ok and len(fs.closed) == world - 1 and fs.freed == [want_base[rank]]
    q.put((rank, lo, hi, clo, chi, ok, slow))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[1:3] for r in res] == [(0, 5), (5, 10)]          # rows split without overlap
    assert [r[3:5] for r in res] == [(0, 512), (512, 1024)]    # columns split evenly
    assert all(r[5] for r in res)                              # records land at [rank][row]
    assert all(r[6] == 2.0 for r in res)                       # everyone sees the slowest rank's time


def test_column_shard_rejects_uneven_split():
    from pagoda_b200.parallel import column_shard
    try:
        column_shard(1001, 2, 0)
    except ValueError:
        return
    raise AssertionError("expected ValueError")
