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
