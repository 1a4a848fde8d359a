"""One rank of the two-GPU vocabulary-sharded test (launched by torchrun from test_gpu_tp.py): emit the
local shard's records, all-gather them over NCCL, merge, and compare with the CPU oracle on rank 0."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import pagoda_b200
    from pagoda_b200 import synth
    from pagoda_b200.parallel import all_gather_records, column_shard
    rows, vocab, cand = 32, 151936, 64
    x = synth.normal_f32(77, rows * vocab, 2.0).reshape(rows, vocab)   # same seed on every rank
    temp = np.full(rows, 1.0, np.float32); temp[::5] = 0.0
    top_p = np.full(rows, 0.95, np.float32)
    u = synth.uniform_f32(78, rows)
    lo, hi = column_shard(vocab, world, rank)
    s = pagoda_b200.Sampler(device=local, max_rows=rows, max_vocab=vocab, max_history=16)
    t = torch.from_numpy(temp).to(dev)
    stream = torch.cuda.current_stream().cuda_stream
    rec = s.tp_partial(torch.from_numpy(np.ascontiguousarray(x[:, lo:hi])).to(dev), vocab, world, rank, cand,
                       temperature=t, stream_ptr=stream)
    allrec = all_gather_records(rec)
    tp, tu = torch.from_numpy(top_p).to(dev), torch.from_numpy(u).to(dev)
    out = s.tp_merge(allrec, vocab, world, rank, cand, temperature=t, top_p=tp, uniform=tu, stream_ptr=stream)
    torch.cuda.synchronize()
    tok = out["token"].cpu().numpy()
    if rank == 0:
        from oracle import oracle
        for r in range(rows):
            want = oracle.tp_sample_row(x[r], world, cand, float(temp[r]), float(top_p[r]), float(u[r]))
            assert tok[r] == want.token, (r, tok[r], want.token)
    # every rank must have produced the same tokens
    ref = out["token"].clone()
    dist.broadcast(ref, 0)
    assert torch.equal(ref, out["token"])
    dist.barrier()
    if rank == 0:
        print("TP_OK")
    s.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
