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
            assert tok[r] == want.token or want.margin <= 1e-5, (r, tok[r], want.token)
    # every rank must have produced the same tokens
    ref = out["token"].clone()
    dist.broadcast(ref, 0)
    assert torch.equal(ref, out["token"])
    # the same steps without a collective: records stored straight into the peers' gather buffers, flags
    # raised there, and the merge kernel waiting (bounded) for them; three steps exercise both buffer parities
    from pagoda_b200.parallel import PeerExchange
    px = PeerExchange(s, rows, s.tp_record_bytes(cand), dev)
    shard = torch.from_numpy(np.ascontiguousarray(x[:, lo:hi])).to(dev)
    for step in range(3):
        epoch, par, rec_ptrs, flag_ptrs = px.next_step()
        s.tp_partial_push(shard, vocab, world, rank, cand, rec_ptrs, flag_ptrs, epoch, temperature=t, stream_ptr=stream)
        out2 = s.tp_merge_wait(px.buf[par], px.flags[par], epoch, vocab, world, rank, cand, temperature=t, top_p=tp,
                               uniform=tu, stream_ptr=stream)
        torch.cuda.synchronize()
        assert int(out2["status"].max()) <= 3, out2["status"]   # no load timeout
        for k in ("token", "status", "argmax", "n_kept"):
            assert torch.equal(out2[k], out[k]), (step, k)
        for k in ("gmax", "gsum", "total"):
            assert torch.equal(out2[k].view(torch.int32), out[k].view(torch.int32)), (step, k)
    # rough cost of the exchange itself (CUDA events on this rank's stream, both paths back to back)
    def timed(fn, n=30):
        for _ in range(5):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3

    def step_nccl():
        r = s.tp_partial(shard, vocab, world, rank, cand, temperature=t, stream_ptr=stream)
        s.tp_merge(all_gather_records(r), vocab, world, rank, cand, temperature=t, top_p=tp, uniform=tu, stream_ptr=stream)

    def step_peer():
        epoch, par, rec_ptrs, flag_ptrs = px.next_step()
        s.tp_partial_push(shard, vocab, world, rank, cand, rec_ptrs, flag_ptrs, epoch, temperature=t, stream_ptr=stream)
        s.tp_merge_wait(px.buf[par], px.flags[par], epoch, vocab, world, rank, cand, temperature=t, top_p=tp,
                        uniform=tu, stream_ptr=stream)

    us_nccl, us_peer = timed(step_nccl), timed(step_peer)
    if rank == 0:
        print(f"TP_TIMING rows={rows} vocab={vocab} ranks={world}: nccl all-gather path {us_nccl:.1f} us/step, "
              f"peer-store path {us_peer:.1f} us/step")
    dist.barrier()
    px.close()
    if rank == 0:
        print("TP_OK")
    s.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
