"""Vocabulary-sharded sampling against the CPU oracle.  On one GPU the shards are emitted one after
the other by the same device (the records do not care which GPU wrote them); the two-process NCCL
test runs when two GPUs are visible."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sampler():
    import pagoda_b200
    s = pagoda_b200.Sampler(device=0, max_rows=64, max_vocab=151936, max_history=16)
    yield s
    s.close()


def _run_tp(sampler, x, n_shards, cand, temp, top_p, uniform):
    import torch
    dev = torch.device("cuda:0")
    rows, vocab = x.shape
    xt = torch.from_numpy(x).to(dev)
    t = torch.from_numpy(temp).to(dev)
    per = vocab // n_shards
    st = torch.cuda.current_stream().cuda_stream   # everything on torch's stream, in order
    recs = [sampler.tp_partial(xt[:, r * per:(r + 1) * per], vocab, n_shards, r, cand, temperature=t, stream_ptr=st)
            for r in range(n_shards)]
    allrec = torch.stack(recs, 0).contiguous()
    tp, tu = torch.from_numpy(top_p).to(dev), torch.from_numpy(uniform).to(dev)
    out = sampler.tp_merge(allrec, vocab, n_shards, 0, cand, temperature=t, top_p=tp, uniform=tu, stream_ptr=st)
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in out.items()}


def test_peer_buffers_alloc_zeroed_and_bad_handle_is_an_error(sampler):
    import torch
    import pagoda_b200
    from pagoda_b200.parallel import _DeviceView
    addr, handle = sampler.peer_alloc(4096)
    assert addr % 256 == 0 and len(handle) == 64
    view = torch.as_tensor(_DeviceView(addr, (4096,), "|u1"), device="cuda:0")
    assert int(view.sum().item()) == 0
    with pytest.raises(pagoda_b200.SamplerError):
        sampler.peer_open(bytes(64))      # not a handle: an error code, nothing is mapped
    del view
    sampler.peer_free(addr)


def test_tp_peer_store_path_on_one_device(sampler, oracle):
    """The peer-store exchange with every 'peer' on this device: each shard pushes its records into the one
    gather buffer and raises its flag, the waiting merge finds all flags up.  (Across GPUs: tp_worker.py.)"""
    import torch
    from pagoda_b200 import synth
    dev = torch.device("cuda:0")
    rows, vocab, n_shards, cand = 12, 151936, 4, 64
    x = synth.normal_f32(61, rows * vocab, 2.0).reshape(rows, vocab)
    temp = np.array([1.0, 1.0, 0.7, 0.0, 0.3, 1.5, 1.0, 0.0, 2.0, 1.0, 0.5, 1.0], np.float32)
    top_p = np.array([0.95, 1.0, 0.5, 1.0, 0.95, 0.95, 0.2, 0.9, 0.95, 0.01, 0.95, 0.6], np.float32)
    u = synth.uniform_f32(9, rows)
    xt, t = torch.from_numpy(x).to(dev), torch.from_numpy(temp).to(dev)
    tp, tu = torch.from_numpy(top_p).to(dev), torch.from_numpy(u).to(dev)
    per = vocab // n_shards
    buf = torch.zeros((2, n_shards, rows, sampler.tp_record_bytes(cand)), dtype=torch.uint8, device=dev)
    flags = torch.zeros((2, n_shards), dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    for epoch in (1, 2, 3):
        par = epoch & 1
        for r in range(n_shards):
            sampler.tp_partial_push(xt[:, r * per:(r + 1) * per], vocab, n_shards, r, cand,
                                    [buf[par].data_ptr()] * n_shards, [flags[par].data_ptr()] * n_shards, epoch,
                                    temperature=t, stream_ptr=st)
        out = sampler.tp_merge_wait(buf[par], flags[par], epoch, vocab, n_shards, 0, cand, temperature=t, top_p=tp,
                                    uniform=tu, stream_ptr=st)
        torch.cuda.synchronize()
        assert flags[par].cpu().tolist() == [epoch] * n_shards
        tok, status = out["token"].cpu().numpy(), out["status"].cpu().numpy()
        for r in range(rows):
            want = oracle.tp_sample_row(x[r], n_shards, cand, float(temp[r]), float(top_p[r]), float(u[r]))
            assert status[r] == want.status and tok[r] == want.token, (epoch, r, tok[r], want.token)


@pytest.mark.parametrize("n_shards,vocab", [(2, 151936), (4, 151936), (8, 151936), (4, 4096), (1, 1000)])
def test_tp_matches_oracle(sampler, oracle, n_shards, vocab):
    from pagoda_b200 import synth
    rows, cand = 12, 64
    x = synth.normal_f32(50 + n_shards, rows * vocab, 2.0).reshape(rows, vocab)
    x[3, 7] = x[3, vocab - 1] = x[3].max() + 1.0   # tie for the argmax across shards: lowest id wins
    temp = np.array([1.0, 1.0, 0.7, 0.0, 0.3, 1.5, 1.0, 0.0, 2.0, 1.0, 0.5, 1.0], np.float32)
    top_p = np.array([0.95, 1.0, 0.5, 1.0, 0.95, 0.95, 0.2, 0.9, 0.95, 0.01, 0.95, 0.6], np.float32)
    u = synth.uniform_f32(9, rows)
    got = _run_tp(sampler, x, n_shards, cand, temp, top_p, u)
    for r in range(rows):
        want = oracle.tp_sample_row(x[r], n_shards, cand, float(temp[r]), float(top_p[r]), float(u[r]))
        assert got["status"][r] == want.status
        assert got["argmax"][r] == want.argmax, r
        assert got["token"][r] == want.token, (r, got["token"][r], want.token)
        assert got["drew"][r] == want.drew
        assert np.float32(got["gmax"][r]).view(np.uint32) == np.float32(want.gmax).view(np.uint32)
        if temp[r] >= 1e-5:
            assert np.float32(got["gsum"][r]).view(np.uint32) == np.float32(want.gsum).view(np.uint32), r
            assert np.float32(got["total"][r]).view(np.uint32) == np.float32(want.total).view(np.uint32)
            assert got["n_kept"][r] == want.n_kept


def test_tp_faulted_shard_faults_the_row(sampler):
    import torch
    x = np.zeros((2, 1024), np.float32)
    x[1, 900] = np.nan
    got = _run_tp(sampler, x, 4, 16, np.ones(2, np.float32), np.ones(2, np.float32), np.zeros(2, np.float32))
    assert got["status"].tolist() == [0, 1]


def test_draft_accept(sampler, oracle):
    import torch
    rng = np.random.default_rng(3)
    am = rng.integers(0, 50, size=(64, 4)).astype(np.int32)
    draft = am.copy()
    flip = rng.random((64, 4)) < 0.3
    draft[flip] += 1
    acc, nxt = sampler.draft_accept(torch.from_numpy(am).cuda(), torch.from_numpy(draft).cuda(),
                                    stream_ptr=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    for s in range(64):
        n, nx = oracle.draft_accept(am[s], draft[s])
        assert acc[s].item() == n and nxt[s].item() == nx


def test_tp_two_ranks_over_nccl():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29517", os.path.join(root, "tests", "tp_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-6000:]
    assert "TP_OK" in out.stdout
