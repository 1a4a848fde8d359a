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


TOL = 1e-5   # relative tolerance on the merged sum in the default (non-exact) mode


def _run_tp(sampler, x, n_shards, cand, temp, top_p, uniform, top_k=None, chain=None):
    """chain(r) -> keyword arguments of tp_partial for shard r (penalties, history, grammar)."""
    import torch
    dev = torch.device("cuda:0")
    rows, vocab = x.shape
    xt = torch.from_numpy(x).to(dev)
    t = torch.from_numpy(temp).to(dev)
    per = vocab // n_shards
    st = torch.cuda.current_stream().cuda_stream   # everything on torch's stream, in order
    recs = [sampler.tp_partial(xt[:, r * per:(r + 1) * per], vocab, n_shards, r, cand, temperature=t, stream_ptr=st,
                               **(chain(r) if chain else {}))
            for r in range(n_shards)]
    allrec = torch.stack(recs, 0).contiguous()
    tp, tu = torch.from_numpy(top_p).to(dev), torch.from_numpy(uniform).to(dev)
    tk = None if top_k is None else torch.from_numpy(top_k.astype(np.int32)).to(dev)
    out = sampler.tp_merge(allrec, vocab, n_shards, 0, cand, temperature=t, top_p=tp, uniform=tu, stream_ptr=st,
                           top_k=tk)
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in out.items()}


def _check_row(got, r, want, stochastic, exact):
    assert got["status"][r] == want.status, (r, got["status"][r], want.status)
    if want.status not in (0, 3):
        return
    assert got["argmax"][r] == want.argmax, r
    assert np.float32(got["gmax"][r]).view(np.uint32) == np.float32(want.gmax).view(np.uint32), r
    assert got["drew"][r] == want.drew, r
    if exact:
        assert got["token"][r] == want.token, (r, got["token"][r], want.token)
        if stochastic:
            assert np.float32(got["gsum"][r]).view(np.uint32) == np.float32(want.gsum).view(np.uint32), r
            assert np.float32(got["total"][r]).view(np.uint32) == np.float32(want.total).view(np.uint32), r
            assert got["n_kept"][r] == want.n_kept, r
    else:
        if stochastic and want.status == 0:
            assert abs(got["gsum"][r] - want.gsum) <= TOL * abs(want.gsum), (r, got["gsum"][r], want.gsum)
        if want.margin > TOL:
            assert got["token"][r] == want.token, (r, got["token"][r], want.token, want.margin)
            if stochastic:
                assert got["n_kept"][r] == want.n_kept, r


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
            assert status[r] == want.status, (epoch, r)
            assert tok[r] == want.token or want.margin <= TOL, (epoch, r, tok[r], want.token)
        sampler.tp_exchange_status()   # nothing timed out


@pytest.mark.parametrize("exact", [True, False], ids=["exact", "stream"])
@pytest.mark.parametrize("n_shards,vocab", [(2, 151936), (4, 151936), (8, 151936), (4, 4096), (1, 1000)])
def test_tp_matches_oracle(sampler, oracle, n_shards, vocab, exact):
    from pagoda_b200 import synth
    rows, cand = 12, 64
    x = synth.normal_f32(50 + n_shards, rows * vocab, 2.0).reshape(rows, vocab)
    x[3, 7] = x[3, vocab - 1] = x[3].max() + 1.0   # tie for the argmax across shards: lowest id wins
    temp = np.array([1.0, 1.0, 0.7, 0.0, 0.3, 1.5, 1.0, 0.0, 2.0, 1.0, 0.5, 1.0], np.float32)
    top_p = np.array([0.95, 1.0, 0.5, 1.0, 0.95, 0.95, 0.2, 0.9, 0.95, 0.01, 0.95, 0.6], np.float32)
    u = synth.uniform_f32(9, rows)
    sampler.set_exact(exact)
    try:
        got = _run_tp(sampler, x, n_shards, cand, temp, top_p, u)
    finally:
        sampler.set_exact(False)
    for r in range(rows):
        want = oracle.tp_sample_row(x[r], n_shards, cand, float(temp[r]), float(top_p[r]), float(u[r]))
        _check_row(got, r, want, temp[r] >= 1e-5, exact)


def _shard_words(words, lo, hi):
    """Bits lo..hi of every state's mask words, repacked so that bit 0 is column lo."""
    bits = np.unpackbits(np.ascontiguousarray(words).view(np.uint8), axis=1, bitorder="little")[:, lo:hi]
    pad = (-bits.shape[1]) % 32
    bits = np.pad(bits, ((0, 0), (0, pad)))
    return np.ascontiguousarray(np.packbits(bits, axis=1, bitorder="little")).view(np.uint32)


@pytest.mark.parametrize("exact", [True, False], ids=["exact", "stream"])
@pytest.mark.parametrize("n_shards", [2, 4, 8])
def test_tp_full_chain_matches_oracle(oracle, n_shards, exact):
    """Penalties over global history ids, a grammar bitmask cut into the shards' own words, the EOS fix on the
    shard that owns the id, a dead state, top-k over the union: everything engine.rs:1296-1313 does before the
    sampler, done shard by shard, against the oracle run on whole rows."""
    import torch
    import pagoda_b200
    from pagoda_b200 import synth
    dev = torch.device("cuda:0")
    rows, vocab, cand, n_states, eos = 24, 151936, 64, 6, 151935
    per = vocab // n_shards
    x = synth.normal_f32(90 + n_shards, rows * vocab, 2.0).reshape(rows, vocab)
    rng = np.random.default_rng(5)
    temp = rng.choice(np.array([0.0, 0.7, 1.0, 1.3], np.float32), rows)
    top_p = rng.choice(np.array([1.0, 0.9, 0.5], np.float32), rows)
    top_k = rng.choice(np.array([0, 1, 20, 64], np.uint32), rows)
    freq = rng.choice(np.array([0.0, 0.2], np.float32), rows)
    pres = rng.choice(np.array([0.0, 0.1], np.float32), rows)
    rep = rng.choice(np.array([1.0, 1.2], np.float32), rows)
    u = synth.uniform_f32(19, rows)
    hist_len = rng.integers(0, 300, rows)
    offs = np.zeros(rows + 1, np.uint32); offs[1:] = np.cumsum(hist_len)
    ids = rng.integers(0, vocab + 50, int(offs[-1])).astype(np.uint32)      # some ids beyond the vocabulary
    for r in range(rows):                                                    # the largest logits get penalised too
        h = ids[offs[r]:offs[r + 1]]
        if h.size >= 8:
            h[:8] = np.argsort(x[r])[-8:]
    words = (rng.random((n_states, vocab // 32, 32)) < 0.1)
    words = np.ascontiguousarray(np.packbits(words.reshape(n_states, -1), axis=1, bitorder="little")).view(np.uint32)
    words[:, 0] |= 1
    words[4] = 0                                       # state 4: nothing allowed; complete, so EOS is re-enabled
    flags = np.zeros(n_states, np.uint8); flags[4] = 1; flags[5] = 2   # state 5: dead
    state = rng.integers(-1, n_states, rows).astype(np.int32)
    state[:6] = [4, 5, -1, 0, 4, 1]
    s = pagoda_b200.Sampler(device=0, max_rows=rows, max_vocab=vocab, max_history=512)
    tables = []
    try:
        tables = [s.upload_mask_table(_shard_words(words, r * per, (r + 1) * per), flags) for r in range(n_shards)]
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).astype(dt)).to(dev)
        common = dict(frequency_penalty=t(freq, np.float32), presence_penalty=t(pres, np.float32),
                      repetition_penalty=t(rep, np.float32), hist_offsets=t(offs, np.int32), hist_ids=t(ids, np.int32),
                      mask_state=t(state, np.int32), eos_token_id=eos)
        mt = [t(np.where(state >= 0, tables[r], -1), np.int32) for r in range(n_shards)]
        s.set_exact(exact)
        got = _run_tp(s, x, n_shards, cand, temp, top_p, u, top_k=top_k, chain=lambda r: dict(common, mask_table=mt[r]))
    finally:
        for tb in tables:
            s.free_mask_table(tb)
        s.close()
    seen = set()
    for r in range(rows):
        kw = dict(top_k=int(top_k[r]), freq=float(freq[r]), pres=float(pres[r]), rep=float(rep[r]),
                  history=ids[offs[r]:offs[r + 1]], eos_id=eos)
        if state[r] >= 0:
            kw.update(mask_words=words[state[r]], complete=bool(flags[state[r]] & 1), dead=bool(flags[state[r]] & 2))
        want = oracle.tp_sample_row(x[r], n_shards, cand, float(temp[r]), float(top_p[r]), float(u[r]), **kw)
        _check_row(got, r, want, temp[r] >= 1e-5, exact)
        seen.add(int(want.status))
        if state[r] == 4:
            assert got["token"][r] == eos     # only the EOS fix left anything finite
    assert {0, 2} <= seen


def test_tp_top_k_beyond_the_record_is_a_bad_parameter(sampler, oracle):
    x = np.zeros((2, 1024), np.float32); x[:, 5] = 1.0
    got = _run_tp(sampler, x, 4, 16, np.ones(2, np.float32), np.ones(2, np.float32), np.zeros(2, np.float32),
                  top_k=np.array([16, 17], np.uint32))
    assert got["status"].tolist() == [0, 4]
    assert oracle.tp_sample_row(x[1], 4, 16, 1.0, 1.0, 0.0, top_k=17).status == 4


def test_tp_merge_wait_gives_up_when_no_shard_answers(sampler):
    """The one wait of the exchange, made to run out: nothing emits, the flags stay at zero, the wait is cut to
    about a millisecond.  Every row reports PGS_ROW_LOAD_TIMEOUT, the host learns of it through
    pgs_tp_exchange_status, and the handle works as before."""
    import torch
    import pagoda_b200
    dev = torch.device("cuda:0")
    rows, vocab, n_shards, cand = 8, 4096, 4, 16
    buf = torch.zeros((n_shards, rows, sampler.tp_record_bytes(cand)), dtype=torch.uint8, device=dev)
    flags = torch.zeros(n_shards, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    sampler.set_wait_limit(2000)
    try:
        out = sampler.tp_merge_wait(buf, flags, 1, vocab, n_shards, 0, cand, stream_ptr=st)
        torch.cuda.synchronize()
        assert out["status"].cpu().tolist() == [5] * rows
        with pytest.raises(pagoda_b200.SamplerError) as err:
            sampler.tp_exchange_status()
        assert err.value.code == -5
        sampler.tp_exchange_status()          # reported once
    finally:
        sampler.set_wait_limit(1 << 21)
    x = np.zeros((2, 1024), np.float32); x[:, 9] = 1.0
    got = _run_tp(sampler, x, 4, 16, np.zeros(2, np.float32), np.ones(2, np.float32), np.zeros(2, np.float32))
    assert got["status"].tolist() == [0, 0] and got["token"].tolist() == [9, 9]


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
