"""The allocation-free entry point (pgs_sample_batch_static) against the regular one.

Some callers of this library cannot allocate device memory while they run (their own pool owns
the GPU, or their runtime forbids it), so this entry point keeps the rows' working storage in a
fixed array inside the library.  That array is shared by every call and keeps whatever the last
call left in it, so the check is made on two different batches in a row: the second must not be
affected by what the first left behind.  Token ids, statuses and the f32 diagnostics must be
bit-identical to the regular entry point in exact mode (both run the same general kernel), and
to the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _device_batch(torch, sampler, w, dev):
    t = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a) if dt is None else np.ascontiguousarray(a).view(dt)).to(dev)
    rows = w.rows
    out = dict(token=torch.full((rows,), -7, dtype=torch.int32, device=dev),
               status=torch.full((rows,), -7, dtype=torch.int32, device=dev),
               drew=torch.zeros(rows, dtype=torch.uint8, device=dev),
               argmax=torch.zeros(rows, dtype=torch.int32, device=dev),
               row_max=torch.zeros(rows, dtype=torch.float32, device=dev),
               sumexp=torch.zeros(rows, dtype=torch.float32, device=dev),
               total=torch.zeros(rows, dtype=torch.float32, device=dev),
               n_kept=torch.zeros(rows, dtype=torch.int32, device=dev))
    desc = sampler.make_device_desc(
        t(w.logits), temperature=t(w.temperature), top_k=t(w.top_k, np.int32), top_p=t(w.top_p),
        frequency_penalty=t(w.frequency_penalty), presence_penalty=t(w.presence_penalty),
        repetition_penalty=t(w.repetition_penalty), hist_offsets=t(w.hist_offsets, np.int32),
        hist_ids=t(w.hist_ids, np.int32), uniform=t(w.uniform), **out)
    return desc, out


def _workload(synth, seed, rows, vocab):
    w = synth.config2(seed=seed, rows=rows, vocab=vocab)
    w.temperature[::4] = 0.0                       # some greedy rows
    w.top_k[1::4] = 0                              # some rows over the whole vocabulary
    w.top_p[2::4] = 1.0
    w.repetition_penalty[:] = 1.2
    w.logits[rows - 1, 5] = np.nan                 # one faulted row
    return w


def test_static_entry_point_matches_the_regular_one_twice_in_a_row(oracle):
    import torch
    import pagoda_b200
    from pagoda_b200 import capi, synth
    dev = torch.device("cuda:0")
    sampler = pagoda_b200.Sampler(device=0, max_rows=16, max_vocab=65536, max_history=1024)
    sampler.set_exact(True)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        for seed, rows, vocab in ((31, 12, 32768), (32, 16, 50257)):
            w = _workload(synth, seed, rows, vocab)
            d_ref, ref = _device_batch(torch, sampler, w, dev)
            d_new, new = _device_batch(torch, sampler, w, dev)
            sampler.launch_device(d_ref, stream)
            capi.sample_batch_static(0, d_new, stream)
            torch.cuda.synchronize()
            assert (ref["status"].cpu().numpy()[:-1] == 0).all() and ref["status"][-1].item() == 1
            for k in ref:
                a, b = ref[k].cpu().numpy(), new[k].cpu().numpy()
                np.testing.assert_array_equal(a.view(np.uint8), b.view(np.uint8), err_msg=f"{k} (seed {seed})")
            # and against the oracle directly: every decision and the f32 quantities behind it, bit for bit
            want = oracle.sample_batch(w.logits_f32(), n_threads=4, **w.oracle_kwargs())
            got = {k: v.cpu().numpy() for k, v in new.items()}
            np.testing.assert_array_equal(got["status"], want["status"])
            np.testing.assert_array_equal(got["token"], want["token"].astype(np.int32))
            np.testing.assert_array_equal(got["drew"].astype(np.int32), want["drew"])
            live = want["status"] == 0
            np.testing.assert_array_equal(got["argmax"][live], want["argmax"][live].astype(np.int32))
            np.testing.assert_array_equal(got["n_kept"][live], want["n_kept"][live].astype(np.int32))
            for k, ko in (("row_max", "row_max"), ("sumexp", "sumexp"), ("total", "total")):
                np.testing.assert_array_equal(got[k][live].view(np.uint32), want[ko][live].view(np.uint32), err_msg=k)
    finally:
        sampler.close()


def test_static_entry_point_row_with_too_long_a_history_is_a_bad_parameter():
    """1024 history ids per row is the fixed capacity: a row with 1025 reports PGS_ROW_BAD_PARAM and nothing
    else of the batch is affected."""
    import torch
    import pagoda_b200
    from pagoda_b200 import capi, synth
    dev = torch.device("cuda:0")
    rows, vocab = 3, 4096
    w = synth.config2(seed=33, rows=rows, vocab=vocab)
    lens = np.array([1024, 1025, 7])
    w.hist_offsets = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    w.hist_ids = np.random.default_rng(4).integers(0, vocab, int(lens.sum())).astype(np.uint32)
    sampler = pagoda_b200.Sampler(device=0, max_rows=4, max_vocab=vocab, max_history=2048)
    try:
        desc, out = _device_batch(torch, sampler, w, dev)
        capi.sample_batch_static(0, desc, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert out["status"].cpu().tolist() == [0, 4, 0]
    finally:
        sampler.close()


def test_static_entry_point_refuses_grammar_tables():
    import torch
    import pagoda_b200
    from pagoda_b200 import capi, synth
    dev = torch.device("cuda:0")
    sampler = pagoda_b200.Sampler(device=0, max_rows=2, max_vocab=4096, max_history=16)
    try:
        w = synth.config1(rows=2, vocab=4096)
        desc, _ = _device_batch(torch, sampler, w, dev)
        tab = torch.zeros(2, dtype=torch.int32, device=dev)
        desc.mask_table, desc.mask_state = tab.data_ptr(), tab.data_ptr()
        with pytest.raises(capi.SamplerError, match="grammar tables"):
            capi.sample_batch_static(0, desc, None)
    finally:
        sampler.close()


def test_static_entry_point_rejects_what_it_cannot_hold():
    import torch
    import pagoda_b200
    from pagoda_b200 import capi, synth
    dev = torch.device("cuda:0")
    sampler = pagoda_b200.Sampler(device=0, max_rows=2, max_vocab=70000, max_history=16)
    try:
        w = synth.config1(rows=2, vocab=70000)
        desc, _ = _device_batch(torch, sampler, w, dev)
        with pytest.raises(capi.SamplerError, match="65536"):
            capi.sample_batch_static(0, desc, None)
    finally:
        sampler.close()
