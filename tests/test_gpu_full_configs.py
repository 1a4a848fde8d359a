"""The benchmark configurations at their full sizes, through the C ABI, against the CPU oracle (run on
all host threads) and through size-independent properties.  The streaming row kernel is the default path; the
general kernel (exact mode) must reproduce every token bit for bit."""
import numpy as np
import pytest

from tests.util import assert_same, run_both

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sampler():
    import pagoda_b200
    s = pagoda_b200.Sampler(device=0, max_rows=256, max_vocab=256000, max_history=2048)
    yield s
    s.close()


@pytest.fixture(scope="module")
def synth():
    from pagoda_b200 import synth
    return synth


@pytest.mark.parametrize("exact", [False, True])
def test_config1_full(sampler, oracle, synth, exact):
    sampler.set_exact(exact)
    w = synth.config1()
    got, want = run_both(sampler, oracle, w)
    assert_same(got, want, w, exact=exact)


@pytest.mark.parametrize("exact", [False, True])
def test_config2_full(sampler, oracle, synth, exact):
    sampler.set_exact(exact)
    w = synth.config2()
    got, want = run_both(sampler, oracle, w, n_threads=16)
    assert_same(got, want, w, exact=exact)
    # the kept set never exceeds top-k unless probabilities tie, and always holds the argmax
    assert (got.n_kept <= 50).all() and (got.n_kept >= 1).all()


@pytest.mark.parametrize("exact", [False, True])
def test_config3_full(sampler, oracle, synth, exact):
    sampler.set_exact(exact)
    w = synth.config3()
    got, want = run_both(sampler, oracle, w, n_threads=16)
    assert_same(got, want, w, exact=exact)
    # every sampled token is allowed by its row's bitmask
    for r in range(w.rows):
        words = w.mask_words[w.mask_state[r]]
        t = int(got.token[r])
        assert (words[t >> 5] >> (t & 31)) & 1, r


def test_config4_full(sampler, oracle, synth):
    sampler.set_exact(False)
    w = synth.config4()
    got, want = run_both(sampler, oracle, w, n_threads=16)
    assert_same(got, want, w, exact=False)
    exact_rows = w.head(24)
    sampler.set_exact(True)
    got, want = run_both(sampler, oracle, exact_rows, n_threads=16)
    assert_same(got, want, exact_rows, exact=True)


def test_headline_batch_properties(sampler, oracle, synth):
    """B=256 at the headline shape: determinism, greedy == argmax, and permuting the rows permutes
    the tokens (rows are independent)."""
    sampler.set_exact(False)
    w = synth.headline()
    a = sampler.sample_batch(w.logits, diagnostics=True, **w.sampler_kwargs())
    b = sampler.sample_batch(w.logits, diagnostics=True, **w.sampler_kwargs())
    np.testing.assert_array_equal(a.token, b.token)
    assert (a.status == 0).all()
    greedy = sampler.sample_batch(w.logits, hist_offsets=w.hist_offsets, hist_ids=w.hist_ids,
                                  frequency_penalty=w.frequency_penalty, presence_penalty=w.presence_penalty,
                                  diagnostics=True)
    np.testing.assert_array_equal(greedy.token, a.argmax)
    perm = np.random.default_rng(0).permutation(w.rows)
    kw = w.sampler_kwargs()
    ho = w.hist_offsets
    ids = np.concatenate([w.hist_ids[ho[r]:ho[r + 1]] for r in perm])
    offs = np.concatenate([[0], np.cumsum([ho[r + 1] - ho[r] for r in perm])]).astype(np.uint32)
    for k in ("temperature", "top_k", "top_p", "frequency_penalty", "presence_penalty", "repetition_penalty", "uniform"):
        kw[k] = kw[k][perm]
    kw["hist_offsets"], kw["hist_ids"] = offs, ids
    p = sampler.sample_batch(np.ascontiguousarray(w.logits[perm]), **kw)
    np.testing.assert_array_equal(p.token, a.token[perm])
    # against the oracle, all 256 rows, with everything the parity helper checks
    got, want = run_both(sampler, oracle, w, n_threads=16)
    np.testing.assert_array_equal(got.token, a.token)
    assert_same(got, want, w, exact=False)


def test_config5_full_width_rows(sampler, oracle, synth):
    """Config 5 at full width (V=151936 split over 2/4/8 shards) on a slice of its 1024 rows; the
    shards are emitted one after the other on this GPU."""
    import torch
    w = synth.config5(sequences=16, positions=4)
    dev = torch.device("cuda:0")
    x = torch.from_numpy(w.logits).to(dev)
    t = torch.from_numpy(w.temperature).to(dev)
    tp, tu = torch.from_numpy(w.top_p).to(dev), torch.from_numpy(w.uniform).to(dev)
    st = torch.cuda.current_stream().cuda_stream
    for n in (2, 4, 8):
        per = w.vocab // n
        recs = [sampler.tp_partial(x[:, r * per:(r + 1) * per], w.vocab, n, r, 64, temperature=t, stream_ptr=st)
                for r in range(n)]
        out = sampler.tp_merge(torch.stack(recs, 0).contiguous(), w.vocab, n, 0, 64, temperature=t, top_p=tp,
                               uniform=tu, stream_ptr=st)
        acc, nxt = sampler.draft_accept(out["argmax"].view(16, 4), torch.from_numpy(w.extra["draft"].astype(np.int32)).to(dev),
                                        stream_ptr=st)
        torch.cuda.synchronize()
        tok, am = out["token"].cpu().numpy(), out["argmax"].cpu().numpy()
        for r in range(w.rows):
            want = oracle.tp_sample_row(w.logits[r], n, 64, 1.0, 0.95, float(w.uniform[r]))
            assert am[r] == want.argmax and (tok[r] == want.token or want.margin <= 1e-5), (n, r)
        np.testing.assert_array_equal(am, w.logits.argmax(axis=1))
        for s in range(16):
            na, nx = oracle.draft_accept(am[4 * s:4 * s + 4], w.extra["draft"][s])
            assert acc[s].item() == na and nxt[s].item() == nx
