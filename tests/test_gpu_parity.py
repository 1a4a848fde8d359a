"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on identical
seeded inputs.  Integer decisions (token ids, argmax, kept sets, statuses) and the f32
quantities behind them (row max, the left-fold sum, probabilities, total) must match bit for
bit; the reference chain is deterministic given the uniform, so no tolerance is needed."""
import math

import numpy as np
import pytest

from tests.util import assert_same, oracle_probs, run_both

pytestmark = pytest.mark.gpu

NEG_INF = float("-inf")


@pytest.fixture(scope="module", params=["exact", "stream"])
def sampler(request):
    """Both kernels behind the same ABI: `exact` routes every row through the general kernel
    (bit-exact token ids), `stream` is the default fast path with its stated tolerance."""
    import pagoda_b200
    s = pagoda_b200.Sampler(device=0, max_rows=256, max_vocab=262144, max_history=4096)
    s.set_exact(request.param == "exact")
    s.exact = request.param == "exact"
    yield s
    s.close()


@pytest.fixture(scope="module")
def synth():
    from pagoda_b200 import synth
    return synth


def _row(sampler, logits, **kw):
    return sampler.sample_batch(np.asarray([logits], dtype=np.float32), diagnostics=True, dump_cap=16, **kw)


# ---- the reference's own unit tests, run on the device ---------------------------------------

def test_greedy_is_argmax(sampler):  # sampler.rs:157-162
    assert _row(sampler, [0.1, 5.0, 2.0]).token[0] == 1


def test_argmax_ties_take_the_lowest_id(sampler):  # sampler.rs:64 strict >
    assert _row(sampler, [1.0, 7.0, 7.0, 7.0, -2.0]).token[0] == 1
    r = _row(sampler, [NEG_INF] * 4, mask_table=None)
    assert r.status[0] == 1  # -inf from the model is a fault (engine.rs:1278-1280)


def test_negative_zero_ties_with_positive_zero(sampler, oracle):
    """The reference's argmax compares with `>` (sampler.rs:64), for which -0.0 and +0.0 are equal: when the row
    maximum is a mix of the two, the lowest id wins whatever its sign bit."""
    assert _row(sampler, [-1.0, -0.0, 0.0, -3.0]).token[0] == 1
    assert _row(sampler, [-1.0, 0.0, -0.0, -3.0]).token[0] == 1
    x = np.full(20000, -2.0, np.float32)           # long enough for several pieces of the streaming kernel
    x[5] = -0.0
    x[15000] = 0.0
    got = _row(sampler, x)
    assert got.token[0] == 5 == oracle.argmax(x) and got.argmax[0] == 5
    got = _row(sampler, x, temperature=1.0, top_k=4, uniform=0.0)   # stochastic rows report the same argmax
    assert got.argmax[0] == 5


def test_rows_shared_by_a_cluster_agree_with_one_cta_per_row(oracle, synth, monkeypatch):
    """Small batches run with a cluster of CTAs per row.  The same batch through a handle created with that
    switched off (PGS_CLUSTER=0) must give the same decisions; both must agree with the oracle."""
    import pagoda_b200
    from tests.util import assert_same, run_both
    w = synth.config2(seed=77, rows=12, vocab=151936)
    w.temperature[::5] = 0.0                       # a few greedy rows
    w.logits[7, 1234] = np.inf                     # and a faulted one
    a = pagoda_b200.Sampler(device=0, max_rows=12, max_vocab=151936, max_history=1024)
    monkeypatch.setenv("PGS_CLUSTER", "0")
    b = pagoda_b200.Sampler(device=0, max_rows=12, max_vocab=151936, max_history=1024)
    monkeypatch.delenv("PGS_CLUSTER")
    try:
        ra, want = run_both(a, oracle, w)
        rb, _ = run_both(b, oracle, w)
        assert_same(ra, want, w, exact=False)
        assert_same(rb, want, w, exact=False)
        live = ra.status == 0                         # (a faulted row has a token and a status, nothing else)
        for k in ("token", "status", "drew"):
            np.testing.assert_array_equal(getattr(ra, k), getattr(rb, k), err_msg=k)
        for k in ("argmax", "n_kept"):
            np.testing.assert_array_equal(getattr(ra, k)[live], getattr(rb, k)[live], err_msg=k)
        np.testing.assert_array_equal(ra.row_max[live].view(np.uint32), rb.row_max[live].view(np.uint32))
        np.testing.assert_allclose(ra.sumexp[live], rb.sumexp[live], rtol=2e-6, atol=0)
    finally:
        a.close()
        b.close()


def test_sampler_is_reproducible_and_matches_the_oracle_stream(sampler, oracle):  # sampler.rs:165-176
    logits = np.ones(100, dtype=np.float32)
    rng = oracle.Rng(99)
    ref = oracle.Sampler(99)
    for _ in range(20):
        u = rng.next_f32()
        got = _row(sampler, logits, temperature=1.0, uniform=u)
        assert got.token[0] == ref.sample(logits, temperature=1.0)
        assert got.drew[0] == 1


def test_top_k_mass_is_some(sampler, oracle):  # sampler.rs:179-189
    rng = oracle.Rng(1)
    for _ in range(32):
        r = _row(sampler, [0.0, 10.0, 9.0, 8.0, 1.0], temperature=1.0, top_k=3, uniform=rng.next_f32())
        assert r.token[0] in (1, 2, 3)
        assert r.n_kept[0] == 3 and r.dump_ids[0, :3].tolist() == [1, 2, 3]


def test_top_p_keeps_only_the_nucleus(sampler, oracle):  # sampler.rs:192-207
    rng = oracle.Rng(123)
    for _ in range(200):
        r = _row(sampler, [1.0, 0.0, -1.0], temperature=1.0, top_p=0.75, uniform=rng.next_f32())
        assert r.token[0] in (0, 1)


def test_masked_logits_get_zero_mass(sampler, oracle):  # sampler.rs:210-228, via a bitmask
    tid = sampler.upload_mask_table(np.array([[0b0011]], dtype=np.uint32))
    try:
        for seed in range(16):
            rng = oracle.Rng(seed)
            for _ in range(8):
                r = _row(sampler, [0.0, -5.0, 3.0, 4.0], temperature=1.0, uniform=rng.next_f32(),
                         mask_table=[tid], mask_state=[0])
                assert r.token[0] in (0, 1)
    finally:
        sampler.free_mask_table(tid)


def test_frequency_and_presence_penalties(sampler):  # engine.rs:1781-1809
    logits = np.zeros(8, dtype=np.float32)
    logits[3] = 5.0
    # frequency 1.0 over [3,7,3]: logit[3] 5 -> 3, logit[7] 0 -> -1: argmax stays 3, row max is 3.0
    r = _row(sampler, logits, frequency_penalty=1.0, hist_offsets=[0, 3], hist_ids=[3, 7, 3])
    assert r.token[0] == 3 and r.row_max[0] == 3.0
    logits[7] = 4.0
    # presence 1.0 over [3,3,7]: 5 -> 4, 4 -> 3
    r = _row(sampler, logits, presence_penalty=1.0, hist_offsets=[0, 3], hist_ids=[3, 3, 7])
    assert r.token[0] == 3 and r.row_max[0] == 4.0
    # large enough frequency flips the argmax to the untouched runner-up
    r = _row(sampler, logits, frequency_penalty=3.0, hist_offsets=[0, 3], hist_ids=[3, 3, 9999])
    assert r.token[0] == 7 and r.row_max[0] == 4.0


def test_mask_keeps_allowed_scores_bit_for_bit(sampler):  # grammar.rs:1088-1098
    vocab = 3 + 256
    words = np.zeros((1, (vocab + 31) // 32), dtype=np.uint32)
    tok_a = 3 + ord("a")
    words[0, tok_a >> 5] |= np.uint32(1 << (tok_a & 31))
    tid = sampler.upload_mask_table(words)
    try:
        r = _row(sampler, np.full(vocab, 3.0, np.float32), mask_table=[tid], mask_state=[0])
        assert r.token[0] == tok_a and r.row_max[0] == 3.0
        r = _row(sampler, np.full(vocab, 3.0, np.float32), temperature=1.0, uniform=0.999, mask_table=[tid],
                 mask_state=[0])
        assert r.token[0] == tok_a and r.n_kept[0] == 1 and r.dump_probs[0, 0] == 1.0
    finally:
        sampler.free_mask_table(tid)


def test_eos_fix_dead_and_empty_states(sampler):  # engine.rs:1299-1312, grammar.rs:615
    words = np.zeros((3, 9), dtype=np.uint32)   # state 0: complete + empty, 1: dead, 2: empty, not complete
    tid = sampler.upload_mask_table(words, state_flags=[1, 2, 0])
    try:
        x = np.full((3, 259), 1.0, np.float32)
        r = sampler.sample_batch(x, mask_table=[tid] * 3, mask_state=[0, 1, 2], eos_token_id=2, diagnostics=True)
        assert r.status.tolist() == [0, 2, 3]
        assert r.token[0] == 2 and r.row_max[0] == 0.0   # EOS forced to exactly 0.0
        assert r.token[2] == 0
    finally:
        sampler.free_mask_table(tid)


def test_nan_row_faults_alone(sampler):  # fault_tests.rs:63-82
    x = np.zeros((3, 259), np.float32)
    x[1, 17] = np.nan
    x[2, 5] = np.inf
    r = sampler.sample_batch(x)
    assert r.status.tolist() == [0, 1, 1] and r.token[0] == 0


def test_bad_parameters_are_per_row(sampler):
    x = np.zeros((3, 64), np.float32)
    r = sampler.sample_batch(x, temperature=[1.0, np.nan, 1.0], repetition_penalty=[1.0, 1.0, 0.0],
                             uniform=[0.5, 0.5, 0.5])
    assert r.status.tolist() == [0, 4, 4]


# ---- randomised parity on small and ragged shapes ------------------------------------------------

def _random_workload(synth, seed, rows, vocab, masked=True, bf16=False):
    S = synth
    x = S.normal_f32(seed, rows * vocab, 2.0).reshape(rows, vocab)
    u = S.uniform_f64(seed + 1, rows * 8).reshape(8, rows)
    temp = np.where(u[0] < 0.25, 0.0, 0.2 + 1.5 * u[0]).astype(np.float32)
    top_k = np.where(u[1] < 0.3, 0, 1 + (u[1] * min(vocab, 300)).astype(np.int64)).astype(np.uint32)
    top_p = np.where(u[2] < 0.3, 1.0, 0.3 + 0.7 * u[2]).astype(np.float32)
    freq = np.where(u[3] < 0.5, 0.0, u[3] - 0.5).astype(np.float32)
    pres = np.where(u[4] < 0.5, 0.0, u[4] * 0.4).astype(np.float32)
    rep = np.where(u[5] < 0.5, 1.0, 1.0 + 0.5 * u[5]).astype(np.float32)
    hl = S.randint(seed + 2, rows, 0, 40)
    ho = np.concatenate([[0], np.cumsum(hl)]).astype(np.uint32)
    hi = S.randint(seed + 3, int(ho[-1]) + 1, 0, vocab + 3).astype(np.uint32)[:int(ho[-1])]
    w = S.Workload(f"random_s{seed}_r{rows}_v{vocab}", S.f32_to_bf16_bits(x).reshape(rows, vocab) if bf16 else x,
                   temp, top_k, top_p, freq, pres, rep, ho, hi, S.uniform_f32(seed + 4, rows))
    if masked:
        w.mask_words = S.random_mask_table(seed + 5, 6, vocab, 0.02, 0.6)
        w.state_flags = np.array([0, 1, 0, 2, 1, 0], np.uint8)
        w.mask_state = np.where(u[6] < 0.5, -1, S.randint(seed + 6, rows, 0, 6)).astype(np.int32)
        w.eos_token_id = 2 if vocab > 2 else -1
    return w


@pytest.mark.parametrize("vocab", [1, 2, 3, 5, 31, 33, 100, 259, 1000, 4099, 32768])
def test_random_small_shapes(sampler, oracle, synth, vocab):
    for seed in (11, 12):
        w = _random_workload(synth, seed * 100 + vocab, rows=24, vocab=vocab)
        got, want = run_both(sampler, oracle, w, dump_cap=min(vocab, 512))
        assert_same(got, want, w, exact=sampler.exact)
        for r in range(w.rows):
            if want["status"][r] != 0 or w.temperature[r] < 1e-5:
                continue
            _, probs = oracle_probs(oracle, w, r)
            ids = np.flatnonzero(probs > 0)
            n = min(len(ids), 512)
            if not sampler.exact and want["margin"][r] <= 1e-5:
                continue
            np.testing.assert_array_equal(got.dump_ids[r, :n], ids[:n].astype(np.uint32))
            if sampler.exact:
                np.testing.assert_array_equal(got.dump_probs[r, :n].view(np.uint32), probs[ids[:n]].view(np.uint32))
            else:
                np.testing.assert_allclose(got.dump_probs[r, :n], probs[ids[:n]], rtol=1e-5, atol=0)


def test_random_bf16_rows(sampler, oracle, synth):
    w = _random_workload(synth, 77, rows=16, vocab=5000, bf16=True)
    got, want = run_both(sampler, oracle, w)
    assert_same(got, want, w, exact=sampler.exact)


def test_row_stride_and_unaligned_rows(sampler, oracle, synth):
    w = _random_workload(synth, 91, rows=8, vocab=1001, masked=False)
    padded = np.full((8, 1024 + 3), 1e30, np.float32)
    padded[:, :1001] = w.logits
    got = sampler.sample_batch(padded, vocab=1001, row_stride=1027, diagnostics=True, **w.sampler_kwargs())
    want = oracle.sample_batch(w.logits, **w.oracle_kwargs())
    assert_same(got, want, w, exact=sampler.exact)


def test_ties_everywhere(sampler, oracle, synth):
    """All-equal and few-valued rows: every tie at the top-k threshold survives (sampler.rs:124) and
    equal probabilities are walked in id order (sampler.rs:135)."""
    S = synth
    rows, vocab = 12, 3000
    x = np.round(S.normal_f32(5, rows * vocab, 1.0).reshape(rows, vocab))
    x[0, :] = 1.0
    w = S.Workload("ties", x.astype(np.float32), np.full(rows, 1.0, np.float32),
                   np.array([0, 5, 50, 500] * 3, np.uint32), np.array([1.0, 1.0, 0.5, 0.9] * 3, np.float32),
                   np.zeros(rows, np.float32), np.zeros(rows, np.float32), np.ones(rows, np.float32), None, None,
                   S.uniform_f32(6, rows))
    got, want = run_both(sampler, oracle, w)
    assert_same(got, want, w, exact=sampler.exact)


def test_uniform_of_exactly_one_falls_through(sampler, oracle):  # rng.rs:28-30, sampler.rs:54
    x = np.array([[0.0, 1.0, 2.0, -1.0]], np.float32)
    got = sampler.sample_batch(x, temperature=1.0, top_k=2, uniform=[1.0])
    want, _ = oracle.sample(x[0], temperature=1.0, top_k=2, u=1.0)
    assert got.token[0] == want == 3


def test_peaked_and_flat_temperatures(sampler, oracle, synth):
    S = synth
    rows, vocab = 16, 20000
    x = S.normal_f32(21, rows * vocab, 4.0).reshape(rows, vocab)
    temp = np.array([1e-4, 1e-3, 0.01, 0.05, 0.1, 0.3, 0.7, 1.0, 2.0, 5.0, 20.0, 100.0, 1e3, 1e-5, 9.9e-6, 0.5],
                    np.float32)
    w = S.Workload("temps", x, temp, np.array([0, 40] * 8, np.uint32), np.array([1.0, 1.0, 0.9, 0.9] * 4, np.float32),
                   np.zeros(rows, np.float32), np.zeros(rows, np.float32), np.ones(rows, np.float32), None, None,
                   S.uniform_f32(22, rows))
    got, want = run_both(sampler, oracle, w)
    # at T >= 100 neighbouring probabilities differ by less than the tolerance, so several rows
    # legitimately sit on a boundary
    assert_same(got, want, w, exact=sampler.exact, min_clear=0.5)


# ---- the benchmark configurations at sizes the oracle finishes in seconds -----------------------

def test_config1_greedy_repetition(sampler, oracle, synth):
    w = synth.config1(rows=4)
    got, want = run_both(sampler, oracle, w)
    assert_same(got, want, w, exact=sampler.exact)


def test_config2_topk_topp(sampler, oracle, synth):
    w = synth.config2(rows=16)
    got, want = run_both(sampler, oracle, w, dump_cap=64)
    assert_same(got, want, w, exact=sampler.exact)
    for r in range(w.rows):
        _, probs = oracle_probs(oracle, w, r)
        ids = np.flatnonzero(probs > 0)
        if not sampler.exact and want["margin"][r] <= 1e-5:
            continue
        np.testing.assert_array_equal(got.dump_ids[r, :len(ids)], ids.astype(np.uint32))
        if sampler.exact:
            np.testing.assert_array_equal(got.dump_probs[r, :len(ids)].view(np.uint32), probs[ids].view(np.uint32))
        else:
            np.testing.assert_allclose(got.dump_probs[r, :len(ids)], probs[ids], rtol=1e-5, atol=0)


def test_config3_grammar(sampler, oracle, synth):
    w = synth.config3(rows=16)
    got, want = run_both(sampler, oracle, w)
    assert_same(got, want, w, exact=sampler.exact)


def test_config4_heterogeneous_bf16(sampler, oracle, synth):
    w = synth.config4(rows=12)
    got, want = run_both(sampler, oracle, w)
    assert_same(got, want, w, exact=sampler.exact)


def test_full_vocab_categorical_and_top_p_without_top_k(sampler, oracle, synth):
    """top-k off: pure categorical over 151936 entries, and top-p with the whole vocabulary as
    candidates (tests/grammar_tests.rs:62-64 requests exactly that combination)."""
    w = synth.config2(seed=9, rows=6)
    w.top_k[:] = 0
    w.top_p[:] = np.array([1.0, 1.0, 0.9, 0.5, 0.99, 0.2], np.float32)
    got, want = run_both(sampler, oracle, w)
    assert_same(got, want, w, exact=sampler.exact)
    # tokens only, no diagnostics: takes the list-free path
    plain = sampler.sample_batch(w.logits, **w.sampler_kwargs())
    np.testing.assert_array_equal(plain.token, want["token"])


def test_device_resident_batch_matches_host_batch(sampler, oracle, synth):
    import torch
    w = synth.config2(seed=13, rows=8, vocab=32000)
    host = sampler.sample_batch(w.logits, **w.sampler_kwargs())
    dev = torch.device("cuda:0")
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).view(dt) if a.dtype != dt else a).to(dev)
    token = torch.zeros(w.rows, dtype=torch.int32, device=dev)
    status = torch.full((w.rows,), -1, dtype=torch.int32, device=dev)
    desc = sampler.make_device_desc(
        torch.from_numpy(w.logits).to(dev), token, status,
        temperature=t(w.temperature, np.float32), top_k=t(w.top_k.view(np.int32), np.int32),
        top_p=t(w.top_p, np.float32), frequency_penalty=t(w.frequency_penalty, np.float32),
        presence_penalty=t(w.presence_penalty, np.float32), repetition_penalty=t(w.repetition_penalty, np.float32),
        hist_offsets=t(w.hist_offsets.view(np.int32), np.int32), hist_ids=t(w.hist_ids.view(np.int32), np.int32),
        uniform=t(w.uniform, np.float32))
    sampler.launch_device(desc, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(token.cpu().numpy().view(np.uint32), host.token)
    assert (status.cpu().numpy() == 0).all()
