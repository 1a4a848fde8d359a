"""Shared helpers of the GPU parity tests: run a workload through the C ABI and through the CPU
oracle and compare everything the chain decides."""
import numpy as np


def run_both(sampler, oracle, w, dump_cap=0, n_threads=8):
    table_id = None
    if w.mask_words is not None:
        table_id = sampler.upload_mask_table(w.mask_words, w.state_flags)
    try:
        got = sampler.sample_batch(w.logits, diagnostics=True, dump_cap=dump_cap, **w.sampler_kwargs(table_id))
    finally:
        if table_id is not None:
            sampler.free_mask_table(table_id)
    want = oracle.sample_batch(w.logits_f32(), n_threads=n_threads, **w.oracle_kwargs())
    return got, want


TOL = 1e-5   # the stated tolerance on softmax probabilities (relative)


def assert_same(got, want, w=None, check_floats=True, exact=True, min_clear=0.9):
    """exact=True (general kernel): bit-exact agreement on every decision and on the f32 quantities
    behind them.  exact=False (fused kernel): statuses, argmax and row max bit-exact; the f32
    left-fold sum and the probabilities within TOL relative; token ids and kept counts equal on
    every row whose closest decision is further than TOL from its boundary (the oracle reports
    that margin per row)."""
    name = w.name if w is not None else ""
    if not exact:
        return assert_close(got, want, name, min_clear)
    np.testing.assert_array_equal(got.status, want["status"], err_msg=f"{name}: status")
    ok = want["status"] == 0
    np.testing.assert_array_equal(got.token, want["token"], err_msg=f"{name}: token")
    np.testing.assert_array_equal(got.drew.astype(np.int32), want["drew"], err_msg=f"{name}: drew")
    live = ok | (want["status"] == 3)
    np.testing.assert_array_equal(got.argmax[live], want["argmax"][live], err_msg=f"{name}: argmax")
    if check_floats:
        np.testing.assert_array_equal(got.row_max[live].view(np.uint32), want["row_max"][live].view(np.uint32),
                                      err_msg=f"{name}: row_max")
        np.testing.assert_array_equal(got.sumexp[live].view(np.uint32), want["sumexp"][live].view(np.uint32),
                                      err_msg=f"{name}: sumexp (f32 left fold)")
        np.testing.assert_array_equal(got.total[live].view(np.uint32), want["total"][live].view(np.uint32),
                                      err_msg=f"{name}: total")
    np.testing.assert_array_equal(got.n_kept[live], want["n_kept"][live], err_msg=f"{name}: n_kept")


def oracle_probs(oracle, w, row):
    """Final probability vector of one row from the oracle (for kept-set comparisons)."""
    kw = dict(temperature=float(w.temperature[row]), top_k=int(w.top_k[row]), top_p=float(w.top_p[row]),
              freq=float(w.frequency_penalty[row]), pres=float(w.presence_penalty[row]),
              rep=float(w.repetition_penalty[row]), uniform=float(w.uniform[row]), eos_id=w.eos_token_id)
    if w.hist_offsets is not None:
        kw["history"] = w.hist_ids[w.hist_offsets[row]:w.hist_offsets[row + 1]]
    if w.mask_state is not None and w.mask_state[row] >= 0:
        s = int(w.mask_state[row])
        kw["mask_words"] = w.mask_words[s]
        kw["complete"] = bool(w.state_flags[s] & 1)
        kw["dead"] = bool(w.state_flags[s] & 2)
    out, probs = oracle.sample_row(w.logits_f32()[row], want_probs=True, **kw)
    return out, probs


def assert_close(got, want, name="", min_clear=0.9):
    np.testing.assert_array_equal(got.status, want["status"], err_msg=f"{name}: status")
    live = (want["status"] == 0) | (want["status"] == 3)
    np.testing.assert_array_equal(got.argmax[live], want["argmax"][live], err_msg=f"{name}: argmax")
    np.testing.assert_array_equal(got.row_max[live].view(np.uint32), want["row_max"][live].view(np.uint32),
                                  err_msg=f"{name}: row_max")
    with np.errstate(divide="ignore", invalid="ignore"):
        rel = np.abs(got.sumexp[live] - want["sumexp"][live]) / np.abs(want["sumexp"][live])
    print(f"[{name}] fused sumexp max relative error {np.nanmax(rel) if rel.size else 0:.3g}")
    np.testing.assert_allclose(got.sumexp[live], want["sumexp"][live], rtol=TOL, atol=0, err_msg=f"{name}: sumexp")
    np.testing.assert_allclose(got.total[live], want["total"][live], rtol=TOL, atol=0, err_msg=f"{name}: total")
    np.testing.assert_array_equal(got.drew.astype(np.int32), want["drew"], err_msg=f"{name}: drew")
    clear = want["margin"] > TOL
    bad = np.flatnonzero((got.token != want["token"]) & clear)
    assert bad.size == 0, f"{name}: token mismatch on rows {bad[:8]} with margins {want['margin'][bad[:8]]}"
    badk = np.flatnonzero((got.n_kept != want["n_kept"]) & clear & live)
    assert badk.size == 0, f"{name}: n_kept mismatch on rows {badk[:8]}"
    # rows that sit on a boundary are rare; make sure the check is not vacuous
    assert clear.mean() >= min_clear or len(clear) < 8, f"{name}: too many rows within tolerance of a boundary"
