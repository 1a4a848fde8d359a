"""Shared helpers of the GPU parity tests: run a workload through the C ABI and through the CPU
oracle and compare everything the chain decides."""
import numpy as np


def run_both(sampler, oracle, w, dump_cap=None, n_threads=8):
    table_id = None
    if w.mask_words is not None:
        table_id = sampler.upload_mask_table(w.mask_words, w.state_flags)
    if dump_cap is None:   # room for every top-k set plus ties; rows over the whole vocabulary are not dumped
        k = w.top_k[(w.top_k > 0) & (w.temperature >= 1e-5)] if w.top_k is not None else np.zeros(0)
        dump_cap = int(min(w.vocab, k.max() + 64)) if k.size else 0
    try:
        got = sampler.sample_batch(w.logits, diagnostics=True, dump_cap=dump_cap, **w.sampler_kwargs(table_id))
    finally:
        if table_id is not None:
            sampler.free_mask_table(table_id)
    want = oracle.sample_batch(w.logits_f32(), n_threads=n_threads, **w.oracle_kwargs())
    # the oracle once more with top-p off: what it keeps is the top-k set every row starts top-p from
    if (w.top_p < 1.0).any():
        kw = w.oracle_kwargs()
        kw["top_p"] = np.ones_like(w.top_p)
        got.want_topk = oracle.sample_batch(w.logits_f32(), n_threads=n_threads, **kw)
    else:
        got.want_topk = want
    got.workload, got.oracle = w, oracle
    return got, want


TOL = 1e-5   # the stated tolerance on softmax probabilities (relative)


def assert_same(got, want, w=None, check_floats=True, exact=True, min_clear=0.9):
    """exact=True (general kernel): bit-exact agreement on every decision and on the f32 quantities
    behind them.  exact=False (streaming row kernel): statuses, argmax and row max bit-exact; the f32
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


def oracle_probs(oracle, w, row, logits_row=None, **over):
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
    kw.update(over)
    out, probs = oracle.sample_row(w.logits_f32()[row] if logits_row is None else logits_row, want_probs=True, **kw)
    return out, probs


def assert_close(got, want, name="", min_clear=0.9):
    """The default (streaming) kernel against the oracle.  Bit-exact, on every row: status, argmax, row maximum,
    whether a uniform was consumed, and the top-k kept set (which does not depend on the sum).  Within TOL: the
    f32 left-fold sum and the total.  The top-p cut and the drawn token are compared on every row whose own
    margin (distance of that decision from flipping, reported by the oracle) exceeds TOL; the rows left out are
    counted, printed and bounded."""
    np.testing.assert_array_equal(got.status, want["status"], err_msg=f"{name}: status")
    live = (want["status"] == 0) | (want["status"] == 3)
    np.testing.assert_array_equal(got.argmax[live], want["argmax"][live], err_msg=f"{name}: argmax")
    np.testing.assert_array_equal(got.row_max[live].view(np.uint32), want["row_max"][live].view(np.uint32),
                                  err_msg=f"{name}: row_max")
    with np.errstate(divide="ignore", invalid="ignore"):
        rel = np.abs(got.sumexp[live] - want["sumexp"][live]) / np.abs(want["sumexp"][live])
    print(f"[{name}] sumexp max relative error {np.nanmax(rel) if rel.size else 0:.3g}")
    np.testing.assert_allclose(got.sumexp[live], want["sumexp"][live], rtol=TOL, atol=0, err_msg=f"{name}: sumexp")
    np.testing.assert_allclose(got.total[live], want["total"][live], rtol=TOL, atol=0, err_msg=f"{name}: total")
    np.testing.assert_array_equal(got.drew.astype(np.int32), want["drew"], err_msg=f"{name}: drew")
    w = getattr(got, "workload", None)
    stoch = live & (want["drew"] == 1)
    # ---- top-k kept set: unconditional
    if w is not None:
        want_k = got.want_topk
        no_p = stoch & (w.top_p >= 1.0)
        np.testing.assert_array_equal(got.n_kept[no_p], want["n_kept"][no_p], err_msg=f"{name}: top-k kept count")
        with_p = stoch & (w.top_p < 1.0)
        assert (got.n_kept[with_p] <= want_k["n_kept"][with_p]).all(), f"{name}: top-p kept more than top-k left"
        if got.dump_ids is not None and got.dump_ids.shape[1] > 0:
            order = np.argsort(np.where(stoch, want["margin"], np.inf))[:48]   # the rows closest to a boundary first
            lf = w.logits_f32()
            for r in order:
                if not stoch[r] or got.n_kept[r] > got.dump_ids.shape[1]:
                    continue
                ids, _ = got.kept(int(r))
                kw_row = dict(top_p=1.0) if w.top_p[r] < 1.0 else {}
                _, probs = oracle_probs(got.oracle, w, int(r), logits_row=lf[r], **kw_row)
                topk_ids = np.flatnonzero(probs > 0)
                if w.top_p[r] >= 1.0:
                    np.testing.assert_array_equal(ids, topk_ids, err_msg=f"{name}: top-k kept ids, row {r}")
                else:
                    assert np.isin(ids, topk_ids).all(), f"{name}: row {r} keeps ids outside of its top-k set"
    # ---- top-p cut and drawn token: on rows whose own decision is clear
    clear_p = want["margin_p"] > TOL
    clear_tok = clear_p & (want["margin_cdf"] > TOL)
    badk = np.flatnonzero((got.n_kept != want["n_kept"]) & clear_p & live)
    assert badk.size == 0, f"{name}: n_kept mismatch on rows {badk[:8]}"
    bad = np.flatnonzero((got.token != want["token"]) & clear_tok)
    assert bad.size == 0, f"{name}: token mismatch on rows {bad[:8]} with margins {want['margin'][bad[:8]]}"
    # Rows whose decision sits within TOL of a boundary may legitimately differ.  With hundreds of kept candidates a
    # uniform lands that close to one of their CDF steps on a percent or two of the rows, so what is bounded is the
    # number of rows that actually differ there, and the number that sit there is printed beside it.
    near = ~clear_tok & stoch
    differ = int(((got.token != want["token"]) & near).sum()) + int(((got.n_kept != want["n_kept"]) & ~clear_p & live).sum())
    print(f"[{name}] stochastic rows with a decision within {TOL} of a boundary: {int(near.sum())} of {int(stoch.sum())}; "
          f"of those, rows whose token or kept count differs from the oracle's: {differ}")
    assert differ <= max(1, len(clear_tok) // 100), f"{name}: {differ} rows differ from the oracle inside the tolerance band"
    assert near.mean() <= 1.0 - min_clear or len(near) < 8, f"{name}: {int(near.sum())} rows within tolerance of a boundary"
