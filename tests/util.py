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


def assert_same(got, want, w=None, check_floats=True):
    """Bit-exact agreement on every decision and on the f32 quantities behind them."""
    name = w.name if w is not None else ""
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
