"""Generates tests/golden/chain_small.npz: small seeded batches with the CPU oracle's results.

    python tests/golden/make_golden.py

The oracle is the C restatement of the reference chain (the reference is Rust and cannot run
here), so these vectors pin today's oracle behaviour: a change in the oracle, in the generator or
in the device path shows up as a difference against the committed file."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def build():
    from oracle import oracle
    from pagoda_b200 import synth
    S = synth
    rows, vocab = 16, 777
    x = S.normal_f32(1234, rows * vocab, 2.0).reshape(rows, vocab)
    u = S.uniform_f64(1235, rows * 6).reshape(6, rows)
    temp = np.where(u[0] < 0.25, 0.0, 0.3 + u[0]).astype(np.float32)
    top_k = np.where(u[1] < 0.3, 0, 1 + (u[1] * 100).astype(np.int64)).astype(np.uint32)
    top_p = np.where(u[2] < 0.3, 1.0, 0.4 + 0.6 * u[2]).astype(np.float32)
    freq = (u[3] * 0.5).astype(np.float32)
    pres = np.where(u[4] < 0.5, 0.0, 0.2).astype(np.float32)
    rep = (1.0 + 0.3 * u[5]).astype(np.float32)
    ho = (np.arange(rows + 1) * 20).astype(np.uint32)
    hi = S.randint(1236, rows * 20, 0, vocab + 5).astype(np.uint32)
    table = S.random_mask_table(1237, 4, vocab, 0.05, 0.5)
    flags = np.array([0, 1, 2, 0], np.uint8)
    state = np.where(np.arange(rows) % 3 == 0, np.arange(rows) % 4, -1).astype(np.int32)
    uni = S.uniform_f32(1238, rows)
    want = oracle.sample_batch(x, temperature=temp, top_k=top_k, top_p=top_p, freq=freq, pres=pres, rep=rep,
                               hist_offsets=ho, hist_ids=hi, mask_table=table, mask_state=state, state_flags=flags,
                               eos_id=2, uniform=uni)
    return dict(logits=x, temperature=temp, top_k=top_k, top_p=top_p, freq=freq, pres=pres, rep=rep, hist_offsets=ho,
                hist_ids=hi, mask_table=table, state_flags=flags, mask_state=state, uniform=uni,
                token=want["token"], status=want["status"], drew=want["drew"], argmax=want["argmax"],
                sumexp=want["sumexp"], total=want["total"], n_kept=want["n_kept"])


if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "chain_small.npz")
    np.savez_compressed(out, **build())
    print(out, os.path.getsize(out), "bytes")
