"""`sampler::log_softmax` (sampler.rs:73-87) and the gather of `Engine::score` on the device against
the oracle.  exp and the f32 left-fold sum are exact; ln is the double logarithm rounded to f32, so
the comparison allows 1e-6 (absolute, values are O(10))."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_log_softmax_matches_oracle(oracle):
    import torch
    import pagoda_b200
    from pagoda_b200 import synth
    s = pagoda_b200.Sampler(device=0, max_rows=8, max_vocab=151936, max_history=16)
    st = torch.cuda.current_stream().cuda_stream
    try:
        for rows, vocab, std in ((3, 3, 1.0), (6, 1000, 2.0), (4, 151936, 3.0)):
            x = synth.normal_f32(40 + vocab, rows * vocab, std).reshape(rows, vocab)
            if vocab == 3:
                x[0] = [0.0, 1.0, 2.0]                      # sampler.rs:231-235 log_softmax_sums_to_one
                x[1] = [5.0, 5.0 - 200.0, 5.0 - 300.0]      # sum == 1: the MIN_POSITIVE clamp; ln(0) = -inf
            ids = np.arange(rows, dtype=np.int32) % vocab
            g, full, status = s.log_softmax(torch.from_numpy(x).cuda(), ids=torch.from_numpy(ids).cuda(), full=True,
                                            stream_ptr=st)
            torch.cuda.synchronize()
            full, g = full.cpu().numpy(), g.cpu().numpy()
            assert (status.cpu().numpy() == 0).all()
            for r in range(rows):
                want = oracle.log_softmax(x[r])
                fin = np.isfinite(want)
                np.testing.assert_array_equal(np.isfinite(full[r]), fin)
                np.testing.assert_allclose(full[r][fin], want[fin], rtol=0, atol=1e-6 * max(1.0, np.abs(want[fin]).max()))
                assert g[r] == full[r][ids[r]]
            if vocab == 3:
                assert abs(np.exp(full[0].astype(np.float64)).sum() - 1.0) < 1e-6
        bad = np.zeros((2, 64), np.float32)
        bad[1, 3] = np.nan
        g, _, status = s.log_softmax(torch.from_numpy(bad).cuda(), ids=torch.zeros(2, dtype=torch.int32).cuda(), stream_ptr=st)
        torch.cuda.synchronize()
        assert status.cpu().numpy().tolist() == [0, 1] and np.isnan(g.cpu().numpy()[1])
    finally:
        s.close()
