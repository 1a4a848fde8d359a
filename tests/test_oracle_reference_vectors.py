"""The CPU oracle against every known-answer test the reference holds for the logits->token
path.  Each test names the reference test it transcribes (paths relative to the reference
project root)."""
import math

import numpy as np
import pytest

NEG_INF = float("-inf")


# ---- pagoda/src/sampler.rs:156-235 ----------------------------------------------------------

def test_greedy_is_argmax(oracle):  # sampler.rs:157-162
    s = oracle.Sampler(0)
    assert s.sample([0.1, 5.0, 2.0]) == 1  # SamplingParams::default(): temperature 0


def test_sampler_is_reproducible(oracle):  # sampler.rs:165-176
    logits = np.ones(100, dtype=np.float32)
    a, b = oracle.Sampler(99), oracle.Sampler(99)
    seq_a = [a.sample(logits, temperature=1.0) for _ in range(20)]
    seq_b = [b.sample(logits, temperature=1.0) for _ in range(20)]
    assert seq_a == seq_b
    assert len(set(seq_a)) > 1  # a stream, not a constant


def test_top_k_mass_is_some(oracle):  # sampler.rs:179-189
    s = oracle.Sampler(1)
    tok = s.sample([0.0, 10.0, 9.0, 8.0, 1.0], temperature=1.0, top_k=3)
    assert tok in (1, 2, 3)


def test_top_p_keeps_only_the_nucleus(oracle):  # sampler.rs:192-207
    s = oracle.Sampler(123)
    for _ in range(200):
        assert s.sample([1.0, 0.0, -1.0], temperature=1.0, top_p=0.75, top_k=0) in (0, 1)


def test_temperature_path_gives_masked_logits_zero_mass(oracle):  # sampler.rs:210-228
    logits = [0.0, -5.0, NEG_INF, NEG_INF]
    for seed in range(16):
        s = oracle.Sampler(seed)
        for _ in range(50):
            assert s.sample(logits, temperature=1.0, top_k=0) in (0, 1)


def test_log_softmax_sums_to_one(oracle):  # sampler.rs:231-235
    lp = oracle.log_softmax([0.0, 1.0, 2.0])
    assert abs(float(np.exp(lp).sum(dtype=np.float32)) - 1.0) < 1e-6


# ---- pagoda/src/engine.rs:1780-1809 ---------------------------------------------------------

def test_frequency_penalty_scales_with_occurrence_count(oracle):  # engine.rs:1781-1793
    logits = np.zeros(8, dtype=np.float32)
    logits[3] = 5.0
    out = oracle.apply_penalties(logits, [3, 7, 3], freq=1.0)
    assert out[3] == 3.0 and out[7] == -1.0 and out[4] == 0.0


def test_presence_penalty_applies_once_per_token(oracle):  # engine.rs:1796-1809
    logits = np.zeros(8, dtype=np.float32)
    logits[3], logits[7] = 5.0, 4.0
    out = oracle.apply_penalties(logits, [3, 3, 7], pres=1.0)
    assert out[3] == 4.0 and out[7] == 3.0 and out[4] == 0.0


def test_penalties_skip_ids_outside_the_vocabulary(oracle):  # engine.rs:1562,1568 guards
    out = oracle.apply_penalties(np.zeros(4, dtype=np.float32), [9, 2, 4], freq=1.0, pres=0.5)
    assert out.tolist() == [0.0, 0.0, -1.5, 0.0]


def test_frequency_runs_even_when_only_presence_is_set(oracle):
    # engine.rs:1554-1564: the early-out needs BOTH penalties small; otherwise the frequency
    # subtraction runs with whatever frequency value there is, then the presence one.
    out = oracle.apply_penalties(np.full(4, 1.0, dtype=np.float32), [1, 1], freq=1e-7, pres=1.0)
    want = np.float32(np.float32(1.0) - np.float32(1e-7) * np.float32(2.0)) - np.float32(1.0)
    assert out[1] == want


# ---- pagoda/src/grammar.rs:1023-1098 --------------------------------------------------------

def test_regex_matches_across_full_string(oracle):  # grammar.rs:1024-1030
    g = oracle.Regex("(ab)+c")
    assert g.is_complete(b"abc") and g.is_complete(b"ababc")
    assert not g.is_complete(b"ab") and not g.is_complete(b"abcd")


def test_regex_character_class_and_digits(oracle):  # grammar.rs:1033-1038
    g = oracle.Regex("[a-z][0-9]{2}")
    assert g.is_complete(b"x42") and not g.is_complete(b"x4") and not g.is_complete(b"X42")


def test_regex_allowed_bytes_are_prefix_legal(oracle):  # grammar.rs:1041-1047
    g = oracle.Regex("[abc]+")
    assert g.allowed_bytes(b"cb") == b"abc"
    assert g.allowed_bytes(b"z") is None


def test_regex_compilation_rejects_dangling_and_mismatched(oracle):  # grammar.rs:1050-1054
    for bad in ("(", "[a", "a|"):
        with pytest.raises(ValueError):
            oracle.Regex(bad)


def test_json_complete_for_scalars_and_containers(oracle):  # grammar.rs:1057-1066
    for text in [b"null", b"true", b"false", b"42", b"-3.5e2", b'"hi"', b"{}", b"[]",
                 b'{"a":1,"b":[true,null]}']:
        assert oracle.Json.is_complete(text), text
    assert not oracle.Json.is_complete(b"") and not oracle.Json.is_complete(b"{")


def test_json_prefix_allows_continuation(oracle):  # grammar.rs:1069-1080
    allowed = oracle.Json.allowed_bytes(b"")
    for c in b'{["t':
        assert c in allowed
    allowed = oracle.Json.allowed_bytes(b"{")
    assert ord('"') in allowed and ord("}") in allowed


def test_json_dead_for_trailing_content(oracle):  # grammar.rs:1083-1085
    assert oracle.Json.allowed_bytes(b'{"a":1}  ]') is None


def test_mask_logits_keeps_allowed_and_zeros_specials(oracle):  # grammar.rs:1088-1098
    out = oracle.mask_logits_bytes(b"a", np.full(3 + 256, 3.0, dtype=np.float32))
    assert not math.isfinite(out[0]) and not math.isfinite(out[1]) and not math.isfinite(out[2])
    assert out[3 + ord("a")] == 3.0
    assert not math.isfinite(out[3 + ord("b")])


# ---- pagoda/src/rng.rs:38-49 ----------------------------------------------------------------

def test_rng_deterministic_and_bounded(oracle):
    a, b = oracle.Rng(7), oracle.Rng(7)
    assert [a.next_u64() for _ in range(100)] == [b.next_u64() for _ in range(100)]
    c = oracle.Rng(7)
    assert all(0.0 <= c.next_f64() < 1.0 for _ in range(100))


def test_rng_is_splitmix64(oracle):
    # rng.rs:10-21 written out with Python integers
    M = (1 << 64) - 1
    s = (7 + 0x9E3779B97F4A7C15) & M
    r = oracle.Rng(7)
    for _ in range(10):
        s = (s + 0x9E3779B97F4A7C15) & M
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        assert r.next_u64() == z ^ (z >> 31)


# ---- pagoda/tests/grammar_tests.rs and fault_tests.rs, at the level of the chain ------------

def _byte_masks(allowed: bytes, vocab=259):
    words = np.zeros((vocab + 31) // 32, dtype=np.uint32)
    for b in allowed:
        words[(3 + b) >> 5] |= np.uint32(1 << ((3 + b) & 31))
    return words


def test_greedy_regex_walk_produces_a_full_match(oracle):  # grammar_tests.rs:9-49
    # the toy engine's logits are replaced by a fixed ramp; the property under test is the
    # chain: mask -> EOS fix -> greedy never leaves the grammar and stops on a full match
    for pattern in ('"[a-z]{3}"', "[a-z]{3}"):
        g = oracle.Regex(pattern)
        out = b""
        logits = np.linspace(-1.0, 1.0, 259, dtype=np.float32)
        for _ in range(8):
            allowed = g.allowed_bytes(out)
            if allowed is None:
                break
            r = oracle.sample_row(logits, mask_words=_byte_masks(allowed), complete=g.is_complete(out),
                                  eos_id=2)
            if r.token == 2:
                break
            out += bytes([r.token - 3])
        assert g.is_complete(out), out


def test_sampling_under_temperature_stays_inside_the_grammar(oracle):  # grammar_tests.rs:52-75
    g = oracle.Regex('"[a-z]{3}"')
    for seed in range(8):
        rng = oracle.Rng(seed)
        out = b""
        logits = np.zeros(259, dtype=np.float32)
        for _ in range(8):
            allowed = g.allowed_bytes(out)
            if allowed is None:
                break
            r = oracle.sample_row(logits, temperature=1.0, mask_words=_byte_masks(allowed),
                                  complete=g.is_complete(out), eos_id=2, uniform=rng.next_f32())
            if r.token == 2:
                break
            out += bytes([r.token - 3])
        assert g.is_complete(out) or g.allowed_bytes(out) is not None, out


def test_nan_logits_fault_only_their_row(oracle):  # fault_tests.rs:49-82, engine.rs:1292-1295
    logits = np.zeros((2, 259), dtype=np.float32)
    logits[1, :] = np.nan
    out = oracle.sample_batch(logits)
    assert out["status"].tolist() == [oracle.ROW_OK, oracle.ROW_NONFINITE]


def test_complete_json_value_leaves_only_eos(oracle):  # grammar.rs:615 + engine.rs:1307-1312
    assert oracle.Json.allowed_bytes(b"12") == b""
    r = oracle.sample_row(np.full(259, 1.0, dtype=np.float32), mask_words=_byte_masks(b""), complete=True,
                          eos_id=2)
    assert r.token == 2 and r.status == oracle.ROW_OK
