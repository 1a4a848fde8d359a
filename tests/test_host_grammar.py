"""Host-side grammar tabulation (DFA for the byte regex, mask classes for JSON) against the CPU
oracle, which re-runs the reference's from-scratch algorithms on every prefix.  No GPU needed:
these entry points of the library are pure host code."""
import random

import numpy as np
import pytest

from pagoda_b200 import Grammar

PATTERNS = ['"[a-z]{3}"', "[a-z]{3}", "(ab)+c", "[a-z][0-9]{2}", "[abc]+", "a*b?c+", "(a|b){2}", "(a*){3}x", "x{0}y",
            "a{2,5}", "[^a-c]z", "\\n\\t\\0.", "(foo|bar|ba[rz])*!", "^ab", "[]a]+", "[a\\-z]+", "(a|ab)(c|bcd)(d*)",
            "((a|b)*c){2}", "[0-9]+(\\.[0-9]+)?(e[+-]?[0-9]+)?", ".*x.{3}"]


def _check_state(st, want_allowed, want_complete, ctx):
    got = st.allowed_bytes()
    assert got == want_allowed, (ctx, got, want_allowed)
    assert st.is_complete() == want_complete, ctx


@pytest.mark.parametrize("pattern", PATTERNS)
def test_regex_dfa_matches_the_reference_algorithm(oracle, pattern):
    ref = oracle.Regex(pattern)
    g = Grammar.regex(pattern)
    rnd = random.Random(hash(pattern) & 0xFFFF)
    alphabet = bytes(set(pattern.encode()) | set(b"abcxyz019!\n\t\x00 ."))
    for trial in range(40):
        st = g.new_state()
        text = b""
        for step in range(12):
            allowed = ref.allowed_bytes(text)
            _check_state(st, allowed, ref.is_complete(text), (pattern, text))
            # mostly legal continuations, sometimes an arbitrary byte (which must kill the state)
            if allowed and rnd.random() < 0.8:
                c = rnd.choice(allowed)
            else:
                c = rnd.choice(alphabet)
            st.advance(bytes([c]))
            text += bytes([c])
        _check_state(st, ref.allowed_bytes(text), ref.is_complete(text), (pattern, text))


def test_regex_compile_errors_match(oracle):
    for bad in ["(", "[a", "a|", "a$", "a{", "a{2", "a{3,1}", "\\", "[z-a]", "a)"]:
        with pytest.raises(ValueError):
            oracle.Regex(bad)
        with pytest.raises(ValueError):
            Grammar.regex(bad)


JSON_DOCS = [b'{"a":1,"b":[true,null]}', b"-3.5e2", b'"h\\u00e9\\n"', b"[1, 2 ,3]", b'{"k": {"n": [ ]}, "z":false}',
             b"0.5", b"12", b"[12", b"1e+9", b'  {  } ', b"nul", b"tru", b"fal", b"[-", b'{"a"', b'{"a":', b"[1,",
             b'"\\', b'"\\u12', b"1.", b"1e", b"1e-", b"01", b"[1 2]", b'{"a":1}  ]', b"{,}", b'"\x01"', b"-a", b"1.e5"]


def test_json_mask_classes_match_the_reference_scanner(oracle):
    g = Grammar.json()
    assert g.n_states == 19
    for doc in JSON_DOCS:
        st = g.new_state()
        for i in range(len(doc) + 1):
            prefix = doc[:i]
            _check_state(st, oracle.Json.allowed_bytes(prefix), oracle.Json.is_complete(prefix), prefix)
            if i < len(doc):
                st.advance(doc[i:i + 1])


def test_json_random_walks(oracle):
    g = Grammar.json()
    rnd = random.Random(5)
    for trial in range(150):
        st = g.new_state()
        text = b""
        for step in range(40):
            allowed = oracle.Json.allowed_bytes(text)
            _check_state(st, allowed, oracle.Json.is_complete(text), text)
            if allowed is None:
                break
            if allowed and rnd.random() < 0.93:
                pool = [c for c in allowed if c < 0x7F] or list(allowed)
                c = rnd.choice(pool)
            else:
                c = rnd.randrange(256)
            st.advance(bytes([c]))
            text += bytes([c])


def test_table_has_the_layout_mask_table_upload_expects():
    g = Grammar.regex('"[a-z]{3}"')
    words, flags = g.build_table(vocab=259, first_byte_id=3)
    assert words.shape == (g.n_states, 9) and flags[0] == 2 and not words[0].any()
    st = g.new_state()
    w = words[st.mask_state]
    allowed = [i for i in range(259) if (w[i >> 5] >> (i & 31)) & 1]
    assert allowed == [3 + ord('"')]
    st.advance(b'"abc"')
    assert flags[st.mask_state] & 1 and not words[st.mask_state].any()   # complete: only EOS remains
    st.reset()
    assert st.allowed_bytes() == b'"'
