"""Builds and runs tests/cpp/reference_tests.cpp: the reference's unit tests for this path, written
against the C++ mirror of its API (include/pagoda_sampler.hpp)."""
import os
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(out):
    lib_dir = os.path.join(ROOT, "pagoda_b200")
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "cpp", "reference_tests.cpp"), "-o", out,
                           "-L", lib_dir, "-lpagoda_sampler", f"-Wl,-rpath,{lib_dir}"])


def test_cpp_mirror_compiles_and_links():
    from pagoda_b200 import build
    build.build()
    with tempfile.TemporaryDirectory() as d:
        _build(os.path.join(d, "t"))


@pytest.mark.gpu
def test_reference_unit_tests_through_the_cpp_mirror():
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "t")
        _build(exe)
        out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
        assert out.returncode == 0 and "CPP_OK" in out.stdout, out.stdout + out.stderr
        _check_draw_order(out.stdout)


def _check_draw_order(stdout):
    """The DRAW_ORDER line of the C++ test against the oracle's Sampler run over the same rows one after the other,
    as the reference's loop does (engine.rs:511-544): a faulted row and a grammar dead end draw nothing."""
    import numpy as np
    from oracle import oracle
    line = [l for l in stdout.splitlines() if l.startswith("DRAW_ORDER")][0].split()
    got = [tuple(map(int, w.split(":"))) for w in line[1:7]]
    nxt = int(line[8])
    vocab = 64
    rows = np.array([[((i * 37 + r * 11) % 17) * 0.25 for i in range(vocab)] for r in range(6)], np.float32)
    rows[1, 5] = np.nan
    s = oracle.Sampler(1234)
    want = []
    for r in range(6):
        if r == 1:
            want.append((0, 1))        # logits_sane fails: Fault, nothing sampled (engine.rs:1292-1295)
        elif r == 3:
            want.append((0, 2))        # allowed_bytes is None: Stop, nothing sampled (engine.rs:1299-1303)
        else:
            want.append((s.sample(rows[r], temperature=0.8, top_k=10, top_p=0.9), 0))
    assert got == want, (got, want)
    assert nxt == s.sample(rows[0], temperature=0.8, top_k=10, top_p=0.9)
