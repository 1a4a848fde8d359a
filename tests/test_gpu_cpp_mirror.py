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
