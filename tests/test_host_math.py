"""pgs_expf (the double-precision table + cubic evaluation the kernels use for exact softmax
numerators) against the platform libm, on the host: the header compiles as plain C++."""
import os
import subprocess
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SRC = r'''
#include "pgs_math.cuh"
#include <cmath>
#include <cstdio>
int main() {
    unsigned long bad = 0, n = 0;
    for (uint32_t b = 0x80000000u; b < 0xc2d20000u; b += 61) {   // x from -0 down to about -105
        const float x = pgs::u2f(b);
        n++;
        bad += pgs::f2u(expf(x)) != pgs::f2u(pgs::pgs_expf(x));
    }
    bad += pgs::pgs_expf(-INFINITY) != 0.0f;
    bad += pgs::pgs_expf(0.0f) != 1.0f;
    // order_key is monotone and invertible on finite values
    const float vals[] = {-3.4e38f, -1.0f, -1e-40f, -0.0f, 0.0f, 1e-40f, 1.0f, 3.4e38f};
    for (int i = 0; i + 1 < 8; i++) bad += !(pgs::order_key(vals[i]) <= pgs::order_key(vals[i + 1]));
    // ... except that -0.0 shares the key of +0.0 (the reference's argmax compares them equal, sampler.rs:64)
    for (int i = 0; i < 8; i++) bad += i != 3 && pgs::f2u(pgs::key_to_float(pgs::order_key(vals[i]))) != pgs::f2u(vals[i]);
    bad += pgs::order_key(-0.0f) != pgs::order_key(0.0f);
    bad += pgs::order_key(INFINITY) != 0 || pgs::order_key(NAN) != 0;
    printf("%lu %lu\n", n, bad);
    return bad != 0;
}
'''


def test_expf_matches_libm_bit_for_bit():
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.cpp")
        open(src, "w").write(SRC)
        exe = os.path.join(d, "t")
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "pagoda_b200", "csrc"), src, "-o", exe])
        out = subprocess.run([exe], capture_output=True, text=True)
        assert out.returncode == 0, out.stdout
        n, bad = map(int, out.stdout.split())
        assert n > 18_000_000 and bad == 0
