// Scalar arithmetic shared by every kernel of the sampler library.
//
// The reference chain (pagoda/src/sampler.rs:92-114) computes exp((v - max) / t) with the
// platform libm and sums the results as an f32 left fold.  To make token ids reproducible
// bit for bit, the device evaluates the same published expf algorithm (the double-precision
// 2^(k/32) table + cubic of Arm's optimized routines, which is what glibc >= 2.27 ships) and
// every float operation of the chain is issued with an explicit round-to-nearest intrinsic so
// that the compiler can neither contract nor reassociate it.
//
// The file compiles as plain C++ too (PGS_HD expands to nothing) so that a host-side test can
// compare pgs_expf with libm over a dense sweep of inputs.
#pragma once

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define PGS_HD __host__ __device__ __forceinline__
#else
#define PGS_HD inline
#endif

namespace pgs {

// 2^(j/32), j = 0..31, as IEEE doubles with j << 47 subtracted from the bit pattern, so that
// adding (k << 47) for k = 32*q + j yields 2^(k/32) directly.
#define PGS_EXP2_TABLE \
    0x3ff0000000000000ULL, 0x3fefd9b0d3158574ULL, 0x3fefb5586cf9890fULL, 0x3fef9301d0125b51ULL, \
    0x3fef72b83c7d517bULL, 0x3fef54873168b9aaULL, 0x3fef387a6e756238ULL, 0x3fef1e9df51fdee1ULL, \
    0x3fef06fe0a31b715ULL, 0x3feef1a7373aa9cbULL, 0x3feedea64c123422ULL, 0x3feece086061892dULL, \
    0x3feebfdad5362a27ULL, 0x3feeb42b569d4f82ULL, 0x3feeab07dd485429ULL, 0x3feea47eb03a5585ULL, \
    0x3feea09e667f3bcdULL, 0x3fee9f75e8ec5f74ULL, 0x3feea11473eb0187ULL, 0x3feea589994cce13ULL, \
    0x3feeace5422aa0dbULL, 0x3feeb737b0cdc5e5ULL, 0x3feec49182a3f090ULL, 0x3feed503b23e255dULL, \
    0x3feee89f995ad3adULL, 0x3feeff76f2fb5e47ULL, 0x3fef199bdd85529cULL, 0x3fef3720dcef9069ULL, \
    0x3fef5818dcfba487ULL, 0x3fef7c97337b9b5fULL, 0x3fefa4afa2a490daULL, 0x3fefd0765b6e4540ULL,
static const unsigned long long kExp2TableHost[32] = {PGS_EXP2_TABLE};
#if defined(__CUDACC__)
static __device__ const unsigned long long kExp2TableDev[32] = {PGS_EXP2_TABLE};
#endif

PGS_HD uint32_t f2u(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
PGS_HD float u2f(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}
PGS_HD bool finite_f(float x) { return (f2u(x) & 0x7f800000u) != 0x7f800000u; }

// exp(x) for x <= 0 (every use in the chain has x = (v - max) / t <= 0), rounded exactly as
// glibc's expf rounds it.  `tab` is the table above or a shared-memory copy of it.
PGS_HD float pgs_expf_tab(float x, const unsigned long long* tab) {
    if (!(x >= -104.5f)) return 0.0f;  // below ~-103.97 the result rounds to +0; also -inf
    const double kInvLn2N = 0x1.71547652b82fep+5;          // 32 / ln 2
    const double kShift = 0x1.8p52;
    const double c0 = 0x1.c6af84b912394p-5 / 32 / 32 / 32;  // minimax cubic for 2^(r/32) - 1
    const double c1 = 0x1.ebfce50fac4f3p-3 / 32 / 32;
    const double c2 = 0x1.62e42ff0c52d6p-1 / 32;
    double z = kInvLn2N * (double)x;
#if defined(__CUDA_ARCH__)
    double kd = __dadd_rn(z, kShift);
    unsigned long long ki = (unsigned long long)__double_as_longlong(kd);
    kd = __dsub_rn(kd, kShift);
    double r = __dsub_rn(z, kd);
    double s = __longlong_as_double((long long)(tab[ki & 31] + (ki << 47)));
    double p = __fma_rn(c0, r, c1);
    double r2 = __dmul_rn(r, r);
    double y = __fma_rn(c2, r, 1.0);
    y = __fma_rn(p, r2, y);
    y = __dmul_rn(y, s);
    return __double2float_rn(y);
#else
    volatile double kdv = z + kShift;
    double kd = kdv;
    unsigned long long ki; memcpy(&ki, &kd, 8);
    kd -= kShift;
    double r = z - kd;
    unsigned long long sb = tab[ki & 31] + (ki << 47);
    double s; memcpy(&s, &sb, 8);
    double p = c0 * r + c1, r2 = r * r, y = c2 * r + 1.0;
    y = p * r2 + y;
    y = y * s;
    return (float)y;
#endif
}

PGS_HD float pgs_expf(float x) {
#if defined(__CUDA_ARCH__)
    return pgs_expf_tab(x, kExp2TableDev);
#else
    return pgs_expf_tab(x, kExp2TableHost);
#endif
}

// One rounding per operation, spelled out (nvcc would otherwise fuse a*b+c into an FMA).
PGS_HD float fadd(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fadd_rn(a, b);
#else
    return a + b;
#endif
}
PGS_HD float fsub(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fsub_rn(a, b);
#else
    return a - b;
#endif
}
PGS_HD float fmul(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fmul_rn(a, b);
#else
    return a * b;
#endif
}
PGS_HD float fdiv(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fdiv_rn(a, b);
#else
    return a / b;
#endif
}

#if defined(__CUDACC__)
// hardware 2^x (a few ulp); 2^-inf = +0
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// same, results below the normal range flushed to zero: a single hardware instruction
__device__ __forceinline__ float ex2_approx_ftz(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
#endif

// Monotone map float -> uint32 (larger float = larger key).  Non-finite values get key 0, below
// every finite value: the chain treats them as masked (sampler.rs:64, :100-108).
PGS_HD uint32_t order_key(float x) {
    uint32_t b = f2u(x);
    if ((b & 0x7f800000u) == 0x7f800000u) return 0u;
    if ((b << 1) == 0u) b = 0u;   // -0.0 and +0.0 compare equal in the reference's argmax (sampler.rs:64)
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
PGS_HD float key_to_float(uint32_t k) {
    return u2f((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// The softmax numerator of one processed logit: exp((x - m) / t), 0 for masked entries
// (sampler.rs:100-108).
PGS_HD float softmax_num(float x, float m, float t, const unsigned long long* tab) {
    if (!finite_f(x)) return 0.0f;
    return pgs_expf_tab(fdiv(fsub(x, m), t), tab);
}

}  // namespace pgs
