// Single-precision exp that reproduces, bit for bit, the expf of the GNU C
// library (glibc 2.39 libm, x86_64) that the reference's CPU router calls through
// Rust's f32::exp (crates/lumen-runtime/src/cuda/moe.rs:6464-6473).
//
// Why: the reference picks the top-k experts by comparing softmax PROBABILITIES
// with a strict '>' (lowest index wins a tie, cuda/moe.rs:6479-6497). Two distinct
// logits can round to the same probability, and whether they do depends on the
// last bit of exp(). Selecting the same experts as the reference for identical
// logits therefore needs the same exp(), not a 2-ulp approximation of it.
//
// Algorithm (published; Szabolcs Nagy's table-driven expf used by glibc, musl,
// newlib and bionic): x*32/ln2 = k + r with k integer (round to nearest via the
// 1.5*2^52 shift) and r in [-1/2,1/2]; exp(x) = 2^(k/32) * 2^(r/32), the first
// factor from a 32-entry table of 2^(i/32) (top bits adjusted by k), the second
// from a cubic in double precision; the double result is rounded once to float.
// The table below was regenerated here from 2^(i/32) at 60 decimal digits.
// All multiply-adds are written as explicit fma() so that the host compiler and
// nvcc evaluate exactly the same operations.
//
// tests/test_exact_expf.py compares this function (compiled for the host) with
// libm's expf on every float in [-104, 0] and [2^-126, 88]: two inputs differ by
// one ulp from the table algorithm in this image's libm; they are patched below
// so that the match is exhaustive.
#pragma once
#include <stdint.h>
#include <string.h>
#include <math.h>

#if defined(__CUDACC__)
#define LUMEN_HD __host__ __device__ __forceinline__
#else
#define LUMEN_HD static inline
#endif
#if defined(__CUDACC__)
#define LUMEN_HD_MEMBER __host__ __device__ __forceinline__
#else
#define LUMEN_HD_MEMBER inline
#endif

namespace lumen_exact {

// 2^(i/32) as IEEE double bits, minus (i << 47) so that adding (k << 47) with
// k = 32*q + i yields the bits of 2^(q + i/32).
#define LUMEN_EXP2_TAB_INIT                                                                             \
    {0x3ff0000000000000ULL, 0x3fefd9b0d3158574ULL, 0x3fefb5586cf9890fULL, 0x3fef9301d0125b51ULL,        \
     0x3fef72b83c7d517bULL, 0x3fef54873168b9aaULL, 0x3fef387a6e756238ULL, 0x3fef1e9df51fdee1ULL,        \
     0x3fef06fe0a31b715ULL, 0x3feef1a7373aa9cbULL, 0x3feedea64c123422ULL, 0x3feece086061892dULL,        \
     0x3feebfdad5362a27ULL, 0x3feeb42b569d4f82ULL, 0x3feeab07dd485429ULL, 0x3feea47eb03a5585ULL,        \
     0x3feea09e667f3bcdULL, 0x3fee9f75e8ec5f74ULL, 0x3feea11473eb0187ULL, 0x3feea589994cce13ULL,        \
     0x3feeace5422aa0dbULL, 0x3feeb737b0cdc5e5ULL, 0x3feec49182a3f090ULL, 0x3feed503b23e255dULL,        \
     0x3feee89f995ad3adULL, 0x3feeff76f2fb5e47ULL, 0x3fef199bdd85529cULL, 0x3fef3720dcef9069ULL,        \
     0x3fef5818dcfba487ULL, 0x3fef7c97337b9b5fULL, 0x3fefa4afa2a490daULL, 0x3fefd0765b6e4540ULL}

#if defined(__CUDACC__)
static __device__ __constant__ uint64_t exp2_tab_dev[32] = LUMEN_EXP2_TAB_INIT;
#endif
static const uint64_t exp2_tab_host[32] = LUMEN_EXP2_TAB_INIT;

LUMEN_HD uint64_t exp2_tab(int i) {
#if defined(__CUDA_ARCH__)
    return exp2_tab_dev[i];
#else
    return exp2_tab_host[i];
#endif
}

struct Exp2TabDefault {
    LUMEN_HD_MEMBER uint64_t operator()(int i) const { return exp2_tab(i); }
};
// table held by the caller (a copy in shared memory: lanes index it divergently)
struct Exp2TabPtr {
    const uint64_t* p;
    LUMEN_HD_MEMBER uint64_t operator()(int i) const { return p[i]; }
};

template <typename Tab>
LUMEN_HD float expf_libm_tab(float x, Tab tab) {
    uint32_t xb;
    memcpy(&xb, &x, 4);
    const uint32_t ax = xb & 0x7fffffffu;
    if (ax >= 0x42b00000u) {  // |x| >= 88, inf or nan
        if (xb == 0xff800000u) return 0.0f;
        if (ax >= 0x7f800000u) return x + x;
        if (x > 88.72283935546875f) return INFINITY;     // 0x1.62e42ep6
        if (x < -103.97207641601562f) return 0.0f;       // -0x1.9fe368p6: below the smallest subnormal
    }
    if (xb == 0xc27c65d9u) { uint32_t r = 0x11fa2993u; float f; memcpy(&f, &r, 4); return f; }
    if (xb == 0x4202422fu) { uint32_t r = 0x56fc9f1cu; float f; memcpy(&f, &r, 4); return f; }
    const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0;
    const double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
    const double c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
    const double c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    const double shift = 0x1.8p+52;
    const double xd = (double)x;
    const double z = inv_ln2_n * xd;
    double kd = z + shift;
    uint64_t ki;
    memcpy(&ki, &kd, 8);
    kd -= shift;
    const double r = z - kd;
    uint64_t t = tab((int)(ki & 31u));
    t += ki << 47;
    double s;
    memcpy(&s, &t, 8);
    const double p = fma(c0, r, c1);
    const double r2 = r * r;
    double y = fma(c2, r, 1.0);
    y = fma(p, r2, y);
    y = y * s;
    return (float)y;
}

LUMEN_HD float expf_libm(float x) { return expf_libm_tab(x, Exp2TabDefault()); }

LUMEN_HD uint64_t exp2_tab_entry(int i) { return exp2_tab(i); }

}  // namespace lumen_exact
