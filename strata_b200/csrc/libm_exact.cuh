// Host-libm-exact elementary functions for the router and the DSV4-exact expert kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace smoe {

// ---------------------------------------------------------------------------------------
// expf as glibc (>= 2.27) computes it: 32-entry table of 2^(i/32), degree-3 polynomial,
// everything in double, one rounding to float at the end.  Evaluated here with IEEE double
// operations so the result is bit-identical to the host libm the reference routers call
// (verified over every float in (-88, 88): two inputs, |x| > 32, differ by one ulp).
static __constant__ unsigned long long kExp2Bits[32] = {
    0x3ff0000000000000ULL, 0x3ff059b0d3158574ULL, 0x3ff0b5586cf9890fULL, 0x3ff11301d0125b51ULL,
    0x3ff172b83c7d517bULL, 0x3ff1d4873168b9aaULL, 0x3ff2387a6e756238ULL, 0x3ff29e9df51fdee1ULL,
    0x3ff306fe0a31b715ULL, 0x3ff371a7373aa9cbULL, 0x3ff3dea64c123422ULL, 0x3ff44e086061892dULL,
    0x3ff4bfdad5362a27ULL, 0x3ff5342b569d4f82ULL, 0x3ff5ab07dd485429ULL, 0x3ff6247eb03a5585ULL,
    0x3ff6a09e667f3bcdULL, 0x3ff71f75e8ec5f74ULL, 0x3ff7a11473eb0187ULL, 0x3ff82589994cce13ULL,
    0x3ff8ace5422aa0dbULL, 0x3ff93737b0cdc5e5ULL, 0x3ff9c49182a3f090ULL, 0x3ffa5503b23e255dULL,
    0x3ffae89f995ad3adULL, 0x3ffb7f76f2fb5e47ULL, 0x3ffc199bdd85529cULL, 0x3ffcb720dcef9069ULL,
    0x3ffd5818dcfba487ULL, 0x3ffdfc97337b9b5fULL, 0x3ffea4afa2a490daULL, 0x3fff50765b6e4540ULL};

static __device__ float expf_libm(float x) {
    if (x > 88.72283f) return __int_as_float(0x7F800000);
    if (x < -103.972076f) return 0.0f;
    const double invln2n = 0x1.71547652b82fep+0 * 32.0;
    const double shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
    const double c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
    const double c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    const double z = __dmul_rn(invln2n, (double)x);
    double kd = __dadd_rn(z, shift);
    const unsigned long long ki = (unsigned long long)__double_as_longlong(kd);
    kd = __dsub_rn(kd, shift);
    const double r = __dsub_rn(z, kd);
    unsigned long long tb = kExp2Bits[ki & 31u] - ((ki & 31u) << 47);
    tb += ki << 47;
    const double sc = __longlong_as_double((long long)tb);
    const double zz = __fma_rn(c0, r, c1);
    const double r2 = __dmul_rn(r, r);
    double y = __fma_rn(c2, r, 1.0);
    y = __fma_rn(zz, r2, y);
    y = __dmul_rn(y, sc);
    return __double2float_rn(y);
}

// ---------------------------------------------------------------------------------------
// log1pf as glibc 2.39 computes it (the fdlibm single-precision algorithm), with every operation
// a separately rounded float operation like the host build.  The CPU restatement of the same
// steps (oracle/moe_oracle.c) is checked bit for bit against the host libm; x >= 0 here
// (the argument is expf of a logit), so the x <= -1 branches are left out.
static __device__ float log1pf_libm(float x) {
    const float ln2_hi = 6.9313812256e-01f, ln2_lo = 9.0580006145e-06f;
    const float Lp1 = 6.6666668653e-01f, Lp2 = 4.0000000596e-01f, Lp3 = 2.8571429849e-01f, Lp4 = 2.2222198546e-01f,
                Lp5 = 1.8183572590e-01f, Lp6 = 1.5313838422e-01f, Lp7 = 1.4798198640e-01f;
    float f = 0.0f, c = 0.0f, u;
    int k = 1, hx = __float_as_int(x), hu = 0;
    const int ax = hx & 0x7fffffff;
    if (hx < 0x3ed413d7) {
        if (ax < 0x31000000) return ax < 0x24800000 ? x : __fsub_rn(x, __fmul_rn(__fmul_rn(x, x), 0.5f));
        if (hx > 0) { k = 0; f = x; hu = 1; }
    }
    if (hx >= 0x7f800000) return __fadd_rn(x, x);
    if (k != 0) {
        if (hx < 0x5a000000) {
            u = __fadd_rn(1.0f, x);
            hu = __float_as_int(u);
            k = (hu >> 23) - 127;
            c = k > 0 ? __fsub_rn(1.0f, __fsub_rn(u, x)) : __fsub_rn(x, __fsub_rn(u, 1.0f));
            c = __fdiv_rn(c, u);
        } else {
            u = x;
            hu = __float_as_int(u);
            k = (hu >> 23) - 127;
            c = 0.0f;
        }
        hu &= 0x007fffff;
        if (hu < 0x3504f7) {
            u = __int_as_float(hu | 0x3f800000);
        } else {
            k += 1;
            u = __int_as_float(hu | 0x3f000000);
            hu = (0x00800000 - hu) >> 2;
        }
        f = __fsub_rn(u, 1.0f);
    }
    const float kf = (float)k;
    const float hfsq = __fmul_rn(__fmul_rn(0.5f, f), f);
    if (hu == 0) {
        if (f == 0.0f) {
            if (k == 0) return 0.0f;
            c = __fadd_rn(c, __fmul_rn(kf, ln2_lo));
            return __fadd_rn(__fmul_rn(kf, ln2_hi), c);
        }
        const float R = __fmul_rn(hfsq, __fsub_rn(1.0f, __fmul_rn(0.66666666666666666f, f)));
        if (k == 0) return __fsub_rn(f, R);
        return __fsub_rn(__fmul_rn(kf, ln2_hi), __fsub_rn(__fsub_rn(R, __fadd_rn(__fmul_rn(kf, ln2_lo), c)), f));
    }
    const float s = __fdiv_rn(f, __fadd_rn(2.0f, f));
    const float z = __fmul_rn(s, s);
    float R = __fadd_rn(Lp6, __fmul_rn(z, Lp7));
    R = __fadd_rn(Lp5, __fmul_rn(z, R));
    R = __fadd_rn(Lp4, __fmul_rn(z, R));
    R = __fadd_rn(Lp3, __fmul_rn(z, R));
    R = __fadd_rn(Lp2, __fmul_rn(z, R));
    R = __fadd_rn(Lp1, __fmul_rn(z, R));
    R = __fmul_rn(z, R);
    if (k == 0) return __fsub_rn(f, __fsub_rn(hfsq, __fmul_rn(s, __fadd_rn(hfsq, R))));
    return __fsub_rn(__fmul_rn(kf, ln2_hi),
                     __fsub_rn(__fsub_rn(hfsq, __fadd_rn(__fmul_rn(s, __fadd_rn(hfsq, R)), __fadd_rn(__fmul_rn(kf, ln2_lo), c))), f));
}

static __device__ __forceinline__ float sigmoid_two_branch(float v) {
    // src/platform/numerics.cpp:44-48 of the reference
    if (v >= 0.0f) return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf_libm(-v)));
    const float e = expf_libm(v);
    return __fdiv_rn(e, __fadd_rn(1.0f, e));
}


}  // namespace smoe
