/*
 * CPU oracle for the MoE expert block.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic that ro99/strata performs on
 * the MoE hot path (router projection -> score/top-k -> group by expert ->
 * quantized gate/up + SwiGLU -> down -> weighted combine + shared expert).
 * It is the checker the CUDA library is compared against; nothing in the
 * shipped library links, loads or calls it.
 *
 * Parity status: PINNED.  Every function below is checked (a) against the
 * known-answer vectors the reference keeps in its own tests and (b) against
 * the reference's own CPU code compiled unmodified into oracle/_ref
 * (see oracle/build.py and tests/test_oracle_*.py).  One exception: the
 * softmax top-k router has no implementation in the reference at all, so
 * ORC_SCORE_SOFTMAX is "parity unpinned" (defined here as softmax over fp32
 * logits, top-k by probability descending then index ascending).
 *
 * Each function names the reference file:line it follows (paths are relative
 * to the reference project root).
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC  (fp contraction is
 * disabled so a*b+c is two roundings, as in the reference's x86-64 -O2 build).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ enums */
enum { ORC_FMT_MXFP4 = 0, ORC_FMT_NVFP4 = 1, ORC_FMT_INT4G128 = 2, ORC_FMT_BF16 = 3 };
enum {
    ORC_SCORE_SIGMOID = 0,       /* two-branch sigmoid_f32, src/platform/numerics.cpp:44-48 */
    ORC_SCORE_SIGMOID_PLAIN = 1, /* 1/(1+exp(-x)), src/models/kimi_k3/kimi_k3_ops.cpp:12-14 */
    ORC_SCORE_SOFTMAX = 2,       /* no reference implementation: parity unpinned */
    ORC_SCORE_SQRTSOFTPLUS = 3   /* src/models/dsv4/deepseek_ops.cpp:82-133 */
};
enum { ORC_COMBINE_RANK_ORDER = 0, ORC_COMBINE_JOB_ORDER = 1 };

/* ------------------------------------------------------- scalar decoders */
static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

/* BF16 -> FP32 is the identity on the top sixteen bits. */
ORC_API float orc_bf16_to_f32(uint16_t v) { return bits_f32((uint32_t)v << 16); }

/* FP32 -> BF16, round to nearest even (NaN kept quiet). */
ORC_API uint16_t orc_f32_to_bf16(float f) {
    uint32_t b = f32_bits(f);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((b >> 16) | 0x40u);
    b += 0x7FFFu + ((b >> 16) & 1u);
    return (uint16_t)(b >> 16);
}

/* stable_bf16_hash (src/platform/diagnostics.cpp:14-27, 84-88): FNV-1a over the little-endian bytes of every
 * value after round-to-nearest-even to BF16; values whose exponent field is all ones (infinities, NaNs) are
 * truncated, not rounded. */
ORC_API uint64_t orc_stable_bf16_hash(const float* values, size_t n) {
    uint64_t h = 14695981039346656037ull;
    for (size_t i = 0; i < n; ++i) {
        uint32_t b = f32_bits(values[i]);
        if ((b & 0x7F800000u) != 0x7F800000u) b += 0x7FFFu + ((b >> 16) & 1u);
        const uint32_t v = b >> 16;
        h = (h ^ (v & 0xFFu)) * 1099511628211ull;
        h = (h ^ (v >> 8)) * 1099511628211ull;
    }
    return h;
}

/* E2M1 value table.  CPU tables in the reference give -0.0 for nibble 0x8
 * (src/platform/numerics.cpp:75-83, include/strata/compressed_tensors.hpp:52-54);
 * the device decoder gives +0.0 (kernels/cuda/backend.cu:194-210, pinned by
 * tests/test_fp4_decode.cpp:56-73).  device_zero selects the latter. */
ORC_API float orc_e2m1(uint32_t nibble, int device_zero) {
    static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float v = mag[nibble & 7u];
    if ((nibble & 8u) && !(device_zero && (nibble & 7u) == 0u)) v = -v;
    return v;
}

/* E8M0 scale as the float whose exponent field is the byte
 * (src/platform/compressed_tensors.cpp:127-129): 0 -> +0.0, 0xFF -> +inf.
 * The DSV4 decoder differs only at the two reserved bytes
 * (kernels/cuda/backend.cu:155-157): 0 -> 2^-127, 0xFF -> NaN. */
ORC_API float orc_e8m0(uint32_t byte, int dsv4_edges) {
    byte &= 0xFFu;
    if (dsv4_edges) {
        if (byte == 0xFFu) return NAN;
        return ldexpf(1.0f, (int)byte - 127);
    }
    return bits_f32(byte << 23);
}

/* E4M3 (fn) -> fp32, src/platform/numerics.cpp:58-73. */
ORC_API float orc_e4m3(uint32_t byte) {
    const uint32_t e = (byte >> 3) & 0xFu, m = byte & 7u;
    float v;
    if (e == 0u) v = ldexpf((float)m / 8.0f, -6);
    else if (e == 0xFu && m == 7u) return NAN;
    else v = ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
    return (byte & 0x80u) ? -v : v;
}

/* sigmoid_f32, src/platform/numerics.cpp:44-48. */
ORC_API float orc_sigmoid(float v) {
    if (v >= 0.0f) return 1.0f / (1.0f + expf(-v));
    const float e = expf(v);
    return e / (1.0f + e);
}
/* silu_f32, src/platform/numerics.cpp:50-52. */
ORC_API float orc_silu(float v) { return v * orc_sigmoid(v); }

/* dsv4_softplus_f32 threshold form (src/models/dsv4/deepseek_ops.cpp, same
 * rule as laguna_softplus_f32, src/models/laguna/laguna_ops.cpp:33-39). */
static float orc_softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

/* --------------------------------------------------------------------------
 * expf restated as the table-driven double-precision algorithm glibc >= 2.27
 * ships (Szabolcs Nagy's expf from ARM optimized-routines: N = 32 table,
 * degree-3 polynomial, evaluated in double).  The CUDA router evaluates the
 * same steps with IEEE double operations so that its sigmoid scores, and
 * therefore its expert ids on near-ties, are bit-identical to the host
 * libm the reference routers call.  use_fma selects whether the three
 * multiply-adds are contracted (the x86-64 FMA ifunc variant) or not;
 * tests/test_oracle_golden.py checks which one this host's libm matches.
 * Valid for |x| < 88 (the router never exceeds that without saturating). */
/* Correctly rounded bit patterns of 2^(i/32), i = 0..31. */
static const uint64_t orc_exp2_bits[32] = {
    0x3ff0000000000000ULL, 0x3ff059b0d3158574ULL, 0x3ff0b5586cf9890fULL, 0x3ff11301d0125b51ULL,
    0x3ff172b83c7d517bULL, 0x3ff1d4873168b9aaULL, 0x3ff2387a6e756238ULL, 0x3ff29e9df51fdee1ULL,
    0x3ff306fe0a31b715ULL, 0x3ff371a7373aa9cbULL, 0x3ff3dea64c123422ULL, 0x3ff44e086061892dULL,
    0x3ff4bfdad5362a27ULL, 0x3ff5342b569d4f82ULL, 0x3ff5ab07dd485429ULL, 0x3ff6247eb03a5585ULL,
    0x3ff6a09e667f3bcdULL, 0x3ff71f75e8ec5f74ULL, 0x3ff7a11473eb0187ULL, 0x3ff82589994cce13ULL,
    0x3ff8ace5422aa0dbULL, 0x3ff93737b0cdc5e5ULL, 0x3ff9c49182a3f090ULL, 0x3ffa5503b23e255dULL,
    0x3ffae89f995ad3adULL, 0x3ffb7f76f2fb5e47ULL, 0x3ffc199bdd85529cULL, 0x3ffcb720dcef9069ULL,
    0x3ffd5818dcfba487ULL, 0x3ffdfc97337b9b5fULL, 0x3ffea4afa2a490daULL, 0x3fff50765b6e4540ULL};
ORC_API float orc_expf_replica(float x, int use_fma) {
    const double invln2n = 0x1.71547652b82fep+0 * 32.0;
    const double shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
    const double c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
    const double c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    if (!(fabsf(x) < 88.0f)) return expf(x);
    const double xd = (double)x;
    const double z = invln2n * xd;
    double kd = z + shift;
    uint64_t ki;
    memcpy(&ki, &kd, 8);
    kd -= shift;
    const double r = z - kd;
    /* scale 2^(k/32): table entry bits(2^(i/32)) - (i << 47), plus k << 47 */
    uint64_t t = orc_exp2_bits[ki & 31u] - ((uint64_t)(ki & 31u) << 47);
    t += ki << 47;
    double sd;
    memcpy(&sd, &t, 8);
    double zz, y;
    const double r2 = r * r;
    if (use_fma) {
        zz = fma(c0, r, c1);
        y = fma(c2, r, 1.0);
        y = fma(zz, r2, y);
    } else {
        zz = c0 * r + c1;
        y = c2 * r + 1.0;
        y = zz * r2 + y;
    }
    y = y * sd;
    return (float)y;
}

/* --------------------------------------------------------------------------
 * log1pf restated as the single-precision algorithm glibc 2.39 ships for it (the classic
 * fdlibm s_log1pf: argument reduction 1 + x = 2^k (1 + f), f / (2 + f) series with seven
 * coefficients, ln2 split in two), every operation a separately rounded float operation
 * (the host build does not contract them).  The CUDA router evaluates the same steps so that
 * its sqrt(softplus) scores are bit-identical to the host's; tests/test_oracle_golden.py
 * checks this restatement against the libm of the machine it runs on.  Inputs here are
 * expf(logit) >= 0; the branches for x <= -1 are kept for completeness. */
ORC_API float orc_log1pf_replica(float x) {
    const float ln2_hi = 6.9313812256e-01f, ln2_lo = 9.0580006145e-06f;
    const float Lp1 = 6.6666668653e-01f, Lp2 = 4.0000000596e-01f, Lp3 = 2.8571429849e-01f, Lp4 = 2.2222198546e-01f,
                Lp5 = 1.8183572590e-01f, Lp6 = 1.5313838422e-01f, Lp7 = 1.4798198640e-01f;
    float hfsq, f = 0.0f, c = 0.0f, s, z, R, u;
    int32_t k = 1, hx = (int32_t)f32_bits(x), hu = 0, ax = hx & 0x7fffffff;
    if (hx < 0x3ed413d7) {                       /* x < 0.41422 */
        if (ax >= 0x3f800000) return x == -1.0f ? -INFINITY : NAN;
        if (ax < 0x31000000) return ax < 0x24800000 ? x : x - x * x * 0.5f;
        if (hx > 0 || hx <= (int32_t)0xbe95f61f) { k = 0; f = x; hu = 1; }
    }
    if (hx >= 0x7f800000) return x + x;
    if (k != 0) {
        if (hx < 0x5a000000) {
            u = 1.0f + x;
            hu = (int32_t)f32_bits(u);
            k = (hu >> 23) - 127;
            c = (k > 0) ? 1.0f - (u - x) : x - (u - 1.0f);
            c /= u;
        } else {
            u = x;
            hu = (int32_t)f32_bits(u);
            k = (hu >> 23) - 127;
            c = 0.0f;
        }
        hu &= 0x007fffff;
        if (hu < 0x3504f7) {
            u = bits_f32((uint32_t)hu | 0x3f800000u);
        } else {
            k += 1;
            u = bits_f32((uint32_t)hu | 0x3f000000u);
            hu = (0x00800000 - hu) >> 2;
        }
        f = u - 1.0f;
    }
    hfsq = 0.5f * f * f;
    if (hu == 0) {
        if (f == 0.0f) {
            if (k == 0) return 0.0f;
            c += (float)k * ln2_lo;
            return (float)k * ln2_hi + c;
        }
        R = hfsq * (1.0f - 0.66666666666666666f * f);
        if (k == 0) return f - R;
        return (float)k * ln2_hi - ((R - ((float)k * ln2_lo + c)) - f);
    }
    s = f / (2.0f + f);
    z = s * s;
    R = z * (Lp1 + z * (Lp2 + z * (Lp3 + z * (Lp4 + z * (Lp5 + z * (Lp6 + z * Lp7))))));
    if (k == 0) return f - (hfsq - s * (hfsq + R));
    return (float)k * ln2_hi - ((hfsq - (s * (hfsq + R) + ((float)k * ln2_lo + c))) - f);
}

/* ------------------------------------------------------ weight matrices */
typedef struct {
    int32_t fmt;
    uint32_t rows, cols;
    const uint8_t* packed; /* MXFP4/NVFP4: [rows, cols/2] u8, low nibble = even column.
                              INT4: [rows, cols/8] little-endian u32, nibble j = column 8w+j.
                              BF16: [rows, cols] u16 */
    const uint8_t* scales; /* MXFP4: [rows, cols/32] E8M0.  NVFP4: [rows, cols/16] E4M3.
                              INT4: [rows, cols/128] BF16 (u16 LE). */
    float global_scale;    /* NVFP4 only: w = e2m1 * (e4m3 / global_scale) */
} orc_matrix;

/* Exact fp32 dequantisation of one row (zero sign as the CPU tables give it
 * unless device_zero).  MXFP4: src/platform/compressed_tensors.cpp:131-178.
 * NVFP4: kernels/cuda/backend.cu:2008-2014 (value = e2m1 * (e4m3 / global), the
 * product taken in fp32).  INT4: kernels/cuda/backend.cu:1908-1916
 * ((raw - 8) * bf16 scale, in fp32). */
ORC_API int orc_dequant_row(const orc_matrix* m, uint32_t row, int device_zero, float* out) {
    if (!m || row >= m->rows) return -1;
    const uint32_t C = m->cols;
    if (m->fmt == ORC_FMT_MXFP4) {
        const uint8_t* p = m->packed + (size_t)row * (C / 2);
        const uint8_t* s = m->scales + (size_t)row * (C / 32);
        for (uint32_t c = 0; c < C; ++c) {
            const uint32_t nib = (c & 1u) ? (p[c / 2] >> 4) : (p[c / 2] & 0xFu);
            out[c] = orc_e2m1(nib, device_zero) * orc_e8m0(s[c / 32], 0);
        }
    } else if (m->fmt == ORC_FMT_NVFP4) {
        const uint8_t* p = m->packed + (size_t)row * (C / 2);
        const uint8_t* s = m->scales + (size_t)row * (C / 16);
        for (uint32_t c = 0; c < C; ++c) {
            const uint32_t nib = (c & 1u) ? (p[c / 2] >> 4) : (p[c / 2] & 0xFu);
            out[c] = orc_e2m1(nib, device_zero) * (orc_e4m3(s[c / 16]) / m->global_scale);
        }
    } else if (m->fmt == ORC_FMT_INT4G128) {
        const uint8_t* p = m->packed + (size_t)row * (C / 8) * 4;
        const uint8_t* s = m->scales + (size_t)row * (C / 128) * 2;
        for (uint32_t c = 0; c < C; ++c) {
            uint32_t w;
            memcpy(&w, p + (size_t)(c / 8) * 4, 4);
            const int q = (int)((w >> ((c % 8u) * 4u)) & 0xFu) - 8;
            uint16_t sb;
            memcpy(&sb, s + (size_t)(c / 128) * 2, 2);
            out[c] = (float)q * orc_bf16_to_f32(sb);
        }
    } else if (m->fmt == ORC_FMT_BF16) {
        const uint16_t* p = (const uint16_t*)m->packed + (size_t)row * C;
        for (uint32_t c = 0; c < C; ++c) out[c] = orc_bf16_to_f32(p[c]);
    } else {
        return -2;
    }
    return 0;
}

/* y[r] = sum_c x[c] * W[r, c] for r in [row_begin, row_end), fp32 accumulate in
 * the order and with the expression shape of the reference's scalar host code:
 *   MXFP4  src/models/kimi_k3/kimi_k3_layer.cpp:279-300 (group partial, then
 *          one multiply by the group scale)
 *   NVFP4  src/models/laguna/laguna_ops.cpp:77-91 (x * e2m1 * scale, scale =
 *          e4m3 / global, sequential)
 *   INT4   kernels/cpu/glm_int4.cpp:140-160 (x * (raw-8) * scale, sequential)
 *   BF16   sequential x * w.
 * accumulate_double = 1 sums the same exact products in double instead (the
 * rounding-free yardstick the tolerance tests measure both sides against). */
ORC_API int orc_matvec(const orc_matrix* m, const float* x, float* y, uint32_t row_begin,
                       uint32_t row_end, int accumulate_double) {
    if (!m || row_end > m->rows || row_begin > row_end) return -1;
    const uint32_t C = m->cols;
    static const float val[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                  -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
    for (uint32_t r = row_begin; r < row_end; ++r) {
        float sum = 0.0f;
        double dsum = 0.0;
        if (m->fmt == ORC_FMT_MXFP4) {
            const uint8_t* p = m->packed + (size_t)r * (C / 2);
            const uint8_t* s = m->scales + (size_t)r * (C / 32);
            for (uint32_t g = 0; g < C / 32; ++g) {
                const float scale = orc_e8m0(s[g], 0);
                const uint8_t* b = p + (size_t)g * 16;
                const float* src = x + (size_t)g * 32;
                if (accumulate_double) {
                    double part = 0.0;
                    for (uint32_t i = 0; i < 16; ++i)
                        part += (double)src[2 * i] * val[b[i] & 0xFu] +
                                (double)src[2 * i + 1] * val[b[i] >> 4];
                    dsum += part * scale;
                } else {
                    float part = 0.0f;
                    for (uint32_t i = 0; i < 16; ++i)
                        part += src[2 * i] * val[b[i] & 0xFu] + src[2 * i + 1] * val[b[i] >> 4];
                    sum += part * scale;
                }
            }
        } else if (m->fmt == ORC_FMT_NVFP4) {
            const uint8_t* p = m->packed + (size_t)r * (C / 2);
            const uint8_t* s = m->scales + (size_t)r * (C / 16);
            for (uint32_t g = 0; g < C / 16; ++g) {
                const float scale = orc_e4m3(s[g]) / m->global_scale;
                for (uint32_t c = g * 16; c < g * 16 + 16; ++c) {
                    const uint32_t nib = (c & 1u) ? (p[c / 2] >> 4) : (p[c / 2] & 0xFu);
                    if (accumulate_double) dsum += (double)x[c] * val[nib] * (double)scale;
                    else sum += x[c] * val[nib] * scale;
                }
            }
        } else if (m->fmt == ORC_FMT_INT4G128) {
            const uint8_t* p = m->packed + (size_t)r * (C / 8) * 4;
            const uint8_t* s = m->scales + (size_t)r * (C / 128) * 2;
            for (uint32_t c = 0; c < C; ++c) {
                uint32_t w;
                memcpy(&w, p + (size_t)(c / 8) * 4, 4);
                const float q = (float)((int)((w >> ((c % 8u) * 4u)) & 0xFu) - 8);
                uint16_t sb;
                memcpy(&sb, s + (size_t)(c / 128) * 2, 2);
                const float scale = orc_bf16_to_f32(sb);
                if (accumulate_double) dsum += (double)x[c] * q * (double)scale;
                else sum += x[c] * q * scale;
            }
        } else if (m->fmt == ORC_FMT_BF16) {
            const uint16_t* p = (const uint16_t*)m->packed + (size_t)r * C;
            for (uint32_t c = 0; c < C; ++c) {
                if (accumulate_double) dsum += (double)x[c] * orc_bf16_to_f32(p[c]);
                else sum += x[c] * orc_bf16_to_f32(p[c]);
            }
        } else {
            return -2;
        }
        y[r] = accumulate_double ? (float)dsum : sum;
    }
    return 0;
}

/* ---------------------------------------------------------------- router */

/* logits[t, e] = sum_h x[t, h] * Wg[e, h] in the reference's production GPU
 * order (kernels/cuda/backend.cu:651-683 and 685-728): lane l of a 32-lane
 * warp accumulates columns l, l+32, ... with a separate multiply and add (no
 * FMA), then five shuffle-down rounds (16, 8, 4, 2, 1) fold the 32 partials;
 * lane 0 holds the result.  x and Wg are BF16; the products are fp32. */
ORC_API void orc_router_logits(const uint16_t* x_bf16, const uint16_t* wg_bf16, uint32_t T,
                               uint32_t H, uint32_t E, float* logits) {
    float* xf = (float*)malloc((size_t)T * H * sizeof(float));
    for (size_t i = 0; i < (size_t)T * H; ++i) xf[i] = orc_bf16_to_f32(x_bf16[i]);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < (int64_t)E; ++e) {
        float* wf = (float*)malloc((size_t)H * sizeof(float));
        for (uint32_t h = 0; h < H; ++h) wf[h] = orc_bf16_to_f32(wg_bf16[(size_t)e * H + h]);
        for (uint32_t t = 0; t < T; ++t) {
            const float* xr = xf + (size_t)t * H;
            float lane[32];
            for (int l = 0; l < 32; ++l) lane[l] = 0.0f;
            uint32_t h = 0;
            for (; h + 32 <= H; h += 32)
                for (int l = 0; l < 32; ++l) lane[l] = lane[l] + xr[h + l] * wf[h + l];
            for (int l = 0; h + (uint32_t)l < H; ++l) lane[l] = lane[l] + xr[h + l] * wf[h + l];
            /* __shfl_down_sync returns the caller's own value when the source
             * lane is out of range; only lanes that feed lane 0 matter. */
            for (int off = 16; off > 0; off >>= 1)
                for (int l = 0; l < off; ++l) lane[l] = lane[l] + lane[l + off];
            logits[(size_t)t * E + e] = lane[0];
        }
        free(wf);
    }
    free(xf);
}

typedef struct {
    uint32_t experts, top_k;
    int32_t score_kind;
    int32_t normalize;   /* divide the k selected scores by their sum */
    float norm_init;     /* GLM starts the normaliser at 1e-20 (glm_ops.cpp:228) */
    float weight_scale;  /* multiplied into each weight after normalisation (GLM 2.5, DSV4 1.5) */
    float softcap;       /* Laguna tanh soft-cap on the logit; 0 = off (laguna_ops.cpp:208-210) */
} orc_router_spec;

/* One row of routing.  Follows
 *   GLM    src/models/glm52/glm_ops.cpp:176-233
 *   Laguna src/models/laguna/laguna_ops.cpp:182-243
 *   Kimi   src/models/kimi_k3/kimi_k3_ops.cpp:192-237
 *   DSV4   src/models/dsv4/deepseek_ops.cpp:82-133
 * which share one rule: score every expert, select top-k on (score + bias)
 * with the lower index winning ties, take the UNBIASED scores of the selected
 * experts in selection-rank order, sum them in that order, divide, scale.
 * k passes of strict-greater arg-max and partial_sort by (value desc, index
 * asc) pick the same sequence.  scratch holds 2*experts floats.
 * Returns 0, or -1 on a non-finite logit/bias, -2 when the normaliser is not
 * positive and finite. */
ORC_API int orc_route_row(const orc_router_spec* s, const float* logits, const float* bias,
                          float* scratch, uint32_t* ids, float* weights) {
    const uint32_t E = s->experts, k = s->top_k;
    float* score = scratch;
    float* choice = scratch + E;
    if (s->score_kind == ORC_SCORE_SOFTMAX) {
        float mx = -INFINITY;
        for (uint32_t e = 0; e < E; ++e) {
            if (!isfinite(logits[e])) return -1;
            if (logits[e] > mx) mx = logits[e];
        }
        float sum = 0.0f;
        for (uint32_t e = 0; e < E; ++e) {
            score[e] = expf(logits[e] - mx);
            sum += score[e];
        }
        for (uint32_t e = 0; e < E; ++e) score[e] = score[e] / sum;
    } else {
        for (uint32_t e = 0; e < E; ++e) {
            float l = logits[e];
            if (!isfinite(l)) return -1;
            if (s->softcap > 0.0f) l = tanhf(l / s->softcap) * s->softcap;
            if (s->score_kind == ORC_SCORE_SIGMOID) score[e] = orc_sigmoid(l);
            else if (s->score_kind == ORC_SCORE_SIGMOID_PLAIN) score[e] = 1.0f / (1.0f + expf(-l));
            else score[e] = sqrtf(orc_softplus(l));
        }
    }
    for (uint32_t e = 0; e < E; ++e) {
        const float b = bias ? bias[e] : 0.0f;
        if (!isfinite(b)) return -1;
        choice[e] = score[e] + b;
    }
    for (uint32_t r = 0; r < k; ++r) {
        uint32_t best = 0;
        float best_v = -INFINITY;
        int found = 0;
        for (uint32_t e = 0; e < E; ++e) {
            int taken = 0;
            for (uint32_t j = 0; j < r; ++j) taken |= (ids[j] == e);
            if (taken) continue;
            if (!found || choice[e] > best_v) { best = e; best_v = choice[e]; found = 1; }
        }
        ids[r] = best;
        weights[r] = score[best];
    }
    if (s->normalize) {
        float sum = s->norm_init;
        for (uint32_t r = 0; r < k; ++r) sum += weights[r];
        if (!(sum > 0.0f) || !isfinite(sum)) return -2;
        for (uint32_t r = 0; r < k; ++r) weights[r] = weights[r] / sum * s->weight_scale;
    } else {
        for (uint32_t r = 0; r < k; ++r) weights[r] = weights[r] * s->weight_scale;
    }
    return 0;
}

/* Inkling's sink router, inkling_route_sigmoid_sink (src/models/inkling/inkling_ops.cpp:184-275).
 * logits holds the E routed experts followed by S shared "sink" experts.  Selection: top-k of
 * sigmoid(logit) + bias over the ROUTED range (lower index wins ties).  Weights: the RAW logits of the k
 * selected experts and of every sink go through log-sigmoid (min(x,0) - log1p(exp(-|x|)),
 * src/platform/numerics.cpp:54-59), then a softmax over that joint set (maximum subtracted, sum in index
 * order), times scale = routed_scale * global_scale.  ids / weights: k selected then S sinks (ids E..E+S-1).
 * Returns 0, -1 on a non-finite logit or bias, -2 when the softmax sum is not positive and finite. */
ORC_API int orc_route_sigmoid_sink(const float* logits, const float* bias, uint32_t E, uint32_t S, uint32_t k,
                                   float scale, float* scratch /* E */, uint32_t* ids, float* weights) {
    if (k == 0 || k > E) return -3;
    for (uint32_t e = 0; e < E + S; ++e)
        if (!isfinite(logits[e])) return -1;
    for (uint32_t e = 0; e < E; ++e) {
        if (!isfinite(bias[e])) return -1;
        scratch[e] = orc_sigmoid(logits[e]) + bias[e];
    }
    for (uint32_t r = 0; r < k; ++r) {
        uint32_t best = 0;
        float best_v = -INFINITY;
        for (uint32_t e = 0; e < E; ++e)
            if (scratch[e] > best_v) { best_v = scratch[e]; best = e; }
        ids[r] = best;
        scratch[best] = -INFINITY;
    }
    for (uint32_t i = 0; i < S; ++i) ids[k + i] = E + i;
    float mx = -INFINITY;
    for (uint32_t i = 0; i < k + S; ++i) {
        const float v = logits[ids[i]];
        weights[i] = fminf(v, 0.0f) - log1pf(expf(-fabsf(v)));
        if (weights[i] > mx) mx = weights[i];
    }
    float total = 0.0f;
    for (uint32_t i = 0; i < k + S; ++i) {
        weights[i] = expf(weights[i] - mx);
        total += weights[i];
    }
    if (!(total > 0.0f) || !isfinite(total)) return -2;
    for (uint32_t i = 0; i < k + S; ++i) weights[i] = weights[i] / total * scale;
    return 0;
}

/* Hash routing, dsv4_route_hash_sqrtsoftplus_f32_into (src/models/dsv4/deepseek_ops.cpp:414-461): the
 * experts are given, the weights are their scores summed in rank order, normalised and scaled.  Stated
 * for every score kind; softmax is not covered (it has no reference).  Returns -3 for an id >= E. */
ORC_API int orc_route_given_row(const orc_router_spec* s, const float* logits, const uint32_t* token_experts,
                                uint32_t* ids, float* weights) {
    const uint32_t E = s->experts, k = s->top_k;
    for (uint32_t e = 0; e < E; ++e)
        if (!isfinite(logits[e])) return -1;
    for (uint32_t r = 0; r < k; ++r) {
        const uint32_t e = token_experts[r];
        if (e >= E) return -3;
        float l = logits[e];
        if (s->softcap > 0.0f) l = tanhf(l / s->softcap) * s->softcap;
        ids[r] = e;
        if (s->score_kind == ORC_SCORE_SIGMOID) weights[r] = orc_sigmoid(l);
        else if (s->score_kind == ORC_SCORE_SIGMOID_PLAIN) weights[r] = 1.0f / (1.0f + expf(-l));
        else if (s->score_kind == ORC_SCORE_SQRTSOFTPLUS) weights[r] = sqrtf(orc_softplus(l));
        else return -4;
    }
    if (s->normalize) {
        float sum = s->norm_init;
        for (uint32_t r = 0; r < k; ++r) sum += weights[r];
        if (!(sum > 0.0f) || !isfinite(sum)) return -2;
        for (uint32_t r = 0; r < k; ++r) weights[r] = weights[r] / sum * s->weight_scale;
    } else {
        for (uint32_t r = 0; r < k; ++r) weights[r] = weights[r] * s->weight_scale;
    }
    return 0;
}

ORC_API int orc_route(const orc_router_spec* s, const float* logits, const float* bias, uint32_t T,
                      uint32_t* ids, float* weights) {
    int rc = 0;
#pragma omp parallel
    {
        float* scratch = (float*)malloc((size_t)2 * s->experts * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t t = 0; t < (int64_t)T; ++t) {
            const int r = orc_route_row(s, logits + (size_t)t * s->experts, bias, scratch,
                                        ids + (size_t)t * s->top_k, weights + (size_t)t * s->top_k);
            if (r != 0) {
#pragma omp critical
                rc = r;
            }
        }
        free(scratch);
    }
    return rc;
}

/* Token -> expert grouping.  The reference builds, for every expert, the list
 * of (token, rank) pairs that chose it by scanning tokens then ranks in
 * row-major order (src/models/glm52/glm_runtime.cpp:1521-1541,
 * src/models/dsv4/deepseek_runtime.cpp:6216-6284; offsets are the exclusive
 * prefix of the group sizes, deepseek_runtime.cpp:6309-6321).  Groups are laid
 * out here in ascending expert id (as src/models/inkling/inkling_runtime.cpp:
 * 792-798 and src/models/kimi_k3/kimi_k3_layer.cpp:839-846 order them); the
 * lists and counts are the same under either group order.
 * perm[pos] = token * k + rank; offsets has E + 1 entries. */
ORC_API void orc_group(const uint32_t* ids, uint32_t T, uint32_t k, uint32_t E, uint32_t* counts,
                       uint32_t* offsets, uint32_t* perm) {
    memset(counts, 0, (size_t)E * sizeof(uint32_t));
    for (size_t i = 0; i < (size_t)T * k; ++i) counts[ids[i]]++;
    offsets[0] = 0;
    for (uint32_t e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + counts[e];
    uint32_t* cursor = (uint32_t*)malloc((size_t)E * sizeof(uint32_t));
    memcpy(cursor, offsets, (size_t)E * sizeof(uint32_t));
    for (uint32_t i = 0; i < T * k; ++i) perm[cursor[ids[i]]++] = i;
    free(cursor);
}

/* --------------------------------------------------------------- experts */
typedef struct {
    orc_matrix gate, up, down; /* gate/up [I, H], down [H, I] */
    int32_t activation;        /* 0 = SwiGLU, 1 = SiTU-GLU */
    float gate_beta, linear_beta;
} orc_expert;

/* kimi_situ_glu, src/models/kimi_k3/kimi_k3_ops.cpp:39-62: both factors of the first bracket read
 * the gate projection (tanh bounds it, the plain sigmoid of :12-14 gates it). */
ORC_API float orc_situ_glu(float g, float u, float gate_beta, float linear_beta) {
    const float sig = 1.0f / (1.0f + expf(-g));
    const float bounded = gate_beta * tanhf(g / gate_beta) * sig;
    const float linear = linear_beta * tanhf(u / linear_beta);
    return bounded * linear;
}

/* One expert applied to one row: act = silu(gate.x) * up.x
 * (kernels/cuda/backend.cu:2016-2032; silu as gate * sigmoid(gate) with the
 * two-branch sigmoid), then y = down.act (backend.cu:2035-2069).  If
 * coef_before_down the routing coefficient multiplies the activation, as the
 * INT4 device path does (backend.cu:1933); otherwise the caller scales y. */
ORC_API int orc_expert_ffn(const orc_expert* ex, const float* x, float coef, int coef_before_down,
                           int accumulate_double, float* act_scratch, float* up_scratch, float* y) {
    const uint32_t I = ex->gate.rows;
    int rc = orc_matvec(&ex->gate, x, act_scratch, 0, I, accumulate_double);
    if (rc) return rc;
    rc = orc_matvec(&ex->up, x, up_scratch, 0, I, accumulate_double);
    if (rc) return rc;
    for (uint32_t i = 0; i < I; ++i) {
        const float g = act_scratch[i];
        float a = ex->activation == 1 ? orc_situ_glu(g, up_scratch[i], ex->gate_beta, ex->linear_beta)
                                      : g * orc_sigmoid(g) * up_scratch[i];
        if (coef_before_down) a = a * coef;
        act_scratch[i] = a;
    }
    return orc_matvec(&ex->down, act_scratch, y, 0, ex->down.rows, accumulate_double);
}

typedef struct {
    uint32_t T, H, I, E, k;
    orc_router_spec router;
    float output_scale;        /* Laguna scales the summed routed output (laguna_runtime.cpp:1141-1143) */
    int32_t combine_order;     /* ORC_COMBINE_* */
    int32_t coef_before_down;
    int32_t accumulate_double;
    uint32_t I_shared;         /* 0 = no shared expert */
} orc_layer_desc;

/* Whole layer for a subset of tokens (token_subset == NULL: all tokens).
 * Routing and grouping are always computed for all T tokens; expert FFNs only
 * for the subset, which keeps full-size shapes checkable in seconds.
 *
 * Combine: out[t] = output_scale * sum_r w[t, r] * y[t, r] + shared(x[t]).
 *   RANK_ORDER: r ascending (src/models/dsv4/deepseek_runtime.cpp:5902-5910,
 *               src/models/inkling/inkling_runtime.cpp:856-868).
 *   JOB_ORDER:  experts in order of first appearance over the (token, rank)
 *               scan, `dest += src * w` per job
 *               (src/models/glm52/glm_runtime.cpp:1586-1608,
 *               src/models/laguna/laguna_runtime.cpp:1129-1139).
 * Shared expert: BF16 gate/up/down, silu(gate.x) * up.x then down, added last
 * (laguna_runtime.cpp:887-905, 1145-1156; glm_runtime.cpp:1610-1612).
 * experts[e] may have NULL data when no subset token routes to e. */
ORC_API int orc_moe_layer(const orc_layer_desc* d, const uint16_t* x_bf16, const uint16_t* router_w,
                          const float* bias, const orc_expert* experts, const orc_expert* shared,
                          const uint32_t* token_subset, uint32_t n_subset, float* logits_out,
                          uint32_t* ids, float* weights, uint32_t* counts, uint32_t* offsets,
                          uint32_t* perm, float* out) {
    const uint32_t T = d->T, H = d->H, I = d->I, E = d->E, k = d->k;
    float* logits = logits_out ? logits_out : (float*)malloc((size_t)T * E * sizeof(float));
    orc_router_logits(x_bf16, router_w, T, H, E, logits);
    int rc = orc_route(&d->router, logits, bias, T, ids, weights);
    if (!logits_out) free(logits);
    if (rc) return rc;
    orc_group(ids, T, k, E, counts, offsets, perm);
    if (!out) return 0;

    /* first-appearance order of experts over the row-major (token, rank) scan */
    uint32_t* job_rank = (uint32_t*)malloc((size_t)E * sizeof(uint32_t));
    for (uint32_t e = 0; e < E; ++e) job_rank[e] = 0xFFFFFFFFu;
    uint32_t jobs = 0;
    for (size_t i = 0; i < (size_t)T * k; ++i)
        if (job_rank[ids[i]] == 0xFFFFFFFFu) job_rank[ids[i]] = jobs++;

    const uint32_t n = token_subset ? n_subset : T;
    int fail = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t si = 0; si < (int64_t)n; ++si) {
        const uint32_t t = token_subset ? token_subset[si] : (uint32_t)si;
        float* xf = (float*)malloc((size_t)H * sizeof(float));
        float* y = (float*)malloc((size_t)k * H * sizeof(float));
        const uint32_t imax = I > d->I_shared ? I : d->I_shared;
        float* a = (float*)malloc((size_t)imax * sizeof(float));
        float* u = (float*)malloc((size_t)imax * sizeof(float));
        for (uint32_t h = 0; h < H; ++h) xf[h] = orc_bf16_to_f32(x_bf16[(size_t)t * H + h]);
        uint32_t order[64];
        for (uint32_t r = 0; r < k; ++r) {
            order[r] = r;
            const orc_expert* ex = &experts[ids[(size_t)t * k + r]];
            if (!ex->gate.packed ||
                orc_expert_ffn(ex, xf, weights[(size_t)t * k + r], d->coef_before_down,
                               d->accumulate_double, a, u, y + (size_t)r * H)) {
#pragma omp critical
                fail = 1;
            }
        }
        if (d->combine_order == ORC_COMBINE_JOB_ORDER) {
            for (uint32_t i = 1; i < k; ++i) { /* insertion sort of ranks by job index */
                const uint32_t r = order[i];
                uint32_t j = i;
                while (j > 0 && job_rank[ids[(size_t)t * k + order[j - 1]]] >
                                    job_rank[ids[(size_t)t * k + r]]) {
                    order[j] = order[j - 1];
                    --j;
                }
                order[j] = r;
            }
        }
        float* o = out + (size_t)si * H;
        for (uint32_t h = 0; h < H; ++h) o[h] = 0.0f;
        for (uint32_t i = 0; i < k; ++i) {
            const uint32_t r = order[i];
            const float w = d->coef_before_down ? 1.0f : weights[(size_t)t * k + r];
            const float* yr = y + (size_t)r * H;
            for (uint32_t h = 0; h < H; ++h) o[h] += yr[h] * w;
        }
        if (d->output_scale != 1.0f)
            for (uint32_t h = 0; h < H; ++h) o[h] *= d->output_scale;
        if (shared && d->I_shared) {
            if (orc_expert_ffn(shared, xf, 1.0f, 0, d->accumulate_double, a, u, y)) {
#pragma omp critical
                fail = 1;
            }
            for (uint32_t h = 0; h < H; ++h) o[h] += y[h];
        }
        free(xf); free(y); free(a); free(u);
    }
    free(job_rank);
    return fail ? -3 : 0;
}

/* Timed CPU arm ("port"): the routed-expert part of one layer for all T tokens
 * using every OpenMP thread, expert-major so each expert's weights are read
 * once per call.  Returns 0.  Used only by bench.py's cpu_baseline leg. */
ORC_API int orc_experts_all(const orc_layer_desc* d, const uint16_t* x_bf16, const orc_expert* experts,
                            const uint32_t* ids, const float* weights, const uint32_t* offsets,
                            const uint32_t* perm, float* y_pairs /* [T*k, H] by pair position */) {
    const uint32_t H = d->H, I = d->I, E = d->E, k = d->k;
    int fail = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t e = 0; e < (int64_t)E; ++e) {
        if (offsets[e + 1] == offsets[e]) continue;
        float* xf = (float*)malloc((size_t)H * sizeof(float));
        float* a = (float*)malloc((size_t)I * sizeof(float));
        float* u = (float*)malloc((size_t)I * sizeof(float));
        for (uint32_t pos = offsets[e]; pos < offsets[e + 1]; ++pos) {
            const uint32_t pair = perm[pos], t = pair / k;
            for (uint32_t h = 0; h < H; ++h) xf[h] = orc_bf16_to_f32(x_bf16[(size_t)t * H + h]);
            if (orc_expert_ffn(&experts[e], xf, weights[pair], d->coef_before_down, 0, a, u,
                               y_pairs + (size_t)pos * H)) {
#pragma omp critical
                fail = 1;
            }
        }
        free(xf); free(a); free(u);
    }
    (void)ids;
    return fail ? -3 : 0;
}

/* ======================================================================================
 * DSV4-exact expert (bit-exact numerical mode of the DeepSeek-V4 routed expert).
 * Follows kernels/cpu/dsv4_fp4_expert.cpp, which itself replays the device kernels
 * deepseek_fp4_gate_up_kernel / deepseek_fp4_down_kernel / quantize_activation_e4m3_kernel
 * (kernels/cuda/backend.cu:247-272, 2308-2413).
 * ====================================================================================== */

/* bf16_round, kernels/cpu/dsv4_fp4_expert.cpp:94-104 (__float2bfloat16_rn widened back). */
ORC_API float orc_bf16_round(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    if ((bits & 0x7FFFFFFFu) > 0x7F800000u) bits = (bits | 0x00400000u) & 0xFFFF0000u;
    else bits = (bits + 0x7FFFu + ((bits >> 16) & 1u)) & 0xFFFF0000u;
    memcpy(&value, &bits, 4);
    return value;
}

/* quantize_e4m3_value, kernels/cpu/dsv4_fp4_expert.cpp:58-72 (backend.cu:212-225). */
ORC_API float orc_quantize_e4m3_value(float value) {
    const float magnitude = fminf(fabsf(value), 448.0f);
    float quantized;
    if (magnitude < 0.015625f) {
        quantized = rintf(ldexpf(magnitude, 9)) * ldexpf(1.0f, -9);
    } else {
        int exponent = 0;
        (void)frexpf(magnitude, &exponent);
        exponent = exponent - 1;
        if (exponent > 8) exponent = 8;
        if (exponent < -6) exponent = -6;
        const float step = ldexpf(1.0f, exponent - 3);
        quantized = fminf(rintf(magnitude / step) * step, 448.0f);
    }
    return copysignf(quantized, value);
}

/* quantize_activation_e4m3, kernels/cpu/dsv4_fp4_expert.cpp:78-92: one power-of-two scale
 * per 128-column block of one row, in place. */
ORC_API void orc_quantize_activation_e4m3(float* values, uint64_t columns) {
    for (uint64_t begin = 0; begin < columns; begin += 128u) {
        const uint64_t end = begin + 128u < columns ? begin + 128u : columns;
        float maximum = 0.0f;
        for (uint64_t i = begin; i < end; ++i) maximum = fmaxf(maximum, fabsf(values[i]));
        float scale = 1.0f;
        if (maximum > 0.0f) scale = exp2f(ceilf(log2f(maximum / 448.0f)));
        for (uint64_t i = begin; i < end; ++i) values[i] = orc_quantize_e4m3_value(values[i] / scale) * scale;
    }
}

/* e8m0_scale with the DSV4 edge rule, kernels/cpu/dsv4_fp4_expert.cpp:46-52. */
static float dsv4_e8m0(uint8_t bits) {
    uint32_t u = bits == 0xFFu ? 0x7FC00000u : (bits == 0u ? 0x00400000u : (uint32_t)bits << 23);
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* One output row: 256 strided partial sums (row_partials_scalar, :146-163) reduced by the
 * device's block tree (reduce_lane0 / reduce_block, :111-144). */
static float dsv4_row(const float* input, const uint8_t* packed, const uint8_t* scales, uint64_t columns,
                      uint64_t packed_base, uint64_t scale_base) {
    static const float kValue[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                     -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
    float partials[256];
    for (uint32_t thread = 0; thread < 256u; ++thread) {
        float sum = 0.0f;
        for (uint64_t c = thread; c < columns; c += 256u) {
            const uint8_t byte = packed[packed_base + c / 2u];
            const unsigned enc = (c % 2u == 0u) ? (byte & 0x0Fu) : (byte >> 4);
            const float scale = dsv4_e8m0(scales[scale_base + c / 32u]);
            sum = fmaf(input[c] * kValue[enc], scale, sum);
        }
        partials[thread] = sum;
    }
    float ws[8];
    for (uint32_t w = 0; w < 8u; ++w) {
        const float* l = partials + w * 32u;
        float a[16];
        for (int i = 0; i < 16; ++i) a[i] = l[i] + l[i + 16];
        for (int i = 0; i < 8; ++i) a[i] += a[i + 8];
        for (int i = 0; i < 4; ++i) a[i] += a[i + 4];
        a[0] += a[2];
        a[1] += a[3];
        ws[w] = a[0] + a[1];
    }
    for (int i = 0; i < 8; ++i) ws[i] += 0.0f;
    for (int i = 0; i < 4; ++i) ws[i] += ws[i + 4];
    ws[0] += ws[2];
    ws[1] += ws[3];
    return ws[0] + ws[1];
}

/* dsv4_host_expert_fp4, kernels/cpu/dsv4_fp4_expert.cpp:864-884 with its phases :774-862.
 * in [hidden] fp32 (raw hidden state), out [hidden].  scratch [intermediate] receives the
 * quantised activation.  Returns 1 when gate/up produced a non-finite value. */
ORC_API int orc_dsv4_expert(float* out, const float* in, const uint8_t* w1, const uint8_t* s1, const uint8_t* w3,
                            const uint8_t* s3, const uint8_t* w2, const uint8_t* s2, uint32_t hidden,
                            uint32_t intermediate, float coefficient, float swiglu_limit, float* scratch) {
    float* q = (float*)malloc((size_t)hidden * sizeof(float));
    memcpy(q, in, (size_t)hidden * sizeof(float));
    orc_quantize_activation_e4m3(q, hidden);
    for (uint64_t row = 0; row < intermediate; ++row) {
        const float g = orc_bf16_round(dsv4_row(q, w1, s1, hidden, row * (hidden / 2u), row * (hidden / 32u)));
        const float u = orc_bf16_round(dsv4_row(q, w3, s3, hidden, row * (hidden / 2u), row * (hidden / 32u)));
        if (!isfinite(g) || !isfinite(u)) {
            free(q);
            return 1;
        }
        const float lg = fminf(g, swiglu_limit);
        const float lu = fmaxf(-swiglu_limit, fminf(u, swiglu_limit));
        uint32_t gb;
        memcpy(&gb, &lg, 4);
        gb &= 0xFFFF0000u;                      /* the table is indexed by the top 16 bits */
        float gt;
        memcpy(&gt, &gb, 4);
        const float silu = isfinite(gt) ? orc_silu(gt) : gt;
        float act = silu * lu;
        act *= coefficient;
        scratch[row] = orc_bf16_round(act);
    }
    free(q);
    orc_quantize_activation_e4m3(scratch, intermediate);
    for (uint64_t row = 0; row < hidden; ++row)
        out[row] = orc_bf16_round(dsv4_row(scratch, w2, s2, intermediate, row * (intermediate / 2u),
                                           row * (intermediate / 32u)));
    return 0;
}

/* ======================================================================================
 * DSV4 shared expert: FP8 E4M3 weights with one E8M0 scale per 128 x 128 block.
 * The reference has no CPU replay of these kernels (its host function dsv4_fp8_e4m3_matvec_f32,
 * src/models/dsv4/deepseek_ops.cpp:523-560, accumulates in double and is only tolerance-close), so this
 * function is PINNED THROUGH THE REFERENCE'S GPU KERNELS instead: the ported command cases
 * (tests/cpp/backend_shim_test.cpp, built against the reference's own backend by oracle/build.py) compare
 * the reference backend's shared-expert output with this function bit for bit at hidden = intermediate = 128
 * and at the DeepSeek-V4 shape 4096 / 2048.  This restates the DEVICE kernels
 * deepseek_fp8_gate_up_kernel / deepseek_fp8_down_kernel (kernels/cuda/backend.cu:2781-2863):
 * thread t of a 256-thread block sums columns t, t + 256, ... with sum = fma(x * w, scale, sum),
 * then the same block tree as the FP4 kernels; decode fp8_e4m3_value (:159-173).
 * ====================================================================================== */
static float dsv4_fp8_value(uint8_t enc) {
    const unsigned exponent = (enc >> 3) & 0x0Fu, mantissa = enc & 7u;
    float value;
    if (exponent == 0u) value = ldexpf((float)mantissa / 8.0f, -6);
    else if (exponent == 0x0Fu && mantissa == 7u) return nanf("");
    else value = ldexpf(1.0f + (float)mantissa / 8.0f, (int)exponent - 7);
    return (enc & 0x80u) ? -value : value;
}

static float dsv4_fp8_row(const float* input, const uint8_t* weights, const uint8_t* scales, uint64_t columns,
                          uint64_t row) {
    const uint64_t scale_columns = (columns + 127u) / 128u;
    float partials[256];
    for (uint32_t thread = 0; thread < 256u; ++thread) {
        float sum = 0.0f;
        for (uint64_t c = thread; c < columns; c += 256u) {
            const float scale = dsv4_e8m0(scales[(row / 128u) * scale_columns + c / 128u]);
            sum = fmaf(input[c] * dsv4_fp8_value(weights[row * columns + c]), scale, sum);
        }
        partials[thread] = sum;
    }
    float ws[8];
    for (uint32_t w = 0; w < 8u; ++w) {
        const float* l = partials + w * 32u;
        float a[16];
        for (int i = 0; i < 16; ++i) a[i] = l[i] + l[i + 16];
        for (int i = 0; i < 8; ++i) a[i] += a[i + 8];
        for (int i = 0; i < 4; ++i) a[i] += a[i + 4];
        a[0] += a[2];
        a[1] += a[3];
        ws[w] = a[0] + a[1];
    }
    for (int i = 0; i < 8; ++i) ws[i] += 0.0f;
    for (int i = 0; i < 4; ++i) ws[i] += ws[i + 4];
    ws[0] += ws[2];
    ws[1] += ws[3];
    return ws[0] + ws[1];
}

/* The shared expert of one row: quantise the hidden state, FP8 gate/up with BF16 rounding, clamp,
 * SiLU of the BF16 gate, BF16 activation, quantise, FP8 down, BF16 output (the sequence of
 * enqueue_deepseek_moe, kernels/cuda/backend.cu:14509-14625).  Returns 1 on a non-finite gate/up. */
ORC_API int orc_dsv4_fp8_shared(float* out, const float* in, const uint8_t* w1, const uint8_t* s1, const uint8_t* w3,
                                const uint8_t* s3, const uint8_t* w2, const uint8_t* s2, uint32_t hidden,
                                uint32_t intermediate, float swiglu_limit, float* scratch) {
    float* q = (float*)malloc((size_t)hidden * sizeof(float));
    memcpy(q, in, (size_t)hidden * sizeof(float));
    orc_quantize_activation_e4m3(q, hidden);
    for (uint64_t row = 0; row < intermediate; ++row) {
        const float g = orc_bf16_round(dsv4_fp8_row(q, w1, s1, hidden, row));
        const float u = orc_bf16_round(dsv4_fp8_row(q, w3, s3, hidden, row));
        if (!isfinite(g) || !isfinite(u)) {
            free(q);
            return 1;
        }
        const float lg = fminf(g, swiglu_limit);
        const float lu = fmaxf(-swiglu_limit, fminf(u, swiglu_limit));
        uint32_t gb;
        memcpy(&gb, &lg, 4);
        gb &= 0xFFFF0000u;
        float gt;
        memcpy(&gt, &gb, 4);
        const float silu = isfinite(gt) ? orc_silu(gt) : gt;
        scratch[row] = orc_bf16_round(silu * lu);
    }
    free(q);
    orc_quantize_activation_e4m3(scratch, intermediate);
    for (uint64_t row = 0; row < hidden; ++row) out[row] = orc_bf16_round(dsv4_fp8_row(scratch, w2, s2, intermediate, row));
    return 0;
}

/* ======================================================================================
 * LatentMoE (Kimi-K3), following kimi_latent_moe_layer, src/models/kimi_k3/kimi_k3_layer.cpp:781-1001:
 *   route on the raw hidden state (router logits in this file's canonical order -- the reference's
 *   kimi_bf16_matmul uses an 8-lane FMA order, see the note on orc_router_logits);
 *   latent = x . down^T (BF16 weights, FP32 accumulation);  every selected expert runs on the FP32
 *   latent (gate/up, SiTU-GLU, down) and weight * output is added to the token's mixture in
 *   ASCENDING EXPERT order (one worker's order, :906-938);  the mixture is RMS-normalised
 *   (kimi_rms_norm, src/models/kimi_k3/kimi_k3_ops.cpp:16-38) and projected back with up;
 *   the shared experts (one concatenated BF16 expert) run on the raw hidden state and add in.
 * Plain sequential FP32 sums for the BF16 projections (the reference's AVX2 order differs in the
 * last bits; comparisons with it are tolerance-level).
 * d->H is the latent width, H_model the layer's input width.  Expert FFNs only for token_subset.
 * ====================================================================================== */
static void orc_bf16_linear(const float* x, const uint16_t* w, uint32_t rows, uint32_t cols, float* y) {
    for (uint32_t r = 0; r < rows; ++r) {
        float sum = 0.0f;
        const uint16_t* wr = w + (size_t)r * cols;
        for (uint32_t c = 0; c < cols; ++c) sum += x[c] * orc_bf16_to_f32(wr[c]);
        y[r] = sum;
    }
}

ORC_API int orc_latent_moe_layer(const orc_layer_desc* d, uint32_t H_model, float rms_epsilon, const uint16_t* x_bf16,
                                 const uint16_t* router_w, const float* bias, const uint16_t* latent_down,
                                 const uint16_t* latent_up, const float* latent_norm, const orc_expert* experts,
                                 const orc_expert* shared, const uint32_t* token_subset, uint32_t n_subset,
                                 uint32_t* ids, float* weights, float* out) {
    const uint32_t T = d->T, HL = d->H, I = d->I, E = d->E, k = d->k;
    float* logits = (float*)malloc((size_t)T * E * sizeof(float));
    orc_router_logits(x_bf16, router_w, T, H_model, E, logits);
    int rc = orc_route(&d->router, logits, bias, T, ids, weights);
    free(logits);
    if (rc) return rc;
    if (!out) return 0;
    const uint32_t n = token_subset ? n_subset : T;
    int fail = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (uint32_t s = 0; s < n; ++s) {
        const uint32_t t = token_subset ? token_subset[s] : s;
        float* xf = (float*)malloc((size_t)H_model * sizeof(float));
        float* latent = (float*)malloc((size_t)HL * sizeof(float));
        float* mix = (float*)calloc(HL, sizeof(float));
        float* y = (float*)malloc((size_t)(HL > H_model ? HL : H_model) * sizeof(float));
        const uint32_t Imax = (d->I_shared > I ? d->I_shared : I);
        float* a = (float*)malloc((size_t)Imax * sizeof(float));
        float* u = (float*)malloc((size_t)Imax * sizeof(float));
        for (uint32_t h = 0; h < H_model; ++h) xf[h] = orc_bf16_to_f32(x_bf16[(size_t)t * H_model + h]);
        orc_bf16_linear(xf, latent_down, HL, H_model, latent);
        /* ascending expert order over the token's selection */
        for (uint32_t e = 0; e < E; ++e) {
            float w = 0.0f;
            for (uint32_t r = 0; r < k; ++r)
                if (ids[(size_t)t * k + r] == e) { w = weights[(size_t)t * k + r]; break; }
            if (w == 0.0f) continue;
            if (orc_expert_ffn(&experts[e], latent, 1.0f, 0, d->accumulate_double, a, u, y)) {
#pragma omp critical
                fail = 1;
                break;
            }
            for (uint32_t h = 0; h < HL; ++h) mix[h] += w * y[h];
        }
        float ms = 0.0f;
        for (uint32_t h = 0; h < HL; ++h) ms += mix[h] * mix[h];
        const float scale = 1.0f / sqrtf(ms / (float)HL + rms_epsilon);
        for (uint32_t h = 0; h < HL; ++h) mix[h] = latent_norm[h] * (mix[h] * scale);
        float* o = out + (size_t)s * H_model;
        orc_bf16_linear(mix, latent_up, H_model, HL, o);
        if (shared) {
            if (orc_expert_ffn(shared, xf, 1.0f, 0, d->accumulate_double, a, u, y)) {
#pragma omp critical
                fail = 1;
            } else {
                for (uint32_t h = 0; h < H_model; ++h) o[h] += y[h];
            }
        }
        free(xf); free(latent); free(mix); free(y); free(a); free(u);
    }
    return fail;
}
