// Small-batch expert FFN for the FP4 formats (MXFP4, NVFP4): the weight-streaming kernel the
// decode roofline is measured on.
//
// Same work split as decode.cu (one warp streams two 16-row tiles over the whole K dimension
// with 16-byte loads straight into registers), but the decode is the hardware one:
// cvt.rn.f16x2.e2m1x2 turns one byte (two E2M1 nibbles, adjacent columns) into an exact f16
// pair, so a 32-bit weight word costs four conversions instead of a dozen integer
// instructions, and the A fragments of m16n8k16 F16 MMAs (FP32 accumulation) come out in
// natural column order -- the activation rows need no permutation.
//
// Block scales are folded into the f16 weights exactly with one packed multiply:
//   NVFP4: e2m1 * e4m3 has 6 significant bits and lies in [2^-10, 2688]: exact in f16.  The
//          per-tensor divisor is applied to the FP32 accumulator.
//   MXFP4: the E8M0 scale is a power of two; every expert/projection gets an exponent base e0
//          (from the smallest scale byte it holds, computed once on the device) and the weight
//          is multiplied by 2^(e - emin - 13), which keeps every product in f16's normal range
//          [2^-14, 49152]; 2^(emin + 13 - 127) goes to the accumulator.  This needs the expert's
//          scale bytes to span at most 26 octaves, else the layer uses the general kernel in
//          decode.cu.
// Activations are carried as f16 after an exact per-row power-of-two pre-scale that puts the
// row maximum in [2^14, 2^15): every BF16 activation within 2^-28 of the row maximum is
// represented exactly, smaller ones to within rowmax * 2^-39 -- below the rounding of the FP32
// accumulation itself.  FP32 activations (the SwiGLU output, fp32 callers) use an f16 hi/lo pair.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "rows_f16.cuh"

namespace smoe {

__device__ __forceinline__ uint4 ldg_stream16_b(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_f16_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 8 E2M1 nibbles (one 32-bit word, nibble q = column q) -> r[b] = f16x2 {column 2b, column 2b+1}
__device__ __forceinline__ void e2m1x8_f16(uint32_t w, uint32_t r[4]) {
    asm("{\n .reg .b8 b0, b1, b2, b3;\n mov.b32 {b0, b1, b2, b3}, %4;\n"
        " cvt.rn.f16x2.e2m1x2 %0, b0;\n cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        " cvt.rn.f16x2.e2m1x2 %2, b2;\n cvt.rn.f16x2.e2m1x2 %3, b3;\n}"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
        : "r"(w));
}
__device__ __forceinline__ uint32_t mul_f16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

constexpr int kMxBias = 2;  // f16 exponent field of the weight multiplier is e - emin + kMxBias (2..28)

struct Fp4Stream {
    const uint8_t* row_lo;
    const uint8_t* row_hi;
    const uint8_t* sc_lo;
    const uint8_t* sc_hi;
    int32_t mx_off;  // MXFP4: kMxBias - emin, added to the scale byte to form the f16 exponent field
};

template <int FMT>
__device__ __forceinline__ void fp4_init(Fp4Stream& p, const uint8_t* packed, const uint8_t* scales,
                                         uint32_t row, uint32_t K, uint32_t t, uint32_t emin) {
    p.row_lo = packed + (size_t)row * (K / 2u) + t * 16u;
    p.row_hi = packed + (size_t)(row + 8u) * (K / 2u) + t * 16u;
    if (FMT == STRATA_MOE_FMT_MXFP4) {
        p.sc_lo = scales + (size_t)row * (K / 32u) + t;
        p.sc_hi = scales + (size_t)(row + 8u) * (K / 32u) + t;
    } else {
        p.sc_lo = scales + (size_t)row * (K / 16u) + t * 2u;
        p.sc_hi = scales + (size_t)(row + 8u) * (K / 16u) + t * 2u;
    }
    p.mx_off = kMxBias - (int32_t)emin;
}

struct Fp4Load {
    uint4 lo, hi;
    uint32_t s_lo, s_hi;
};

template <int FMT>
__device__ __forceinline__ void fp4_load(const Fp4Stream& p, uint32_t kb, Fp4Load& L) {
    L.lo = ldg_stream16_b(p.row_lo + (size_t)kb * 64u);
    L.hi = ldg_stream16_b(p.row_hi + (size_t)kb * 64u);
    if (FMT == STRATA_MOE_FMT_MXFP4) {
        L.s_lo = __ldg(p.sc_lo + kb * 4u);
        L.s_hi = __ldg(p.sc_hi + kb * 4u);
    } else {
        L.s_lo = __ldg(reinterpret_cast<const unsigned short*>(p.sc_lo + kb * 8u));
        L.s_hi = __ldg(reinterpret_cast<const unsigned short*>(p.sc_hi + kb * 8u));
    }
}

// packed f16x2 multipliers of one 32-column chunk: m[0] for words 0-1, m[1] for words 2-3
template <int FMT>
__device__ __forceinline__ void fp4_mult(uint32_t s, int32_t mx_off, uint32_t m[2]) {
    if (FMT == STRATA_MOE_FMT_MXFP4) {
        const uint32_t h = (uint32_t)((int32_t)s + mx_off) << 10;  // f16 2^(e - emin + kMxBias - 15)
        m[0] = m[1] = h * 0x00010001u;
    } else {
        uint32_t pair;
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"((unsigned short)s));
        m[0] = __byte_perm(pair, pair, 0x1010);
        m[1] = __byte_perm(pair, pair, 0x3232);
    }
}

__device__ __forceinline__ uint32_t pick4(const uint4& v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

template <int FMT, int NT, bool SPLIT>
__device__ __forceinline__ void fp4_step(const Fp4Load& L0, const Fp4Load& L1, const Fp4Stream& p0,
                                         const Fp4Stream& p1, const __half* const xh[NT],
                                         const __half* const xl[NT], const bool valid[NT], uint32_t kb,
                                         uint32_t t, float acc0[NT][4], float acc1[NT][4]) {
    const uint4 zero = make_uint4(0, 0, 0, 0);
    uint32_t m0l[2], m0h[2], m1l[2], m1h[2];
    fp4_mult<FMT>(L0.s_lo, p0.mx_off, m0l);
    fp4_mult<FMT>(L0.s_hi, p0.mx_off, m0h);
    fp4_mult<FMT>(L1.s_lo, p1.mx_off, m1l);
    fp4_mult<FMT>(L1.s_hi, p1.mx_off, m1h);
    // activation fragments of this step: 32 columns per lane, natural order
    uint4 bh[NT][4], bl[SPLIT ? NT : 1][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
            const size_t off = (size_t)kb * 128u + t * 32u + wd * 8u;
            bh[nt][wd] = valid[nt] ? __ldg(reinterpret_cast<const uint4*>(xh[nt] + off)) : zero;
            if (SPLIT) bl[nt][wd] = valid[nt] ? __ldg(reinterpret_cast<const uint4*>(xl[nt] + off)) : zero;
        }
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const Fp4Load& L = s ? L1 : L0;
            uint32_t a[4], b[4];
            e2m1x8_f16(pick4(L.lo, wd), a);
            e2m1x8_f16(pick4(L.hi, wd), b);
            const uint32_t ml = s ? m1l[wd >> 1] : m0l[wd >> 1];
            const uint32_t mh = s ? m1h[wd >> 1] : m0h[wd >> 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                a[j] = mul_f16x2(a[j], ml);
                b[j] = mul_f16x2(b[j], mh);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float* c = s ? acc1[nt] : acc0[nt];
                mma_f16_16816(c, a[0], b[0], a[1], b[1], bh[nt][wd].x, bh[nt][wd].y);
                mma_f16_16816(c, a[2], b[2], a[3], b[3], bh[nt][wd].z, bh[nt][wd].w);
                if (SPLIT) {
                    mma_f16_16816(c, a[0], b[0], a[1], b[1], bl[nt][wd].x, bl[nt][wd].y);
                    mma_f16_16816(c, a[2], b[2], a[3], b[3], bl[nt][wd].z, bl[nt][wd].w);
                }
            }
        }
    }
}

__device__ __forceinline__ float silu_mul_f(float g, float u) {
    const float e = __expf(-fabsf(g));
    const float sig = g >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
    return g * sig * u;
}

// DUAL = true : gate tile + up tile, SwiGLU epilogue, writes act fp32 [pairs, I]
// DUAL = false: two adjacent down tiles, writes y fp32 [pairs, H]
template <int FMT, int NT, bool SPLIT, bool DUAL>
__global__ void __launch_bounds__(128, NT == 1 ? 4 : (NT == 2 ? 3 : 2)) decode_fp4_kernel(DecodeArgs a) {
    const uint32_t lane = threadIdx.x & 31u, gid = lane >> 2, t = lane & 3u;
    const uint32_t K = DUAL ? a.H : a.I;
    const uint32_t R = DUAL ? a.I : a.H;
    const uint32_t tiles_per_group = DUAL ? R / 16u : R / 32u;
    const uint32_t n_act = a.active_list ? *a.n_active : a.n_groups;
    const uint32_t total = n_act * tiles_per_group;
    if (total == 0u) return;
    const uint32_t steps = K / 128u;
    const uint32_t warp = threadIdx.x >> 5;
    // Work split.  Normally one warp owns a tile for all of K.  When the tile count leaves the last round
    // of warps badly filled, two warps of a CTA share a tile instead, each taking half of K (partial sums
    // meet in shared memory): the granule halves, so the rounding loss of the last round halves too.
    const uint32_t r4 = (total + gridDim.x * 4u - 1u) / (gridDim.x * 4u);
    const uint32_t r2 = (total + gridDim.x * 2u - 1u) / (gridDim.x * 2u);
    const bool ksplit = (steps % 2u == 0u) && (steps >= 4u) && (r2 * 10u <= r4 * 18u);   // >= 10 % fewer rounds
    const uint32_t W = ksplit ? gridDim.x * 2u : gridDim.x * 4u;
    const uint32_t rounds = (total + W - 1u) / W;
    const uint32_t W_eff = (total + rounds - 1u) / rounds;
    const uint32_t wid = ksplit ? blockIdx.x * 2u + (warp >> 1) : blockIdx.x * 4u + warp;
    const uint32_t khalf = ksplit ? (warp & 1u) : 0u;
    if (wid >= W_eff) return;     // both warps of a pair leave together
    const uint32_t kb_begin = ksplit ? khalf * (steps / 2u) : 0u;
    const uint32_t kb_end = ksplit ? kb_begin + steps / 2u : steps;
    __shared__ float xch[2][32][NT * 8];
    bool bad = false;
    const __half* bh_base = reinterpret_cast<const __half*>(DUAL ? a.x_hi : a.act_hi);
    const __half* bl_base = reinterpret_cast<const __half*>(DUAL ? a.x_lo : a.act_lo);
    const float* rowscale = DUAL ? a.x_rowscale : a.act_rowscale;

    for (uint32_t tile = wid; tile < total; tile += W_eff) {
        const uint32_t slot = tile / tiles_per_group;
        const uint32_t g = a.active_list ? a.active_list[slot] : slot;
        const uint32_t rt = tile - slot * tiles_per_group;
        const uint32_t row0 = a.offsets[g], cnt = a.offsets[g + 1] - row0;
        if (cnt == 0u || (a.skip_from != 0u && cnt >= a.skip_from)) continue;   // big groups: tensor-core path
        const uint32_t row = (DUAL ? rt * 16u : rt * 32u) + gid;

        Fp4Stream p0, p1;
        float s0, s1;
        if (DUAL) {
            fp4_init<FMT>(p0, a.gate.packed[g], a.gate.scales[g], row, K, t, a.gate.emin ? a.gate.emin[g] : 0u);
            fp4_init<FMT>(p1, a.up.packed[g], a.up.scales[g], row, K, t, a.up.emin ? a.up.emin[g] : 0u);
            s0 = a.gate.post_scale[g];
            s1 = a.up.post_scale[g];
        } else {
            const uint32_t em = a.down.emin ? a.down.emin[g] : 0u;
            fp4_init<FMT>(p0, a.down.packed[g], a.down.scales[g], row, K, t, em);
            fp4_init<FMT>(p1, a.down.packed[g], a.down.scales[g], row + 16u, K, t, em);
            s0 = s1 = a.down.post_scale[g];
        }

        for (uint32_t tb = 0; tb < cnt; tb += 8u * NT) {
            const __half* xh[NT];
            const __half* xl[NT];
            bool valid[NT];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t tok = tb + nt * 8u + gid;
                valid[nt] = tok < cnt;
                const size_t r = (size_t)(row0 + (valid[nt] ? tok : 0u)) * K;
                xh[nt] = bh_base + r;
                xl[nt] = SPLIT ? bl_base + r : nullptr;
            }
            float acc0[NT][4], acc1[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc0[nt][j] = acc1[nt][j] = 0.0f;

            Fp4Load A0, A1, B0, B1;  // current and next step of the two streams
            fp4_load<FMT>(p0, kb_begin, A0);
            fp4_load<FMT>(p1, kb_begin, A1);
            for (uint32_t kb = kb_begin; kb < kb_end; kb += 2u) {
                const uint32_t k1 = kb + 1u < kb_end ? kb + 1u : kb;
                fp4_load<FMT>(p0, k1, B0);
                fp4_load<FMT>(p1, k1, B1);
                fp4_step<FMT, NT, SPLIT>(A0, A1, p0, p1, xh, xl, valid, kb, t, acc0, acc1);
                const uint32_t k2 = kb + 2u < kb_end ? kb + 2u : kb;
                fp4_load<FMT>(p0, k2, A0);
                fp4_load<FMT>(p1, k2, A1);
                if (kb + 1u < kb_end)
                    fp4_step<FMT, NT, SPLIT>(B0, B1, p0, p1, xh, xl, valid, kb + 1u, t, acc0, acc1);
            }

            if (ksplit) {   // the upper-half warp hands its partial sums to its partner
                float* slot = xch[warp >> 1][lane];
                const uint32_t bar_id = 1u + (warp >> 1);
                if (khalf == 1u) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            slot[nt * 8 + j] = acc0[nt][j];
                            slot[nt * 8 + 4 + j] = acc1[nt][j];
                        }
                }
                asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
                if (khalf == 0u) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            acc0[nt][j] += slot[nt * 8 + j];
                            acc1[nt][j] += slot[nt * 8 + 4 + j];
                        }
                }
                asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");   // the slot may be rewritten after this
                if (khalf == 1u) continue;                                    // only the lower half writes results
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t tok = tb + nt * 8u + t * 2u + (j & 1u);
                    if (tok >= cnt) continue;
                    const uint32_t orow = row + ((j & 2u) ? 8u : 0u);
                    const size_t pos = row0 + tok;
                    const float rs = rowscale[pos];
                    if (DUAL) {
                        const float gv = acc0[nt][j] * s0 * rs, uv = acc1[nt][j] * s1 * rs;
                        float v = a.glu.kind == STRATA_MOE_ACT_SWIGLU ? silu_mul_f(gv, uv) : glu_other(gv, uv, a.glu);
                        if (a.coef) v *= a.coef[pos];
                        if (!(fabsf(v) <= 3.0e38f)) bad = true;
                        a.act_f32[pos * R + orow] = v;
                    } else {
                        const float v0 = acc0[nt][j] * s0 * rs, v1 = acc1[nt][j] * s1 * rs;
                        if (!(fabsf(v0) <= 3.0e38f) || !(fabsf(v1) <= 3.0e38f)) bad = true;
                        a.y[pos * R + orow] = v0;
                        a.y[pos * R + orow + 16u] = v1;
                    }
                }
            }
        }
    }
    if (bad) atomicOr(a.status, kStatusNonFiniteOutput);
}

static uint32_t fp4_ctas_per_sm(uint32_t nt) { return nt == 1 ? 4u : (nt == 2 ? 3u : 2u); }

template <int FMT, bool SPLIT, bool DUAL>
static void launch_fp4_nt(const DecodeArgs& a, cudaStream_t s) {
    const uint32_t R = DUAL ? a.I : a.H;
    const uint32_t total = a.n_groups * (DUAL ? R / 16u : R / 32u);
    if (total == 0u) return;
    const uint32_t m = a.max_rows_per_group;
    const uint32_t nt = m <= 8u ? 1u : (m <= 16u ? 2u : 4u);
    uint32_t grid = (total + 3u) / 4u;
    const uint32_t cap = kNumSMs * fp4_ctas_per_sm(nt);
    if (grid > cap) grid = cap;
    if (nt == 1u) decode_fp4_kernel<FMT, 1, SPLIT, DUAL><<<grid, 128, 0, s>>>(a);
    else if (nt == 2u) decode_fp4_kernel<FMT, 2, SPLIT, DUAL><<<grid, 128, 0, s>>>(a);
    else decode_fp4_kernel<FMT, 4, SPLIT, DUAL><<<grid, 128, 0, s>>>(a);
    ++g_kernel_launches;
}

void launch_decode_fp4_gate_up(const DecodeArgs& a, cudaStream_t s) {
    const bool split = a.x_lo != nullptr;
    if (a.fmt == STRATA_MOE_FMT_MXFP4)
        split ? launch_fp4_nt<STRATA_MOE_FMT_MXFP4, true, true>(a, s)
              : launch_fp4_nt<STRATA_MOE_FMT_MXFP4, false, true>(a, s);
    else
        split ? launch_fp4_nt<STRATA_MOE_FMT_NVFP4, true, true>(a, s)
              : launch_fp4_nt<STRATA_MOE_FMT_NVFP4, false, true>(a, s);
}

void launch_decode_fp4_down(const DecodeArgs& a, cudaStream_t s) {
    if (a.fmt == STRATA_MOE_FMT_MXFP4) launch_fp4_nt<STRATA_MOE_FMT_MXFP4, true, false>(a, s);
    else launch_fp4_nt<STRATA_MOE_FMT_NVFP4, true, false>(a, s);
}

// ---------------------------------------------------------------------------------------
// Rows -> f16 with an exact power-of-two pre-scale per row (one warp per destination row).
// SRC_F32 = false: BF16 source, hi only.  SRC_F32 = true: fp32 source, hi + lo.
// src row = perm ? perm[pos] / k_div : (reps ? pos % src_rows : pos).
template <bool SRC_F32>
__global__ void __launch_bounds__(256) rows_to_f16_kernel(const void* __restrict__ src,
                                                          const uint32_t* __restrict__ perm,
                                                          uint32_t k_div, uint32_t src_rows, uint32_t rows,
                                                          uint32_t C, __half* __restrict__ hi,
                                                          __half* __restrict__ lo,
                                                          float* __restrict__ rowscale,
                                                          const uint32_t* __restrict__ rows_dev) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t pos = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (pos >= rows) return;
    if (rows_dev && pos >= *rows_dev) return;   // `rows` is only an upper bound; the count lives on the device
    const uint32_t srow = perm ? perm[pos] / k_div : (src_rows ? pos % src_rows : pos);
    if (!SRC_F32) {
        warp_row_to_f16_bf16(static_cast<const __nv_bfloat16*>(src) + (size_t)srow * C, C, hi + (size_t)pos * C,
                             rowscale + pos);
        return;
    }
    float mx = 0.0f;
    {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(src) + (size_t)srow * C);
        for (uint32_t i = lane; i < C / 4u; i += 32u) {
            const float4 v = __ldg(p + i);
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    // scale = 2^(14 - floor(log2 mx)): row maximum lands in [2^14, 2^15); exact, and clamped so
    // both it and its reciprocal stay normal floats
    int ex = 0;
    if (mx > 0.0f && mx < 3.0e38f) ex = 14 - (int)((__float_as_uint(mx) >> 23) & 0xFFu) + 127;
    ex = max(-100, min(100, ex));
    const float sc = __uint_as_float((uint32_t)(ex + 127) << 23);
    if (lane == 0) rowscale[pos] = __uint_as_float((uint32_t)(127 - ex) << 23);
    {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(src) + (size_t)srow * C);
        for (uint32_t i = lane; i < C / 4u; i += 32u) {
            const float4 v = __ldg(p + i);
            const float f[4] = {v.x * sc, v.y * sc, v.z * sc, v.w * sc};
            __half h[4], l[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                h[q] = __float2half_rn(f[q]);
                l[q] = __float2half_rn(f[q] - __half2float(h[q]));
            }
            *reinterpret_cast<uint2*>(hi + (size_t)pos * C + i * 4u) =
                make_uint2((uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16),
                           (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16));
            if (lo != nullptr)
                *reinterpret_cast<uint2*>(lo + (size_t)pos * C + i * 4u) =
                    make_uint2((uint32_t)__half_as_ushort(l[0]) | ((uint32_t)__half_as_ushort(l[1]) << 16),
                               (uint32_t)__half_as_ushort(l[2]) | ((uint32_t)__half_as_ushort(l[3]) << 16));
        }
    }
}

void launch_rows_to_f16_bf16(const __nv_bfloat16* x, const uint32_t* perm, uint32_t k_div, uint32_t rows,
                             uint32_t C, void* hi, float* rowscale, cudaStream_t s, const uint32_t* rows_dev) {
    if (rows == 0) return;
    rows_to_f16_kernel<false><<<(rows + 7) / 8, 256, 0, s>>>(x, perm, k_div, 0, rows, C,
                                                            static_cast<__half*>(hi), nullptr, rowscale, rows_dev);
    ++g_kernel_launches;
}

// One warp per SOURCE row, stored to each of its k destination rows dest[t * k + j] (0xFFFFFFFF or a value of
// dst_bound and above = none).  rows_dev, when given, holds the number of source rows.
__global__ void __launch_bounds__(256) rows_to_f16_spread_kernel(const __nv_bfloat16* __restrict__ src,
                                                                 const uint32_t* __restrict__ dest, uint32_t k,
                                                                 uint32_t rows, const uint32_t* __restrict__ rows_dev,
                                                                 uint32_t dst_bound, uint32_t C,
                                                                 __half* __restrict__ hi,
                                                                 float* __restrict__ rowscale) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t t = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (t >= rows) return;
    if (rows_dev && t >= *rows_dev) return;
    uint32_t mydst = lane < k ? dest[(size_t)t * k + lane] : 0xFFFFFFFFu;
    if (mydst >= dst_bound) mydst = 0xFFFFFFFFu;
    if (__ballot_sync(0xFFFFFFFFu, mydst != 0xFFFFFFFFu) == 0u) return;
    warp_row_to_f16_bf16_spread(src + (size_t)t * C, C, hi, rowscale, mydst, k);
}

void launch_rows_to_f16_spread(const __nv_bfloat16* x, const uint32_t* dest, uint32_t k, uint32_t rows,
                               const uint32_t* rows_dev, uint32_t dst_bound, uint32_t C, void* hi, float* rowscale,
                               cudaStream_t s) {
    if (rows == 0) return;
    rows_to_f16_spread_kernel<<<(rows + 7) / 8, 256, 0, s>>>(x, dest, k, rows, rows_dev, dst_bound, C,
                                                            static_cast<__half*>(hi), rowscale);
    ++g_kernel_launches;
}

void launch_rows_to_f16_f32(const float* x, uint32_t src_rows, uint32_t rows, uint32_t C, void* hi, void* lo,
                            float* rowscale, cudaStream_t s, const uint32_t* rows_dev) {
    if (rows == 0) return;
    rows_to_f16_kernel<true><<<(rows + 7) / 8, 256, 0, s>>>(x, nullptr, 1, src_rows, rows, C,
                                                           static_cast<__half*>(hi), static_cast<__half*>(lo),
                                                           rowscale, rows_dev);
    ++g_kernel_launches;
}

// ---------------------------------------------------------------------------------------
// Per (expert, projection): smallest and largest E8M0 scale byte.  Decides whether the f16
// path can hold the expert (span <= 26 octaves, no reserved bytes) and fixes its exponent base.
// post_scale = 2^(emin + 15 - kMxBias - 127): the factor taken out of the weights.
__global__ void __launch_bounds__(256) mx_scale_range_kernel(const uint8_t* const* __restrict__ scales,
                                                             size_t bytes, uint32_t* __restrict__ emin,
                                                             float* __restrict__ post_scale,
                                                             uint32_t* __restrict__ not_ok) {
    __shared__ uint32_t smin[8], smax[8];
    const uint8_t* p = scales[blockIdx.x];
    uint32_t lo = 255u, hi = 0u;
    for (size_t i = (size_t)threadIdx.x * 16u; i < bytes; i += 256u * 16u) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p + i));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t e = (w[q] >> (8 * b)) & 0xFFu;
                lo = min(lo, e);
                hi = max(hi, e);
            }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        lo = min(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, off));
        hi = max(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, off));
    }
    if ((threadIdx.x & 31u) == 0) { smin[threadIdx.x >> 5] = lo; smax[threadIdx.x >> 5] = hi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i) { lo = min(lo, smin[i]); hi = max(hi, smax[i]); }
        emin[blockIdx.x] = lo;
        const int pe = (int)lo + 15 - kMxBias;  // exponent byte of the post scale
        if (hi - lo > 26u || hi == 0xFFu || pe < 1 || pe > 254) {
            atomicOr(not_ok, 1u);
            post_scale[blockIdx.x] = 0.0f;
        } else {
            post_scale[blockIdx.x] = __uint_as_float((uint32_t)pe << 23);
        }
    }
}

// Dequantised weights through the f16 decoders above (the values the f16 MMA path consumes),
// widened to fp32 and multiplied by the accumulator-side factor.
__global__ void dequant_export_f16_kernel(int fmt, const uint8_t* __restrict__ packed,
                                          const uint8_t* __restrict__ scales, uint32_t emin,
                                          float post_scale, uint32_t rows, uint32_t cols,
                                          float* __restrict__ out) {
    const size_t words = (size_t)rows * (cols / 8u);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / (cols / 8u)), wc = (uint32_t)(i % (cols / 8u));
        uint32_t r[4], m[2];
        e2m1x8_f16(reinterpret_cast<const uint32_t*>(packed)[i], r);
        uint32_t mult;
        if (fmt == STRATA_MOE_FMT_MXFP4) {
            fp4_mult<STRATA_MOE_FMT_MXFP4>(scales[(size_t)row * (cols / 32u) + wc / 4u],
                                           kMxBias - (int32_t)emin, m);
            mult = m[0];
        } else {
            // two scale bytes of the 32-column chunk; this word belongs to group (wc / 2) % 2
            const uint32_t pair = reinterpret_cast<const unsigned short*>(scales)[(size_t)row * (cols / 32u) + wc / 4u];
            fp4_mult<STRATA_MOE_FMT_NVFP4>(pair, 0, m);
            mult = m[(wc >> 1) & 1u];
        }
        float* o = out + (size_t)row * cols + (size_t)wc * 8u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t v = mul_f16x2(r[j], mult);
            o[2 * j] = __half2float(__ushort_as_half((unsigned short)(v & 0xFFFFu))) * post_scale;
            o[2 * j + 1] = __half2float(__ushort_as_half((unsigned short)(v >> 16))) * post_scale;
        }
    }
}

void launch_dequant_export_f16(int fmt, const uint8_t* packed, const uint8_t* scales, uint32_t emin,
                               float post_scale, uint32_t rows, uint32_t cols, float* out, cudaStream_t s) {
    dequant_export_f16_kernel<<<148 * 4, 256, 0, s>>>(fmt, packed, scales, emin, post_scale, rows, cols, out);
    ++g_kernel_launches;
}

void launch_mx_scale_range(const uint8_t* const* scales, uint32_t n, size_t bytes, uint32_t* emin,
                           float* post_scale, uint32_t* not_ok, cudaStream_t s) {
    if (n == 0) return;
    mx_scale_range_kernel<<<n, 256, 0, s>>>(scales, bytes, emin, post_scale, not_ok);
    ++g_kernel_launches;
}

}  // namespace smoe
