// Small-batch ("decode") expert FFN: each expert sees a handful of rows, so the kernels are
// bound by streaming the 4-bit weights from HBM exactly once.
//
// One warp owns a 16-row tile of one expert's projection and walks the whole K dimension.
// Per 128 columns every lane streams one 16-byte chunk (32 nibbles) of row `gid` and of row
// `gid + 8` straight into registers (no shared-memory round trip), dequantises them exactly to
// BF16 pairs and feeds them as the A operand of m16n8k16 BF16 MMAs with FP32 accumulation; the
// B operand is up to 8*NT activation rows.  The dot product is invariant under a permutation of
// K applied to both operands, so the activation rows are stored K-permuted (see kperm_index)
// such that the 4 values a lane needs per MMA are contiguous and every nibble pair (j, j+4) of a
// weight word decodes straight into one A register.
//
// Replaces, for small row counts, the reference's one-CTA-per-output-row GEMV kernels
// (kernels/cuda/backend.cu:1886-2069, 2308-2413), which re-read the weights for every row.
#include <cstdlib>

#include "common.cuh"
#include "dequant.cuh"

namespace smoe {

std::atomic<unsigned long long> g_kernel_launches{0};

// Position of column c inside its 128-column block in the K-permuted activation layout:
// chunk t = (c % 128) / 32 is the lane-in-quad that streams it, word wd = (c % 32) / 8, nibble
// p = c % 8.  Layout [wd][t][perm(p)] with perm = 0,4,1,5,2,6,3,7 -> slots 0..7.
__host__ __device__ __forceinline__ uint32_t kperm_index(uint32_t c) {
    const uint32_t blk = c & ~127u, t = (c >> 5) & 3u, wd = (c >> 3) & 3u, p = c & 7u;
    const uint32_t slot = ((p & 3u) << 1) | (p >> 2);
    return blk + wd * 32u + t * 8u + slot;
}

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kFmtBf16 = 3;

// Streams and decodes one projection's A fragments for one 128-column step (32 columns for
// BF16 weights) and issues the MMAs against the B fragments in `b`.
template <int FMT, int NT, bool SPLIT>
struct Projection {
    const uint8_t* row_lo;  // row gid
    const uint8_t* row_hi;  // row gid + 8
    const uint8_t* sc_lo;
    const uint8_t* sc_hi;

    __device__ __forceinline__ void init(const uint8_t* packed, const uint8_t* scales, uint32_t row,
                                         uint32_t K, uint32_t t) {
        if (FMT == kFmtBf16) {
            row_lo = packed + ((size_t)row * K + t * 8u) * 2u;
            row_hi = packed + ((size_t)(row + 8u) * K + t * 8u) * 2u;
            sc_lo = sc_hi = nullptr;
        } else {
            row_lo = packed + (size_t)row * (K / 2u) + t * 16u;
            row_hi = packed + (size_t)(row + 8u) * (K / 2u) + t * 16u;
            if (FMT == STRATA_MOE_FMT_MXFP4) {
                sc_lo = scales + (size_t)row * (K / 32u) + t;
                sc_hi = scales + (size_t)(row + 8u) * (K / 32u) + t;
            } else if (FMT == STRATA_MOE_FMT_NVFP4) {
                sc_lo = scales + (size_t)row * (K / 16u) + t * 2u;
                sc_hi = scales + (size_t)(row + 8u) * (K / 16u) + t * 2u;
            } else {
                sc_lo = scales + (size_t)row * (K / 128u) * 2u;
                sc_hi = scales + (size_t)(row + 8u) * (K / 128u) * 2u;
            }
        }
    }
};

template <int FMT>
struct StepLoad {
    uint4 lo, hi;       // packed weights of the two rows
    uint32_t s_lo, s_hi;  // raw scale bits
};

template <int FMT, int NT, bool SPLIT>
__device__ __forceinline__ void step_load(const Projection<FMT, NT, SPLIT>& p, uint32_t kb,
                                          StepLoad<FMT>& L) {
    if (FMT == kFmtBf16) {
        L.lo = ldg_stream16(p.row_lo + (size_t)kb * 64u);
        L.hi = ldg_stream16(p.row_hi + (size_t)kb * 64u);
        L.s_lo = L.s_hi = 0;
    } else {
        L.lo = ldg_stream16(p.row_lo + (size_t)kb * 64u);
        L.hi = ldg_stream16(p.row_hi + (size_t)kb * 64u);
        if (FMT == STRATA_MOE_FMT_MXFP4) {
            L.s_lo = __ldg(p.sc_lo + kb * 4u);
            L.s_hi = __ldg(p.sc_hi + kb * 4u);
        } else if (FMT == STRATA_MOE_FMT_NVFP4) {
            L.s_lo = __ldg(reinterpret_cast<const unsigned short*>(p.sc_lo + kb * 8u));
            L.s_hi = __ldg(reinterpret_cast<const unsigned short*>(p.sc_hi + kb * 8u));
        } else {
            L.s_lo = __ldg(reinterpret_cast<const unsigned short*>(p.sc_lo + kb * 2u));
            L.s_hi = __ldg(reinterpret_cast<const unsigned short*>(p.sc_hi + kb * 2u));
        }
    }
}

// Decoded A registers of one weight word for rows gid (a) and gid + 8 (b).
template <int FMT>
struct StepScale {
    Mx4Mult mlo, mhi;        // MXFP4
    uint32_t nlo[2], nhi[2]; // NVFP4: groups of words 0-1 and 2-3
};

template <int FMT>
__device__ __forceinline__ void step_scale(const StepLoad<FMT>& L, StepScale<FMT>& S) {
    if (FMT == STRATA_MOE_FMT_MXFP4) {
        S.mlo = mxfp4_mult(L.s_lo);
        S.mhi = mxfp4_mult(L.s_hi);
    } else if (FMT == STRATA_MOE_FMT_NVFP4) {
        S.nlo[0] = nvfp4_mult(L.s_lo & 0xFFu);
        S.nlo[1] = nvfp4_mult(L.s_lo >> 8);
        S.nhi[0] = nvfp4_mult(L.s_hi & 0xFFu);
        S.nhi[1] = nvfp4_mult(L.s_hi >> 8);
    }
}

template <int FMT>
__device__ __forceinline__ void decode_word(uint32_t wl, uint32_t wh, const StepScale<FMT>& S, int wd,
                                            uint32_t a[4], uint32_t b[4]) {
    if (FMT == kFmtBf16) return;
    if (FMT == STRATA_MOE_FMT_INT4G128) {
        int4x8_bf16(wl, a);
        int4x8_bf16(wh, b);
        return;
    }
    e2m1x8_raw(wl, a);
    e2m1x8_raw(wh, b);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (FMT == STRATA_MOE_FMT_MXFP4) {
            a[j] = apply_mx4(a[j], S.mlo);
            b[j] = apply_mx4(b[j], S.mhi);
        } else {
            a[j] = mul_bf16x2(a[j], S.nlo[wd >> 1]);
            b[j] = mul_bf16x2(b[j], S.nhi[wd >> 1]);
        }
    }
}

__device__ __forceinline__ uint32_t sel4(const uint4& v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// One K step (128 columns; 32 for BF16 weights) of one or two projections against up to 8*NT
// activation rows.  B fragments are fetched per weight word so that only NT (x2 when SPLIT)
// 16-byte registers are live at a time; gate and up share them.
template <int FMT, int NT, bool SPLIT, bool DUAL>
__device__ __forceinline__ void step_compute(const StepLoad<FMT>& Lg, const StepLoad<FMT>& Lu,
                                             const __nv_bfloat16* const xh[NT],
                                             const __nv_bfloat16* const xl[NT], const bool valid[NT],
                                             uint32_t kb, uint32_t t, float accg[NT][4],
                                             float accu[NT][4]) {
    constexpr int WORDS = FMT == kFmtBf16 ? 1 : 4;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    StepScale<FMT> Sg, Su;
    step_scale<FMT>(Lg, Sg);
    if (DUAL) step_scale<FMT>(Lu, Su);
    float tg[NT][4], tu[NT][4];
    if (FMT == STRATA_MOE_FMT_INT4G128) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) tg[nt][j] = tu[nt][j] = 0.0f;
    }
#pragma unroll
    for (int wd = 0; wd < WORDS; ++wd) {
        uint4 bh[NT], bl[SPLIT ? NT : 1];
        const size_t off = FMT == kFmtBf16 ? ((size_t)kb * 32u + t * 8u)
                                           : ((size_t)kb * 128u + wd * 32u + t * 8u);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            bh[nt] = valid[nt] ? __ldg(reinterpret_cast<const uint4*>(xh[nt] + off)) : zero;
            if (SPLIT) bl[nt] = valid[nt] ? __ldg(reinterpret_cast<const uint4*>(xl[nt] + off)) : zero;
        }
#pragma unroll
        for (int proj = 0; proj < (DUAL ? 2 : 1); ++proj) {
            const StepLoad<FMT>& L = proj ? Lu : Lg;
            uint32_t a[4], b[4];
            if (FMT == kFmtBf16) {
                a[0] = L.lo.x; a[1] = L.lo.y; a[2] = L.lo.z; a[3] = L.lo.w;
                b[0] = L.hi.x; b[1] = L.hi.y; b[2] = L.hi.z; b[3] = L.hi.w;
            } else {
                decode_word<FMT>(sel4(L.lo, wd), sel4(L.hi, wd), proj ? Su : Sg, wd, a, b);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float* c = FMT == STRATA_MOE_FMT_INT4G128 ? (proj ? tu[nt] : tg[nt])
                                                          : (proj ? accu[nt] : accg[nt]);
                mma_bf16_16816(c, a[0], b[0], a[1], b[1], bh[nt].x, bh[nt].y);
                mma_bf16_16816(c, a[2], b[2], a[3], b[3], bh[nt].z, bh[nt].w);
                if (SPLIT) {
                    mma_bf16_16816(c, a[0], b[0], a[1], b[1], bl[nt].x, bl[nt].y);
                    mma_bf16_16816(c, a[2], b[2], a[3], b[3], bl[nt].z, bl[nt].w);
                }
            }
        }
    }
    if (FMT == STRATA_MOE_FMT_INT4G128) {
        // one BF16 scale per (row, 128 columns): applied to the step's partial sums in fp32,
        // so the product (q - 8) * s is never rounded to BF16.
#pragma unroll
        for (int proj = 0; proj < (DUAL ? 2 : 1); ++proj) {
            const StepLoad<FMT>& L = proj ? Lu : Lg;
            const float s_lo = __uint_as_float(L.s_lo << 16), s_hi = __uint_as_float(L.s_hi << 16);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float* acc = proj ? accu[nt] : accg[nt];
                const float* tmp = proj ? tu[nt] : tg[nt];
                acc[0] = fmaf(tmp[0], s_lo, acc[0]);
                acc[1] = fmaf(tmp[1], s_lo, acc[1]);
                acc[2] = fmaf(tmp[2], s_hi, acc[2]);
                acc[3] = fmaf(tmp[3], s_hi, acc[3]);
            }
        }
    }
}

__device__ __forceinline__ float silu_mul(float g, float u) {
    // gate * sigmoid(gate) * up with the two-branch sigmoid (kernels/cuda/backend.cu:2021-2031)
    const float e = __expf(-fabsf(g));
    const float sig = g >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
    return g * sig * u;
}

// Every warp streams TWO 16-row tiles at once against the same activation fragments:
// DUAL = true : the gate tile and the up tile of the same output rows, fused SwiGLU epilogue,
//               writes act (hi/lo BF16, K-permuted for the down kernel unless the down weights
//               are BF16).
// DUAL = false: two adjacent row tiles of the down projection, writes y fp32 [pairs, rows].
// The K loop runs in super-steps of two steps (256 columns: each quad reads one full 128-byte
// line per row) and keeps the next super-step's loads in flight while decoding the current one.
template <int FMT, int NT, bool SPLIT, bool DUAL>
__global__ void __launch_bounds__(128, NT == 1 ? 3 : 2) decode_ffn_kernel(DecodeArgs a) {
    const uint32_t lane = threadIdx.x & 31u, gid = lane >> 2, t = lane & 3u;
    const uint32_t K = DUAL ? a.H : a.I;
    const uint32_t R = DUAL ? a.I : a.H;  // output rows of this projection
    const uint32_t tiles_per_group = DUAL ? R / 16u : R / 32u;
    const uint32_t n_act = a.active_list ? *a.n_active : a.n_groups;
    const uint32_t total = n_act * tiles_per_group;
    if (total == 0u) return;
    // With only a handful of tiles (one always-on expert and a few rows) a warp per tile would
    // leave most SMs idle: then the four warps of a CTA share one tile, each streaming a quarter
    // of K, and warp 0 adds the four partial sums in a fixed order.
    const bool ks = a.ksplit != 0u;
    const uint32_t kw = threadIdx.x >> 5;
    const uint32_t W = ks ? gridDim.x : gridDim.x * 4u;
    const uint32_t rounds = (total + W - 1u) / W;
    const uint32_t W_eff = (total + rounds - 1u) / rounds;  // equal tiles per warp, no ragged tail
    const uint32_t wid = ks ? blockIdx.x : blockIdx.x * 4u + kw;
    if (wid >= W_eff) return;
    constexpr uint32_t KSTEP = FMT == kFmtBf16 ? 32u : 128u;
    constexpr int U = 2;
    const uint32_t steps = K / KSTEP;
    const uint32_t nsuper = (steps + U - 1u) / U;
    const uint32_t sb_begin = ks ? kw * nsuper / 4u : 0u;
    const uint32_t sb_end = ks ? (kw + 1u) * nsuper / 4u : nsuper;
    __shared__ float red[3][2 * NT * 4][32];
    bool bad = false;

    for (uint32_t tile = wid; tile < total; tile += W_eff) {
        const uint32_t slot = tile / tiles_per_group;
        const uint32_t g = a.active_list ? a.active_list[slot] : slot;
        const uint32_t rt = tile - slot * tiles_per_group;
        const uint32_t row0 = a.offsets[g], cnt = a.offsets[g + 1] - row0;
        if (cnt == 0u) continue;
        const uint32_t row = (DUAL ? rt * 16u : rt * 32u) + gid;  // first stream's row gid

        Projection<FMT, NT, SPLIT> pg, pu;
        float gs = 1.0f, us = 1.0f;
        if (DUAL) {
            pg.init(a.gate.packed[g], a.gate.scales[g], row, K, t);
            pu.init(a.up.packed[g], a.up.scales[g], row, K, t);
            if (FMT == STRATA_MOE_FMT_NVFP4) {
                gs = kNvfp4AccScale / a.gate.global_scale[g];
                us = kNvfp4AccScale / a.up.global_scale[g];
            }
        } else {
            pg.init(a.down.packed[g], a.down.scales[g], row, K, t);
            pu.init(a.down.packed[g], a.down.scales[g], row + 16u, K, t);
            if (FMT == STRATA_MOE_FMT_NVFP4) gs = us = kNvfp4AccScale / a.down.global_scale[g];
        }

        for (uint32_t tb = 0; tb < cnt; tb += 8u * NT) {
            const __nv_bfloat16* xh[NT];
            const __nv_bfloat16* xl[NT];
            bool valid[NT];
            const __nv_bfloat16* bh = DUAL ? a.x_hi : a.act_hi;
            const __nv_bfloat16* bl = DUAL ? a.x_lo : a.act_lo;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t tok = tb + nt * 8u + gid;
                valid[nt] = tok < cnt;
                const size_t r = (size_t)(row0 + (valid[nt] ? tok : 0u)) * K;
                xh[nt] = bh + r;
                xl[nt] = SPLIT ? bl + r : nullptr;
            }
            float accg[NT][4], accu[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) accg[nt][j] = accu[nt][j] = 0.0f;

            StepLoad<FMT> Lg[U], Lu[U], Ng[U], Nu[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t kb = min(sb_begin * U + (uint32_t)u, steps - 1u);
                step_load(pg, kb, Lg[u]);
                step_load(pu, kb, Lu[u]);
            }
            for (uint32_t sb = sb_begin; sb < sb_end; ++sb) {
                // next super-step's weights are requested before this one is decoded
                const uint32_t sn = sb + 1u < sb_end ? sb + 1u : sb;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const uint32_t kb = min(sn * U + u, steps - 1u);
                    step_load(pg, kb, Ng[u]);
                    step_load(pu, kb, Nu[u]);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const uint32_t kb = sb * U + u;
                    if (kb < steps)
                        step_compute<FMT, NT, SPLIT, true>(Lg[u], Lu[u], xh, xl, valid, kb, t, accg, accu);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    Lg[u] = Ng[u];
                    Lu[u] = Nu[u];
                }
            }

            if (ks) {  // fold the four K-quarters: warps 1..3 publish, warp 0 adds them in order
                if (kw > 0u) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            red[kw - 1u][nt * 8 + j][lane] = accg[nt][j];
                            red[kw - 1u][nt * 8 + 4 + j][lane] = accu[nt][j];
                        }
                }
                __syncthreads();
                if (kw == 0u) {
#pragma unroll
                    for (int w = 0; w < 3; ++w)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                accg[nt][j] += red[w][nt * 8 + j][lane];
                                accu[nt][j] += red[w][nt * 8 + 4 + j][lane];
                            }
                }
                __syncthreads();
            }
            // epilogue: c0,c1 = (row gid, tokens 2t, 2t+1); c2,c3 = (row gid + 8, same tokens)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t tok = tb + nt * 8u + t * 2u + (j & 1u);
                    if (tok >= cnt || (ks && kw != 0u)) continue;
                    const uint32_t orow = row + ((j & 2u) ? 8u : 0u);
                    const size_t pos = row0 + tok;
                    if (DUAL) {
                        const float gv = accg[nt][j] * gs, uv = accu[nt][j] * us;
                        float v = a.glu.kind == STRATA_MOE_ACT_SWIGLU ? silu_mul(gv, uv) : glu_other(gv, uv, a.glu);
                        if (a.coef) v *= a.coef[pos];
                        if (!(fabsf(v) <= 3.0e38f)) bad = true;
                        const __nv_bfloat16 hi = __float2bfloat16_rn(v);
                        const __nv_bfloat16 lo = __float2bfloat16_rn(v - __bfloat162float(hi));
                        const uint32_t col = a.fmt == kFmtBf16 ? orow : kperm_index(orow);
                        a.act_hi[pos * R + col] = hi;
                        a.act_lo[pos * R + col] = lo;
                    } else {
                        const float v0 = accg[nt][j] * gs, v1 = accu[nt][j] * us;
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

static uint32_t decode_ctas_per_sm() { return 4u; }

template <int FMT, bool SPLIT, bool DUAL>
static void launch_nt(const DecodeArgs& a, cudaStream_t s) {
    const uint32_t R = DUAL ? a.I : a.H;
    const uint32_t total = a.n_groups * (DUAL ? R / 16u : R / 32u);
    if (total == 0u) return;
    const uint32_t cap = kNumSMs * decode_ctas_per_sm();
    DecodeArgs b = a;
    b.ksplit = total <= 2u * kNumSMs ? 1u : 0u;  // too few tiles to fill the GPU one warp each
    uint32_t grid = b.ksplit ? total : (total + 3u) / 4u;
    if (grid > cap) grid = cap;
    const uint32_t m = a.max_rows_per_group;
    if (m <= 8u) decode_ffn_kernel<FMT, 1, SPLIT, DUAL><<<grid, 128, 0, s>>>(b);
    else if (m <= 16u) decode_ffn_kernel<FMT, 2, SPLIT, DUAL><<<grid, 128, 0, s>>>(b);
    else decode_ffn_kernel<FMT, 4, SPLIT, DUAL><<<grid, 128, 0, s>>>(b);
    ++g_kernel_launches;
}

template <bool DUAL>
static void launch_fmt(const DecodeArgs& a, cudaStream_t s) {
    const bool split = DUAL ? (a.x_lo != nullptr) : true;  // down always reads the hi/lo activation
    switch (a.fmt) {
        case STRATA_MOE_FMT_MXFP4:
            split ? launch_nt<STRATA_MOE_FMT_MXFP4, true, DUAL>(a, s)
                  : launch_nt<STRATA_MOE_FMT_MXFP4, false, DUAL>(a, s);
            break;
        case STRATA_MOE_FMT_NVFP4:
            split ? launch_nt<STRATA_MOE_FMT_NVFP4, true, DUAL>(a, s)
                  : launch_nt<STRATA_MOE_FMT_NVFP4, false, DUAL>(a, s);
            break;
        case STRATA_MOE_FMT_INT4G128:
            split ? launch_nt<STRATA_MOE_FMT_INT4G128, true, DUAL>(a, s)
                  : launch_nt<STRATA_MOE_FMT_INT4G128, false, DUAL>(a, s);
            break;
        default:
            split ? launch_nt<kFmtBf16, true, DUAL>(a, s) : launch_nt<kFmtBf16, false, DUAL>(a, s);
            break;
    }
}

void launch_decode_gate_up(const DecodeArgs& a, cudaStream_t s) { launch_fmt<true>(a, s); }
void launch_decode_down(const DecodeArgs& a, cudaStream_t s) { launch_fmt<false>(a, s); }

// ---------------------------------------------------------------------------------------
// Activation row copies into the layouts the expert kernels read.
__global__ void gather_rows_kperm_kernel(const __nv_bfloat16* __restrict__ x,
                                         const uint32_t* __restrict__ perm, uint32_t k_div,
                                         uint32_t pairs, uint32_t H, __nv_bfloat16* __restrict__ dst,
                                         const uint32_t* __restrict__ pairs_dev) {
    const uint32_t per_row = H / 8u;
    if (pairs_dev) pairs = min(pairs, *pairs_dev);   // `pairs` is only an upper bound in that case
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)pairs * per_row;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t pos = (uint32_t)(i / per_row), c8 = (uint32_t)(i % per_row) * 8u;
        const uint32_t src = perm ? perm[pos] / k_div : pos;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)src * H + c8));
        // source elements p = 0..7 of one word go to slots 0,2,4,6,1,3,5,7
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        unsigned short e[8];
#pragma unroll
        for (int p = 0; p < 8; ++p) e[p] = (unsigned short)(w[p >> 1] >> ((p & 1) * 16));
        uint4 o;
        o.x = (uint32_t)e[0] | ((uint32_t)e[4] << 16);
        o.y = (uint32_t)e[1] | ((uint32_t)e[5] << 16);
        o.z = (uint32_t)e[2] | ((uint32_t)e[6] << 16);
        o.w = (uint32_t)e[3] | ((uint32_t)e[7] << 16);
        *reinterpret_cast<uint4*>(dst + (size_t)pos * H + kperm_index(c8)) = o;
    }
}

void launch_gather_rows_kperm(const __nv_bfloat16* x, const uint32_t* perm, uint32_t k_div,
                              uint32_t pairs, uint32_t H, __nv_bfloat16* dst, cudaStream_t s,
                              const uint32_t* pairs_dev) {
    if (pairs == 0) return;
    const size_t n = (size_t)pairs * (H / 8u);
    const uint32_t grid = (uint32_t)((n + 255) / 256 < 148u * 8u ? (n + 255) / 256 : 148u * 8u);
    gather_rows_kperm_kernel<<<grid, 256, 0, s>>>(x, perm, k_div, pairs, H, dst, pairs_dev);
    ++g_kernel_launches;
}

// fp32 rows -> hi/lo BF16 K-permuted, each source row repeated `reps` times group-major
// (dense command: every listed expert sees all rows).  dst row = rep * rows + row.
__global__ void gather_rows_kperm_f32_kernel(const float* __restrict__ x, uint32_t rows, uint32_t reps,
                                             uint32_t H, __nv_bfloat16* __restrict__ hi,
                                             __nv_bfloat16* __restrict__ lo, bool natural) {
    const size_t n = (size_t)rows * reps * H;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = (uint32_t)(i % H);
        const size_t drow = i / H;
        const uint32_t srow = (uint32_t)(drow % rows);
        const float v = x[(size_t)srow * H + c];
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        const uint32_t dc = natural ? c : kperm_index(c);   // BF16 weights read natural column order
        hi[drow * H + dc] = h;
        lo[drow * H + dc] = __float2bfloat16_rn(v - __bfloat162float(h));
    }
}

void launch_gather_rows_kperm_f32(const float* x, uint32_t rows, uint32_t reps, uint32_t H,
                                  __nv_bfloat16* hi, __nv_bfloat16* lo, cudaStream_t s, bool natural) {
    const size_t n = (size_t)rows * reps * H;
    if (n == 0) return;
    const uint32_t grid = (uint32_t)((n + 255) / 256 < 148u * 8u ? (n + 255) / 256 : 148u * 8u);
    gather_rows_kperm_f32_kernel<<<grid, 256, 0, s>>>(x, rows, reps, H, hi, lo, natural);
    ++g_kernel_launches;
}

__global__ void gather_rows_plain_kernel(const __nv_bfloat16* __restrict__ x,
                                         const uint32_t* __restrict__ perm, uint32_t k_div,
                                         uint32_t pairs, uint32_t H, __nv_bfloat16* __restrict__ dst) {
    const uint32_t per_row = H / 8u;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)pairs * per_row;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t pos = (uint32_t)(i / per_row), c8 = (uint32_t)(i % per_row) * 8u;
        const uint32_t src = perm ? perm[pos] / k_div : pos;
        *reinterpret_cast<uint4*>(dst + (size_t)pos * H + c8) =
            __ldg(reinterpret_cast<const uint4*>(x + (size_t)src * H + c8));
    }
}

void launch_gather_rows_plain(const __nv_bfloat16* x, const uint32_t* perm, uint32_t k_div,
                              uint32_t pairs, uint32_t H, __nv_bfloat16* dst, cudaStream_t s) {
    if (pairs == 0) return;
    const size_t n = (size_t)pairs * (H / 8u);
    const uint32_t grid = (uint32_t)((n + 255) / 256 < 148u * 16u ? (n + 255) / 256 : 148u * 16u);
    gather_rows_plain_kernel<<<grid, 256, 0, s>>>(x, perm, k_div, pairs, H, dst);
    ++g_kernel_launches;
}

// ---------------------------------------------------------------------------------------
// Dequantised weights through the same decoders the MMA path uses, widened to fp32.
// NVFP4 exports e2m1 * e4m3 / global with the division applied in fp32.
__global__ void dequant_export_kernel(int fmt, const uint8_t* __restrict__ packed,
                                      const uint8_t* __restrict__ scales, float global_scale,
                                      uint32_t rows, uint32_t cols, float* __restrict__ out) {
    const size_t words = (size_t)rows * (cols / 8u);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / (cols / 8u)), wc = (uint32_t)(i % (cols / 8u));
        const uint32_t w = reinterpret_cast<const uint32_t*>(packed)[i];
        uint32_t r[4];
        float mul = 1.0f;
        if (fmt == STRATA_MOE_FMT_INT4G128) {
            int4x8_bf16(w, r);
            const unsigned short sb =
                reinterpret_cast<const unsigned short*>(scales)[(size_t)row * (cols / 128u) + wc / 16u];
            mul = __uint_as_float((uint32_t)sb << 16);
        } else {
            e2m1x8_raw(w, r);
            if (fmt == STRATA_MOE_FMT_MXFP4) {
                const Mx4Mult m = mxfp4_mult(scales[(size_t)row * (cols / 32u) + wc / 4u]);
#pragma unroll
                for (int j = 0; j < 4; ++j) r[j] = apply_mx4(r[j], m);
            } else {
                const uint32_t m = nvfp4_mult(scales[(size_t)row * (cols / 16u) + wc / 2u]);
#pragma unroll
                for (int j = 0; j < 4; ++j) r[j] = mul_bf16x2(r[j], m);
                mul = kNvfp4AccScale / global_scale;
            }
        }
        float* o = out + (size_t)row * cols + (size_t)wc * 8u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            o[j] = __uint_as_float(r[j] << 16) * mul;
            o[j + 4] = __uint_as_float(r[j] & 0xFFFF0000u) * mul;
        }
    }
}

void launch_dequant_export(int fmt, const uint8_t* packed, const uint8_t* scales, float global_scale,
                           uint32_t rows, uint32_t cols, float* out, cudaStream_t s) {
    dequant_export_kernel<<<148 * 4, 256, 0, s>>>(fmt, packed, scales, global_scale, rows, cols, out);
    ++g_kernel_launches;
}

}  // namespace smoe
