// Small-batch expert FFN for the FP4 formats, weight tiles STREAMED HBM -> shared memory by TMA:
// the kernel the decode roofline is measured on.
//
// One persistent CTA per SM.  A producer warp walks the CTA's jobs and fills a ring of shared-
// memory stages with asynchronous copies whose completion is counted in bytes on an mbarrier.
// Per stage: the packed 4-bit bytes of up to 64 + 64 weight rows x 512 columns as FOUR tiled TMA
// copies (cp.async.bulk.tensor.2d, boxes of 64 rows x 128 bytes, 128-byte swizzle), their block
// scales as TWO tiled copies, and the same 512 columns of the group's activation rows (f16) as one
// bulk copy per row.  A few large copies per 32 KB of weights keep the copy engine far from its
// request-rate limit, and with four stages in the ring ~128 KB of weight bytes are in flight per
// SM, independent of how many warps are resident -- the loads no longer live in registers.
//
// Sixteen consumer warps read ONLY shared memory.  The work of one expert projection pair is cut
// into units of 16 output rows (gate/up: 16 gate rows + the same 16 up rows; down: 2 x 16 rows);
// every CTA owns a contiguous, evenly sized range of units and walks it in jobs of up to four
// units (the tail of a range, or of an expert, takes smaller jobs fetched with 16-row boxes).  A
// stage holds four k-steps of 128 columns; warp w owns unit w / 4 and k-step w % 4 of every stage:
// it decodes its rows with the hardware E2M1 -> f16 conversion, folds the block scale in with one
// packed multiply (exact, as in decode_fp4.cu) and issues m16n8k16 F16 MMAs with FP32
// accumulation.  At the end of a job the four partial accumulators of a unit's K split meet in
// shared memory and are summed in a fixed order, so results are bit-reproducible.
//
// Bank conflicts: in a swizzled box the 16-byte chunk c of row r sits at chunk position c ^ (r & 7);
// lane (g, t) reads the 32-bit words t, t+4, t+8, t+12 of its row's 64-byte k-step slice, so a
// warp-wide 32-bit load touches one chunk in each of 8 rows with distinct r & 7 = all 32 banks once.
// Activation rows sit 1088 bytes apart (1024 + 64) and the four lanes of a quad read 64 contiguous
// bytes, so an 8-lane phase of a 128-bit load covers two rows x 64 bytes = all banks once.  Word
// wd * 4 + t of a k-step holds columns 8 (wd * 4 + t) .. + 7, which is also activation chunk
// wd * 4 + t: natural column order.
//
// Every wait is bounded; on expiry the kernel raises kStatusWaitTimeout, all roles leave, the
// producer gives the copies still in flight a bounded chance to land, and the kernel returns.
// All copies read this GPU's own memory and have a single destination CTA.
//
// Replaces the reference's per-row NVFP4 / DeepSeek FP4 expert kernels for decode batches
// (kernels/cuda/backend.cu:1978-2069, 2308-2413).
#include <cuda.h>
#include <cuda_fp16.h>

#include "stream_ring.cuh"

namespace smoe {

using namespace ring;

namespace {

constexpr uint32_t kCWarps = 16;                  // consumer warps: 4 units x 4 k-steps
constexpr uint32_t kSThreads = (kCWarps + 1) * 32;
constexpr uint32_t kStageSteps = 4;               // k-steps of 128 columns per stage
constexpr uint32_t kJobUnits = 4;                 // units of 16 (+16) rows per full job
constexpr uint32_t kBoxRows = 16 * kJobUnits;     // 64
constexpr uint32_t kBoxBytes = kBoxRows * 128;    // one weight box: 64 rows x 128 bytes
constexpr uint32_t kXSlabs = kStageSteps * 2;     // 128-byte slabs of one activation row per stage (64 f16 columns each)
constexpr int kMxBiasS = 2;                       // f16 exponent field of an MXFP4 multiplier is e - emin + 2

template <int FMT>
struct ScaleGeo {
    static constexpr uint32_t kStepBytes = FMT == STRATA_MOE_FMT_MXFP4 ? 4u : 8u;   // scale bytes per row per k-step
    static constexpr uint32_t kPitch = kStepBytes * kStageSteps;                    // 16 or 32
};

template <int FMT, int NT, bool SPLIT>
struct StreamGeo {
    // weights: [tile p][k half][64 rows][128 B], each box 1024-byte aligned (swizzle atom)
    static constexpr uint32_t kWOff = 0;
    static constexpr uint32_t kSOff = 4u * kBoxBytes;                               // scales: [tile p][64 rows][pitch]
    static constexpr uint32_t kXOff = (kSOff + 2u * kBoxRows * ScaleGeo<FMT>::kPitch + 1023u) / 1024u * 1024u;   // swizzle atom
    static constexpr uint32_t kXBoxBytes = 8u * NT * kXSlabs * 128u;                // one activation box: [slab][8 NT rows][128 B]
    static constexpr uint32_t kStageBytes = (kXOff + (SPLIT ? 2u : 1u) * kXBoxBytes + 1023u) / 1024u * 1024u;
    static constexpr uint32_t kRedBytes = kCWarps * 32u * 8u * NT * 4u;
    static constexpr uint32_t kBudget = 225u * 1024u;
    static constexpr uint32_t kStagesRaw = (kBudget - kRedBytes - 1024u) / kStageBytes;
    static constexpr uint32_t kStages = kStagesRaw > 8u ? 8u : kStagesRaw;
    static constexpr uint32_t kSmem = kStages * kStageBytes + kRedBytes + 1024u + 1024u;
    static_assert(kStages >= 2, "ring too shallow");
};

struct StreamCtl {                 // first 1024 bytes of the dynamic shared memory
    uint64_t full[8], empty[8];
    uint64_t red_ready, red_free;
    uint32_t abort_flag;
};

__device__ __forceinline__ void tma_box(void* dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_addr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_addr(bar))
        : "memory");
}

__device__ __forceinline__ void tma_box3(void* dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint32_t z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_addr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_addr(bar))
        : "memory");
}

__device__ __forceinline__ float silu_mul_s(float g, float u) {
    const float e = __expf(-fabsf(g));
    const float sig = g >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
    return g * sig * u;
}

// f16x2 multipliers of the four 32-column blocks of one row's k-step
template <int FMT>
__device__ __forceinline__ void step_mults(uint32_t saddr, int32_t mx_off, uint32_t t, uint32_t m[4]) {
    if (FMT == STRATA_MOE_FMT_MXFP4) {
        const uint32_t w = lds32(saddr);   // four E8M0 bytes, one per 32 columns
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
            const uint32_t e = (w >> (8 * wd)) & 0xFFu;
            m[wd] = ((uint32_t)((int32_t)e + mx_off) << 10) * 0x00010001u;   // f16 2^(e - emin + 2 - 15), twice
        }
    } else {
        const uint2 w = lds64(saddr);      // eight E4M3 bytes, one per 16 columns; this lane's words use byte 2 wd + (t >> 1)
        const uint32_t sel = (t >> 1) ? 0x3232u : 0x1010u;
        const uint32_t h[4] = {w.x & 0xFFFFu, w.x >> 16, w.y & 0xFFFFu, w.y >> 16};
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
            uint32_t pair;
            asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"((unsigned short)h[wd]));
            m[wd] = __byte_perm(pair, pair, sel);
        }
    }
}

// A wait whose outcome the whole warp agrees on (a lane that timed out fails the warp).
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, const volatile uint32_t* abort_flag) {
    return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, abort_flag));
}

struct JobInfo {
    uint32_t g;        // group (local expert)
    uint32_t us, nu;   // first unit inside the expert, units in this job (1..4)
    uint32_t row0, cnt, tb;
};

// DUAL = true : gate/up + SwiGLU, writes act fp32 [pairs, I].   K = H, a unit is 16 gate + 16 up rows.
// DUAL = false: down, writes y fp32 [pairs, H].                 K = I, a unit is 2 x 16 rows.
// maps: [3 roles][n_groups][3] tensor maps (64-row weight boxes, 16-row weight boxes, scale boxes).
template <int FMT, int NT, bool SPLIT, bool DUAL>
__global__ void __launch_bounds__(kSThreads, 1) decode_stream_kernel(DecodeArgs a, const CUtensorMap* __restrict__ maps,
                                                                     const __grid_constant__ CUtensorMap xmap_hi,
                                                                     const __grid_constant__ CUtensorMap xmap_lo) {
    using G = StreamGeo<FMT, NT, SPLIT>;
    constexpr uint32_t S = G::kStages;
    extern __shared__ uint8_t smem_raw_s[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_s) + 1023) & ~uintptr_t(1023));
    StreamCtl& C = *reinterpret_cast<StreamCtl*>(base);
    uint8_t* stages = base + 1024;
    float* red = reinterpret_cast<float*>(stages + S * G::kStageBytes);   // [warp][8 NT][lane]
    volatile uint32_t* abort_flag = &C.abort_flag;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t K = DUAL ? a.H : a.I;
    const uint32_t R = DUAL ? a.I : a.H;
    const uint32_t upe = DUAL ? R / 16u : R / 32u;           // units per expert
    const uint32_t n_act = a.active_list ? *a.n_active : a.n_groups;
    const uint32_t total_units = n_act * upe;
    const uint32_t steps = K / 128u;
    const uint32_t chunks = (steps + kStageSteps - 1u) / kStageSteps;
    // this CTA's contiguous range of units (sizes differ by at most one over the grid)
    const uint32_t u_begin = (uint32_t)(((uint64_t)total_units * blockIdx.x) / gridDim.x);
    const uint32_t u_end = (uint32_t)(((uint64_t)total_units * (blockIdx.x + 1u)) / gridDim.x);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(&C.full[s], 1);
            mbar_init(&C.empty[s], kCWarps);
        }
        mbar_init(&C.red_ready, kCWarps);
        mbar_init(&C.red_free, kCWarps);
        C.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // the job sequence of this CTA, walked identically by the producer and by every consumer
    auto next_job = [&](uint32_t& u, JobInfo& j, bool first) -> bool {
        if (!first) {
            j.tb += 8u * NT;
            if (j.tb < j.cnt) return true;      // same rows, next block of tokens
            u += j.nu;
        }
        while (u < u_end) {
            const uint32_t slot = u / upe;
            j.g = a.active_list ? a.active_list[slot] : slot;
            j.us = u - slot * upe;
            j.nu = min(kJobUnits, min(u_end - u, upe - j.us));
            j.row0 = a.offsets[j.g];
            j.cnt = a.offsets[j.g + 1] - j.row0;
            j.tb = 0;
            if (j.cnt == 0u || (a.skip_from != 0u && j.cnt >= a.skip_from)) {   // empty, or left to the tensor-core path
                u = (slot + 1u) * upe;
                continue;
            }
            return true;
        }
        return false;
    };

    if (warp == kCWarps) {
        // ------------------------------------------------------------------ producer
        uint32_t it = 0, u = u_begin;
        JobInfo j;
        bool ok = true;
        for (bool have = next_job(u, j, true); have && ok; have = next_job(u, j, false)) {
            // tile p of the job: gate / up rows [16 us, 16 (us + nu)), or the two halves of 32 nu down rows
            const CUtensorMap* m0 = maps + ((size_t)(DUAL ? 0u : 2u) * a.n_groups + j.g) * 3u;
            const CUtensorMap* m1 = maps + ((size_t)(DUAL ? 1u : 2u) * a.n_groups + j.g) * 3u;
            const uint32_t rowp0 = DUAL ? j.us * 16u : j.us * 32u;
            const uint32_t rowp1 = DUAL ? j.us * 16u : j.us * 32u + j.nu * 16u;
            const bool full_job = j.nu == kJobUnits;
            for (uint32_t c = 0; c < chunks; ++c, ++it) {
                const uint32_t s = it % S, ph = (it / S) & 1u;
                uint32_t got = 1;
                if (lane == 0) got = mbar_wait(&C.empty[s], ph ^ 1u, abort_flag) ? 1u : 0u;
                got = __shfl_sync(0xFFFFFFFFu, got, 0);
                if (!got) { ok = false; break; }
                const uint32_t nks = min(kStageSteps, steps - c * kStageSteps);
                const uint32_t khalves = (nks + 1u) / 2u;                // 128-byte K slices in this stage (1 or 2)
                uint8_t* st = stages + (size_t)s * G::kStageBytes;
                // Few, large requests: one elected lane issues a request in some tens of nanoseconds, and a stage of a
                // dozen requests (one per box, row and scale slice) was bounded by that, not by memory.  A full job is
                // two weight boxes of 16 KB (3-D: 128 bytes x 64 rows x 2 K slices; a slice past the end of K arrives
                // as zeros and still counts), two scale boxes and one box of activation rows per operand half.
                if (lane == 0) {
                    const uint32_t wtx = full_job ? 2u * 2u * kBoxBytes : 2u * khalves * j.nu * 16u * 128u;
                    const uint32_t stx = 2u * kBoxRows * ScaleGeo<FMT>::kPitch;
                    mbar_arrive_expect_tx(&C.full[s], wtx + stx + (SPLIT ? 2u : 1u) * G::kXBoxBytes);
                }
                __syncwarp();
                if (lane < 2u) {
                    // weights of tile p
                    const uint32_t p = lane;
                    const CUtensorMap* m = p ? m1 : m0;
                    uint8_t* dst = st + G::kWOff + p * 2u * kBoxBytes;
                    const uint32_t y0 = p ? rowp1 : rowp0;
                    if (full_job) {
                        tma_box3(dst, m + 0, 0u, y0, c * 2u, &C.full[s]);
                    } else {
                        for (uint32_t kh = 0; kh < khalves; ++kh)
                            for (uint32_t q = 0; q < j.nu; ++q)
                                tma_box(dst + kh * kBoxBytes + q * 2048u, m + 1, c * (kStageSteps * 64u) + kh * 128u,
                                        y0 + q * 16u, &C.full[s]);
                    }
                } else if (lane < 4u) {
                    // block scales of the 64 rows from the tile's first row on (rows past the job are not read)
                    const uint32_t p = lane - 2u;
                    tma_box(st + G::kSOff + p * kBoxRows * ScaleGeo<FMT>::kPitch, (p ? m1 : m0) + 2,
                            c * ScaleGeo<FMT>::kPitch, p ? rowp1 : rowp0, &C.full[s]);
                } else if (lane < (SPLIT ? 6u : 5u)) {
                    // 8 NT activation rows from the job's first token row on, 512 columns: rows past the group belong
                    // to the next group (their results are dropped), rows or columns past the buffer arrive as zeros
                    const bool lo = lane == 5u;
                    tma_box3(st + G::kXOff + (lo ? G::kXBoxBytes : 0u), lo ? &xmap_lo : &xmap_hi, 0u, j.row0 + j.tb,
                             c * kXSlabs, &C.full[s]);
                }
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicOr(a.status, kStatusWaitTimeout); }
        __syncwarp();
        if (*abort_flag && lane == 0) {
            // copies issued but possibly not consumed: give each a bounded chance to land before the
            // CTA's shared memory is released
            const uint32_t pending = it < S ? it : S;
            for (uint32_t q = 0; q < pending; ++q) {
                const uint32_t jdx = it - 1u - q;
                for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                    if (mbar_test(&C.full[jdx % S], (jdx / S) & 1u)) break;
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    const uint32_t gid = lane >> 2, t = lane & 3u;
    const uint32_t unit = warp >> 2;           // which unit of a job
    const uint32_t ks = warp & 3u;             // which k-step of a stage
    const uint32_t stage_base = smem_addr(stages);
    const float* rowscale = DUAL ? a.x_rowscale : a.act_rowscale;
    // byte offsets inside a weight box of this lane's rows (16 unit + gid and + 8) for the k-step's four words:
    // chunk (ks & 1) * 4 + wd of the 128-byte row, swizzled by row & 7 (= gid for both rows)
    const uint32_t kh = ks >> 1;
    const uint32_t row_lo = unit * 16u + gid;
    uint32_t woff[4];
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) woff[wd] = row_lo * 128u + ((((ks & 1u) * 4u + (uint32_t)wd) ^ gid) << 4) + t * 4u;
    uint32_t it = 0, u = u_begin, jobs_done = 0;
    JobInfo j;
    bool ok = true, bad = false;
    for (bool have = next_job(u, j, true); have && ok; have = next_job(u, j, false), ++jobs_done) {
        float acc0[NT][4], acc1[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc0[nt][q] = acc1[nt][q] = 0.0f;
        const int32_t mx0 = 0, mx1 = 0;   // NVFP4 multipliers need no exponent base
        const bool my_unit = unit < j.nu;
        for (uint32_t c = 0; c < chunks; ++c, ++it) {
            const uint32_t s = it % S, ph = (it / S) & 1u;
            if (!warp_wait(&C.full[s], ph, abort_flag)) { ok = false; break; }
            const uint32_t nks = min(kStageSteps, steps - c * kStageSteps);
            if (my_unit && ks < nks) {
                const uint32_t st = stage_base + s * G::kStageBytes;
                const uint32_t box0 = st + G::kWOff + kh * kBoxBytes;             // tile 0, this k half
                const uint32_t box1 = box0 + 2u * kBoxBytes;                      // tile 1
                const uint32_t sc0 = st + G::kSOff + row_lo * ScaleGeo<FMT>::kPitch + ks * ScaleGeo<FMT>::kStepBytes;
                const uint32_t sc1 = sc0 + kBoxRows * ScaleGeo<FMT>::kPitch;
                // activation box: [slab][8 NT rows][128 B], 16-byte chunk c of row r at chunk position c ^ (r & 7); this
                // lane's word wd of the k-step lies in slab 2 ks + (wd >> 1), chunk 4 (wd & 1) + t, of row gid (+ 8 nt)
                uint32_t xoff[4];
#pragma unroll
                for (int wd = 0; wd < 4; ++wd)
                    xoff[wd] = st + G::kXOff + ((ks * 2u + ((uint32_t)wd >> 1)) * (8u * NT) + gid) * 128u +
                               ((((uint32_t)(wd & 1) * 4u + t) ^ gid) << 4);
                if (FMT == STRATA_MOE_FMT_MXFP4) {
                    // E8M0 block scales are powers of two and one 32-column block is exactly the two MMAs of
                    // a (word index, tile): the raw E2M1 values go into the MMAs and the FP32 partial sum of
                    // the block is scaled (exactly) on its way into the accumulator -- four multiply-adds in
                    // place of sixteen packed multiplies on the weights.  Byte 0 decodes to 0, 0xFF to +inf.
                    const uint32_t s0l = lds32(sc0), s0h = lds32(sc0 + 8u * ScaleGeo<FMT>::kPitch);
                    const uint32_t s1l = lds32(sc1), s1h = lds32(sc1 + 8u * ScaleGeo<FMT>::kPitch);
#pragma unroll
                    for (int wd = 0; wd < 4; ++wd) {
                        uint4 bh[NT], bl[SPLIT ? NT : 1];
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            bh[nt] = lds128(xoff[wd] + (uint32_t)nt * 1024u);
                            if (SPLIT) bl[nt] = lds128(xoff[wd] + G::kXBoxBytes + (uint32_t)nt * 1024u);
                        }
#pragma unroll
                        for (int p = 0; p < 2; ++p) {
                            const uint32_t box = p ? box1 : box0;
                            uint32_t al[4], ah[4];
                            e2m1x8(lds32(box + woff[wd]), al);
                            e2m1x8(lds32(box + woff[wd] + 8u * 128u), ah);
                            const float fl = __uint_as_float((((p ? s1l : s0l) >> (8 * wd)) & 0xFFu) << 23);
                            const float fh = __uint_as_float((((p ? s1h : s0h) >> (8 * wd)) & 0xFFu) << 23);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                float tmp[4];
                                mma_f16_zero(tmp, al[0], ah[0], al[1], ah[1], bh[nt].x, bh[nt].y);
                                mma_f16(tmp, al[2], ah[2], al[3], ah[3], bh[nt].z, bh[nt].w);
                                if (SPLIT) {
                                    mma_f16(tmp, al[0], ah[0], al[1], ah[1], bl[nt].x, bl[nt].y);
                                    mma_f16(tmp, al[2], ah[2], al[3], ah[3], bl[nt].z, bl[nt].w);
                                }
                                float* cacc = p ? acc1[nt] : acc0[nt];
                                cacc[0] = fmaf(tmp[0], fl, cacc[0]);
                                cacc[1] = fmaf(tmp[1], fl, cacc[1]);
                                cacc[2] = fmaf(tmp[2], fh, cacc[2]);
                                cacc[3] = fmaf(tmp[3], fh, cacc[3]);
                            }
                        }
                    }
                } else {
                    uint32_t m0l[4], m0h[4], m1l[4], m1h[4];
                    step_mults<FMT>(sc0, mx0, t, m0l);
                    step_mults<FMT>(sc0 + 8u * ScaleGeo<FMT>::kPitch, mx0, t, m0h);
                    step_mults<FMT>(sc1, mx1, t, m1l);
                    step_mults<FMT>(sc1 + 8u * ScaleGeo<FMT>::kPitch, mx1, t, m1h);
#pragma unroll
                    for (int wd = 0; wd < 4; ++wd) {
                        uint4 bh[NT], bl[SPLIT ? NT : 1];
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            bh[nt] = lds128(xoff[wd] + (uint32_t)nt * 1024u);
                            if (SPLIT) bl[nt] = lds128(xoff[wd] + G::kXBoxBytes + (uint32_t)nt * 1024u);
                        }
#pragma unroll
                        for (int p = 0; p < 2; ++p) {
                            const uint32_t box = p ? box1 : box0;
                            const uint32_t wlo = lds32(box + woff[wd]);
                            const uint32_t whi = lds32(box + woff[wd] + 8u * 128u);
                            uint32_t al[4], ah[4];
                            e2m1x8(wlo, al);
                            e2m1x8(whi, ah);
                            const uint32_t ml = p ? m1l[wd] : m0l[wd], mh = p ? m1h[wd] : m0h[wd];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                al[q] = mul2(al[q], ml);
                                ah[q] = mul2(ah[q], mh);
                            }
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                float* cacc = p ? acc1[nt] : acc0[nt];
                                mma_f16(cacc, al[0], ah[0], al[1], ah[1], bh[nt].x, bh[nt].y);
                                mma_f16(cacc, al[2], ah[2], al[3], ah[3], bh[nt].z, bh[nt].w);
                                if (SPLIT) {
                                    mma_f16(cacc, al[0], ah[0], al[1], ah[1], bl[nt].x, bl[nt].y);
                                    mma_f16(cacc, al[2], ah[2], al[3], ah[3], bl[nt].z, bl[nt].w);
                                }
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&C.empty[s]);
        }
        if (!ok) break;

        // ---- the four partial sums of every unit meet in shared memory -----------------------------
        if (!warp_wait(&C.red_free, (jobs_done & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        float* mine = red + (size_t)warp * (8u * NT) * 32u;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                mine[(nt * 8 + q) * 32 + lane] = acc0[nt][q];
                mine[(nt * 8 + 4 + q) * 32 + lane] = acc1[nt][q];
            }
        __syncwarp();
        if (lane == 0) mbar_arrive(&C.red_ready);
        if (!warp_wait(&C.red_ready, jobs_done & 1u, abort_flag)) { ok = false; break; }
        // warp (unit, ks) finishes the accumulator pairs q = ks, ks + 4, ... of its unit; the four partial
        // sums are added in k-step order
        if (my_unit) {
            float s0 = 1.0f, s1 = 1.0f;     // MXFP4: the block scales went into the accumulators whole
            if (FMT != STRATA_MOE_FMT_MXFP4) {
                if (DUAL) { s0 = a.gate.post_scale[j.g]; s1 = a.up.post_scale[j.g]; }
                else { s0 = s1 = a.down.post_scale[j.g]; }
            }
            for (uint32_t q = ks; q < 4u * NT; q += 4u) {
                const uint32_t nt = q >> 2, jj = q & 3u;
                float v0 = 0.0f, v1 = 0.0f;
#pragma unroll
                for (uint32_t k2 = 0; k2 < 4u; ++k2) {
                    const float* src = red + (size_t)(unit * 4u + k2) * (8u * NT) * 32u;
                    v0 += src[(nt * 8u + jj) * 32u + lane];
                    v1 += src[(nt * 8u + 4u + jj) * 32u + lane];
                }
                const uint32_t tok = j.tb + nt * 8u + t * 2u + (jj & 1u);
                if (tok < j.cnt) {
                    const size_t pos = (size_t)j.row0 + tok;
                    const float rs = rowscale[pos];
                    const uint32_t r16 = unit * 16u + gid + ((jj & 2u) ? 8u : 0u);
                    if (DUAL) {
                        const uint32_t orow = j.us * 16u + r16;
                        const float gv = v0 * s0 * rs, uv = v1 * s1 * rs;
                        float v = a.glu.kind == STRATA_MOE_ACT_SWIGLU ? silu_mul_s(gv, uv) : glu_other(gv, uv, a.glu);
                        if (a.coef) v *= a.coef[pos];
                        if (a.act_direct) {
                            // f16 hi + lo straight from the epilogue (unit row factor): the down kernel's operand
                            // without a conversion pass; a value beyond the f16 range is reported, not clipped
                            if (!(fabsf(v) <= 65504.0f)) bad = true;
                            const __half h = __float2half_rn(v);
                            reinterpret_cast<__half*>(a.act_hi)[pos * R + orow] = h;
                            reinterpret_cast<__half*>(a.act_lo)[pos * R + orow] = __float2half_rn(v - __half2float(h));
                            if (orow == 0u) a.act_rowscale_out[pos] = 1.0f;
                        } else {
                            if (!(fabsf(v) <= 3.0e38f)) bad = true;
                            a.act_f32[pos * R + orow] = v;
                        }
                    } else {
                        const uint32_t orow = j.us * 32u + r16;
                        const float y0 = v0 * s0 * rs, y1 = v1 * s1 * rs;
                        if (!(fabsf(y0) <= 3.0e38f) || !(fabsf(y1) <= 3.0e38f)) bad = true;
                        a.y[pos * R + orow] = y0;
                        a.y[pos * R + orow + j.nu * 16u] = y1;
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&C.red_free);
    }
    if (!ok && lane == 0) { *abort_flag = 1; atomicOr(a.status, kStatusWaitTimeout); }
    if (bad) atomicOr(a.status, kStatusNonFiniteOutput);
}

typedef CUresult (*EncodeTiledFnS)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFnS encode_fn_s() {
    static EncodeTiledFnS fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFnS>(p);
    }
    return fn;
}

bool encode_u8_map(CUtensorMap* m, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes,
                   uint32_t box_rows, bool swizzle) {
    EncodeTiledFnS fn = encode_fn_s();
    if (!fn) return false;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_bytes, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [rows, row_bytes] bytes seen as {128 B, rows, row_bytes / 128 slabs}: one box = box_rows rows x box_slabs slabs,
// laid out [slab][row][128 B] with the 128-byte swizzle (what the consumers' addressing expects)
bool encode_slab_map(CUtensorMap* m, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows,
                     uint32_t box_slabs) {
    EncodeTiledFnS fn = encode_fn_s();
    if (!fn || row_bytes % 128u) return false;
    const cuuint64_t dims[3] = {128, rows, row_bytes / 128u};
    const cuuint64_t strides[2] = {row_bytes, 128};
    const cuuint32_t box[3] = {128, box_rows, box_slabs};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int FMT, int NT, bool SPLIT, bool DUAL>
int launch_stream_one(const DecodeArgs& a, const void* maps, cudaStream_t s) {
    using G = StreamGeo<FMT, NT, SPLIT>;
    static bool attr[64] = {};   // the shared-memory opt-in is per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    if (!attr[dev]) {
        if (cudaFuncSetAttribute(decode_stream_kernel<FMT, NT, SPLIT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)G::kSmem) != cudaSuccess)
            return -1;
        attr[dev] = true;
    }
    const uint32_t R = DUAL ? a.I : a.H;
    const uint32_t jobs = a.n_groups * ((DUAL ? R / 16u : R / 32u) + kJobUnits - 1u) / kJobUnits;
    if (jobs == 0u) return 0;
    const uint32_t grid = jobs < (uint32_t)kNumSMs ? jobs : (uint32_t)kNumSMs;
    // the activation rows of this launch: f16 [x_rows, K], hi (and lo) halves
    const uint32_t K = DUAL ? a.H : a.I;
    const void* xh = DUAL ? static_cast<const void*>(a.x_hi) : static_cast<const void*>(a.act_hi);
    const void* xl = DUAL ? static_cast<const void*>(a.x_lo) : static_cast<const void*>(a.act_lo);
    CUtensorMap xmap_hi, xmap_lo;
    if (a.x_rows == 0u || !encode_slab_map(&xmap_hi, xh, (uint64_t)K * 2u, a.x_rows, 8u * NT, kXSlabs)) return -1;
    if (SPLIT) {
        if (!encode_slab_map(&xmap_lo, xl, (uint64_t)K * 2u, a.x_rows, 8u * NT, kXSlabs)) return -1;
    } else {
        xmap_lo = xmap_hi;
    }
    decode_stream_kernel<FMT, NT, SPLIT, DUAL><<<grid, kSThreads, G::kSmem, s>>>(a, static_cast<const CUtensorMap*>(maps),
                                                                                 xmap_hi, xmap_lo);
    ++g_kernel_launches;
    return 0;
}

template <int FMT, bool SPLIT, bool DUAL>
int launch_stream_nt(const DecodeArgs& a, const void* maps, cudaStream_t s) {
    return a.max_rows_per_group <= 8u ? launch_stream_one<FMT, 1, SPLIT, DUAL>(a, maps, s)
                                      : launch_stream_one<FMT, 2, SPLIT, DUAL>(a, maps, s);
}

}  // namespace

bool decode_stream_supported(int fmt, uint32_t H, uint32_t I) {
    // a stage carries whole 16-byte pieces of block scales per row: MXFP4 (4 bytes per k-step) needs K % 512 == 0,
    // NVFP4 (8 bytes per k-step) K % 256 == 0, for both K = H (gate/up) and K = I (down)
    if (encode_fn_s() == nullptr) return false;
    if (fmt == STRATA_MOE_FMT_MXFP4) return H % 512u == 0u && I % 512u == 0u;
    if (fmt == STRATA_MOE_FMT_NVFP4) return H % 256u == 0u && I % 256u == 0u;
    return false;
}

// The three tensor maps of one projection ([rows, K] weights of format fmt) into out (3 x 128 bytes, host memory):
// 64-row x two-slice boxes (3-D, one request per tile and stage) and 16-row boxes of 128 packed bytes (both with the
// 128-byte swizzle), and 64-row boxes of one stage's scale bytes.
int decode_stream_encode_maps(void* out, int fmt, const void* packed, const void* scales, uint32_t rows, uint32_t K) {
    static_assert(sizeof(CUtensorMap) == 128, "descriptor size");
    CUtensorMap* m = static_cast<CUtensorMap*>(out);
    const uint32_t spitch = fmt == STRATA_MOE_FMT_MXFP4 ? ScaleGeo<STRATA_MOE_FMT_MXFP4>::kPitch
                                                        : ScaleGeo<STRATA_MOE_FMT_NVFP4>::kPitch;
    const uint64_t srow = fmt == STRATA_MOE_FMT_MXFP4 ? K / 32u : K / 16u;
    if (!encode_slab_map(m + 0, packed, K / 2u, rows, kBoxRows, 2)) return -1;
    if (!encode_u8_map(m + 1, packed, K / 2u, rows, 128, 16, true)) return -1;
    if (!encode_u8_map(m + 2, scales, srow, rows, spitch, kBoxRows, false)) return -1;
    return 0;
}

int launch_decode_stream_gate_up(const DecodeArgs& a, const void* maps, cudaStream_t s) {
    if (a.fmt == STRATA_MOE_FMT_MXFP4) return launch_stream_nt<STRATA_MOE_FMT_MXFP4, false, true>(a, maps, s);
    return launch_stream_nt<STRATA_MOE_FMT_NVFP4, false, true>(a, maps, s);
}

int launch_decode_stream_down(const DecodeArgs& a, const void* maps, cudaStream_t s) {
    if (a.fmt == STRATA_MOE_FMT_MXFP4) return launch_stream_nt<STRATA_MOE_FMT_MXFP4, true, false>(a, maps, s);
    return launch_stream_nt<STRATA_MOE_FMT_NVFP4, true, false>(a, maps, s);
}

}  // namespace smoe
