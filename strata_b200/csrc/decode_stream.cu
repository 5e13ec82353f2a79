// Small-batch expert FFN for the FP4 formats, weight tiles STREAMED HBM -> shared memory by the
// copy engine: the kernel the decode roofline is measured on.
//
// One persistent CTA per SM.  A producer warp walks the CTA's jobs and fills a ring of shared-
// memory stages with bulk asynchronous copies (cp.async.bulk, completion counted in bytes on an
// mbarrier): per stage the packed 4-bit bytes of 64 weight rows x 512 columns (row segments of
// 256 contiguous bytes), their block scales, and the same 512 columns of the group's activation
// rows (f16).  With five to seven stages in the ring, 80-110 KB of weight bytes are in flight per
// SM, independent of how many warps are resident -- the loads no longer live in registers.
//
// Sixteen consumer warps read ONLY shared memory.  A job is 64 weight rows of one expert (gate/up:
// 32 gate rows + the same 32 up rows; down: 64 rows) against up to 8 * NT token rows, all of K.
// A stage holds four k-steps of 128 columns; the warps form two groups of eight that take
// alternate stages, and inside a group a warp owns one (16-row tile pair, k-step) cell: it decodes
// its rows with the hardware E2M1 -> f16 conversion, folds the block scale in with one packed
// multiply (exact, as in decode_fp4.cu) and issues m16n8k16 F16 MMAs with FP32 accumulation.  At
// the end of a job the sixteen partial accumulators of the K split meet in shared memory and are
// summed in a fixed order, so results are bit-reproducible.
//
// Bank conflicts: weight row segments sit 272 bytes apart (256 + 16) and lane (g, t) reads the
// 32-bit words t, t+4, t+8, t+12 of its row's 64-byte k-step slice, so a warp-wide 32-bit load
// covers 8 rows x 16 bytes = all 32 banks once; activation rows sit 1088 bytes apart (1024 + 64)
// and the four lanes of a quad read 64 contiguous bytes, so an 8-lane phase of a 128-bit load
// covers two rows x 64 bytes = all banks once.  Word wd * 4 + t of a k-step holds columns
// 8 (wd * 4 + t) .. + 7, which is also activation chunk wd * 4 + t: natural column order.
//
// Every wait is bounded; on expiry the kernel raises kStatusWaitTimeout, all roles leave, the
// producer gives the copies still in flight a bounded chance to land, and the kernel returns.
//
// Replaces the reference's per-row NVFP4 / DeepSeek FP4 expert kernels for decode batches
// (kernels/cuda/backend.cu:1978-2069, 2308-2413).
#include "stream_ring.cuh"

namespace smoe {

using namespace ring;

namespace {

constexpr uint32_t kCWarps = 16;                  // consumer warps: two groups of eight
constexpr uint32_t kSThreads = (kCWarps + 1) * 32;
constexpr uint32_t kStageSteps = 4;               // k-steps of 128 columns per stage
constexpr uint32_t kJobSegs = 64;                 // weight row segments per stage
constexpr uint32_t kWP = kStageSteps * 64 + 16;   // bytes between row segments (272)
constexpr uint32_t kXP = kStageSteps * 256 + 64;  // bytes between activation rows (1088)
constexpr int kMxBiasS = 2;                       // f16 exponent field of an MXFP4 multiplier is e - emin + 2

template <int FMT>
struct ScaleGeo {
    static constexpr uint32_t kStepBytes = FMT == STRATA_MOE_FMT_MXFP4 ? 4u : 8u;   // scale bytes per row per k-step
    static constexpr uint32_t kPitch = kStepBytes * kStageSteps;                    // 16 or 32
};

template <int FMT, int NT, bool SPLIT>
struct StreamGeo {
    static constexpr uint32_t kXRows = 8u * NT * (SPLIT ? 2u : 1u);
    static constexpr uint32_t kWOff = 0;
    static constexpr uint32_t kSOff = kJobSegs * kWP;
    static constexpr uint32_t kXOff = kSOff + kJobSegs * ScaleGeo<FMT>::kPitch;
    static constexpr uint32_t kStageBytes = (kXOff + kXRows * kXP + 127u) / 128u * 128u;
    static constexpr uint32_t kRedBytes = kCWarps * 32u * 8u * NT * 4u;
    static constexpr uint32_t kBudget = 224u * 1024u;
    static constexpr uint32_t kStagesRaw = (kBudget - kRedBytes - 512u) / kStageBytes;
    static constexpr uint32_t kStages = kStagesRaw > 8u ? 8u : kStagesRaw;
    static constexpr uint32_t kSmem = kStages * kStageBytes + kRedBytes + 512u + 128u;
    static_assert(kStages >= 3, "ring too shallow");
};

struct StreamCtl {                 // 512 bytes at the front of the dynamic shared memory
    uint64_t full[8], empty[8];
    uint64_t red_ready, red_free;
    uint32_t abort_flag;
};

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
    uint32_t g, rt, row0, cnt, tb;
};

// DUAL = true : gate/up + SwiGLU, writes act fp32 [pairs, I].   K = H, 32 + 32 rows per job.
// DUAL = false: down, writes y fp32 [pairs, H].                 K = I, 64 rows per job.
template <int FMT, int NT, bool SPLIT, bool DUAL>
__global__ void __launch_bounds__(kSThreads, 1) decode_stream_kernel(DecodeArgs a) {
    using G = StreamGeo<FMT, NT, SPLIT>;
    constexpr uint32_t S = G::kStages;
    extern __shared__ uint8_t smem_raw_s[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_s) + 127) & ~uintptr_t(127));
    StreamCtl& C = *reinterpret_cast<StreamCtl*>(base);
    uint8_t* stages = base + 512;
    float* red = reinterpret_cast<float*>(stages + S * G::kStageBytes);   // [warp][8 NT][lane]
    volatile uint32_t* abort_flag = &C.abort_flag;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t K = DUAL ? a.H : a.I;
    const uint32_t R = DUAL ? a.I : a.H;
    const uint32_t tiles_per_group = DUAL ? R / 32u : R / 64u;
    const uint32_t n_act = a.active_list ? *a.n_active : a.n_groups;
    const uint32_t total = n_act * tiles_per_group;
    const uint32_t steps = K / 128u;
    const uint32_t chunks = (steps + kStageSteps - 1u) / kStageSteps;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(&C.full[s], 1);
            mbar_init(&C.empty[s], kCWarps / 2u);   // one arrival per warp of the group that owns the stage
        }
        mbar_init(&C.red_ready, kCWarps);
        mbar_init(&C.red_free, kCWarps);
        C.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // the job sequence of this CTA, walked identically by the producer and by every consumer
    auto next_job = [&](uint32_t& tile, JobInfo& j, bool first) -> bool {
        if (!first) {
            j.tb += 8u * NT;
            if (j.tb < j.cnt) return true;
            tile += gridDim.x;
        }
        for (; tile < total; tile += gridDim.x) {
            const uint32_t slot = tile / tiles_per_group;
            j.g = a.active_list ? a.active_list[slot] : slot;
            j.rt = tile - slot * tiles_per_group;
            j.row0 = a.offsets[j.g];
            j.cnt = a.offsets[j.g + 1] - j.row0;
            j.tb = 0;
            if (j.cnt == 0u || (a.skip_from != 0u && j.cnt >= a.skip_from)) continue;   // empty, or left to the tensor-core path
            return true;
        }
        return false;
    };

    const __half* xh_base = reinterpret_cast<const __half*>(DUAL ? a.x_hi : a.act_hi);
    const __half* xl_base = reinterpret_cast<const __half*>(DUAL ? a.x_lo : a.act_lo);

    if (warp == kCWarps) {
        // ------------------------------------------------------------------ producer
        uint32_t it = 0, tile = blockIdx.x;
        JobInfo j;
        bool ok = true;
        for (bool have = next_job(tile, j, true); have && ok; have = next_job(tile, j, false)) {
            const uint8_t* wp[2];
            const uint8_t* sp[2];
            if (DUAL) {
                wp[0] = a.gate.packed[j.g]; sp[0] = a.gate.scales[j.g];
                wp[1] = a.up.packed[j.g];   sp[1] = a.up.scales[j.g];
            } else {
                wp[0] = wp[1] = a.down.packed[j.g];
                sp[0] = sp[1] = a.down.scales[j.g];
            }
            const uint32_t nvalid = min(8u * NT, j.cnt - j.tb);
            for (uint32_t c = 0; c < chunks; ++c, ++it) {
                const uint32_t s = it % S, ph = (it / S) & 1u;
                uint32_t got = 1;
                if (lane == 0) got = mbar_wait(&C.empty[s], ph ^ 1u, abort_flag) ? 1u : 0u;
                got = __shfl_sync(0xFFFFFFFFu, got, 0);
                if (!got) { ok = false; break; }
                const uint32_t nks = min(kStageSteps, steps - c * kStageSteps);
                const uint32_t wbytes = nks * 64u, sbytes = nks * ScaleGeo<FMT>::kStepBytes, xbytes = nks * 256u;
                uint8_t* st = stages + (size_t)s * G::kStageBytes;
                if (lane == 0)
                    mbar_arrive_expect_tx(&C.full[s], kJobSegs * (wbytes + sbytes) + nvalid * (SPLIT ? 2u : 1u) * xbytes);
                __syncwarp();
                // segment i: tile pair i >> 5, tile (i >> 4) & 1 (gate / up, or the two halves of 32 down rows), row i & 15
                for (uint32_t i = lane; i < kJobSegs; i += 32u) {
                    const uint32_t pair = i >> 5, p = (i >> 4) & 1u, r = i & 15u;
                    const uint32_t row = DUAL ? j.rt * 32u + pair * 16u + r : j.rt * 64u + pair * 32u + p * 16u + r;
                    bulk_g2s(st + G::kWOff + i * kWP, wp[p] + (size_t)row * (K / 2u) + (size_t)c * (kStageSteps * 64u), wbytes,
                             &C.full[s]);
                    const uint32_t srow_bytes = FMT == STRATA_MOE_FMT_MXFP4 ? K / 32u : K / 16u;
                    bulk_g2s(st + G::kSOff + i * ScaleGeo<FMT>::kPitch,
                             sp[p] + (size_t)row * srow_bytes + (size_t)c * ScaleGeo<FMT>::kPitch, sbytes, &C.full[s]);
                }
                for (uint32_t i = lane; i < nvalid * (SPLIT ? 2u : 1u); i += 32u) {
                    const uint32_t tok = i < nvalid ? i : i - nvalid;
                    const __half* src = (i < nvalid ? xh_base : xl_base) + (size_t)(j.row0 + j.tb + tok) * K +
                                        (size_t)c * (kStageSteps * 128u);
                    const uint32_t slot = i < nvalid ? tok : 8u * NT + tok;
                    bulk_g2s(st + G::kXOff + slot * kXP, src, xbytes, &C.full[s]);
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
    const uint32_t grp = warp >> 3;            // which alternate stages this warp takes
    const uint32_t pair = (warp >> 2) & 1u;    // which 16-row tile pair of the job
    const uint32_t ks = warp & 3u;             // which k-step of a stage
    const uint32_t stage_base = smem_addr(stages);
    const float* rowscale = DUAL ? a.x_rowscale : a.act_rowscale;
    uint32_t it = 0, tile = blockIdx.x, jobs_done = 0;
    JobInfo j;
    bool ok = true, bad = false;
    for (bool have = next_job(tile, j, true); have && ok; have = next_job(tile, j, false), ++jobs_done) {
        float acc0[NT][4], acc1[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc0[nt][q] = acc1[nt][q] = 0.0f;
        int32_t mx0 = 0, mx1 = 0;
        if (FMT == STRATA_MOE_FMT_MXFP4) {
            mx0 = kMxBiasS - (int32_t)(DUAL ? a.gate.emin[j.g] : a.down.emin[j.g]);
            mx1 = kMxBiasS - (int32_t)(DUAL ? a.up.emin[j.g] : a.down.emin[j.g]);
        }
        for (uint32_t c = 0; c < chunks; ++c, ++it) {
            if ((it & 1u) != grp) continue;
            const uint32_t s = it % S, ph = (it / S) & 1u;
            if (!warp_wait(&C.full[s], ph, abort_flag)) { ok = false; break; }
            const uint32_t nks = min(kStageSteps, steps - c * kStageSteps);
            if (ks < nks) {
                const uint32_t st = stage_base + s * G::kStageBytes;
                const uint32_t seg0 = st + G::kWOff + (pair * 32u) * kWP + ks * 64u + t * 4u;   // tile 0, row 0
                const uint32_t sc0 = st + G::kSOff + (pair * 32u) * ScaleGeo<FMT>::kPitch + ks * ScaleGeo<FMT>::kStepBytes;
                uint32_t m0l[4], m0h[4], m1l[4], m1h[4];
                step_mults<FMT>(sc0 + gid * ScaleGeo<FMT>::kPitch, mx0, t, m0l);
                step_mults<FMT>(sc0 + (gid + 8u) * ScaleGeo<FMT>::kPitch, mx0, t, m0h);
                step_mults<FMT>(sc0 + (16u + gid) * ScaleGeo<FMT>::kPitch, mx1, t, m1l);
                step_mults<FMT>(sc0 + (24u + gid) * ScaleGeo<FMT>::kPitch, mx1, t, m1h);
                const uint32_t xrow = st + G::kXOff + gid * kXP + ks * 256u + t * 16u;
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) {
                    uint4 bh[NT], bl[SPLIT ? NT : 1];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        bh[nt] = lds128(xrow + (uint32_t)nt * 8u * kXP + (uint32_t)wd * 64u);
                        if (SPLIT) bl[nt] = lds128(xrow + (uint32_t)(NT + nt) * 8u * kXP + (uint32_t)wd * 64u);
                    }
#pragma unroll
                    for (int p = 0; p < 2; ++p) {
                        const uint32_t wlo = lds32(seg0 + (uint32_t)(p * 16 + (int)gid) * kWP + (uint32_t)wd * 16u);
                        const uint32_t whi = lds32(seg0 + (uint32_t)(p * 16 + 8 + (int)gid) * kWP + (uint32_t)wd * 16u);
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
            __syncwarp();
            if (lane == 0) mbar_arrive(&C.empty[s]);
        }
        if (!ok) break;

        // ---- the sixteen partial sums of the job meet in shared memory -----------------------------
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
        // reducer `ri` of this tile pair finishes accumulator pairs q = ri, ri + 8, ...; the eight partial
        // sums are added in a fixed order (group 0 k-steps 0..3, then group 1)
        const uint32_t ri = ks + 4u * grp;
        float s0, s1;
        if (DUAL) { s0 = a.gate.post_scale[j.g]; s1 = a.up.post_scale[j.g]; }
        else { s0 = s1 = a.down.post_scale[j.g]; }
        for (uint32_t q = ri; q < 4u * NT; q += 8u) {
            const uint32_t nt = q >> 2, jj = q & 3u;
            float v0 = 0.0f, v1 = 0.0f;
#pragma unroll
            for (uint32_t gsel = 0; gsel < 2u; ++gsel)
#pragma unroll
                for (uint32_t k2 = 0; k2 < 4u; ++k2) {
                    const float* src = red + (size_t)(gsel * 8u + pair * 4u + k2) * (8u * NT) * 32u;
                    v0 += src[(nt * 8u + jj) * 32u + lane];
                    v1 += src[(nt * 8u + 4u + jj) * 32u + lane];
                }
            const uint32_t tok = j.tb + nt * 8u + t * 2u + (jj & 1u);
            if (tok < j.cnt) {
                const size_t pos = (size_t)j.row0 + tok;
                const float rs = rowscale[pos];
                if (DUAL) {
                    const uint32_t orow = j.rt * 32u + pair * 16u + gid + ((jj & 2u) ? 8u : 0u);
                    const float gv = v0 * s0 * rs, uv = v1 * s1 * rs;
                    float v = a.glu.kind == STRATA_MOE_ACT_SWIGLU ? silu_mul_s(gv, uv) : glu_other(gv, uv, a.glu);
                    if (a.coef) v *= a.coef[pos];
                    if (!(fabsf(v) <= 3.0e38f)) bad = true;
                    a.act_f32[pos * R + orow] = v;
                } else {
                    const uint32_t orow = j.rt * 64u + pair * 32u + gid + ((jj & 2u) ? 8u : 0u);
                    const float y0 = v0 * s0 * rs, y1 = v1 * s1 * rs;
                    if (!(fabsf(y0) <= 3.0e38f) || !(fabsf(y1) <= 3.0e38f)) bad = true;
                    a.y[pos * R + orow] = y0;
                    a.y[pos * R + orow + 16u] = y1;
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&C.red_free);
    }
    if (!ok && lane == 0) { *abort_flag = 1; atomicOr(a.status, kStatusWaitTimeout); }
    if (bad) atomicOr(a.status, kStatusNonFiniteOutput);
}

template <int FMT, int NT, bool SPLIT, bool DUAL>
int launch_stream_one(const DecodeArgs& a, cudaStream_t s) {
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
    const uint32_t total = a.n_groups * (DUAL ? R / 32u : R / 64u);
    if (total == 0u) return 0;
    const uint32_t grid = total < (uint32_t)kNumSMs ? total : (uint32_t)kNumSMs;
    decode_stream_kernel<FMT, NT, SPLIT, DUAL><<<grid, kSThreads, G::kSmem, s>>>(a);
    ++g_kernel_launches;
    return 0;
}

template <int FMT, bool SPLIT, bool DUAL>
int launch_stream_nt(const DecodeArgs& a, cudaStream_t s) {
    return a.max_rows_per_group <= 8u ? launch_stream_one<FMT, 1, SPLIT, DUAL>(a, s)
                                      : launch_stream_one<FMT, 2, SPLIT, DUAL>(a, s);
}

}  // namespace

bool decode_stream_supported(int fmt, uint32_t H, uint32_t I) {
    // whole stages of block scales must be 16-byte pieces: MXFP4 (4 bytes per k-step) needs K % 512 == 0,
    // NVFP4 (8 bytes per k-step) K % 256 == 0, for both K = H (gate/up) and K = I (down)
    if (fmt == STRATA_MOE_FMT_MXFP4) return H % 512u == 0u && I % 512u == 0u;
    if (fmt == STRATA_MOE_FMT_NVFP4) return H % 256u == 0u && I % 256u == 0u;
    return false;
}

int launch_decode_stream_gate_up(const DecodeArgs& a, cudaStream_t s) {
    const bool split = a.x_lo != nullptr;
    if (a.fmt == STRATA_MOE_FMT_MXFP4)
        return split ? launch_stream_nt<STRATA_MOE_FMT_MXFP4, true, true>(a, s)
                     : launch_stream_nt<STRATA_MOE_FMT_MXFP4, false, true>(a, s);
    return split ? launch_stream_nt<STRATA_MOE_FMT_NVFP4, true, true>(a, s)
                 : launch_stream_nt<STRATA_MOE_FMT_NVFP4, false, true>(a, s);
}

int launch_decode_stream_down(const DecodeArgs& a, cudaStream_t s) {
    if (a.fmt == STRATA_MOE_FMT_MXFP4) return launch_stream_nt<STRATA_MOE_FMT_MXFP4, true, false>(a, s);
    return launch_stream_nt<STRATA_MOE_FMT_NVFP4, true, false>(a, s);
}

}  // namespace smoe
