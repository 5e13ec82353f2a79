// Router: BF16 projection in the reference's production accumulation order, then score,
// top-k and routing weights, one warp per token.
//
// The projection reproduces kernels/cuda/backend.cu:651-728 of the reference exactly: lane l of
// a warp owns columns l, l+32, ... of one expert row and accumulates them with a separate
// multiply and add (no FMA); five shuffle-down rounds fold the 32 partial sums.  Expert ids are
// a discontinuous function of the logits, so reproducing the order is what makes them
// bit-identical to the reference's.  For the same reason the scores use an expf that follows
// the host libm's algorithm step by step in double precision (see expf_libm below).
#include <cstdlib>

#include "common.cuh"
#include "libm_exact.cuh"
#include "rows_f16.cuh"
#include "stream_ring.cuh"

namespace smoe {

bool launch_router_logits_small(const __nv_bfloat16* x, const __nv_bfloat16* wg, uint32_t T, uint32_t H, uint32_t E,
                                float* logits, uint32_t* status, cudaStream_t s);

// ---------------------------------------------------------------------------------------
// logits[t, e] for a tile of TT tokens and WARPS expert rows per CTA.  The activation tile and
// each warp's weight-row chunk are staged in shared memory as fp32, transposed so that lane l
// reads its columns l, l+32, ... of a 256-column chunk as two 16-byte vectors.
constexpr int kRouterChunk = 256;

__device__ __forceinline__ void router_stage8(float (*dst)[32][4], uint32_t c8, const uint4& v) {
    // 8 consecutive columns c8..c8+7 -> dst[j >> 2][lane][j & 3] with column = lane + 32 j
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const uint32_t c = c8 + p, l = c & 31u, j = c >> 5;
        const uint32_t bits = (p & 1) ? (w[p >> 1] & 0xFFFF0000u) : (w[p >> 1] << 16);
        dst[j >> 2][l][j & 3u] = __uint_as_float(bits);
    }
}

// LIST = true: the tokens are list[0 .. *count) (indices into x and logits) and the blocks of a
// column of the grid stride over the list, whose length is only known on the device.
template <int WARPS, int TT, bool LIST>
__global__ void __launch_bounds__(WARPS * 32) router_logits_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg, uint32_t T, uint32_t H,
    uint32_t E, float* __restrict__ logits, const uint32_t* __restrict__ list, const uint32_t* __restrict__ count) {
    // xs[tok][half][lane][4] : column = chunk + lane + 32 * (half * 4 + i)
    __shared__ __align__(16) float xs[TT][2][32][4];
    __shared__ __align__(16) float ws[WARPS][2][32][4];
    constexpr int THREADS = WARPS * 32;
    constexpr int XV = (TT * (kRouterChunk / 8) + THREADS - 1) / THREADS;  // uint4 per thread
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t e = blockIdx.x * WARPS + warp;
    const bool e_ok = e < E;
    if (LIST) T = *count;
  for (uint32_t t0 = blockIdx.y * TT; t0 < T; t0 += gridDim.y * TT) {
    const uint32_t nt = min((uint32_t)TT, T - t0);
    __shared__ uint32_t tok_of[TT];
    if (LIST) {
        __syncthreads();
        if (threadIdx.x < TT) tok_of[threadIdx.x] = threadIdx.x < nt ? list[t0 + threadIdx.x] : 0u;
        __syncthreads();
    }
    float sum[TT];
#pragma unroll
    for (int i = 0; i < TT; ++i) sum[i] = 0.0f;

    uint4 xr[XV], wr;
    auto fetch = [&](uint32_t c0) {
        const uint32_t cols = min((uint32_t)kRouterChunk, H - c0);
#pragma unroll
        for (int q = 0; q < XV; ++q) {
            const uint32_t i = threadIdx.x + q * THREADS;
            const uint32_t tok = i / (kRouterChunk / 8), c8 = (i % (kRouterChunk / 8)) * 8u;
            xr[q] = make_uint4(0, 0, 0, 0);
            if (i < TT * (kRouterChunk / 8) && tok < nt && c8 < cols)
                xr[q] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)(LIST ? tok_of[tok] : t0 + tok) * H + c0 + c8));
        }
        wr = make_uint4(0, 0, 0, 0);
        if (e_ok && lane * 8u < cols)
            wr = __ldg(reinterpret_cast<const uint4*>(wg + (size_t)e * H + c0 + lane * 8u));
    };
    fetch(0);
    for (uint32_t c0 = 0; c0 < H; c0 += kRouterChunk) {
        const uint32_t cols = min((uint32_t)kRouterChunk, H - c0);  // multiple of 32
        __syncthreads();  // everyone is done reading the previous chunk
#pragma unroll
        for (int q = 0; q < XV; ++q) {
            const uint32_t i = threadIdx.x + q * THREADS;
            if (i < TT * (kRouterChunk / 8))
                router_stage8(xs[i / (kRouterChunk / 8)], (i % (kRouterChunk / 8)) * 8u, xr[q]);
        }
        router_stage8(ws[warp], lane * 8u, wr);
        __syncthreads();
        if (c0 + kRouterChunk < H) fetch(c0 + kRouterChunk);  // overlaps the arithmetic below
        const uint32_t nj = cols >> 5;  // columns lane + 32 j, j < nj, exist
        const float4 w0 = *reinterpret_cast<const float4*>(ws[warp][0][lane]);
        const float4 w1 = *reinterpret_cast<const float4*>(ws[warp][1][lane]);
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int tok = 0; tok < TT; ++tok) {
            const float4 a0 = *reinterpret_cast<const float4*>(xs[tok][0][lane]);
            const float4 a1 = *reinterpret_cast<const float4*>(xs[tok][1][lane]);
            const float xv[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            float s = sum[tok];
            if (nj == 8u) {
#pragma unroll
                for (int j = 0; j < 8; ++j) s = __fmaf_rn(xv[j], wv[j], s);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if ((uint32_t)j < nj) s = __fmaf_rn(xv[j], wv[j], s);
            }
            sum[tok] = s;
        }
    }
#pragma unroll
    for (int tok = 0; tok < TT; ++tok) {
        float v = sum[tok];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v = __fadd_rn(v, __shfl_down_sync(0xFFFFFFFFu, v, off));
        if (e_ok && lane == 0 && (uint32_t)tok < nt) logits[(size_t)(LIST ? tok_of[tok] : t0 + tok) * E + e] = v;
    }
    if (!LIST) break;
  }
}

// A single token (decode): the projection is a latency problem -- E rows of H BF16 values, a few bytes each
// per lane.  One warp owns an expert row and issues ALL of its loads before the first use (lane l reads
// its own columns l, l + 32, ... directly, 64 contiguous bytes per warp load), so the row costs one trip
// to HBM instead of one per 256-column chunk; the activations of the few tokens come from L1/L2.
// Same per-lane order and the same shuffle tree as the kernels above.
constexpr int kTinyCols = 112;   // columns per lane held in registers at once (H <= 3584 in one pass)

template <int TT>
__global__ void __launch_bounds__(64) router_logits_tiny_kernel(const __nv_bfloat16* __restrict__ x,
                                                                const __nv_bfloat16* __restrict__ wg, uint32_t T,
                                                                uint32_t H, uint32_t E, float* __restrict__ logits) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t e = blockIdx.x * 2u + warp;
    if (e >= E) return;
    const unsigned short* wrow = reinterpret_cast<const unsigned short*>(wg) + (size_t)e * H + lane;
    const unsigned short* xb = reinterpret_cast<const unsigned short*>(x) + lane;
    const uint32_t per_lane = H / 32u;
    float sum[TT];
#pragma unroll
    for (int i = 0; i < TT; ++i) sum[i] = 0.0f;
    for (uint32_t j0 = 0; j0 < per_lane; j0 += kTinyCols) {
        float w[kTinyCols];
#pragma unroll
        for (int j = 0; j < kTinyCols; ++j)
            w[j] = j0 + j < per_lane ? __uint_as_float((uint32_t)__ldg(wrow + (size_t)(j0 + j) * 32u) << 16) : 0.0f;
#pragma unroll
        for (int tok = 0; tok < TT; ++tok) {
            if ((uint32_t)tok >= T) continue;   // uniform over the grid
            const unsigned short* xr = xb + (size_t)tok * H + (size_t)j0 * 32u;
            float s = sum[tok];
#pragma unroll
            for (int j = 0; j < kTinyCols; ++j) {
                if (j0 + j < per_lane) {    // past the row's end nothing is added (not even +0)
                    const float xv = __uint_as_float((uint32_t)__ldg(xr + (size_t)j * 32u) << 16);
                    s = __fmaf_rn(xv, w[j], s);
                }
            }
            sum[tok] = s;
        }
    }
#pragma unroll
    for (int tok = 0; tok < TT; ++tok) {
        float v = sum[tok];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v = __fadd_rn(v, __shfl_down_sync(0xFFFFFFFFu, v, off));
        if (lane == 0 && (uint32_t)tok < T) logits[(size_t)tok * E + e] = v;
    }
}

// Multiply-add: the reference rounds the product and the sum separately (__fmul_rn, __fadd_rn).  Both
// operands here are BF16 values, whose product has at most 16 significant bits and is therefore exact in
// FP32, so one fused multiply-add rounds exactly once, at the same place, and returns the same bits with
// half the instructions.  (The only divergence would need a product below 2^-126 added to a subnormal sum.)
//
// Large token counts: every warp owns RW expert rows and a 16-token tile, so one staged
// activation value feeds RW multiply-add chains and the staging cost is shared by 8 * RW rows.
// Same per-lane accumulation order as above (the order is a property of one (token, row) dot
// product, not of how dot products are batched).
// Shared layout per (token or row): lane l holds its 8 columns contiguously (32 bytes); the two
// 16-byte halves are swapped for lanes with bit 2 set, which makes the float4 reads conflict-free.
constexpr int kBigRW = 4;
constexpr int kBigWarps = 8;
constexpr int kBigTT = 16;

__device__ __forceinline__ void router_stage8_b(float* dst, uint32_t c8, const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const uint32_t c = c8 + p, l = c & 31u, j = c >> 5;
        const uint32_t bits = (p & 1) ? (w[p >> 1] & 0xFFFF0000u) : (w[p >> 1] << 16);
        dst[l * 8u + ((((j >> 2) ^ (l >> 2)) & 1u) << 2) + (j & 3u)] = __uint_as_float(bits);
    }
}

__global__ void __launch_bounds__(kBigWarps * 32, 1) router_logits_big_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg, uint32_t T, uint32_t H,
    uint32_t E, float* __restrict__ logits) {
    extern __shared__ __align__(16) float rsm[];
    float* xs = rsm;                              // [kBigTT][256]
    float* ws = rsm + kBigTT * kRouterChunk;      // [kBigWarps * kBigRW][256]
    constexpr int THREADS = kBigWarps * 32;
    constexpr int ROWS = kBigWarps * kBigRW;
    constexpr int XV = kBigTT * (kRouterChunk / 8) / THREADS;  // 2
    constexpr int WV = ROWS * (kRouterChunk / 8) / THREADS;    // 4
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t e0 = blockIdx.x * ROWS;
    const uint32_t t0 = blockIdx.y * kBigTT;
    const uint32_t nt = min((uint32_t)kBigTT, T - t0);
    float sum[kBigRW][kBigTT];
#pragma unroll
    for (int r = 0; r < kBigRW; ++r)
#pragma unroll
        for (int i = 0; i < kBigTT; ++i) sum[r][i] = 0.0f;

    uint4 xr[XV], wr[WV];
    auto fetch = [&](uint32_t c0) {
        const uint32_t cols = min((uint32_t)kRouterChunk, H - c0);
#pragma unroll
        for (int q = 0; q < XV; ++q) {
            const uint32_t i = threadIdx.x + q * THREADS;
            const uint32_t tok = i / (kRouterChunk / 8), c8 = (i % (kRouterChunk / 8)) * 8u;
            xr[q] = make_uint4(0, 0, 0, 0);
            if (tok < nt && c8 < cols)
                xr[q] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)(t0 + tok) * H + c0 + c8));
        }
#pragma unroll
        for (int q = 0; q < WV; ++q) {
            const uint32_t i = threadIdx.x + q * THREADS;
            const uint32_t row = i / (kRouterChunk / 8), c8 = (i % (kRouterChunk / 8)) * 8u;
            wr[q] = make_uint4(0, 0, 0, 0);
            if (e0 + row < E && c8 < cols)
                wr[q] = __ldg(reinterpret_cast<const uint4*>(wg + (size_t)(e0 + row) * H + c0 + c8));
        }
    };
    fetch(0);
    const uint32_t swz = ((lane >> 2) & 1u) << 2;  // which half holds j = 0..3 for this lane
    for (uint32_t c0 = 0; c0 < H; c0 += kRouterChunk) {
        const uint32_t cols = min((uint32_t)kRouterChunk, H - c0);
        __syncthreads();
#pragma unroll
        for (int q = 0; q < XV; ++q) {
            const uint32_t i = threadIdx.x + q * THREADS;
            router_stage8_b(xs + (i / (kRouterChunk / 8)) * kRouterChunk, (i % (kRouterChunk / 8)) * 8u, xr[q]);
        }
#pragma unroll
        for (int q = 0; q < WV; ++q) {
            const uint32_t i = threadIdx.x + q * THREADS;
            router_stage8_b(ws + (i / (kRouterChunk / 8)) * kRouterChunk, (i % (kRouterChunk / 8)) * 8u, wr[q]);
        }
        __syncthreads();
        if (c0 + kRouterChunk < H) fetch(c0 + kRouterChunk);
        const uint32_t nj = cols >> 5;
        float wv[kBigRW][8];
#pragma unroll
        for (int r = 0; r < kBigRW; ++r) {
            const float* wp = ws + (warp * kBigRW + r) * kRouterChunk + lane * 8u;
            const float4 a = *reinterpret_cast<const float4*>(wp + swz);
            const float4 b = *reinterpret_cast<const float4*>(wp + (swz ^ 4u));
            wv[r][0] = a.x; wv[r][1] = a.y; wv[r][2] = a.z; wv[r][3] = a.w;
            wv[r][4] = b.x; wv[r][5] = b.y; wv[r][6] = b.z; wv[r][7] = b.w;
        }
#pragma unroll
        for (int tok = 0; tok < kBigTT; ++tok) {
            const float* xp = xs + tok * kRouterChunk + lane * 8u;
            const float4 a = *reinterpret_cast<const float4*>(xp + swz);
            const float4 b = *reinterpret_cast<const float4*>(xp + (swz ^ 4u));
            const float xv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            if (nj == 8u) {
                // column-major over the rows: the kBigRW accumulators of a token form independent add chains,
                // so consecutive instructions never wait on each other (per (token, row) the order over j is
                // unchanged, which is all the reference order fixes)
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int r = 0; r < kBigRW; ++r) sum[r][tok] = __fmaf_rn(xv[j], wv[r][j], sum[r][tok]);
            } else {
#pragma unroll
                for (int r = 0; r < kBigRW; ++r)
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if ((uint32_t)j < nj) sum[r][tok] = __fmaf_rn(xv[j], wv[r][j], sum[r][tok]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kBigRW; ++r) {
        const uint32_t e = e0 + warp * kBigRW + r;
#pragma unroll
        for (int tok = 0; tok < kBigTT; ++tok) {
            float v = sum[r][tok];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v = __fadd_rn(v, __shfl_down_sync(0xFFFFFFFFu, v, off));
            if (lane == 0 && (uint32_t)tok < nt && e < E) logits[(size_t)(t0 + tok) * E + e] = v;
        }
    }
}

void launch_router_logits(const __nv_bfloat16* x, const __nv_bfloat16* wg, uint32_t T, uint32_t H,
                          uint32_t E, float* logits, cudaStream_t s, uint32_t* status) {
    if (T == 0) return;
    // decode batches: whole rows by bulk copy, one warp per token (25 -> about 6 us for 8 tokens at E = 256, H = 4096)
    if (status != nullptr && launch_router_logits_small(x, wg, T, H, E, logits, status, s)) return;
    // few tokens: one expert row per warp, two warps per CTA, so the rows spread over many SMs;
    // many tokens: register-blocked kernel (4 rows per warp, 32 rows per CTA)
    const size_t big_tiles = (size_t)((T + 15) / 16) * ((E + 31) / 32);
    if (T == 1) {
        // a single token: 10 vs 20 us at E = 256, H = 3072; with more tokens the staged kernel wins (the
        // per-token scalar activation loads of this kernel cost 33 us at 2 tokens, 88 us at 8)
        router_logits_tiny_kernel<2><<<(E + 1) / 2, 64, 0, s>>>(x, wg, T, H, E, logits);   // the 2-token build is the faster one even for one token (10 vs 31 us)
    } else if (T <= 8) {
        dim3 grid((E + 1) / 2, 1);
        router_logits_kernel<2, 8, false><<<grid, 64, 0, s>>>(x, wg, T, H, E, logits, nullptr, nullptr);
    } else if (T <= 32) {
        dim3 grid((E + 1) / 2, (T + 15) / 16);
        router_logits_kernel<2, 16, false><<<grid, 64, 0, s>>>(x, wg, T, H, E, logits, nullptr, nullptr);
    } else if (big_tiles < 96) {
        dim3 grid((E + 7) / 8, (T + 15) / 16);
        router_logits_kernel<8, 16, false><<<grid, 256, 0, s>>>(x, wg, T, H, E, logits, nullptr, nullptr);
    } else {
        static bool attr[64] = {};   // the shared-memory opt-in is per device
        const size_t smem = (size_t)(kBigTT + kBigWarps * kBigRW) * kRouterChunk * sizeof(float);
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && !attr[dev]) {
            cudaFuncSetAttribute(router_logits_big_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            attr[dev] = true;
        }
        dim3 grid((E + 31) / 32, (T + 15) / 16);
        router_logits_big_kernel<<<grid, kBigWarps * 32, smem, s>>>(x, wg, T, H, E, logits);
    }
    ++g_kernel_launches;
}

// Scores, top-k and routing weights of ONE token by one warp.  score / choice: [E] floats of shared memory each.
// Scores and selection values of the experts first, first + step, ... of one token (every rule but softmax, whose
// normaliser needs the whole row).  Returns true when a logit or bias is not finite.
__device__ __forceinline__ bool route_scores_part(const RouterParams& p, const float* __restrict__ lg,
                                                  const float* __restrict__ bias, float* score, float* choice,
                                                  uint32_t first, uint32_t step) {
    bool bad = false;
    for (uint32_t e = first; e < p.experts; e += step) {
        float l = lg[e];
        bad |= !isfinite(l);
        if (p.softcap > 0.0f) l = __fmul_rn(tanhf(__fdiv_rn(l, p.softcap)), p.softcap);
        float sc;
        if (p.score_kind == STRATA_MOE_SCORE_SIGMOID) sc = sigmoid_two_branch(l);
        else if (p.score_kind == STRATA_MOE_SCORE_SIGMOID_PLAIN)
            sc = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf_libm(-l)));
        else sc = sqrtf(l > 20.0f ? l : log1pf_libm(expf_libm(l)));
        const float b = bias ? bias[e] : 0.0f;
        bad |= !isfinite(b);
        score[e] = sc;
        choice[e] = __fadd_rn(sc, b);
    }
    return bad;
}

// scores_ready: score / choice were filled by route_scores_part (bad_in = its verdict); else they are computed here.
__device__ __forceinline__ void route_token(const RouterParams& p, const float* __restrict__ logits,
                                            const float* __restrict__ bias, uint32_t tok, float* score, float* choice,
                                            uint32_t* __restrict__ ids, float* __restrict__ weights, uint32_t* status,
                                            const uint32_t* __restrict__ forced_ids, bool scores_ready = false,
                                            bool bad_in = false) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t E = p.experts, k = p.top_k;
    const float* lg = logits + (size_t)tok * E;
    bool bad = bad_in;

    if (scores_ready) {
    } else if (p.score_kind == STRATA_MOE_SCORE_SOFTMAX) {
        float mx = -INFINITY;
        for (uint32_t e = lane; e < E; e += 32u) {
            const float l = lg[e];
            bad |= !isfinite(l);
            mx = fmaxf(mx, l);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
        for (uint32_t e = lane; e < E; e += 32u) score[e] = expf_libm(__fsub_rn(lg[e], mx));
        __syncwarp();
        float sum = 0.0f;  // index order, as a scalar loop sums it
        if (lane == 0)
            for (uint32_t e = 0; e < E; ++e) sum = __fadd_rn(sum, score[e]);
        sum = __shfl_sync(0xFFFFFFFFu, sum, 0);
        for (uint32_t e = lane; e < E; e += 32u) score[e] = __fdiv_rn(score[e], sum);
    } else {
        bad |= route_scores_part(p, lg, bias, score, choice, lane, 32u);
    }
    if (!scores_ready && p.score_kind == STRATA_MOE_SCORE_SOFTMAX)
        for (uint32_t e = lane; e < E; e += 32u) {
            const float b = bias ? bias[e] : 0.0f;
            bad |= !isfinite(b);
            choice[e] = __fadd_rn(score[e], b);
        }
    __syncwarp();

    // k rounds of arg-max over (value desc, index asc); taken entries drop to -inf.
    float my_w = 0.0f;
    uint32_t my_id = 0;
    // Hash routing (src/models/dsv4/deepseek_ops.cpp:390-461): the experts of a token come from a
    // table, only their weights are computed here -- same scores, same rank-order sum and division.
    for (uint32_t r = 0; forced_ids != nullptr && r < k; ++r) {
        uint32_t bi = forced_ids[(size_t)tok * k + r];
        if (bi >= E) { bad = true; bi = 0; }
        if (lane == r) { my_id = bi; my_w = score[bi]; }
    }
    for (uint32_t r = 0; forced_ids == nullptr && r < k; ++r) {
        float bv = -INFINITY;
        uint32_t bi = 0xFFFFFFFFu;
        for (uint32_t e = lane; e < E; e += 32u) {
            const float v = choice[e];
            if (v > bv || bi == 0xFFFFFFFFu) {
                if (v > bv || bi == 0xFFFFFFFFu) { bv = v; bi = e; }
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
            const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi >= E) { bad = true; bi = 0; }
        if (lane == r) { my_id = bi; my_w = score[bi]; }
        if (lane == 0) choice[bi] = -INFINITY;
        __syncwarp();
    }
    // weights: sum in rank order, divide, scale (lane r holds rank r; k <= 32)
    float sum = p.norm_init;
    for (uint32_t r = 0; r < k; ++r) sum = __fadd_rn(sum, __shfl_sync(0xFFFFFFFFu, my_w, r));
    float w = my_w;
    if (p.normalize) {
        if (!(sum > 0.0f) || !isfinite(sum)) {
            if (lane == 0) atomicOr(status, kStatusBadNormaliser);
            w = 0.0f;
        } else {
            w = __fmul_rn(__fdiv_rn(my_w, sum), p.weight_scale);
        }
    } else {
        w = __fmul_rn(my_w, p.weight_scale);
    }
    if (lane < k) {
        ids[(size_t)tok * k + lane] = my_id;
        weights[(size_t)tok * k + lane] = w;
    }
    if (__any_sync(0xFFFFFFFFu, bad) && lane == 0) atomicOr(status, kStatusNonFiniteLogit);
    __syncwarp();
}

// One warp per token.  Shared memory: score[E] and choice[E] per warp.
constexpr int kRouteWarps = 4;

__global__ void __launch_bounds__(kRouteWarps * 32) route_kernel(
    RouterParams p, const float* __restrict__ logits, const float* __restrict__ bias, uint32_t T,
    uint32_t* __restrict__ ids, float* __restrict__ weights, uint32_t* status,
    const uint32_t* __restrict__ forced_ids, const uint32_t* __restrict__ list, const uint32_t* __restrict__ count) {
    extern __shared__ float smem[];
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t E = p.experts;
    float* score = smem + (size_t)warp * 2u * E;
    float* choice = score + E;
    if (list) T = *count;     // tokens list[0 .. *count), the grid strides over them
    for (uint32_t slot = blockIdx.x * kRouteWarps + warp; slot < T; slot += gridDim.x * kRouteWarps)
        route_token(p, logits, bias, list ? list[slot] : slot, score, choice, ids, weights, status, forced_ids);
}

// ---------------------------------------------------------------------------------------
// Fast router for large token counts.
//
// The canonical projection above runs on the FP32 pipe (T * E * H multiply-adds); for thousands of
// tokens it costs as much as a third of the expert GEMMs.  Here the projection runs on the tensor
// cores first (launch_router_tc: same products, another summation order, so its logits differ from
// the canonical ones in the last bits), and this kernel turns those APPROXIMATE logits into the
// EXACT routing decision:
//   1. selection values from the approximate logits, and for every expert a bound eps on how far its
//      value can be from the canonical one: |dlogit| <= delta (see below) times the local slope of the
//      score function, plus rounding slack;
//   2. the k largest approximate values; L = the smallest of their lower bounds (value - eps).  At least
//      k experts truly reach L, so an expert whose upper bound (value + eps) is below L cannot be selected;
//   3. CANDIDATES = those k plus every expert whose upper bound reaches L (usually none, sometimes one
//      or two);
//   4. the logits of the candidates are recomputed in the canonical lane-strided order (a few * H
//      multiply-adds per token, router rows from L2);
//   5. their exact scores and selection values follow, and the canonical rule -- (value desc, index
//      asc) -- picks and orders the k among them; routing weights come from the same exact scores.
//      Ids, rank order and weights are therefore bit-identical to the canonical router's, exact ties
//      included.  The same canonical logits check delta: a candidate further than delta / 2 from its
//      approximate logit sends the token to the list.  The largest distance seen, as a fraction of
//      delta, is kept in recheck_total[1] (float bits) for the statistics;
//   6. a token with non-finite logits, more than 32 candidates or a failed check goes on a list; the
//      canonical kernels recompute those completely.
// delta = 2^-13 * max(2, max_e |logit|): both summation orders round at most a few hundred partial
// sums of magnitude <= that maximum (relative 2^-24 each; the tensor cores may truncate, 2^-23), so
// the true distance is orders of magnitude below delta; step 3 verifies that on the selected logits of every
// token.  For the experts that were NOT selected delta is an assumption, not a proof: a projection error
// above delta on one of them alone could hide an expert that belongs in the selection.
// The softmax rule normalises over all experts and is not served by this path.
__device__ __forceinline__ float score_and_slope(const RouterParams& p, float l, float& slope) {
    float cap = 1.0f;
    if (p.softcap > 0.0f) {
        const float th = tanhf(__fdiv_rn(l, p.softcap));
        l = __fmul_rn(th, p.softcap);
        cap = 1.0f;     // d/dl of the soft cap is 1 - th^2 <= 1
    }
    float sc;
    if (p.score_kind == STRATA_MOE_SCORE_SIGMOID) {
        sc = sigmoid_two_branch(l);
        slope = sc * (1.0f - sc);
    } else if (p.score_kind == STRATA_MOE_SCORE_SIGMOID_PLAIN) {
        sc = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf_libm(-l)));
        slope = sc * (1.0f - sc);
    } else {
        sc = sqrtf(l > 20.0f ? l : log1pf_libm(expf_libm(l)));
        const float sg = 1.0f / (1.0f + __expf(-l));
        slope = sc > 0.0f ? sg / (2.0f * sc) : 1.0f;
    }
    slope *= cap;
    return sc;
}

constexpr int kFastWarps = 4;

// 16-byte asynchronous copies global -> shared (cp.async): the data of a whole batch is in flight without occupying
// registers, and the wait is an instruction of its own, so the instruction scheduler cannot shorten the batch to save
// registers (with plain loads it placed each multiply-add right behind its own load and the in-order warp then
// waited out one memory round trip per vector instead of one per batch).
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// eight products of one 16-byte weight load with the matching activations, each added to its own chain
__device__ __forceinline__ void chain_fma8(float (&c)[8], const uint4& xv, const uint4& wv) {
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        c[2 * i] = __fmaf_rn(__uint_as_float(xw[i] << 16), __uint_as_float(ww[i] << 16), c[2 * i]);
        c[2 * i + 1] = __fmaf_rn(__uint_as_float(xw[i] & 0xFFFF0000u), __uint_as_float(ww[i] & 0xFFFF0000u), c[2 * i + 1]);
    }
}

constexpr uint32_t kMaxCand = 32;     // candidates per token: one lane each
constexpr uint32_t kFastStageFloats = (512u + 64u) * 4u;   // per warp: two weight buffers of 256 vectors, two activation buffers of 32

__global__ void __launch_bounds__(kFastWarps * 32) route_fast_kernel(
    RouterParams p, const float* __restrict__ logits, const float* __restrict__ bias,
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg, uint32_t T, uint32_t H,
    uint32_t* __restrict__ ids, float* __restrict__ weights, uint32_t* __restrict__ list,
    uint32_t* __restrict__ count, unsigned long long* __restrict__ recheck_total, uint32_t* status) {
    extern __shared__ __align__(16) float fsm[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t E = p.experts, k = p.top_k;
    // per warp: staging buffers for the canonical dot products (2 x 256 + 2 x 32 vectors of 16 bytes, first so that they
    // stay 16-byte aligned), then choice, eps [E]; candidate ids, their canonical logits, selected ids and scores [32 each]
    const size_t per_warp = kFastStageFloats + 2u * (size_t)E + 4u * kMaxCand;
    uint4* wbuf = reinterpret_cast<uint4*>(fsm + warp * per_warp);
    uint4* xbuf = wbuf + 512;
    float* choice = fsm + warp * per_warp + kFastStageFloats;
    float* eps = choice + E;
    uint32_t* cand = reinterpret_cast<uint32_t*>(eps + E);
    float* canon = reinterpret_cast<float*>(cand + kMaxCand);
    uint32_t* sel_id = reinterpret_cast<uint32_t*>(canon + kMaxCand);
    float* sel_sc = reinterpret_cast<float*>(sel_id + kMaxCand);
    float worst = 0.0f;        // largest |canonical - approximate| / delta this warp has seen
    for (uint32_t tok = blockIdx.x * kFastWarps + warp; tok < T; tok += gridDim.x * kFastWarps) {
        const float* lg = logits + (size_t)tok * E;
        bool bad = false;
        float mx = 0.0f;
        for (uint32_t e = lane; e < E; e += 32u) {
            const float l = lg[e];
            bad |= !isfinite(l);
            mx = fmaxf(mx, fabsf(l));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
        const float delta = 1.220703125e-4f * fmaxf(2.0f, mx);
        for (uint32_t e = lane; e < E; e += 32u) {
            float slope;
            const float sc = score_and_slope(p, lg[e], slope);
            const float b = bias ? bias[e] : 0.0f;
            bad |= !isfinite(b);
            choice[e] = __fadd_rn(sc, b);
            eps[e] = 1.25f * slope * delta + 4.8e-7f * (fabsf(sc) + fabsf(b)) + 1e-30f;
        }
        __syncwarp();
        // step 2: the k largest approximate values; lane r keeps the lower bound of the r-th
        float my_low = INFINITY;
        for (uint32_t r = 0; r < k; ++r) {
            float bv = -INFINITY;
            uint32_t bi = 0xFFFFFFFFu;
            for (uint32_t e = lane; e < E; e += 32u) {
                const float v = choice[e];
                if (v > bv || bi == 0xFFFFFFFFu) { bv = v; bi = e; }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
                const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (bi >= E) { bad = true; bi = 0; }
            if (lane == r) { cand[r] = bi; my_low = bv - eps[bi]; }
            if (lane == 0) choice[bi] = -INFINITY;
            __syncwarp();
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) my_low = fminf(my_low, __shfl_xor_sync(0xFFFFFFFFu, my_low, off));
        // step 3: every other expert whose value could reach the weakest of those lower bounds joins the candidates
        uint32_t n = k;
        for (uint32_t base = 0; base < E; base += 32u) {
            const uint32_t e = base + lane;
            const bool in = e < E && (choice[e] + eps[e] >= my_low);      // the k found above hold -inf
            const uint32_t m = __ballot_sync(0xFFFFFFFFu, in);
            if (in) {
                const uint32_t pos = n + __popc(m & ((1u << lane) - 1u));
                if (pos < kMaxCand) cand[pos] = e;
            }
            n += __popc(m);
        }
        bool safe = !__any_sync(0xFFFFFFFFu, bad) && n <= kMaxCand;
        __syncwarp();
        // step 4: canonical-order logits of the candidates, eight per pass.  The canonical dot product gives lane v the
        // columns v, v + 32, ... (one multiply-add chain per lane, increasing column order) and folds the 32 chains by
        // five shuffle-down rounds.  Here four lanes serve one expert and each owns EIGHT of those chains (columns
        // 8*sub .. 8*sub+7 of every 32): one 16-byte load feeds eight chains, the chains keep their order, and the
        // fold below pairs the same chains in the same rounds, so the sum is bit-identical.
        const uint32_t grp = lane >> 2, sub = lane & 3u, per_lane = H / 32u;
        for (uint32_t r0 = 0; r0 < n && safe; r0 += 8u) {
            const uint32_t r = r0 + grp;
            const uint32_t e = cand[r < n ? r : n - 1u];
            const uint4* wrow = reinterpret_cast<const uint4*>(wg + (size_t)e * H) + sub;
            // the token's row comes through L1: the four lanes of a group read 64 contiguous bytes, all groups the same
            const uint4* xrow = reinterpret_cast<const uint4*>(x + (size_t)tok * H) + sub;
            float c[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            // batches of eight steps through two shared-memory buffers per warp: batch b + 1 is requested before batch
            // b is consumed.  The router rows differ per group (32 x 16 bytes per step); the token row is the same for
            // all groups, so group 0 fetches it (4 x 16 bytes per step).
            auto issue = [&](uint32_t b, uint32_t j) {
                uint4* wb = wbuf + (b & 1u) * 256u;
                uint4* xb = xbuf + (b & 1u) * 32u;
#pragma unroll
                for (uint32_t q = 0; q < 8u; ++q)
                    if (j + q < per_lane) {
                        cp_async16(wb + q * 32u + lane, wrow + (size_t)(j + q) * 4u);
                        if (grp == 0u) cp_async16(xb + q * 4u + sub, xrow + (size_t)(j + q) * 4u);
                    }
                cp_async_commit();
            };
            issue(0u, 0u);
            for (uint32_t b = 0, j = 0; j < per_lane; ++b, j += 8u) {
                if (j + 8u < per_lane) issue(b + 1u, j + 8u);
                else cp_async_commit();             // an empty group keeps the count the wait relies on
                cp_async_wait_all_but_one();
                __syncwarp();
                const uint4* wb = wbuf + (b & 1u) * 256u;
                const uint4* xb = xbuf + (b & 1u) * 32u;
#pragma unroll
                for (uint32_t q = 0; q < 8u; ++q)
                    if (j + q < per_lane) chain_fma8(c, xb[q * 4u + sub], wb[q * 32u + lane]);
                __syncwarp();                       // the buffer is refilled by the issue after next
            }
            // rounds 16 and 8 pair chains held by different lanes of the group, rounds 4, 2, 1 chains of one lane
#pragma unroll
            for (int i = 0; i < 8; ++i) c[i] = __fadd_rn(c[i], __shfl_down_sync(0xFFFFFFFFu, c[i], 2));
#pragma unroll
            for (int i = 0; i < 8; ++i) c[i] = __fadd_rn(c[i], __shfl_down_sync(0xFFFFFFFFu, c[i], 1));
#pragma unroll
            for (int i = 0; i < 4; ++i) c[i] = __fadd_rn(c[i], c[i + 4]);
            c[0] = __fadd_rn(c[0], c[2]);
            c[1] = __fadd_rn(c[1], c[3]);
            c[0] = __fadd_rn(c[0], c[1]);
            if (sub == 0u && r < n) canon[r] = c[0];
        }
        __syncwarp();
        // step 5: exact values of the candidates; the premise of the bounds is checked on each of them
        const bool mine = safe && lane < n;
        uint32_t my_e = 0xFFFFFFFFu;
        float my_sc = 0.0f, my_val = -INFINITY;
        if (mine) {
            my_e = cand[lane];
            const float cl = canon[lane];
            const float d = fabsf(cl - lg[my_e]);
            worst = fmaxf(worst, d / delta);
            if (!(d <= 0.5f * delta)) safe = false;
            float slope_unused;
            my_sc = score_and_slope(p, cl, slope_unused);
            my_val = __fadd_rn(my_sc, bias ? bias[my_e] : 0.0f);
        }
        safe = __all_sync(0xFFFFFFFFu, safe);
        if (!safe) {
            if (lane == 0) {
                list[atomicAdd(count, 1u)] = tok;
                atomicAdd(recheck_total, 1ull);
            }
            __syncwarp();
            continue;
        }
        // step 6: rank by (value desc, index asc) among the candidates -- the canonical selection rule on canonical values
        uint32_t rank = 0;
        for (uint32_t jn = 0; jn < n; ++jn) {
            const float vj = __shfl_sync(0xFFFFFFFFu, my_val, jn);
            const uint32_t ej = __shfl_sync(0xFFFFFFFFu, my_e, jn);
            rank += (vj > my_val || (vj == my_val && ej < my_e)) ? 1u : 0u;
        }
        if (mine && rank < k) { sel_id[rank] = my_e; sel_sc[rank] = my_sc; }
        __syncwarp();
        const float my_w = lane < k ? sel_sc[lane] : 0.0f;
        float sum = p.norm_init;
        for (uint32_t r = 0; r < k; ++r) sum = __fadd_rn(sum, sel_sc[r]);
        float w;
        if (p.normalize) {
            if (!(sum > 0.0f) || !isfinite(sum)) {
                if (lane == 0) atomicOr(status, kStatusBadNormaliser);
                w = 0.0f;
            } else {
                w = __fmul_rn(__fdiv_rn(my_w, sum), p.weight_scale);
            }
        } else {
            w = __fmul_rn(my_w, p.weight_scale);
        }
        if (lane < k) {
            ids[(size_t)tok * k + lane] = sel_id[lane];
            weights[(size_t)tok * k + lane] = w;
        }
        __syncwarp();
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) worst = fmaxf(worst, __shfl_xor_sync(0xFFFFFFFFu, worst, off));
    // non-negative floats order like their bit patterns
    if (lane == 0 && worst > 0.0f) atomicMax(reinterpret_cast<unsigned int*>(recheck_total + 1), __float_as_uint(worst));
}

// ---------------------------------------------------------------------------------------
// Canonical logits for a handful of tokens (decode batches), latency-oriented.
//
// The staged kernel above walks a row in 256-column chunks with two block barriers per chunk; for eight tokens that
// chain of load -> barrier -> arithmetic -> barrier takes 25 us at H = 4096 although the router is only 2 MB.  Here a
// CTA owns eight expert rows and fetches them WHOLE into shared memory with bulk copies (four column quarters per row,
// each quarter completing on its own mbarrier, all issued up front), and warp w computes token w against the eight
// rows with the four-lanes-per-expert chain mapping of route_fast_kernel: bit-identical sums, no block barrier, and
// the arithmetic on a quarter starts as soon as that quarter has landed.
constexpr uint32_t kSmallRows = 8;        // expert rows per CTA
constexpr uint32_t kSmallMaxTokens = 16;  // one warp per token
constexpr uint32_t kSmallPad = 64;        // bytes added to the row pitch: two neighbouring rows fill one 128-byte wavefront

__global__ void __launch_bounds__(kSmallMaxTokens * 32) router_logits_small_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg, uint32_t T, uint32_t H, uint32_t E,
    float* __restrict__ logits, uint32_t* status, uint32_t tokens_per_cta) {
    extern __shared__ __align__(128) uint8_t small_smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(small_smem);     // [4]
    uint8_t* rows = small_smem + 128;
    const uint32_t pitch = H * 2u + kSmallPad;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t e0 = blockIdx.x * kSmallRows;
    const uint32_t nrows = min(kSmallRows, E - e0);
    const uint32_t per_lane = H / 32u;                            // 64-byte steps of a row
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        for (int q = 0; q < 4; ++q) ring::mbar_init(&bars[q], 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) {
        if (lane == 0)
            for (uint32_t q = 0; q < 4u; ++q) {
                const uint32_t j0 = per_lane * q / 4u, j1 = per_lane * (q + 1u) / 4u;
                ring::mbar_arrive_expect_tx(&bars[q], nrows * (j1 - j0) * 64u);
            }
        __syncwarp();
        if (lane < nrows)
            for (uint32_t q = 0; q < 4u; ++q) {
                const uint32_t j0 = per_lane * q / 4u, j1 = per_lane * (q + 1u) / 4u;
                if (j1 > j0)
                    ring::bulk_g2s(rows + (size_t)lane * pitch + j0 * 64u,
                                   reinterpret_cast<const uint8_t*>(wg + (size_t)(e0 + lane) * H) + j0 * 64u,
                                   (j1 - j0) * 64u, &bars[q]);
            }
    }
    bool ok = true;
    const uint32_t tok = blockIdx.y * tokens_per_cta + warp;
    if (warp < tokens_per_cta && tok < T) {
        // the whole token row is requested into L2 now: the register batches below then never wait on HBM (every CTA
        // reads the same T rows; without this each batch of four lines was a fresh miss for all CTAs at once)
        if (lane == 0)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(x + (size_t)tok * H), "r"(H * 2u) : "memory");
        const uint32_t grp = lane >> 2, sub = lane & 3u;
        const uint32_t row = grp < nrows ? grp : nrows - 1u;
        const uint32_t wrow = ring::smem_addr(rows + (size_t)row * pitch) + sub * 16u;
        const uint4* xrow = reinterpret_cast<const uint4*>(x + (size_t)tok * H) + sub;
        float c[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        // the token's row comes from global memory in batches of eight steps through two small shared-memory buffers
        // (cp.async; group 0 fetches, the row is the same for all groups): batch b + 1 is in flight while b is consumed
        uint4* xbuf = reinterpret_cast<uint4*>(rows + (size_t)kSmallRows * pitch) + warp * 64u;
        auto issue = [&](uint32_t b, uint32_t j) {
            if (grp == 0u) {
#pragma unroll
                for (uint32_t i = 0; i < 8u; ++i)
                    if (j + i < per_lane) cp_async16(xbuf + (b & 1u) * 32u + i * 4u + sub, xrow + (size_t)(j + i) * 4u);
            }
            cp_async_commit();
        };
        issue(0u, 0u);
        uint32_t q = 0, jq = per_lane / 4u;          // quarter being consumed and its end step
        ok = __all_sync(0xFFFFFFFFu, ring::mbar_wait_poll(&bars[0], 0u, &abort_flag));
        for (uint32_t b = 0, j = 0; j < per_lane && ok; ++b, j += 8u) {
            if (j + 8u < per_lane) issue(b + 1u, j + 8u);
            else cp_async_commit();
            const uint32_t je = min(j + 8u, per_lane);
            while (ok && q < 3u && je > jq) {      // the batch reaches into the next quarter of the router rows
                ++q;
                jq = per_lane * (q + 1u) / 4u;
                ok = __all_sync(0xFFFFFFFFu, ring::mbar_wait_poll(&bars[q], 0u, &abort_flag));
            }
            if (!ok) break;
            cp_async_wait_all_but_one();
            __syncwarp();
            const uint4* xb = xbuf + (b & 1u) * 32u;
#pragma unroll
            for (uint32_t i = 0; i < 8u; ++i)
                if (j + i < je) chain_fma8(c, xb[i * 4u + sub], ring::lds128(wrow + (j + i) * 64u));
            __syncwarp();
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (ok) {
#pragma unroll
            for (int i = 0; i < 8; ++i) c[i] = __fadd_rn(c[i], __shfl_down_sync(0xFFFFFFFFu, c[i], 2));
#pragma unroll
            for (int i = 0; i < 8; ++i) c[i] = __fadd_rn(c[i], __shfl_down_sync(0xFFFFFFFFu, c[i], 1));
#pragma unroll
            for (int i = 0; i < 4; ++i) c[i] = __fadd_rn(c[i], c[i + 4]);
            c[0] = __fadd_rn(c[0], c[2]);
            c[1] = __fadd_rn(c[1], c[3]);
            c[0] = __fadd_rn(c[0], c[1]);
            if (sub == 0u && grp < nrows) logits[(size_t)tok * E + e0 + grp] = c[0];
        }
    }
    if (!ok && lane == 0) { abort_flag = 1; atomicOr(status, kStatusWaitTimeout); }
    // the copies target this CTA's shared memory: none may be in flight when the CTA retires
    __syncthreads();
    if (threadIdx.x == 0)
        for (uint32_t q = 0; q < 4u; ++q)
            for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                if (ring::mbar_test(&bars[q], 0u)) break;
}

bool launch_router_logits_small(const __nv_bfloat16* x, const __nv_bfloat16* wg, uint32_t T, uint32_t H, uint32_t E,
                                float* logits, uint32_t* status, cudaStream_t s) {
    if (T == 0 || T > kSmallMaxTokens || H % 128u || status == nullptr) return false;
    if ((((uintptr_t)x | (uintptr_t)wg) & 15u) != 0) return false;
    const size_t smem = 128u + (size_t)kSmallRows * (H * 2u + kSmallPad) + (size_t)kSmallMaxTokens * 64u * 16u;
    if (smem > 200u * 1024u) return false;
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return false;
    if (!attr[dev]) {
        if (cudaFuncSetAttribute(router_logits_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
            cudaSuccess)
            return false;
        attr[dev] = true;
    }
    // two tokens per CTA while that keeps the grid within two CTAs per SM: more SMs stream and decode (a CTA whose
    // rows another CTA already fetched reads them from L2)
    const uint32_t row_groups = (E + kSmallRows - 1) / kSmallRows;
    uint32_t tpc = 2u;
    while (tpc < T && row_groups * ((T + tpc - 1u) / tpc) > 2u * (uint32_t)kNumSMs) tpc *= 2u;
    if (tpc > T) tpc = T;
    const uint32_t warps = tpc < 4u ? 4u : tpc;      // warp 0 also issues the copies
    dim3 grid(row_groups, (T + tpc - 1u) / tpc);
    router_logits_small_kernel<<<grid, warps * 32u, smem, s>>>(x, wg, T, H, E, logits, status, tpc);
    ++g_kernel_launches;
    return true;
}

bool route_fast_supported(const RouterParams& p, uint32_t H) {
    if (p.score_kind == STRATA_MOE_SCORE_SOFTMAX) return false;
    if (p.experts % 128u || H % 64u) return false;
    return p.top_k <= kMaxCand &&
           (size_t)kFastWarps * ((kFastStageFloats + 2u * (size_t)p.experts + 4u * kMaxCand) * sizeof(float)) <= 200u * 1024u;
}

// logits: approximate [T, E] (tensor-core projection); list [T], count, recheck_total: device scratch.
// On return (stream order) ids / weights hold the canonical routing of every token and the canonical
// logits of the rechecked tokens have replaced their approximate rows.
void launch_route_fast(const RouterParams& p, float* logits, const float* bias, const __nv_bfloat16* x,
                       const __nv_bfloat16* wg, uint32_t T, uint32_t H, uint32_t* ids, float* weights,
                       uint32_t* list, uint32_t* count, unsigned long long* recheck_total, uint32_t* status,
                       cudaStream_t s) {
    if (T == 0) return;
    const size_t smem = (size_t)kFastWarps * ((kFastStageFloats + 2u * (size_t)p.experts + 4u * kMaxCand) * sizeof(float));
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr[dev]) {
        cudaFuncSetAttribute(route_fast_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr[dev] = true;
    }
    cudaMemsetAsync(count, 0, sizeof(uint32_t), s);
    uint32_t grid = (T + kFastWarps - 1) / kFastWarps;
    if (grid > (uint32_t)kNumSMs * 8u) grid = (uint32_t)kNumSMs * 8u;
    route_fast_kernel<<<grid, kFastWarps * 32, smem, s>>>(p, logits, bias, x, wg, T, H, ids, weights, list, count,
                                                          recheck_total, status);
    // the tokens on the list, completely in the canonical order (few: the grids stride over the list)
    const uint32_t E = p.experts;
    dim3 g2((E + 7) / 8, 32);
    router_logits_kernel<8, 16, true><<<g2, 256, 0, s>>>(x, wg, T, H, E, logits, list, count);
    const size_t smem_r = (size_t)kRouteWarps * 2u * E * sizeof(float);
    route_kernel<<<64, kRouteWarps * 32, smem_r, s>>>(p, logits, bias, T, ids, weights, status, nullptr, list, count);
    g_kernel_launches += 3;
}

// ---------------------------------------------------------------------------------------
// Decode front end in ONE launch: scores / top-k / weights, grouping and the gather + f16 conversion of the routed
// rows, for at most 16 tokens.  As separate kernels (route, group, convert) these cost 14 + 12 + 8 us for 8 tokens,
// mostly launch latency and single-CTA barrier chains.  One CTA of 16 warps: warp w routes token w; the pairs
// (<= 512) are counted per expert in shared memory, offsets come from a two-level warp scan (two experts per thread,
// so up to 1024 experts), every pair finds its stable position by counting the earlier pairs of its expert; then the
// warps convert the routed rows.  Outputs are those of route_kernel, the grouping kernels and rows_to_f16_kernel.
constexpr uint32_t kFrontWarps = 16, kFrontMaxPairs = 512, kFrontMaxExperts = 1024;

__global__ void __launch_bounds__(kFrontWarps * 32) front_small_kernel(
    RouterParams p, const float* __restrict__ logits, const float* __restrict__ bias, uint32_t T,
    uint32_t* __restrict__ ids, float* __restrict__ weights, uint32_t* __restrict__ counts,
    uint32_t* __restrict__ offsets, uint32_t* __restrict__ perm, uint32_t* __restrict__ inv,
    uint32_t* __restrict__ active_list, uint32_t* __restrict__ n_active, const __nv_bfloat16* __restrict__ x, uint32_t H,
    __half* __restrict__ xg, float* __restrict__ x_rowscale, uint32_t* status) {
    extern __shared__ float fsm2[];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t E = p.experts, k = p.top_k, P = T * k;
    uint32_t* cnt = reinterpret_cast<uint32_t*>(fsm2 + (size_t)kFrontWarps * 2u * E);   // [E]
    uint32_t* off = cnt + E;                                                            // [E]
    uint32_t* ids_s = off + E;                                                          // [P]
    uint32_t* perm_s = ids_s + kFrontMaxPairs;                                          // [P]
    __shared__ uint32_t wtot[kFrontWarps], wact[kFrontWarps], bad_s[kFrontWarps];
    for (uint32_t e = tid; e < E; e += blockDim.x) cnt[e] = 0;
    if (tid < kFrontWarps) bad_s[tid] = 0;
    // scores: the exact exp / log1p replicas are the long part of routing a token, so all 16 warps share them
    // (16 / T warps per token, each a strided subset of the experts); the softmax rule keeps one warp per token
    const bool coop = p.score_kind != STRATA_MOE_SCORE_SOFTMAX;
    const uint32_t nsub = kFrontWarps / T;
    __syncthreads();
    if (coop && warp < T * nsub) {
        const uint32_t tok = warp % T, part = warp / T;
        float* sc = fsm2 + (size_t)tok * 2u * E;
        if (route_scores_part(p, logits + (size_t)tok * E, bias, sc, sc + E, part * 32u + lane, 32u * nsub))
            bad_s[tok] = 1u;
    }
    __syncthreads();
    if (warp < T) {
        float* score = fsm2 + (size_t)warp * 2u * E;
        route_token(p, logits, bias, warp, score, score + E, ids, weights, status, nullptr, coop, bad_s[warp] != 0u);
        if (lane < k) ids_s[warp * k + lane] = ids[(size_t)warp * k + lane];    // this lane's own store
    }
    __syncthreads();
    if (tid < P) atomicAdd(&cnt[ids_s[tid]], 1u);
    __syncthreads();
    // exclusive scans over the experts of (count) and of (count != 0): thread t owns experts 2t and 2t + 1
    const uint32_t ea = 2u * tid, eb = ea + 1u;
    const uint32_t ca = ea < E ? cnt[ea] : 0u, cb = eb < E ? cnt[eb] : 0u;
    uint32_t run = ca + cb, act = (ca != 0u) + (cb != 0u);
    uint32_t inc = run, inca = act;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, inc, o), va = __shfl_up_sync(0xFFFFFFFFu, inca, o);
        if (lane >= (uint32_t)o) { inc += v; inca += va; }
    }
    if (lane == 31u) { wtot[warp] = inc; wact[warp] = inca; }
    __syncthreads();
    uint32_t base = 0, basea = 0;
    for (uint32_t w = 0; w < warp; ++w) { base += wtot[w]; basea += wact[w]; }
    const uint32_t oa = base + inc - run, ra = basea + inca - act;      // exclusive prefixes at expert 2t
    if (ea < E) {
        counts[ea] = ca;
        offsets[ea] = oa;
        off[ea] = oa;
        if (ca) active_list[ra] = ea;
    }
    if (eb < E) {
        counts[eb] = cb;
        offsets[eb] = oa + ca;
        off[eb] = oa + ca;
        if (cb) active_list[ra + (ca != 0u)] = eb;
    }
    if (tid == blockDim.x - 1u) {
        offsets[E] = base + inc;
        *n_active = basea + inca;
    }
    __syncthreads();
    if (tid < P) {
        const uint32_t e = ids_s[tid];
        uint32_t r = 0;
        for (uint32_t j = 0; j < tid; ++j) r += ids_s[j] == e ? 1u : 0u;
        const uint32_t pos = off[e] + r;
        perm[pos] = tid;
        inv[tid] = pos;
        perm_s[pos] = tid;
    }
    __syncthreads();
    if (xg != nullptr)
        for (uint32_t pos = warp; pos < P; pos += kFrontWarps)
            warp_row_to_f16_bf16(x + (size_t)(perm_s[pos] / k) * H, H, xg + (size_t)pos * H, x_rowscale + pos);
}

// false: the shape is outside the kernel's limits and nothing was launched
bool launch_front_small(const RouterParams& p, const float* logits, const float* bias, uint32_t T, uint32_t* ids,
                        float* weights, uint32_t* counts, uint32_t* offsets, uint32_t* perm, uint32_t* inv,
                        uint32_t* active_list, uint32_t* n_active, const __nv_bfloat16* x, uint32_t H, void* xg,
                        float* x_rowscale, uint32_t* status, cudaStream_t s) {
    if (T == 0 || T > kFrontWarps || T * p.top_k > kFrontMaxPairs || p.experts > kFrontMaxExperts || p.top_k > 32u)
        return false;
    if (xg != nullptr && (H % 8u || (((uintptr_t)x | (uintptr_t)xg) & 15u))) return false;
    const size_t smem = ((size_t)kFrontWarps * 2u * p.experts + 2u * p.experts + 2u * kFrontMaxPairs) * sizeof(float);
    if (smem > 200u * 1024u) return false;
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return false;
    if (!attr[dev]) {
        if (cudaFuncSetAttribute(front_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return false;
        attr[dev] = true;
    }
    front_small_kernel<<<1, kFrontWarps * 32, smem, s>>>(p, logits, bias, T, ids, weights, counts, offsets, perm, inv,
                                                         active_list, n_active, x, H, static_cast<__half*>(xg),
                                                         x_rowscale, status);
    ++g_kernel_launches;
    return true;
}

// ---------------------------------------------------------------------------------------
// Inkling's sink router (src/models/inkling/inkling_ops.cpp:184-275), one warp per token.  logits [T, E + S]:
// the routed experts followed by S shared "sink" experts.  Selection: top-k of sigmoid(logit) + bias over the routed
// range, lower index on ties.  Weights: log-sigmoid (min(x, 0) - log1p(exp(-|x|)), src/platform/numerics.cpp:54-59)
// of the RAW logits of the k selected experts and of every sink, softmax over that joint set (maximum subtracted,
// sum in index order), times scale.  expf / log1pf follow the host libm step by step, so the weights are bit-exact.
__global__ void __launch_bounds__(kRouteWarps * 32) route_sink_kernel(
    const float* __restrict__ logits, const float* __restrict__ bias, uint32_t T, uint32_t E, uint32_t S, uint32_t k,
    float scale, uint32_t* __restrict__ ids, float* __restrict__ w_routed, float* __restrict__ w_sinks,
    uint32_t* status) {
    extern __shared__ float smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    float* choice = smem + (size_t)warp * E;
    const uint32_t tok = blockIdx.x * kRouteWarps + warp;
    if (tok >= T) return;
    const float* lg = logits + (size_t)tok * (E + S);
    bool bad = false;
    for (uint32_t e = lane; e < E + S; e += 32u) bad |= !isfinite(lg[e]);
    for (uint32_t e = lane; e < E; e += 32u) {
        const float b = bias[e];
        bad |= !isfinite(b);
        choice[e] = __fadd_rn(sigmoid_two_branch(lg[e]), b);
    }
    __syncwarp();
    uint32_t my_id = 0;
    for (uint32_t r = 0; r < k; ++r) {
        float bv = -INFINITY;
        uint32_t bi = 0xFFFFFFFFu;
        for (uint32_t e = lane; e < E; e += 32u) {
            const float v = choice[e];
            if (v > bv || bi == 0xFFFFFFFFu) { bv = v; bi = e; }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
            const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi >= E) { bad = true; bi = 0; }
        if (lane == r) my_id = bi;
        if (lane == 0) choice[bi] = -INFINITY;
        __syncwarp();
    }
    if (lane >= k && lane < k + S) my_id = E + (lane - k);
    const bool mine = lane < k + S;
    float lp = -INFINITY;
    if (mine) {
        const float v = lg[my_id];
        lp = __fsub_rn(fminf(v, 0.0f), log1pf_libm(expf_libm(-fabsf(v))));
    }
    float mx = lp;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    const float ex = mine ? expf_libm(__fsub_rn(lp, mx)) : 0.0f;
    float total = 0.0f;
    for (uint32_t i = 0; i < k + S; ++i) total = __fadd_rn(total, __shfl_sync(0xFFFFFFFFu, ex, i));
    float w = 0.0f;
    if (!(total > 0.0f) || !isfinite(total)) {
        if (lane == 0) atomicOr(status, kStatusBadNormaliser);
    } else {
        w = __fmul_rn(__fdiv_rn(ex, total), scale);
    }
    if (lane < k) {
        ids[(size_t)tok * k + lane] = my_id;
        w_routed[(size_t)tok * k + lane] = w;
    } else if (mine) {
        w_sinks[(size_t)tok * S + (lane - k)] = w;
    }
    if (__any_sync(0xFFFFFFFFu, bad) && lane == 0) atomicOr(status, kStatusNonFiniteLogit);
}

void launch_route_sink(const float* logits, const float* bias, uint32_t T, uint32_t E, uint32_t S, uint32_t k, float scale,
                       uint32_t* ids, float* w_routed, float* w_sinks, uint32_t* status, cudaStream_t s) {
    if (T == 0) return;
    route_sink_kernel<<<(T + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, (size_t)kRouteWarps * E * sizeof(float), s>>>(
        logits, bias, T, E, S, k, scale, ids, w_routed, w_sinks, status);
    ++g_kernel_launches;
}

void launch_route(const RouterParams& p, const float* logits, const float* bias, uint32_t T,
                  uint32_t* ids, float* weights, uint32_t* status, cudaStream_t s, const uint32_t* forced_ids) {
    if (T == 0) return;
    const size_t smem = (size_t)kRouteWarps * 2u * p.experts * sizeof(float);
    route_kernel<<<(T + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, smem, s>>>(
        p, logits, bias, T, ids, weights, status, forced_ids, nullptr, nullptr);
    ++g_kernel_launches;
}

}  // namespace smoe
