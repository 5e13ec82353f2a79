// Expert-parallel exchange over peer memory (NVLink / NVSwitch), fused with the work on either
// side of it.  A token's row crosses the link ONCE per owning GPU, however many of that GPU's
// experts the token selected, and ONE row comes back per (token, owning GPU): the owner forms the
// weighted sum of its experts' outputs for the token before anything leaves.  The dispatch kernel
// gathers a token's row and stores it straight into the owner's window together with the few words
// that tell the owner which of its grouped rows use it; the combine kernel loads the owners'
// partial sums straight from their windows.  No staging copy, no host round trip, no library
// collective on the data path.
//
// The reference places experts on several GPUs of one process and moves the activations through
// host memory (src/models/glm52/glm_runtime.cpp:650-652, 1561-1576); this file replaces that
// transport for one-process-per-GPU expert parallelism.
//
// Every rank owns a "window" of device memory with the same layout, mapped into every peer:
//
//   flags   u32 [3][world]       flags[k][s] = last step for which rank s finished phase k
//                                (0 counts published, 1 rows stored, 2 partial sums ready)
//   counts  u32 [2][world][E]    counts[p][s][e] = pairs rank s holds for global expert e
//   visits  u32 [2][16][16]      visits[p][s][o] = token rows rank s sends to owner o
//   rows    bf16 [2][cap][H]     token rows received, slot = (source rank, source token order)
//   y       f16 [2][cap][H]      per slot: sum over this owner's experts of weight x expert output,
//                                scaled by a power of two
//   yscale  f32 [2][cap]         the factor that undoes a slot's scale
//   src_of  u32 [2][cap]         per grouped row (local expert, source rank, source scan order): its slot
//   vis_pos u32 [2][cap][k]      per slot: the grouped rows of the token's experts here, selection order, packed
//                                to the front, ~0 = none
//   vis_w   f32 [2][cap][k]      per slot: their routing weights
//
// [2] is the step parity: a buffer written in step n is next written in step n + 2, and a rank
// can only reach step n + 2 after every peer finished step n (it waited for their step n + 1
// flags, which are stored after their step n work in stream order).
//
// Flags only ever grow (the step number), are written with release stores at system scope after
// a system fence, and are polled with acquire loads.  Every wait is bounded by wall time; a wait
// that runs out sets the status word and an abort word, and the remaining kernels of the step
// skip their peer accesses.
#include <cuda_fp16.h>

#include "common.cuh"

namespace smoe {

namespace {

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Poll *flag until it reaches `step` or `limit_ns` of wall time passes.  True on success.
__device__ bool wait_flag(const uint32_t* flag, uint32_t step, uint64_t limit_ns) {
    // steps are compared modulo 2^32 so that the counter may wrap
    if ((int32_t)(ld_acquire_sys(flag) - step) >= 0) return true;
    const uint64_t t0 = now_ns();
    for (;;) {
        __nanosleep(200);
        if ((int32_t)(ld_acquire_sys(flag) - step) >= 0) return true;
        if (now_ns() - t0 > limit_ns) return false;
    }
}

}  // namespace

// ------------------------------------------------------------------------------ visits
// CTA o lists, in token order, the tokens that selected at least one expert of owner o:
// vis_idx[o][t] = index of token t in that list (~0 when it selected none), nvis[o] = its length.
__global__ void __launch_bounds__(1024) ep_visits_kernel(EpWindows w, EpPlan pl, const uint32_t* __restrict__ ids,
                                                         uint32_t T) {
    __shared__ uint32_t warp_base[33];
    const uint32_t o = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t B = w.E / w.world;
    uint32_t base = 0;
    for (uint32_t t0 = 0; t0 < T; t0 += 1024u) {
        const uint32_t t = t0 + tid;
        bool hit = false;
        if (t < T)
            for (uint32_t j = 0; j < w.k; ++j) {
                const uint32_t e = ids[(size_t)t * w.k + j];
                hit |= e < w.E && e / B == o;
            }
        const uint32_t mask = __ballot_sync(0xFFFFFFFFu, hit);
        if (lane == 0) warp_base[warp] = __popc(mask);
        __syncthreads();
        if (warp == 0) {
            const uint32_t c = warp_base[lane];
            uint32_t incl = c;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, off);
                if ((int)lane >= off) incl += v;
            }
            warp_base[lane] = incl - c;
            if (lane == 31) warp_base[32] = incl;
        }
        __syncthreads();
        if (t < T)
            pl.vis_idx[(size_t)o * pl.stride + t] =
                hit ? base + warp_base[warp] + __popc(mask & ((1u << lane) - 1u)) : 0xFFFFFFFFu;
        base += warp_base[32];
        __syncthreads();
    }
    if (tid == 0) pl.nvis[o] = base;
}

// ------------------------------------------------------------------------------ publish
// Block b stores this rank's per-expert pair counts and per-owner row counts into rank b's window
// and raises flag 0 there.
__global__ void __launch_bounds__(256) ep_publish_kernel(EpWindows w, EpPlan pl, const uint32_t* __restrict__ counts) {
    const uint32_t dst = blockIdx.x;
    uint32_t* c = w.counts(dst, w.step & 1u, w.rank);
    for (uint32_t e = threadIdx.x; e < w.E; e += blockDim.x) c[e] = counts[e];
    if (threadIdx.x < w.world) w.visits(dst, w.step & 1u, w.rank)[threadIdx.x] = pl.nvis[threadIdx.x];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(w.flag(dst, 0, w.rank), w.step);
}

// ------------------------------------------------------------------------------ plan
// One CTA.  Waits for every rank's counts, then derives from the full [world][E] matrix
//   dst_row[e]   first row, in the owner's grouped order, of this rank's pairs for global expert e
//   loffsets[j]  row range of this rank's local expert j over all sources (j = 0..B)
// and from the [world][world] row counts
//   tok_base[o]  first slot, in owner o's window, of this rank's token rows
//   vis_total    token rows this rank receives as an owner.
// Any rank can evaluate every owner's totals, so an overflow of `cap` is seen by all ranks alike.
__global__ void __launch_bounds__(1024) ep_plan_kernel(EpWindows w, EpPlan pl, uint32_t* __restrict__ status) {
    __shared__ uint32_t scan[1024];
    __shared__ uint32_t bad;
    const uint32_t tid = threadIdx.x;
    if (tid == 0) bad = 0;
    __syncthreads();
    if (tid < w.world && !wait_flag(w.flag(w.rank, 0, tid), w.step, w.wait_ns)) atomicOr(&bad, 1u);
    __syncthreads();
    uint32_t tot = 0, before = 0;
    if (!bad && tid < w.E) {
        for (uint32_t s = 0; s < w.world; ++s) {
            const uint32_t c = w.counts(w.rank, w.step & 1u, s)[tid];
            if (c > w.cap) atomicOr(&bad, 2u);
            if (s < w.rank) before += c;
            tot += c;
        }
    }
    scan[tid] = tot;
    __syncthreads();
    for (uint32_t off = 1; off < 1024u; off <<= 1) {
        const uint32_t v = tid >= off ? scan[tid - off] : 0u;
        __syncthreads();
        scan[tid] += v;
        __syncthreads();
    }
    const uint32_t B = w.E / w.world;
    if (tid < w.E) {
        const uint32_t owner = tid / B;
        const uint32_t block_base = owner ? scan[owner * B - 1] : 0u;
        const uint32_t excl = scan[tid] - tot - block_base;      // rows of the owner's earlier experts
        if (excl + tot > w.cap) atomicOr(&bad, 2u);              // the owner's window would overflow
        pl.dst_row[tid] = excl + before;
        if (owner == w.rank) {
            pl.loffsets[tid - owner * B] = excl;
            if (tid - owner * B == B - 1) pl.loffsets[B] = excl + tot;
        }
    }
    if (!bad && tid < w.world) {   // tid plays the owner
        uint32_t vt = 0, vb = 0;
        for (uint32_t s = 0; s < w.world; ++s) {
            const uint32_t c = w.visits(w.rank, w.step & 1u, s)[tid];
            if (c > w.cap) atomicOr(&bad, 2u);
            if (s < w.rank) vb += c;
            vt += c;
        }
        if (vt > w.cap) atomicOr(&bad, 2u);
        pl.tok_base[tid] = vb;
        if (tid == w.rank) *pl.vis_total = vt;
    }
    __syncthreads();
    if (bad) {
        // nothing is sent and nothing is computed this step
        for (uint32_t i = tid; i <= B; i += blockDim.x) pl.loffsets[i] = 0;
        for (uint32_t i = tid; i < w.E; i += blockDim.x) pl.dst_row[i] = 0;
        if (tid < w.world) pl.tok_base[tid] = 0;
        if (tid == 0) {
            *pl.vis_total = 0;
            *pl.abort_word = 1;
            atomicOr(status, (bad & 1u) ? kStatusWaitTimeout : kStatusBadGroup);
        }
    } else if (tid == 0) {
        *pl.abort_word = 0;
    }
}

// ------------------------------------------------------------------------------ dispatch
// One warp per (token, owner) that has a row to send: copy the token's BF16 row into the owner's
// window once, and beside it the grouped rows of the token's experts there with their routing
// weights; every such grouped row learns its slot.  The last CTA to finish raises flag 1 on every rank.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpWindows w, EpPlan pl, const __nv_bfloat16* __restrict__ x,
                                                          const uint32_t* __restrict__ ids,
                                                          const uint32_t* __restrict__ inv,
                                                          const uint32_t* __restrict__ offsets,
                                                          const float* __restrict__ weights, uint32_t T) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t B = w.E / w.world, par = w.step & 1u;
    const uint32_t vecs = w.H / 8u;   // 16-byte vectors per row
    if (*pl.abort_word == 0) {
        const uint32_t tasks = T * w.world;
        for (uint32_t task = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; task < tasks; task += warps) {
            const uint32_t t = task / w.world, o = task - t * w.world;
            const uint32_t vi = pl.vis_idx[(size_t)o * pl.stride + t];
            if (vi == 0xFFFFFFFFu) continue;
            const uint32_t slot = pl.tok_base[o] + vi;
            if (slot >= w.cap) continue;   // cannot happen after a clean plan; never store outside the window
            // the token's experts on this owner, selection order kept, listed first: the owner's loops stop at the
            // first empty entry
            uint32_t pos = 0xFFFFFFFFu;
            float wt = 0.0f;
            if (lane < w.k) {
                const uint32_t pair = t * w.k + lane;
                const uint32_t e = ids[pair], p = inv[pair];
                wt = weights[pair];
                if (e < w.E && e / B == o && p != 0xFFFFFFFFu) {
                    const uint32_t row = pl.dst_row[e] + (p - offsets[e]);
                    if (row < w.cap) {
                        pos = row;
                        w.src_of(o, par)[row] = slot;
                    }
                }
            }
            const uint32_t valid = __ballot_sync(0xFFFFFFFFu, pos != 0xFFFFFFFFu);
            if (lane < w.k) {
                const uint32_t below = (1u << lane) - 1u;
                const uint32_t idx = pos != 0xFFFFFFFFu ? __popc(valid & below)
                                                        : __popc(valid) + __popc(~valid & below);
                w.vis_pos(o, par)[(size_t)slot * w.k + idx] = pos;
                w.vis_w(o, par)[(size_t)slot * w.k + idx] = wt;
            }
            const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * w.H);
            uint4* dst = reinterpret_cast<uint4*>(w.rows(o, par) + (size_t)slot * w.H);
            for (uint32_t v = lane; v < vecs; v += 32u) dst[v] = __ldg(src + v);
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t prev = atomicAdd(pl.done, 1u);
        if (prev == gridDim.x - 1u) {
            *pl.done = 0;
            __threadfence_system();
            for (uint32_t d = 0; d < w.world; ++d) st_release_sys(w.flag(d, 1, w.rank), w.step);
        }
    }
}

// ------------------------------------------------------------------------------ wait / signal
// One warp: lane s waits until rank s raised flag `kind` for this step.
__global__ void ep_wait_kernel(EpWindows w, uint32_t kind, uint32_t* __restrict__ abort_word,
                               uint32_t* __restrict__ status) {
    const uint32_t s = threadIdx.x;
    if (s < w.world && !wait_flag(w.flag(w.rank, kind, s), w.step, w.wait_ns)) {
        *abort_word = 1;
        atomicOr(status, kStatusWaitTimeout);
    }
}

// One warp: lane d tells rank d that this rank's partial sums of the step are in its window.
__global__ void ep_signal_kernel(EpWindows w, uint32_t kind) {
    const uint32_t d = threadIdx.x;
    __threadfence_system();
    if (d < w.world) st_release_sys(w.flag(d, kind, w.rank), w.step);
}

// ------------------------------------------------------------------------------ owner-side partial sums
// One CTA per received token row: sum over the token's experts on this rank, selection order, of
// weight x expert output (separate multiply and add, like the single-GPU combine), stored into this
// rank's own window as f16 with an exact power-of-two row factor.  Everything read here is local.
template <bool Y_HALF>
__device__ __forceinline__ void partial_vec(const void* __restrict__ y, const uint32_t* pos, const float* wgt,
                                            uint32_t k, uint32_t H, uint32_t c, float (&o)[8]) {
#pragma unroll
    for (int q = 0; q < 8; ++q) o[q] = 0.0f;
    for (uint32_t r0 = 0; r0 < k; r0 += 4u) {
        float f[4][8];
#pragma unroll
        for (uint32_t q = 0; q < 4u; ++q) {
            const bool on = r0 + q < k && pos[r0 + q] != 0xFFFFFFFFu;
            if (Y_HALF) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (on) v = *(reinterpret_cast<const uint4*>(static_cast<const __half*>(y) + (size_t)pos[r0 + q] * H) + c);
                const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const float2 g = __half22float2(*reinterpret_cast<const __half2*>(&wv[h]));
                    f[q][2 * h] = g.x;
                    f[q][2 * h + 1] = g.y;
                }
            } else {
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
                if (on) {
                    const float4* yp = reinterpret_cast<const float4*>(static_cast<const float*>(y) + (size_t)pos[r0 + q] * H) + c * 2u;
                    a = yp[0];
                    b = yp[1];
                }
                f[q][0] = a.x; f[q][1] = a.y; f[q][2] = a.z; f[q][3] = a.w;
                f[q][4] = b.x; f[q][5] = b.y; f[q][6] = b.z; f[q][7] = b.w;
            }
        }
#pragma unroll
        for (uint32_t q = 0; q < 4u; ++q) {
            if (r0 + q >= k || pos[r0 + q] == 0xFFFFFFFFu) continue;
            const float g = wgt[r0 + q];
#pragma unroll
            for (int h = 0; h < 8; ++h) o[h] = __fadd_rn(o[h], __fmul_rn(f[q][h], g));
        }
    }
}

template <bool Y_HALF>
__global__ void __launch_bounds__(256) ep_partial_kernel(EpWindows w, EpPlan pl, const void* __restrict__ y,
                                                         uint32_t* __restrict__ status) {
    constexpr uint32_t kKeep = 4;   // vectors per thread kept in registers between the two passes (H <= 8192)
    __shared__ uint32_t pos[32];
    __shared__ float wgt[32];
    __shared__ float red[8];
    if (*pl.abort_word) return;
    const uint32_t tid = threadIdx.x, par = w.step & 1u;
    const uint32_t n = min(*pl.vis_total, w.cap);
    const uint32_t per_row = w.H / 8u;
    bool bad = false;
    for (uint32_t slot = blockIdx.x; slot < n; slot += gridDim.x) {
        __syncthreads();
        if (tid < w.k) {
            const uint32_t p = w.vis_pos(w.rank, par)[(size_t)slot * w.k + tid];
            pos[tid] = p < w.cap ? p : 0xFFFFFFFFu;
            wgt[tid] = w.vis_w(w.rank, par)[(size_t)slot * w.k + tid];
        }
        __syncthreads();
        float keep[kKeep][8];
        float mx = 0.0f;
#pragma unroll
        for (uint32_t i = 0; i < kKeep; ++i) {
            const uint32_t c = tid + i * 256u;
            if (c < per_row) {
                partial_vec<Y_HALF>(y, pos, wgt, w.k, w.H, c, keep[i]);
#pragma unroll
                for (int q = 0; q < 8; ++q) mx = fmaxf(mx, fabsf(keep[i][q]));
            }
        }
        for (uint32_t c = tid + kKeep * 256u; c < per_row; c += 256u) {
            float o[8];
            partial_vec<Y_HALF>(y, pos, wgt, w.k, w.H, c, o);
#pragma unroll
            for (int q = 0; q < 8; ++q) mx = fmaxf(mx, fabsf(o[q]));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
        if ((tid & 31u) == 0) red[tid >> 5] = mx;
        __syncthreads();
        mx = red[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
        if (!(mx <= 3.0e38f)) bad = true;   // also catches NaN through the comparison below
        // scale = 2^(14 - floor(log2 mx)): the row maximum lands in [2^14, 2^15); exact
        int ex = 0;
        if (mx > 0.0f && mx < 3.0e38f) ex = 14 - (int)((__float_as_uint(mx) >> 23) & 0xFFu) + 127;
        ex = max(-100, min(100, ex));
        const float sc = __uint_as_float((uint32_t)(ex + 127) << 23);
        if (tid == 0) w.yscale(w.rank, par)[slot] = __uint_as_float((uint32_t)(127 - ex) << 23);
        unsigned short* dst = w.y(w.rank, par) + (size_t)slot * w.H;
        auto store = [&](uint32_t c, const float (&o)[8]) {
            uint32_t pk[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const __half2 v = __floats2half2_rn(o[2 * h] * sc, o[2 * h + 1] * sc);
                pk[h] = *reinterpret_cast<const uint32_t*>(&v);
                bad |= !(fabsf(o[2 * h]) <= 3.0e38f) || !(fabsf(o[2 * h + 1]) <= 3.0e38f);
            }
            *(reinterpret_cast<uint4*>(dst) + c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        };
#pragma unroll
        for (uint32_t i = 0; i < kKeep; ++i) {
            const uint32_t c = tid + i * 256u;
            if (c < per_row) store(c, keep[i]);
        }
        for (uint32_t c = tid + kKeep * 256u; c < per_row; c += 256u) {
            float o[8];
            partial_vec<Y_HALF>(y, pos, wgt, w.k, w.H, c, o);
            store(c, o);
        }
    }
    if (bad) atomicOr(status, kStatusNonFiniteOutput);
}

// The same sums when the experts left f16 rows (the tensor-core path, many rows): one pass, the
// result stored as plain f16 with a unit row factor -- the addends are f16 values already and the
// weights of a token sum to about one, so the sum needs no other range than they do (it is clamped
// to the largest finite f16 like the rows themselves).  A flat loop over (slot, eight columns): no
// barrier, and neighbouring threads read neighbouring stretches of the same rows.
__global__ void __launch_bounds__(256) ep_partial_half_kernel(EpWindows w, EpPlan pl, const __half* __restrict__ y,
                                                              uint32_t* __restrict__ status) {
    if (*pl.abort_word) return;
    const uint32_t par = w.step & 1u, k = w.k;
    const uint32_t n = min(*pl.vis_total, w.cap);
    const uint32_t per_row = w.H / 8u;
    // a thread forms two stretches of a slot's row (c and c + half) from the same table entries: over many GPUs a
    // slot has only one or two experts here, and one 16-byte load per table look-up would leave the thread waiting
    const uint32_t half = (per_row + 1u) / 2u;
    const uint32_t* __restrict__ vpos = w.vis_pos(w.rank, par);
    const float* __restrict__ vw = w.vis_w(w.rank, par);
    uint4* __restrict__ dst = reinterpret_cast<uint4*>(w.y(w.rank, par));
    bool bad = false;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)n * half;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t slot = (uint32_t)(i / half), c0 = (uint32_t)(i % half), c1 = c0 + half;
        const bool two = c1 < per_row;
        if (c0 == 0) w.yscale(w.rank, par)[slot] = 1.0f;
        float o[2][8];
#pragma unroll
        for (int v = 0; v < 2; ++v)
#pragma unroll
            for (int q = 0; q < 8; ++q) o[v][q] = 0.0f;
        for (uint32_t r0 = 0; r0 < k; r0 += 4u) {
            uint32_t pos[4];
            float g[4];
            uint4 raw[4][2];
#pragma unroll
            for (uint32_t q = 0; q < 4u; ++q) {
                const bool in = r0 + q < k;
                const uint32_t p = in ? vpos[(size_t)slot * k + r0 + q] : 0xFFFFFFFFu;
                pos[q] = p < w.cap ? p : 0xFFFFFFFFu;
                g[q] = in ? vw[(size_t)slot * k + r0 + q] : 0.0f;
            }
            if (pos[0] == 0xFFFFFFFFu) break;   // the list is packed: nothing follows an empty entry
#pragma unroll
            for (uint32_t q = 0; q < 4u; ++q) {
                raw[q][0] = raw[q][1] = make_uint4(0, 0, 0, 0);
                if (pos[q] != 0xFFFFFFFFu) {
                    const uint4* row = reinterpret_cast<const uint4*>(y + (size_t)pos[q] * w.H);
                    raw[q][0] = __ldg(row + c0);
                    if (two) raw[q][1] = __ldg(row + c1);
                }
            }
#pragma unroll
            for (uint32_t q = 0; q < 4u; ++q) {
                if (pos[q] == 0xFFFFFFFFu) continue;
#pragma unroll
                for (int v = 0; v < 2; ++v) {
                    const uint32_t hw[4] = {raw[q][v].x, raw[q][v].y, raw[q][v].z, raw[q][v].w};
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw[h]));
                        o[v][2 * h] = __fadd_rn(o[v][2 * h], __fmul_rn(f.x, g[q]));
                        o[v][2 * h + 1] = __fadd_rn(o[v][2 * h + 1], __fmul_rn(f.y, g[q]));
                    }
                }
            }
        }
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            if (v == 1 && !two) break;
            uint32_t pk[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                bad |= !(fabsf(o[v][2 * h]) <= 3.0e38f) || !(fabsf(o[v][2 * h + 1]) <= 3.0e38f);
                const __half2 r = __floats2half2_rn(fminf(fmaxf(o[v][2 * h], -65504.0f), 65504.0f),
                                                    fminf(fmaxf(o[v][2 * h + 1], -65504.0f), 65504.0f));
                pk[h] = *reinterpret_cast<const uint32_t*>(&r);
            }
            dst[(size_t)slot * per_row + (v ? c1 : c0)] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    }
    if (bad) atomicOr(status, kStatusNonFiniteOutput);
}

// ------------------------------------------------------------------------------ combine
// out[t] = output_scale * sum over owners o (rank order) of partial_o(t) + shared[t].  The partial
// sums are read from the owners' windows as f16 (16-byte peer loads of eight values) and widened
// with the slot's power-of-two factor; each CTA first checks flag 2 of every rank.
__global__ void __launch_bounds__(256) ep_combine_kernel(EpWindows w, EpPlan pl, const float* __restrict__ shared,
                                                         uint32_t T, float output_scale, float* __restrict__ out,
                                                         uint32_t* __restrict__ status) {
    __shared__ const unsigned short* src[kEpMaxWorld];
    __shared__ float rscale[kEpMaxWorld];
    __shared__ uint32_t failed;
    const uint32_t tid = threadIdx.x, par = w.step & 1u;
    if (tid == 0) failed = *pl.abort_word;
    __syncthreads();
    if (tid < w.world && !failed && !wait_flag(w.flag(w.rank, 2, tid), w.step, w.wait_ns)) {
        atomicOr(&failed, 1u);
        *pl.abort_word = 1;
        atomicOr(status, kStatusWaitTimeout);
    }
    __syncthreads();
    const bool skip = failed != 0;
    const uint32_t per_row = w.H / 8u;     // 16-byte vectors of eight f16 values
    bool bad = false;
    for (uint32_t t = blockIdx.x; t < T; t += gridDim.x) {
        __syncthreads();
        if (tid < w.world) {
            const unsigned short* ptr = nullptr;
            float rs = 0.0f;
            const uint32_t vi = skip ? 0xFFFFFFFFu : pl.vis_idx[(size_t)tid * pl.stride + t];
            if (vi != 0xFFFFFFFFu) {
                const uint32_t slot = pl.tok_base[tid] + vi;
                if (slot < w.cap) {
                    ptr = w.y(tid, par) + (size_t)slot * w.H;
                    rs = w.yscale(tid, par)[slot];   // undoes the slot's power-of-two scale: exact
                }
            }
            src[tid] = ptr;
            rscale[tid] = rs;
        }
        __syncthreads();
        for (uint32_t c = tid; c < per_row; c += blockDim.x) {
            float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            // four peer rows are requested together: a load over NVLink takes microseconds, and one after the other
            // (the loop count is a run-time value) they would add up per thread; the sums keep the rank order
            for (uint32_t r0 = 0; r0 < w.world; r0 += 4u) {
                uint4 v[4];
#pragma unroll
                for (uint32_t q = 0; q < 4u; ++q) {
                    const unsigned short* ptr = r0 + q < w.world ? src[r0 + q] : nullptr;
                    v[q] = ptr ? *reinterpret_cast<const uint4*>(ptr + c * 8u) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (uint32_t q = 0; q < 4u; ++q) {
                    if (r0 + q >= w.world || !src[r0 + q]) continue;
                    const float rs = rscale[r0 + q];
                    const uint32_t wv[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&wv[h]));
                        o[2 * h] = __fadd_rn(o[2 * h], __fmul_rn(f.x, rs));
                        o[2 * h + 1] = __fadd_rn(o[2 * h + 1], __fmul_rn(f.y, rs));
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                if (output_scale != 1.0f) o[q] = __fmul_rn(o[q], output_scale);
            }
            if (shared) {
                const float4* sp = reinterpret_cast<const float4*>(shared + (size_t)t * w.H) + c * 2u;
                const float4 s0 = __ldg(sp), s1 = __ldg(sp + 1);
                o[0] = __fadd_rn(o[0], s0.x); o[1] = __fadd_rn(o[1], s0.y); o[2] = __fadd_rn(o[2], s0.z); o[3] = __fadd_rn(o[3], s0.w);
                o[4] = __fadd_rn(o[4], s1.x); o[5] = __fadd_rn(o[5], s1.y); o[6] = __fadd_rn(o[6], s1.z); o[7] = __fadd_rn(o[7], s1.w);
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) bad |= !(fabsf(o[q]) <= 3.0e38f);
            float4* op = reinterpret_cast<float4*>(out + (size_t)t * w.H) + c * 2u;
            op[0] = make_float4(o[0], o[1], o[2], o[3]);
            op[1] = make_float4(o[4], o[5], o[6], o[7]);
        }
    }
    if (bad) atomicOr(status, kStatusNonFiniteOutput);
}

// ------------------------------------------------------------------------------ launchers
size_t ep_window_bytes(uint32_t world, uint32_t E, uint32_t H, uint32_t cap, uint32_t k) {
    EpWindows w{};
    w.world = world;
    w.E = E;
    w.H = H;
    w.cap = cap;
    w.k = k;
    return w.total_bytes();
}

void launch_ep_visits(const EpWindows& w, const EpPlan& pl, const uint32_t* ids, uint32_t T, cudaStream_t s) {
    ep_visits_kernel<<<w.world, 1024, 0, s>>>(w, pl, ids, T);
    ++g_kernel_launches;
}

void launch_ep_publish(const EpWindows& w, const EpPlan& pl, const uint32_t* counts, cudaStream_t s) {
    ep_publish_kernel<<<w.world, 256, 0, s>>>(w, pl, counts);
    ++g_kernel_launches;
}

void launch_ep_plan(const EpWindows& w, const EpPlan& pl, uint32_t* status, cudaStream_t s) {
    ep_plan_kernel<<<1, 1024, 0, s>>>(w, pl, status);
    ++g_kernel_launches;
}

void launch_ep_dispatch(const EpWindows& w, const EpPlan& pl, const __nv_bfloat16* x, const uint32_t* ids,
                        const uint32_t* inv, const uint32_t* offsets, const float* weights, uint32_t T,
                        cudaStream_t s) {
    const uint64_t tasks = (uint64_t)T * w.world;
    uint32_t grid = (uint32_t)((tasks + 7u) / 8u);
    if (grid < 1u) grid = 1u;
    if (grid > (uint32_t)kNumSMs * 8u) grid = (uint32_t)kNumSMs * 8u;
    ep_dispatch_kernel<<<grid, 256, 0, s>>>(w, pl, x, ids, inv, offsets, weights, T);
    ++g_kernel_launches;
}

void launch_ep_wait(const EpWindows& w, uint32_t kind, uint32_t* abort_word, uint32_t* status, cudaStream_t s) {
    ep_wait_kernel<<<1, 32, 0, s>>>(w, kind, abort_word, status);
    ++g_kernel_launches;
}

void launch_ep_signal(const EpWindows& w, uint32_t kind, cudaStream_t s) {
    ep_signal_kernel<<<1, 32, 0, s>>>(w, kind);
    ++g_kernel_launches;
}

void launch_ep_partial(const EpWindows& w, const EpPlan& pl, const void* y, bool y_half, uint32_t* status,
                       cudaStream_t s) {
    // the row count lives on the device; the grid covers the machine and strides over the slots
    const uint32_t grid = w.cap < (uint32_t)kNumSMs * 8u ? w.cap : (uint32_t)kNumSMs * 8u;
    if (y_half) {
        const uint64_t work = ((uint64_t)w.cap * ((w.H / 8u + 1u) / 2u) + 255u) / 256u;
        const uint32_t g = work < (uint64_t)kNumSMs * 8u ? (uint32_t)work : (uint32_t)kNumSMs * 8u;
        ep_partial_half_kernel<<<g, 256, 0, s>>>(w, pl, static_cast<const __half*>(y), status);
    } else {
        ep_partial_kernel<false><<<grid, 256, 0, s>>>(w, pl, y, status);
    }
    ++g_kernel_launches;
}

void launch_ep_combine(const EpWindows& w, const EpPlan& pl, const float* shared, uint32_t T, float output_scale,
                       float* out, uint32_t* status, cudaStream_t s) {
    if (T == 0) return;
    const uint32_t grid = T < (uint32_t)kNumSMs * 8u ? T : (uint32_t)kNumSMs * 8u;
    ep_combine_kernel<<<grid, 256, 0, s>>>(w, pl, shared, T, output_scale, out, status);
    ++g_kernel_launches;
}

}  // namespace smoe
