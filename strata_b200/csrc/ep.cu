// Expert-parallel exchange over peer memory (NVLink / NVSwitch), fused with the work on either
// side of it: the dispatch kernel gathers a token's row and stores it straight into the owning
// GPU's grouped input buffer, and the combine kernel loads the expert outputs straight from the
// owners' buffers while it forms the top-k-weighted sum.  No staging copy, no host round trip,
// no library collective on the data path.
//
// The reference places experts on several GPUs of one process and moves the activations through
// host memory (src/models/glm52/glm_runtime.cpp:650-652, 1561-1576); this file replaces that
// transport for one-process-per-GPU expert parallelism.
//
// Every rank owns a "window" of device memory with the same layout, mapped into every peer:
//
//   flags  u32 [3][world]        flags[k][s] = last step for which rank s finished phase k
//                                (0 counts published, 1 rows stored, 2 expert outputs ready)
//   counts u32 [2][world][E]     counts[p][s][e] = rows rank s holds for global expert e
//   rows   bf16 [2][cap][H]      grouped input rows of this rank's experts (local expert, source
//                                rank, source scan order)
//   y      f16 [2][cap][H]       expert outputs for those rows, each row scaled by a power of two
//   yscale f32 [2][cap]          the factor that undoes a row's scale
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

// ------------------------------------------------------------------------------ publish
// Block b stores this rank's per-expert counts into rank b's window and raises flag 0 there.
__global__ void __launch_bounds__(256) ep_publish_kernel(EpWindows w, const uint32_t* __restrict__ counts) {
    const uint32_t dst = blockIdx.x;
    uint32_t* c = w.counts(dst, w.step & 1u, w.rank);
    for (uint32_t e = threadIdx.x; e < w.E; e += blockDim.x) c[e] = counts[e];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(w.flag(dst, 0, w.rank), w.step);
}

// ------------------------------------------------------------------------------ plan
// One CTA.  Waits for every rank's counts, then derives from the full [world][E] matrix
//   dst_row[e]   first row, in the owner's window, of this rank's rows for global expert e
//   loffsets[j]  row range of this rank's local expert j over all sources (j = 0..B)
// Any rank can evaluate every owner's total, so an overflow of `cap` is seen by all ranks alike.
__global__ void __launch_bounds__(1024) ep_plan_kernel(EpWindows w, uint32_t* __restrict__ dst_row,
                                                       uint32_t* __restrict__ loffsets,
                                                       uint32_t* __restrict__ abort_word,
                                                       uint32_t* __restrict__ status) {
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
        dst_row[tid] = excl + before;
        if (owner == w.rank) {
            loffsets[tid - owner * B] = excl;
            if (tid - owner * B == B - 1) loffsets[B] = excl + tot;
        }
    }
    __syncthreads();
    if (bad) {
        // nothing is sent and nothing is computed this step
        for (uint32_t i = tid; i <= B; i += blockDim.x) loffsets[i] = 0;
        for (uint32_t i = tid; i < w.E; i += blockDim.x) dst_row[i] = 0;
        if (tid == 0) {
            *abort_word = 1;
            atomicOr(status, (bad & 1u) ? kStatusWaitTimeout : kStatusBadGroup);
        }
    } else if (tid == 0) {
        *abort_word = 0;
    }
}

// ------------------------------------------------------------------------------ dispatch
// One warp per (token, expert) pair in grouped order: copy the token's BF16 row into the owner's
// window.  The last CTA to finish raises flag 1 on every rank.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpWindows w, const __nv_bfloat16* __restrict__ x,
                                                          const uint32_t* __restrict__ ids,
                                                          const uint32_t* __restrict__ perm,
                                                          const uint32_t* __restrict__ offsets,
                                                          const uint32_t* __restrict__ dst_row, uint32_t pairs,
                                                          uint32_t k, const uint32_t* __restrict__ abort_word,
                                                          uint32_t* __restrict__ done) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t B = w.E / w.world;
    const uint32_t vecs = w.H / 8u;   // 16-byte vectors per row
    if (*abort_word == 0) {
        for (uint32_t p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < pairs; p += warps) {
            const uint32_t pair = perm[p];
            const uint32_t e = ids[pair];
            if (e >= w.E) continue;
            const uint32_t row = dst_row[e] + (p - offsets[e]);
            if (row >= w.cap) continue;   // cannot happen after a clean plan; never store outside the window
            const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(pair / k) * w.H);
            uint4* dst = reinterpret_cast<uint4*>(w.rows(e / B, w.step & 1u) + (size_t)row * w.H);
            for (uint32_t v = lane; v < vecs; v += 32u) dst[v] = __ldg(src + v);
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t prev = atomicAdd(done, 1u);
        if (prev == gridDim.x - 1u) {
            *done = 0;
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

// One warp: lane d tells rank d that this rank's expert outputs of the step are in its window.
__global__ void ep_signal_kernel(EpWindows w, uint32_t kind) {
    const uint32_t d = threadIdx.x;
    __threadfence_system();
    if (d < w.world) st_release_sys(w.flag(d, kind, w.rank), w.step);
}

// ------------------------------------------------------------------------------ combine
// out[t] = output_scale * sum_r weight[t,r] * y_owner(t,r)[row(t,r)] + shared[t], the sum taken in
// selection-rank order with separate multiply and add like the single-GPU combine.  The expert
// rows are read from the owners' windows as f16 (16-byte peer loads of eight values) and widened
// with the row's power-of-two factor; each CTA first waits for flag 2 of every rank.
__global__ void __launch_bounds__(256) ep_combine_kernel(EpWindows w, const uint32_t* __restrict__ ids,
                                                         const uint32_t* __restrict__ inv,
                                                         const uint32_t* __restrict__ offsets,
                                                         const uint32_t* __restrict__ dst_row,
                                                         const float* __restrict__ weights,
                                                         const float* __restrict__ shared, uint32_t T, uint32_t k,
                                                         float output_scale, float* __restrict__ out,
                                                         uint32_t* __restrict__ abort_word,
                                                         uint32_t* __restrict__ status) {
    __shared__ const unsigned short* src[32];
    __shared__ float wgt[32], rscale[32];
    __shared__ uint32_t failed;
    const uint32_t tid = threadIdx.x;
    if (tid == 0) failed = *abort_word;
    __syncthreads();
    if (tid < w.world && !failed && !wait_flag(w.flag(w.rank, 2, tid), w.step, w.wait_ns)) {
        atomicOr(&failed, 1u);
        *abort_word = 1;
        atomicOr(status, kStatusWaitTimeout);
    }
    __syncthreads();
    const bool skip = failed != 0;
    const uint32_t B = w.E / w.world;
    const uint32_t per_row = w.H / 8u;     // 16-byte vectors of eight f16 values
    bool bad = false;
    for (uint32_t t = blockIdx.x; t < T; t += gridDim.x) {
        __syncthreads();
        if (tid < k) {
            const uint32_t pair = t * k + tid;
            const uint32_t e = ids[pair], p = inv[pair];
            const unsigned short* ptr = nullptr;
            float rs = 0.0f;
            if (!skip && e < w.E && p != 0xFFFFFFFFu) {
                const uint32_t row = dst_row[e] + (p - offsets[e]);
                if (row < w.cap) {
                    ptr = w.y(e / B, w.step & 1u) + (size_t)row * w.H;
                    rs = w.yscale(e / B, w.step & 1u)[row];
                }
            }
            src[tid] = ptr;
            rscale[tid] = rs;               // undoes the row's power-of-two scale: exact
            wgt[tid] = weights[pair];
        }
        __syncthreads();
        for (uint32_t c = tid; c < per_row; c += blockDim.x) {
            float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            // four peer rows are requested together: a load over NVLink takes microseconds, and one after the other
            // (the loop count is a run-time value) they would add up per thread; the sums keep the rank order
            for (uint32_t r0 = 0; r0 < k; r0 += 4u) {
                uint4 v[4];
#pragma unroll
                for (uint32_t q = 0; q < 4u; ++q) {
                    const unsigned short* ptr = r0 + q < k ? src[r0 + q] : nullptr;
                    v[q] = ptr ? *reinterpret_cast<const uint4*>(ptr + c * 8u) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (uint32_t q = 0; q < 4u; ++q) {
                    if (r0 + q >= k || !src[r0 + q]) continue;
                    const float g = wgt[r0 + q], rs = rscale[r0 + q];
                    const uint32_t wv[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&wv[h]));
                        o[2 * h] = __fadd_rn(o[2 * h], __fmul_rn(__fmul_rn(f.x, rs), g));
                        o[2 * h + 1] = __fadd_rn(o[2 * h + 1], __fmul_rn(__fmul_rn(f.y, rs), g));
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
size_t ep_window_bytes(uint32_t world, uint32_t E, uint32_t H, uint32_t cap) {
    EpWindows w{};
    w.world = world;
    w.E = E;
    w.H = H;
    w.cap = cap;
    return w.total_bytes();
}

void launch_ep_publish(const EpWindows& w, const uint32_t* counts, cudaStream_t s) {
    ep_publish_kernel<<<w.world, 256, 0, s>>>(w, counts);
    ++g_kernel_launches;
}

void launch_ep_plan(const EpWindows& w, uint32_t* dst_row, uint32_t* loffsets, uint32_t* abort_word,
                    uint32_t* status, cudaStream_t s) {
    ep_plan_kernel<<<1, 1024, 0, s>>>(w, dst_row, loffsets, abort_word, status);
    ++g_kernel_launches;
}

void launch_ep_dispatch(const EpWindows& w, const __nv_bfloat16* x, const uint32_t* ids, const uint32_t* perm,
                        const uint32_t* offsets, const uint32_t* dst_row, uint32_t pairs, uint32_t k,
                        const uint32_t* abort_word, uint32_t* done, cudaStream_t s) {
    uint32_t grid = (pairs + 7u) / 8u;
    if (grid < 1u) grid = 1u;
    if (grid > (uint32_t)kNumSMs * 8u) grid = (uint32_t)kNumSMs * 8u;
    ep_dispatch_kernel<<<grid, 256, 0, s>>>(w, x, ids, perm, offsets, dst_row, pairs, k, abort_word, done);
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

void launch_ep_combine(const EpWindows& w, const uint32_t* ids, const uint32_t* inv, const uint32_t* offsets,
                       const uint32_t* dst_row, const float* weights, const float* shared, uint32_t T, uint32_t k,
                       float output_scale, float* out, uint32_t* abort_word, uint32_t* status, cudaStream_t s) {
    if (T == 0) return;
    const uint32_t grid = T < (uint32_t)kNumSMs * 8u ? T : (uint32_t)kNumSMs * 8u;
    ep_combine_kernel<<<grid, 256, 0, s>>>(w, ids, inv, offsets, dst_row, weights, shared, T, k, output_scale, out,
                                           abort_word, status);
    ++g_kernel_launches;
}

}  // namespace smoe
