// Token -> expert grouping: per-expert counts, exclusive offsets, and the stable permutation
// that sorts (token, rank) pairs by expert id while keeping row-major scan order inside each
// expert -- the lists the reference builds on the host with vector pushes
// (src/models/glm52/glm_runtime.cpp:1521-1541, src/models/dsv4/deepseek_runtime.cpp:6216-6321).
//
// Integer work only.  Pairs are cut into segments of 128 (one warp each); a warp ranks its
// pairs with __match_any_sync, so the order inside a segment is the scan order, and segment
// bases come from an exclusive scan over (expert, segment).  Pairs whose expert lies outside
// [expert_begin, expert_begin + n_experts) are ignored (expert-parallel ranks group only their
// own experts).
#include "common.cuh"

namespace smoe {

constexpr uint32_t kSegPairs = 128;   // pairs per warp segment
constexpr uint32_t kSmallPairs = 2048; // single-CTA path up to this many pairs (above, the segmented path is faster: 35 vs ~22 us at 2560 pairs)

// ---- small path: one CTA does everything ---------------------------------------------------
__global__ void __launch_bounds__(1024) group_small_kernel(
    const uint32_t* __restrict__ ids, uint32_t pairs, uint32_t ebeg, uint32_t nexp,
    uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets, uint32_t* __restrict__ perm,
    uint32_t* __restrict__ inv, uint32_t* __restrict__ active_list, uint32_t* __restrict__ n_active) {
    extern __shared__ uint32_t sm[];
    uint32_t* cnt = sm;             // [nexp]
    uint32_t* cur = sm + nexp;      // [nexp] running cursor
    uint32_t* scan = sm + 2 * nexp; // [1024] scratch
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    for (uint32_t e = tid; e < nexp; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (uint32_t i = tid; i < pairs; i += blockDim.x) {
        const uint32_t e = ids[i] - ebeg;
        if (e < nexp) atomicAdd(&cnt[e], 1u);
    }
    __syncthreads();
    // exclusive scan over experts (nexp <= 1024): one element per thread, Hillis-Steele
    const uint32_t mine = tid < nexp ? cnt[tid] : 0u;
    scan[tid] = mine;
    __syncthreads();
    for (uint32_t off = 1; off < 1024u; off <<= 1) {
        const uint32_t v = tid >= off ? scan[tid - off] : 0u;
        __syncthreads();
        scan[tid] += v;
        __syncthreads();
    }
    const uint32_t incl = scan[tid];
    if (tid < nexp) {
        counts[tid] = mine;
        offsets[tid] = incl - mine;
        cur[tid] = incl - mine;
        if (tid == nexp - 1) offsets[nexp] = incl;
    }
    __syncthreads();
    // active list (ascending): rank = number of non-empty experts before this one
    scan[tid] = (tid < nexp && mine) ? 1u : 0u;
    __syncthreads();
    for (uint32_t off = 1; off < 1024u; off <<= 1) {
        const uint32_t v = tid >= off ? scan[tid - off] : 0u;
        __syncthreads();
        scan[tid] += v;
        __syncthreads();
    }
    if (active_list) {
        if (tid < nexp && mine) active_list[scan[tid] - 1u] = tid;
        if (tid == 1023u) *n_active = scan[1023];
    }
    __syncthreads();
    // stable placement: warps take their 32 pairs in turn
    const uint32_t nwarps = blockDim.x >> 5;
    for (uint32_t base = 0; base < pairs; base += blockDim.x) {
        const uint32_t i = base + tid;
        const uint32_t e = i < pairs ? ids[i] - ebeg : 0xFFFFFFFFu;
        const bool ok = e < nexp;
        for (uint32_t w = 0; w < nwarps; ++w) {
            if (warp == w && base + w * 32u < pairs) {
                const uint32_t key = ok ? e : 0xFFFFFFFFu;
                const uint32_t peers = __match_any_sync(0xFFFFFFFFu, key);
                if (ok) {
                    const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
                    const uint32_t pos = cur[e] + rank;
                    perm[pos] = i;
                    if (inv) inv[i] = pos;
                }
                __syncwarp();
                if (ok && lane == (uint32_t)(__ffs(peers) - 1)) cur[e] += __popc(peers);
            }
            __syncthreads();
        }
    }
    for (uint32_t i = tid; i < pairs; i += blockDim.x) {
        const uint32_t e = ids[i] - ebeg;
        if (!(e < nexp) && inv) inv[i] = 0xFFFFFFFFu;
    }
}

// ---- large path -------------------------------------------------------------------------
// A: per-segment histograms  hist[seg][e]
__global__ void __launch_bounds__(256) group_hist_kernel(const uint32_t* __restrict__ ids,
                                                         uint32_t pairs, uint32_t ebeg, uint32_t nexp,
                                                         uint32_t* __restrict__ hist) {
    extern __shared__ uint32_t sm[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    uint32_t* h = sm + (size_t)warp * nexp;
    const uint32_t seg = blockIdx.x * 8u + warp;
    for (uint32_t e = lane; e < nexp; e += 32u) h[e] = 0;
    __syncwarp();
    const uint32_t b = seg * kSegPairs;
    for (uint32_t i = b + lane; i < min(b + kSegPairs, pairs); i += 32u) {
        const uint32_t e = ids[i] - ebeg;
        if (e < nexp) atomicAdd(&h[e], 1u);
    }
    __syncwarp();
    if (b < pairs)
        for (uint32_t e = lane; e < nexp; e += 32u) hist[(size_t)seg * nexp + e] = h[e];
}

// B: per expert, exclusive scan over segments (in place) and total count.  One warp per expert,
// 128 segments per round: the four loads of a round are issued together, a shuffle scan orders them.
__global__ void __launch_bounds__(256) group_segscan_kernel(uint32_t* __restrict__ hist, uint32_t nseg,
                                                            uint32_t nexp, uint32_t* __restrict__ counts) {
    const uint32_t e = blockIdx.x * 8u + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (e >= nexp) return;
    uint32_t run = 0;
    for (uint32_t b = 0; b < nseg; b += 128u) {
        uint32_t v[4];
#pragma unroll
        for (uint32_t q = 0; q < 4u; ++q) {
            const uint32_t sidx = b + q * 32u + lane;
            v[q] = sidx < nseg ? hist[(size_t)sidx * nexp + e] : 0u;
        }
#pragma unroll
        for (uint32_t q = 0; q < 4u; ++q) {
            uint32_t incl = v[q];
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, off);
                if ((int)lane >= off) incl += t;
            }
            const uint32_t sidx = b + q * 32u + lane;
            if (sidx < nseg) hist[(size_t)sidx * nexp + e] = run + incl - v[q];
            run += __shfl_sync(0xFFFFFFFFu, incl, 31);
        }
    }
    if (lane == 0) counts[e] = run;
}

// C: offsets = exclusive scan of counts; active list
__global__ void __launch_bounds__(1024) group_offsets_kernel(const uint32_t* __restrict__ counts,
                                                             uint32_t nexp, uint32_t* __restrict__ offsets,
                                                             uint32_t* __restrict__ active_list,
                                                             uint32_t* __restrict__ n_active) {
    __shared__ uint32_t scan[1024];
    __shared__ uint32_t scan2[1024];
    const uint32_t tid = threadIdx.x;
    const uint32_t mine = tid < nexp ? counts[tid] : 0u;
    scan[tid] = mine;
    scan2[tid] = mine ? 1u : 0u;
    __syncthreads();
    for (uint32_t off = 1; off < 1024u; off <<= 1) {
        const uint32_t v = tid >= off ? scan[tid - off] : 0u;
        const uint32_t v2 = tid >= off ? scan2[tid - off] : 0u;
        __syncthreads();
        scan[tid] += v;
        scan2[tid] += v2;
        __syncthreads();
    }
    if (tid < nexp) {
        offsets[tid] = scan[tid] - mine;
        if (tid == nexp - 1) offsets[nexp] = scan[tid];
        if (active_list && mine) active_list[scan2[tid] - 1u] = tid;
    }
    if (active_list && tid == 1023u) *n_active = scan2[1023];
}

// D: stable scatter, one warp per segment, 4 rounds of 32 pairs in order
__global__ void __launch_bounds__(256) group_scatter_kernel(
    const uint32_t* __restrict__ ids, uint32_t pairs, uint32_t ebeg, uint32_t nexp,
    const uint32_t* __restrict__ hist, const uint32_t* __restrict__ offsets,
    uint32_t* __restrict__ perm, uint32_t* __restrict__ inv) {
    extern __shared__ uint32_t sm[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    uint32_t* cur = sm + (size_t)warp * nexp;
    const uint32_t seg = blockIdx.x * 8u + warp;
    const uint32_t b = seg * kSegPairs;
    if (b >= pairs) return;
    for (uint32_t e = lane; e < nexp; e += 32u) cur[e] = offsets[e] + hist[(size_t)seg * nexp + e];
    __syncwarp();
    for (uint32_t r = 0; r < kSegPairs / 32u; ++r) {
        const uint32_t i = b + r * 32u + lane;
        const uint32_t e = i < pairs ? ids[i] - ebeg : 0xFFFFFFFFu;
        const bool ok = e < nexp;
        const uint32_t peers = __match_any_sync(0xFFFFFFFFu, ok ? e : 0xFFFFFFFFu);
        if (ok) {
            const uint32_t pos = cur[e] + __popc(peers & ((1u << lane) - 1u));
            perm[pos] = i;
            if (inv) inv[i] = pos;
        } else if (i < pairs && inv) {
            inv[i] = 0xFFFFFFFFu;
        }
        __syncwarp();
        if (ok && lane == (uint32_t)(__ffs(peers) - 1)) cur[e] += __popc(peers);
        __syncwarp();
    }
}

size_t group_scratch_bytes(uint32_t pairs, uint32_t n_experts) {
    const size_t nseg = (pairs + kSegPairs - 1) / kSegPairs;
    return (nseg + 8) * (size_t)n_experts * sizeof(uint32_t);
}

void launch_group(const uint32_t* ids, uint32_t pairs, uint32_t expert_begin, uint32_t n_experts,
                  uint32_t* counts, uint32_t* offsets, uint32_t* perm, uint32_t* inv,
                  uint32_t* active_list, uint32_t* n_active, void* scratch, cudaStream_t s) {
    if (pairs <= kSmallPairs) {
        const size_t smem = (2u * (size_t)n_experts + 1024u) * sizeof(uint32_t);
        group_small_kernel<<<1, 1024, smem, s>>>(ids, pairs, expert_begin, n_experts, counts, offsets,
                                                perm, inv, active_list, n_active);
        ++g_kernel_launches;
        return;
    }
    uint32_t* hist = static_cast<uint32_t*>(scratch);
    const uint32_t nseg = (pairs + kSegPairs - 1) / kSegPairs;
    const uint32_t blocks = (nseg + 7) / 8;
    const size_t smem = 8u * (size_t)n_experts * sizeof(uint32_t);
    group_hist_kernel<<<blocks, 256, smem, s>>>(ids, pairs, expert_begin, n_experts, hist);
    group_segscan_kernel<<<(n_experts + 7) / 8, 256, 0, s>>>(hist, nseg, n_experts, counts);
    group_offsets_kernel<<<1, 1024, 0, s>>>(counts, n_experts, offsets, active_list, n_active);
    group_scatter_kernel<<<blocks, 256, smem, s>>>(ids, pairs, expert_begin, n_experts, hist, offsets,
                                                   perm, inv);
    g_kernel_launches += 4;
}


// ---------------------------------------------------------------------------------------------
// Grouping without any allocation.
//
// Some hosts of this library cannot let it allocate device memory: a serving runtime that has
// handed the whole GPU to its own arena at start-up (a later cudaMalloc then fails or stalls),
// or a caller sitting in a latency-critical section where cudaMalloc's implicit device
// synchronisation is not acceptable.  Those callers have no layer object (creating one
// allocates workspaces), so this entry point works on caller-provided inputs and outputs only
// and keeps its scratch -- the per-segment histograms of the segmented path -- in a fixed
// device array that is part of the loaded module.
//
// Limits and rules:
//   * at most kStaticMaxPairs pairs and kStaticMaxExperts experts per call (520 KiB of scratch,
//     held by every GPU that loads the library until the process exits);
//   * the first call on a device looks up the array's device address; make that first call
//     before any stream capture on that device;
//   * all calls share the one array: two calls whose kernels overlap on the GPU (different
//     streams, or different host threads) race on it.  Serialise them;
//   * nothing has to be cleared between calls: every histogram row a call reads was written by
//     that call's first kernel.
constexpr uint32_t kStaticMaxPairs = 65536;
constexpr uint32_t kStaticMaxExperts = 256;
static __device__ __align__(256) uint32_t g_group_static_scratch[(kStaticMaxPairs / kSegPairs + 8) * kStaticMaxExperts];

}  // namespace smoe

#include <cstdio>
#include <mutex>

extern "C" int strata_moe_group_static(void* stream, const uint32_t* ids, uint32_t pairs,
                                       uint32_t expert_begin, uint32_t n_experts, uint32_t* counts,
                                       uint32_t* offsets, uint32_t* perm, uint32_t* inv, char* err,
                                       size_t err_cap) {
    using namespace smoe;
    auto fail = [&](int code, const char* what, const char* detail) {
        if (err && err_cap) snprintf(err, err_cap, "strata_moe_group_static: %s%s%s", what, detail ? ": " : "",
                                     detail ? detail : "");
        return code;
    };
    if (!ids || !counts || !offsets || !perm) return fail(STRATA_MOE_E_INVALID, "null pointer", nullptr);
    if (pairs > kStaticMaxPairs)
        return fail(STRATA_MOE_E_INVALID, "too many pairs for the fixed scratch (limit 65536); use strata_moe_group",
                    nullptr);
    if (n_experts == 0 || n_experts > kStaticMaxExperts)
        return fail(STRATA_MOE_E_INVALID, "expert count must be in 1..256 for the fixed scratch; use strata_moe_group",
                    nullptr);
    // device address of the scratch array, looked up once per device with that device current
    static std::mutex mu;
    static uint32_t* dev_ptr[64] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(STRATA_MOE_E_CUDA, "cudaGetDevice", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(STRATA_MOE_E_INVALID, "device ordinal out of range", nullptr);
    uint32_t* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!dev_ptr[dev]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_group_static_scratch);
            if (e != cudaSuccess) return fail(STRATA_MOE_E_CUDA, "cudaGetSymbolAddress", cudaGetErrorString(e));
            dev_ptr[dev] = static_cast<uint32_t*>(p);
        }
        scratch = dev_ptr[dev];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // an error left pending by earlier, unrelated work must not be reported as this call's launch
    e = cudaPeekAtLastError();
    if (e != cudaSuccess) return fail(STRATA_MOE_E_CUDA, "an earlier CUDA error is pending", cudaGetErrorString(e));
    const uint32_t nseg = (pairs + kSegPairs - 1) / kSegPairs;
    const uint32_t blocks = (nseg + 7) / 8;
    const size_t smem = 8u * (size_t)n_experts * sizeof(uint32_t);
    if (nseg) group_hist_kernel<<<blocks, 256, smem, s>>>(ids, pairs, expert_begin, n_experts, scratch);
    group_segscan_kernel<<<(n_experts + 7) / 8, 256, 0, s>>>(scratch, nseg, n_experts, counts);
    group_offsets_kernel<<<1, 1024, 0, s>>>(counts, n_experts, offsets, nullptr, nullptr);
    if (nseg)
        group_scatter_kernel<<<blocks, 256, smem, s>>>(ids, pairs, expert_begin, n_experts, scratch, offsets, perm,
                                                       inv);
    g_kernel_launches += nseg ? 4 : 2;
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(STRATA_MOE_E_CUDA, "kernel launch", cudaGetErrorString(e));
    return 0;
}
