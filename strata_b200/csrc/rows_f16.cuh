// One BF16 row -> f16 with an exact power-of-two pre-scale, by one warp (shared by the stand-alone conversion kernel
// and the fused small-batch front end).  scale = 2^(14 - floor(log2 max|row|)): the row maximum lands in [2^14, 2^15);
// exact, and clamped so both it and its reciprocal stay normal floats.  *rowscale receives the factor that undoes it.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace smoe {

__device__ __forceinline__ float absmax8_bf16(const uint4& v, float mx) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        mx = fmaxf(mx, fabsf(__uint_as_float(w[q] << 16)));
        mx = fmaxf(mx, fabsf(__uint_as_float(w[q] & 0xFFFF0000u)));
    }
    return mx;
}

__device__ __forceinline__ uint4 scale8_bf16_to_f16(const uint4& v, float sc) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const __half a = __float2half_rn(__uint_as_float(w[q] << 16) * sc);
        const __half b = __float2half_rn(__uint_as_float(w[q] & 0xFFFF0000u) * sc);
        o[q] = (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// Rows of up to 4096 columns are read ONCE: the lane keeps its sixteen 16-byte pieces in registers between the
// maximum and the conversion, and all sixteen loads are in flight together (a warp that converts several rows in
// turn is otherwise bound by one memory round trip per piece).  Longer rows take two passes in batches of eight loads.
__device__ __forceinline__ void warp_row_to_f16_bf16(const __nv_bfloat16* __restrict__ src, uint32_t C,
                                                     __half* __restrict__ hi, float* __restrict__ rowscale) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint4* p = reinterpret_cast<const uint4*>(src);
    uint4* out = reinterpret_cast<uint4*>(hi);
    const uint32_t n = C / 8u;
    const bool once = n <= 16u * 32u;
    uint4 keep[16];
    float mx = 0.0f;
    if (once) {
#pragma unroll
        for (uint32_t q = 0; q < 16u; ++q) {
            const uint32_t i = lane + 32u * q;
            keep[q] = i < n ? __ldg(p + i) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (uint32_t q = 0; q < 16u; ++q) mx = absmax8_bf16(keep[q], mx);
    } else {
        for (uint32_t base = 0; base < n; base += 256u) {
            uint4 v[8];
#pragma unroll
            for (uint32_t q = 0; q < 8u; ++q) {
                const uint32_t i = base + lane + 32u * q;
                v[q] = i < n ? __ldg(p + i) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (uint32_t q = 0; q < 8u; ++q) mx = absmax8_bf16(v[q], mx);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    int ex = 0;
    if (mx > 0.0f && mx < 3.0e38f) ex = 14 - (int)((__float_as_uint(mx) >> 23) & 0xFFu) + 127;
    ex = max(-100, min(100, ex));
    const float sc = __uint_as_float((uint32_t)(ex + 127) << 23);
    if (lane == 0) *rowscale = __uint_as_float((uint32_t)(127 - ex) << 23);
    if (once) {
#pragma unroll
        for (uint32_t q = 0; q < 16u; ++q) {
            const uint32_t i = lane + 32u * q;
            if (i < n) out[i] = scale8_bf16_to_f16(keep[q], sc);
        }
    } else {
        for (uint32_t base = 0; base < n; base += 256u) {
            uint4 v[8];
#pragma unroll
            for (uint32_t q = 0; q < 8u; ++q) {
                const uint32_t i = base + lane + 32u * q;
                v[q] = i < n ? __ldg(p + i) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (uint32_t q = 0; q < 8u; ++q) {
                const uint32_t i = base + lane + 32u * q;
                if (i < n) out[i] = scale8_bf16_to_f16(v[q], sc);
            }
        }
    }
}

// The same conversion when one source row feeds several destination rows (a token's row in front of each of its k
// experts): the row is read and converted once and stored k times.  Lane j < k holds destination row j in `mydst`
// (0xFFFFFFFF = none); hi / rowscale are the bases of the destination arrays.
__device__ __forceinline__ void warp_row_to_f16_bf16_spread(const __nv_bfloat16* __restrict__ src, uint32_t C,
                                                            __half* __restrict__ hi, float* __restrict__ rowscale,
                                                            uint32_t mydst, uint32_t k) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint4* p = reinterpret_cast<const uint4*>(src);
    const uint32_t n = C / 8u;
    float mx = 0.0f;
    for (uint32_t base = 0; base < n; base += 256u) {
        uint4 v[8];
#pragma unroll
        for (uint32_t q = 0; q < 8u; ++q) {
            const uint32_t i = base + lane + 32u * q;
            v[q] = i < n ? __ldg(p + i) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (uint32_t q = 0; q < 8u; ++q) mx = absmax8_bf16(v[q], mx);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    int ex = 0;
    if (mx > 0.0f && mx < 3.0e38f) ex = 14 - (int)((__float_as_uint(mx) >> 23) & 0xFFu) + 127;
    ex = max(-100, min(100, ex));
    const float sc = __uint_as_float((uint32_t)(ex + 127) << 23);
    if (lane < k && mydst != 0xFFFFFFFFu) rowscale[mydst] = __uint_as_float((uint32_t)(127 - ex) << 23);
    for (uint32_t base = 0; base < n; base += 256u) {
        uint4 v[8];
#pragma unroll
        for (uint32_t q = 0; q < 8u; ++q) {
            const uint32_t i = base + lane + 32u * q;
            v[q] = i < n ? scale8_bf16_to_f16(__ldg(p + i), sc) : make_uint4(0, 0, 0, 0);
        }
        for (uint32_t j = 0; j < k; ++j) {
            const uint32_t d = __shfl_sync(0xFFFFFFFFu, mydst, j);
            if (d == 0xFFFFFFFFu) continue;
            uint4* out = reinterpret_cast<uint4*>(hi + (size_t)d * C);
#pragma unroll
            for (uint32_t q = 0; q < 8u; ++q) {
                const uint32_t i = base + lane + 32u * q;
                if (i < n) out[i] = v[q];
            }
        }
    }
}

}  // namespace smoe
