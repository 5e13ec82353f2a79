// One BF16 row -> f16 with an exact power-of-two pre-scale, by one warp (shared by the stand-alone conversion kernel
// and the fused small-batch front end).  scale = 2^(14 - floor(log2 max|row|)): the row maximum lands in [2^14, 2^15);
// exact, and clamped so both it and its reciprocal stay normal floats.  *rowscale receives the factor that undoes it.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace smoe {

__device__ __forceinline__ void warp_row_to_f16_bf16(const __nv_bfloat16* __restrict__ src, uint32_t C,
                                                     __half* __restrict__ hi, float* __restrict__ rowscale) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint4* p = reinterpret_cast<const uint4*>(src);
    float mx = 0.0f;
    for (uint32_t i = lane; i < C / 8u; i += 32u) {
        const uint4 v = __ldg(p + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            mx = fmaxf(mx, fabsf(__uint_as_float(w[q] << 16)));
            mx = fmaxf(mx, fabsf(__uint_as_float(w[q] & 0xFFFF0000u)));
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    int ex = 0;
    if (mx > 0.0f && mx < 3.0e38f) ex = 14 - (int)((__float_as_uint(mx) >> 23) & 0xFFu) + 127;
    ex = max(-100, min(100, ex));
    const float sc = __uint_as_float((uint32_t)(ex + 127) << 23);
    if (lane == 0) *rowscale = __uint_as_float((uint32_t)(127 - ex) << 23);
    for (uint32_t i = lane; i < C / 8u; i += 32u) {
        const uint4 v = __ldg(p + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const __half a = __float2half_rn(__uint_as_float(w[q] << 16) * sc);
            const __half b = __float2half_rn(__uint_as_float(w[q] & 0xFFFF0000u) * sc);
            o[q] = (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
        }
        *reinterpret_cast<uint4*>(hi + i * 8u) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

}  // namespace smoe
