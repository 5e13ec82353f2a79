// Top-k-weighted combine: out[t] = output_scale * sum_r w[t,r] * y[inv[t*k+r]] + shared[t].
//
// A gather, not a scatter: one thread owns output elements and adds its token's k expert rows
// in selection-rank order with separate multiply and add, so the result is reproducible run
// to run and equals the reference's host loops `dest += src * weight` evaluated in rank order
// (src/models/dsv4/deepseek_runtime.cpp:5897-5914, src/models/inkling/inkling_runtime.cpp:
// 856-868; scale placement as src/models/laguna/laguna_runtime.cpp:1141-1156).
#include <cuda_fp16.h>

#include "common.cuh"

namespace smoe {

// Y_HALF: the expert rows are f16 (the tensor-core down kernel can store them so: half the bytes of the pass that
// bounds this kernel); they widen exactly and the arithmetic below is unchanged.
template <bool Y_HALF>
__global__ void __launch_bounds__(256) combine_kernel(const void* __restrict__ y_v,
                                                      const uint32_t* __restrict__ inv,
                                                      const float* __restrict__ weights,
                                                      const float* __restrict__ shared, uint32_t T,
                                                      uint32_t k, uint32_t H, float output_scale,
                                                      float* __restrict__ out, uint32_t* status) {
    constexpr uint32_t V = Y_HALF ? 8u : 4u;     // columns per thread: one 16-byte load of an expert row either way
    const uint32_t per_row = H / V;
    bool bad = false;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)T * per_row;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / per_row), c = (uint32_t)(i % per_row) * V;
        float o[V];
#pragma unroll
        for (uint32_t q = 0; q < V; ++q) o[q] = 0.0f;
        for (uint32_t r = 0; r < k; ++r) {
            const uint32_t pos = inv[(size_t)t * k + r];
            if (pos == 0xFFFFFFFFu) continue;
            const float w = weights[(size_t)t * k + r];
            float v[V];
            if (Y_HALF) {
                const uint4 h = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(y_v) + (size_t)pos * H + c));
                const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw[q]));
                    v[2 * q] = f.x;
                    v[2 * q + 1] = f.y;
                }
            } else {
                const float4 f = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(y_v) + (size_t)pos * H + c));
                v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
            }
#pragma unroll
            for (uint32_t q = 0; q < V; ++q) o[q] = __fadd_rn(o[q], __fmul_rn(v[q], w));
        }
        if (output_scale != 1.0f) {
#pragma unroll
            for (uint32_t q = 0; q < V; ++q) o[q] = __fmul_rn(o[q], output_scale);
        }
        if (shared) {
#pragma unroll
            for (uint32_t q4 = 0; q4 < V / 4u; ++q4) {
                const float4 s = __ldg(reinterpret_cast<const float4*>(shared + (size_t)t * H + c) + q4);
                o[4 * q4] = __fadd_rn(o[4 * q4], s.x);
                o[4 * q4 + 1] = __fadd_rn(o[4 * q4 + 1], s.y);
                o[4 * q4 + 2] = __fadd_rn(o[4 * q4 + 2], s.z);
                o[4 * q4 + 3] = __fadd_rn(o[4 * q4 + 3], s.w);
            }
        }
#pragma unroll
        for (uint32_t q = 0; q < V; ++q) bad |= !(fabsf(o[q]) <= 3.0e38f);
#pragma unroll
        for (uint32_t q4 = 0; q4 < V / 4u; ++q4)
            reinterpret_cast<float4*>(out + (size_t)t * H + c)[q4] = make_float4(o[4 * q4], o[4 * q4 + 1], o[4 * q4 + 2], o[4 * q4 + 3]);
    }
    if (bad) atomicOr(status, kStatusNonFiniteOutput);
}

void launch_combine(const void* y, const uint32_t* inv, const float* weights, const float* shared,
                    uint32_t T, uint32_t k, uint32_t H, float output_scale, float* out,
                    uint32_t* status, cudaStream_t s, bool y_half) {
    if (T == 0) return;
    const size_t n = (size_t)T * (H / (y_half ? 8u : 4u));
    const uint32_t grid = (uint32_t)((n + 255) / 256 < 148u * 8u ? (n + 255) / 256 : 148u * 8u);
    if (y_half)
        combine_kernel<true><<<grid, 256, 0, s>>>(y, inv, weights, shared, T, k, H, output_scale, out, status);
    else
        combine_kernel<false><<<grid, 256, 0, s>>>(y, inv, weights, shared, T, k, H, output_scale, out, status);
    ++g_kernel_launches;
}

}  // namespace smoe
