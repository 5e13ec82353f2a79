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
        // four expert rows are requested together (their loads do not depend on one another); the products are still
        // added in selection-rank order
        for (uint32_t r0 = 0; r0 < k; r0 += 4u) {
            uint32_t pos[4];
            float w[4];
            uint4 raw[4];
#pragma unroll
            for (uint32_t q = 0; q < 4u; ++q) {
                const bool in = r0 + q < k;
                pos[q] = in ? inv[(size_t)t * k + r0 + q] : 0xFFFFFFFFu;
                w[q] = in ? weights[(size_t)t * k + r0 + q] : 0.0f;
            }
#pragma unroll
            for (uint32_t q = 0; q < 4u; ++q) {
                raw[q] = make_uint4(0, 0, 0, 0);
                if (pos[q] != 0xFFFFFFFFu) {
                    if (Y_HALF)
                        raw[q] = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(y_v) + (size_t)pos[q] * H + c));
                    else
                        raw[q] = __ldg(reinterpret_cast<const uint4*>(static_cast<const float*>(y_v) + (size_t)pos[q] * H + c));
                }
            }
#pragma unroll
            for (uint32_t q = 0; q < 4u; ++q) {
                if (pos[q] == 0xFFFFFFFFu) continue;
                float v[V];
                const uint32_t hw[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
                if (Y_HALF) {
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw[h]));
                        v[2 * h] = f.x;
                        v[2 * h + 1] = f.y;
                    }
                } else {
#pragma unroll
                    for (int h = 0; h < 4; ++h) v[h] = __uint_as_float(hw[h]);
                }
#pragma unroll
                for (uint32_t e = 0; e < V; ++e) o[e] = __fadd_rn(o[e], __fmul_rn(v[e], w[q]));
            }
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
