// Top-k-weighted combine: out[t] = output_scale * sum_r w[t,r] * y[inv[t*k+r]] + shared[t].
//
// A gather, not a scatter: one thread owns output elements and adds its token's k expert rows
// in selection-rank order with separate multiply and add, so the result is reproducible run
// to run and equals the reference's host loops `dest += src * weight` evaluated in rank order
// (src/models/dsv4/deepseek_runtime.cpp:5897-5914, src/models/inkling/inkling_runtime.cpp:
// 856-868; scale placement as src/models/laguna/laguna_runtime.cpp:1141-1156).
#include "common.cuh"

namespace smoe {

__global__ void __launch_bounds__(256) combine_kernel(const float* __restrict__ y,
                                                      const uint32_t* __restrict__ inv,
                                                      const float* __restrict__ weights,
                                                      const float* __restrict__ shared, uint32_t T,
                                                      uint32_t k, uint32_t H, float output_scale,
                                                      float* __restrict__ out, uint32_t* status) {
    const uint32_t per_row = H / 4u;
    bool bad = false;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)T * per_row;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / per_row), c = (uint32_t)(i % per_row) * 4u;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < k; ++r) {
            const uint32_t pos = inv[(size_t)t * k + r];
            if (pos == 0xFFFFFFFFu) continue;
            const float w = weights[(size_t)t * k + r];
            const float4 v = __ldg(reinterpret_cast<const float4*>(y + (size_t)pos * H + c));
            o.x = __fadd_rn(o.x, __fmul_rn(v.x, w));
            o.y = __fadd_rn(o.y, __fmul_rn(v.y, w));
            o.z = __fadd_rn(o.z, __fmul_rn(v.z, w));
            o.w = __fadd_rn(o.w, __fmul_rn(v.w, w));
        }
        if (output_scale != 1.0f) {
            o.x = __fmul_rn(o.x, output_scale);
            o.y = __fmul_rn(o.y, output_scale);
            o.z = __fmul_rn(o.z, output_scale);
            o.w = __fmul_rn(o.w, output_scale);
        }
        if (shared) {
            const float4 s = __ldg(reinterpret_cast<const float4*>(shared + (size_t)t * H + c));
            o.x = __fadd_rn(o.x, s.x);
            o.y = __fadd_rn(o.y, s.y);
            o.z = __fadd_rn(o.z, s.z);
            o.w = __fadd_rn(o.w, s.w);
        }
        bad |= !(fabsf(o.x) <= 3.0e38f) | !(fabsf(o.y) <= 3.0e38f) | !(fabsf(o.z) <= 3.0e38f) |
               !(fabsf(o.w) <= 3.0e38f);
        *reinterpret_cast<float4*>(out + (size_t)t * H + c) = o;
    }
    if (bad) atomicOr(status, kStatusNonFiniteOutput);
}

void launch_combine(const float* y, const uint32_t* inv, const float* weights, const float* shared,
                    uint32_t T, uint32_t k, uint32_t H, float output_scale, float* out,
                    uint32_t* status, cudaStream_t s) {
    if (T == 0) return;
    const size_t n = (size_t)T * (H / 4u);
    const uint32_t grid = (uint32_t)((n + 255) / 256 < 148u * 8u ? (n + 255) / 256 : 148u * 8u);
    combine_kernel<<<grid, 256, 0, s>>>(y, inv, weights, shared, T, k, H, output_scale, out, status);
    ++g_kernel_launches;
}

}  // namespace smoe
