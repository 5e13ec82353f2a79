// Small row kernels of the LatentMoE wrapper (Kimi-K3): the routed experts run on a latent that
// is a BF16 projection of the hidden state; their weighted mixture is RMS-normalised in the latent
// space and projected back (ref: kimi_latent_moe_layer, src/models/kimi_k3/kimi_k3_layer.cpp:781-1001;
// kimi_rms_norm, src/models/kimi_k3/kimi_k3_ops.cpp:16-38).  The two projections themselves run on
// the tensor cores (launch_router_tc: the same single-GEMM mode the fast router uses).
#include "common.cuh"

namespace smoe {

__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* __restrict__ src, size_t n4,
                                                          __nv_bfloat16* __restrict__ dst) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(src) + i);
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&a);
        o.y = *reinterpret_cast<uint32_t*>(&b);
        reinterpret_cast<uint2*>(dst)[i] = o;
    }
}

// One warp per row: scale = 1 / sqrt(mean(x^2) + eps), y = weight * (x * scale), rounded to BF16 for the
// projection that follows.  A non-finite row raises the status word.
__global__ void __launch_bounds__(256) rmsnorm_bf16_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                                           uint32_t rows, uint32_t cols, float eps,
                                                           __nv_bfloat16* __restrict__ y, uint32_t* status) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* xr = x + (size_t)row * cols;
    float sum = 0.0f;
    for (uint32_t c = lane; c < cols; c += 32u) {
        const float v = xr[c];
        sum = fmaf(v, v, sum);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    const float scale = 1.0f / sqrtf(sum / (float)cols + eps);
    if (!(fabsf(scale) <= 3.0e38f) && lane == 0) atomicOr(status, kStatusNonFiniteOutput);
    for (uint32_t c = lane; c < cols; c += 32u)
        y[(size_t)row * cols + c] = __float2bfloat16_rn(weight[c] * (xr[c] * scale));
}

__global__ void __launch_bounds__(256) add_rows_kernel(float* __restrict__ out, const float* __restrict__ a, size_t n4) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 o = reinterpret_cast<float4*>(out)[i];
        const float4 v = __ldg(reinterpret_cast<const float4*>(a) + i);
        o.x += v.x; o.y += v.y; o.z += v.z; o.w += v.w;
        reinterpret_cast<float4*>(out)[i] = o;
    }
}

static unsigned grid_for(size_t n) {
    const size_t g = (n + 255) / 256;
    return (unsigned)(g < (size_t)kNumSMs * 8u ? (g ? g : 1) : (size_t)kNumSMs * 8u);
}

void launch_f32_to_bf16(const float* src, size_t n, __nv_bfloat16* dst, cudaStream_t s) {   // n % 4 == 0
    if (n == 0) return;
    f32_to_bf16_kernel<<<grid_for(n / 4), 256, 0, s>>>(src, n / 4, dst);
    ++g_kernel_launches;
}

void launch_rmsnorm_bf16(const float* x, const float* weight, uint32_t rows, uint32_t cols, float eps,
                         __nv_bfloat16* y, uint32_t* status, cudaStream_t s) {
    if (rows == 0) return;
    rmsnorm_bf16_kernel<<<(rows + 7) / 8, 256, 0, s>>>(x, weight, rows, cols, eps, y, status);
    ++g_kernel_launches;
}

void launch_add_rows(float* out, const float* a, size_t n, cudaStream_t s) {   // n % 4 == 0
    if (n == 0) return;
    add_rows_kernel<<<grid_for(n / 4), 256, 0, s>>>(out, a, n / 4);
    ++g_kernel_launches;
}

}  // namespace smoe
