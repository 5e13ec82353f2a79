// DSV4-exact numerical mode of the routed expert: the arithmetic of the reference's DeepSeek-V4
// kernels reproduced bit for bit, for hosts that must match a DeepSeek-V4 deployment exactly.
//
//   quantize_activation_e4m3_kernel   kernels/cuda/backend.cu:247-272  (value rule :212-225)
//   deepseek_fp4_gate_up_kernel       kernels/cuda/backend.cu:2308-2376
//   deepseek_fp4_down_kernel          kernels/cuda/backend.cu:2378-2413
//   CPU replay of all three           kernels/cpu/dsv4_fp4_expert.cpp:58-163, 774-884
//   deepseek_fp8_gate_up_kernel / deepseek_fp8_down_kernel (the shared expert: FP8 E4M3 weights, one
//   E8M0 scale per 128 x 128 block)   kernels/cuda/backend.cu:2781-2863
//
// The reference computes one output row with a 256-thread block: thread t accumulates the columns
// t, t + 256, ... in increasing order with sum = fma(x * w, scale, sum), then the block adds the 256
// partial sums in a fixed tree (five shuffle rounds per warp, then the eight warp sums).  The
// result depends on that association, so this kernel keeps it and only changes who computes it:
// ONE warp owns an output row; lane l plays the reference's threads 8l .. 8l+7 (eight
// accumulators per token), which makes every weight load a contiguous 128 bytes per warp, and
// up to four token rows of the expert share one pass over the weights.  The reduction tree is
// evaluated in the same order with two shuffle rounds, three in-register rounds and the final
// three rounds over the eight "warp" sums.
#include "common.cuh"
#include "libm_exact.cuh"

namespace smoe {

namespace {

__device__ __forceinline__ float bf16_round_dev(float v) {
    uint32_t b = __float_as_uint(v);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) b = (b | 0x00400000u) & 0xFFFF0000u;
    else b = (b + 0x7FFFu + ((b >> 16) & 1u)) & 0xFFFF0000u;
    return __uint_as_float(b);
}

__device__ __forceinline__ float quantize_e4m3_value_dev(float value) {
    const float magnitude = fminf(fabsf(value), 448.0f);
    float q;
    if (magnitude < 0.015625f) {
        q = __fmul_rn(rintf(__fmul_rn(magnitude, 512.0f)), 0.001953125f);
    } else {
        int e = (int)((__float_as_uint(magnitude) >> 23) & 0xFFu) - 127;   // frexp exponent - 1
        e = max(-6, min(8, e));
        const float step = __uint_as_float((uint32_t)(e - 3 + 127) << 23);
        q = fminf(__fmul_rn(rintf(__fdiv_rn(magnitude, step)), step), 448.0f);
    }
    return copysignf(q, value);
}

// exp2f(ceilf(log2f(maximum / 448))) as the host evaluates it.  log2 is taken in double and rounded
// to float: equal to the host's float log2f except when the true logarithm lies within a quarter
// of a float ulp of a rounding boundary next to an integer.
__device__ __forceinline__ float block_scale_dev(float maximum) {
    if (!(maximum > 0.0f)) return 1.0f;
    const float q = __fdiv_rn(maximum, 448.0f);
    const float l = __double2float_rn(log2((double)q));
    if (!(fabsf(l) <= 3.0e38f)) return l > 0.0f ? l : 0.0f;
    return ldexpf(1.0f, (int)ceilf(l));
}

__device__ __forceinline__ float e8m0_dsv4(uint32_t bits) {
    return __uint_as_float(bits == 0xFFu ? 0x7FC00000u : (bits == 0u ? 0x00400000u : bits << 23));
}

// 8 E2M1 nibbles (low nibble = even column) -> 8 floats, 0x8 -> -0.0 like the host table.
__device__ __forceinline__ void e2m1x8_f32(uint32_t w, float v[8]) {
    uint32_t h[4];
    asm("{\n .reg .b8 b0, b1, b2, b3;\n mov.b32 {b0, b1, b2, b3}, %4;\n"
        " cvt.rn.f16x2.e2m1x2 %0, b0;\n cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        " cvt.rn.f16x2.e2m1x2 %2, b2;\n cvt.rn.f16x2.e2m1x2 %3, b3;\n}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(w));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 p = *reinterpret_cast<const __half2*>(&h[i]);
        v[2 * i] = __low2float(p);
        v[2 * i + 1] = __high2float(p);
    }
}

// 8 E4M3 bytes (two 32-bit words, byte q = column q) -> 8 floats, exact; 0x7F / 0xFF -> NaN.
__device__ __forceinline__ void e4m3x8_f32(uint2 w, float v[8]) {
    const uint32_t words[2] = {w.x, w.y};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint32_t lo, hi;
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(lo) : "h"((unsigned short)(words[i] & 0xFFFFu)));
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hi) : "h"((unsigned short)(words[i] >> 16)));
        const __half2 a = *reinterpret_cast<const __half2*>(&lo), b = *reinterpret_cast<const __half2*>(&hi);
        v[4 * i] = __low2float(a);
        v[4 * i + 1] = __high2float(a);
        v[4 * i + 2] = __low2float(b);
        v[4 * i + 3] = __high2float(b);
    }
}

// The reference's block tree over the 256 partial sums, held as v[s] on lane l = thread 8l + s.
// Returns the block sum on lane 0.
__device__ __forceinline__ float block_tree(float v[8], uint32_t lane) {
    (void)lane;
#pragma unroll
    for (int s = 0; s < 8; ++s) v[s] = __fadd_rn(v[s], __shfl_down_sync(0xFFFFFFFFu, v[s], 2));  // thread + 16
#pragma unroll
    for (int s = 0; s < 8; ++s) v[s] = __fadd_rn(v[s], __shfl_down_sync(0xFFFFFFFFu, v[s], 1));  // thread + 8
#pragma unroll
    for (int s = 0; s < 4; ++s) v[s] = __fadd_rn(v[s], v[s + 4]);                               // thread + 4
    v[0] = __fadd_rn(v[0], v[2]);
    v[1] = __fadd_rn(v[1], v[3]);
    float w = __fadd_rn(v[0], v[1]);            // warp sum of reference warp l / 4, valid on lanes 0, 4, .., 28
    w = __fadd_rn(w, 0.0f);                     // the rounds that add the zeroed lanes 8..31
    w = __fadd_rn(w, __shfl_down_sync(0xFFFFFFFFu, w, 16));   // warp + 4
    w = __fadd_rn(w, __shfl_down_sync(0xFFFFFFFFu, w, 8));    // warp + 2
    w = __fadd_rn(w, __shfl_down_sync(0xFFFFFFFFu, w, 4));    // warp + 1
    return w;
}

constexpr int kRT = 4;   // token rows that share one pass over a weight row

}  // namespace

// ------------------------------------------------------------------------------ quantise
// One warp per (row, 128-column block).  dst row pos <- src row (perm ? perm[pos] / k_div : pos).
__global__ void __launch_bounds__(256) dsv4_quantize_kernel(const float* __restrict__ src,
                                                            const uint32_t* __restrict__ perm, uint32_t k_div,
                                                            uint32_t rows, uint32_t cols, float* __restrict__ dst) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t blocks = (cols + 127u) / 128u;
    const size_t task = (size_t)blockIdx.x * 8u + (threadIdx.x >> 5);
    if (task >= (size_t)rows * blocks) return;
    const uint32_t pos = (uint32_t)(task / blocks), begin = (uint32_t)(task % blocks) * 128u;
    const uint32_t srow = perm ? perm[pos] / k_div : pos;
    const float* s = src + (size_t)srow * cols + begin;
    float* d = dst + (size_t)pos * cols + begin;
    float x[4];
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t c = lane + 32u * i;
        x[i] = begin + c < cols ? s[c] : 0.0f;
        mx = fmaxf(mx, fabsf(x[i]));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    const float scale = block_scale_dev(mx);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t c = lane + 32u * i;
        if (begin + c < cols) d[c] = __fmul_rn(quantize_e4m3_value_dev(__fdiv_rn(x[i], scale)), scale);
    }
}

// ------------------------------------------------------------------------------ matvec rows
struct Dsv4Args {
    uint32_t n_groups, K, R;
    const uint32_t* offsets;
    WeightTable w0, w1;        // gate, up  (DUAL)  or  down, unused
    const float* x;            // [pairs, K] fp32, already E4M3-quantised
    const float* coef;         // [pairs] or nullptr (= 1)
    float limit;
    float* out;                // [pairs, R]
    uint32_t* status;
};

// FP8 = false: E2M1 nibbles + one E8M0 scale per 32 columns of a row.
// FP8 = true : E4M3 bytes + one E8M0 scale per 128 x 128 block (scales [ceil(R / 128), ceil(K / 128)]).
template <bool DUAL, bool FP8>
__global__ void __launch_bounds__(128) dsv4_rows_kernel(Dsv4Args a) {
    const uint32_t lane = threadIdx.x & 31u;
    const size_t total = (size_t)a.n_groups * a.R;
    const uint32_t K = a.K;
    bool bad = false;
    for (size_t task = (size_t)blockIdx.x * 4u + (threadIdx.x >> 5); task < total; task += (size_t)gridDim.x * 4u) {
        const uint32_t g = (uint32_t)(task / a.R), row = (uint32_t)(task % a.R);
        const uint32_t row0 = a.offsets[g], cnt = a.offsets[g + 1] - row0;
        if (cnt == 0u) continue;
        const size_t prow = FP8 ? (size_t)row * K : (size_t)row * (K / 2u);
        const size_t srow = FP8 ? (size_t)(row / 128u) * ((K + 127u) / 128u) : (size_t)row * (K / 32u);
        const uint8_t* p0 = a.w0.packed[g] + prow;
        const uint8_t* s0 = a.w0.scales[g] + srow;
        const uint8_t* p1 = DUAL ? a.w1.packed[g] + prow : nullptr;
        const uint8_t* s1 = DUAL ? a.w1.scales[g] + srow : nullptr;
        for (uint32_t tb = 0; tb < cnt; tb += kRT) {
            float acc0[kRT][8], acc1[DUAL ? kRT : 1][8];
#pragma unroll
            for (int r = 0; r < kRT; ++r)
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    acc0[r][s] = 0.0f;
                    if (DUAL) acc1[r][s] = 0.0f;
                }
            for (uint32_t c0 = lane * 8u; c0 < K; c0 += 256u) {
                float w0v[8], w1v[8];
                float sc0, sc1 = 0.0f;
                if (FP8) {
                    e4m3x8_f32(__ldg(reinterpret_cast<const uint2*>(p0 + c0)), w0v);
                    sc0 = e8m0_dsv4(__ldg(s0 + c0 / 128u));
                    if (DUAL) {
                        e4m3x8_f32(__ldg(reinterpret_cast<const uint2*>(p1 + c0)), w1v);
                        sc1 = e8m0_dsv4(__ldg(s1 + c0 / 128u));
                    }
                } else {
                    e2m1x8_f32(__ldg(reinterpret_cast<const uint32_t*>(p0 + c0 / 2u)), w0v);
                    sc0 = e8m0_dsv4(__ldg(s0 + c0 / 32u));
                    if (DUAL) {
                        e2m1x8_f32(__ldg(reinterpret_cast<const uint32_t*>(p1 + c0 / 2u)), w1v);
                        sc1 = e8m0_dsv4(__ldg(s1 + c0 / 32u));
                    }
                }
#pragma unroll
                for (int r = 0; r < kRT; ++r) {
                    if (tb + r >= cnt) break;
                    const float4* xp = reinterpret_cast<const float4*>(a.x + (size_t)(row0 + tb + r) * K + c0);
                    const float4 xa = __ldg(xp), xb = __ldg(xp + 1);
                    const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                    for (int s = 0; s < 8; ++s) {
                        acc0[r][s] = __fmaf_rn(__fmul_rn(xv[s], w0v[s]), sc0, acc0[r][s]);
                        if (DUAL) acc1[r][s] = __fmaf_rn(__fmul_rn(xv[s], w1v[s]), sc1, acc1[r][s]);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < kRT; ++r) {
                if (tb + r >= cnt) break;       // uniform across the warp
                const size_t pos = (size_t)row0 + tb + r;
                const float t0 = block_tree(acc0[r], lane);
                if (DUAL) {
                    const float t1 = block_tree(acc1[r], lane);
                    if (lane == 0) {
                        const float g_r = bf16_round_dev(t0), u_r = bf16_round_dev(t1);
                        if (!(fabsf(g_r) <= 3.0e38f) || !(fabsf(u_r) <= 3.0e38f)) bad = true;
                        const float lg = fminf(g_r, a.limit);
                        const float lu = fmaxf(-a.limit, fminf(u_r, a.limit));
                        const float gt = __uint_as_float(__float_as_uint(lg) & 0xFFFF0000u);  // table index = top 16 bits
                        const float silu = (fabsf(gt) <= 3.0e38f) ? __fmul_rn(gt, sigmoid_two_branch(gt)) : gt;
                        float act = __fmul_rn(silu, lu);
                        act = __fmul_rn(act, a.coef ? a.coef[pos] : 1.0f);
                        a.out[pos * a.R + row] = bf16_round_dev(act);
                    }
                } else if (lane == 0) {
                    a.out[pos * a.R + row] = bf16_round_dev(t0);
                }
            }
        }
    }
    if (bad) atomicOr(a.status, kStatusNonFiniteOutput);
}

// ------------------------------------------------------------------------------ join
// out[t] = bf16(sum_r y[inv[t * k + r]] + bf16(shared[t])): the routed rows (already BF16-rounded, route
// weight already applied) are added in selection-rank order starting from +0, the shared row is
// rounded on its own, then the total is rounded (src/models/dsv4/deepseek_runtime.cpp:5897-5914;
// device form kernels/cuda/backend.cu:2868-2880).
__global__ void __launch_bounds__(256) dsv4_join_kernel(const float* __restrict__ y, const uint32_t* __restrict__ inv,
                                                        const float* __restrict__ shared, uint32_t T, uint32_t k,
                                                        uint32_t H, float* __restrict__ out, uint32_t* status) {
    bool bad = false;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)T * H;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / H), c = (uint32_t)(i % H);
        float o = 0.0f;
        for (uint32_t r = 0; r < k; ++r) {
            const uint32_t pos = inv[(size_t)t * k + r];
            if (pos == 0xFFFFFFFFu) continue;
            o = __fadd_rn(o, bf16_round_dev(y[(size_t)pos * H + c]));
        }
        const float sh = shared ? bf16_round_dev(shared[i]) : 0.0f;
        o = bf16_round_dev(__fadd_rn(o, sh));
        bad |= !(fabsf(o) <= 3.0e38f);
        out[i] = o;
    }
    if (bad) atomicOr(status, kStatusNonFiniteOutput);
}

void launch_dsv4_join(const float* y, const uint32_t* inv, const float* shared, uint32_t T, uint32_t k, uint32_t H,
                      float* out, uint32_t* status, cudaStream_t s) {
    if (T == 0) return;
    const size_t n = (size_t)T * H;
    const unsigned grid = (unsigned)((n + 255) / 256 < (size_t)kNumSMs * 8u ? (n + 255) / 256 : (size_t)kNumSMs * 8u);
    dsv4_join_kernel<<<grid, 256, 0, s>>>(y, inv, shared, T, k, H, out, status);
    ++g_kernel_launches;
}

// ------------------------------------------------------------------------------ launchers
void launch_dsv4_quantize(const float* src, const uint32_t* perm, uint32_t k_div, uint32_t rows, uint32_t cols,
                          float* dst, cudaStream_t s) {
    if (rows == 0 || cols == 0) return;
    const size_t tasks = (size_t)rows * ((cols + 127u) / 128u);
    dsv4_quantize_kernel<<<(unsigned)((tasks + 7) / 8), 256, 0, s>>>(src, perm, k_div, rows, cols, dst);
    ++g_kernel_launches;
}

void launch_dsv4_gate_up(uint32_t n_groups, const uint32_t* offsets, uint32_t H, uint32_t I, const WeightTable& gate,
                         const WeightTable& up, const float* xq, const float* coef, float limit, float* act,
                         uint32_t* status, cudaStream_t s, bool fp8) {
    Dsv4Args a{n_groups, H, I, offsets, gate, up, xq, coef, limit, act, status};
    const size_t warps = (size_t)n_groups * I;
    const unsigned grid = (unsigned)((warps + 3) / 4 < (size_t)kNumSMs * 16u ? (warps + 3) / 4 : (size_t)kNumSMs * 16u);
    if (fp8) dsv4_rows_kernel<true, true><<<grid, 128, 0, s>>>(a);
    else dsv4_rows_kernel<true, false><<<grid, 128, 0, s>>>(a);
    ++g_kernel_launches;
}

void launch_dsv4_down(uint32_t n_groups, const uint32_t* offsets, uint32_t H, uint32_t I, const WeightTable& down,
                      const float* actq, float* y, uint32_t* status, cudaStream_t s, bool fp8) {
    Dsv4Args a{n_groups, I, H, offsets, down, down, actq, nullptr, 0.0f, y, status};
    const size_t warps = (size_t)n_groups * H;
    const unsigned grid = (unsigned)((warps + 3) / 4 < (size_t)kNumSMs * 16u ? (warps + 3) / 4 : (size_t)kNumSMs * 16u);
    if (fp8) dsv4_rows_kernel<false, true><<<grid, 128, 0, s>>>(a);
    else dsv4_rows_kernel<false, false><<<grid, 128, 0, s>>>(a);
    ++g_kernel_launches;
}

}  // namespace smoe
