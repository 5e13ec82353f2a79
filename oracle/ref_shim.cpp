// extern "C" doorway onto the reference's own CPU code.  TEST INFRASTRUCTURE ONLY.
//
// oracle/build.py compiles this file together with the reference's unmodified
// sources (read in place from the reference checkout, never copied) into
// oracle/_ref/libstrata_ref.so.  It is used to validate oracle/moe_oracle.c
// and as the timed CPU arm of bench.py; the shipped CUDA library never loads it.
//
// Every wrapper only marshals pointers into the std::span / view types the
// reference function takes and returns 0 on ok(), 1 otherwise.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <span>
#include <vector>

#include "strata/compressed_tensors.hpp"
#include "strata/deepseek_host_expert.hpp"
#include "strata/deepseek_ops.hpp"
#include "strata/glm_int4.hpp"
#include "strata/glm_ops.hpp"
#include "strata/kimi_k3_layer.hpp"
#include "strata/kimi_k3_ops.hpp"
#include "strata/laguna_ops.hpp"
#include "strata/model.hpp"
#include "strata/numerics.hpp"
#include "strata/worker_pool.hpp"

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {
std::span<const std::byte> bytes(const void* p, std::size_t n) {
    return {static_cast<const std::byte*>(p), n};
}
}  // namespace

// ---- scalar decoders (src/platform/numerics.cpp, compressed_tensors.cpp) ----
REF_API float ref_fp4_e2m1(uint8_t nibble) { return strata::fp4_e2m1_f32(nibble); }
REF_API float ref_fp8_e4m3(uint8_t byte) { return strata::fp8_e4m3_f32(byte); }
REF_API float ref_mxfp4_scale(uint8_t byte) { return strata::mxfp4_scale_from_e8m0(byte); }
REF_API float ref_sigmoid(float v) { return strata::sigmoid_f32(v); }
REF_API float ref_silu(float v) { return strata::silu_f32(v); }
REF_API float ref_dsv4_e8m0(uint8_t byte) { return strata::dsv4_fp8_e8m0_scale_f32(byte); }

// ---- routers ----------------------------------------------------------------
// glm_route_logits_noaux_tc, src/models/glm52/glm_ops.cpp:176-233
REF_API int ref_glm_route(const float* logits, const float* bias, uint32_t experts, uint32_t k,
                          float routed_scale, uint32_t* ids, float* weights) {
    strata::RouterSpec spec;
    spec.selection = strata::RouterSelectionKind::NoAuxTc;
    spec.scoring = strata::RouterScoreKind::Sigmoid;
    spec.routed_experts = experts;
    spec.experts_per_token = k;
    spec.normalize_topk = true;
    spec.selection_bias = true;
    spec.routed_scale = routed_scale;
    auto r = strata::glm_route_logits_noaux_tc({logits, experts}, {bias, experts}, spec);
    if (!r.ok()) return 1;
    std::copy(r.value.experts.begin(), r.value.experts.end(), ids);
    std::copy(r.value.weights.begin(), r.value.weights.end(), weights);
    return 0;
}

// laguna_route_sigmoid_topk, src/models/laguna/laguna_ops.cpp:182-243
REF_API int ref_laguna_route(const float* logits, const float* bias, uint32_t experts, uint32_t k,
                             int normalize, float softcap, uint32_t* ids, float* weights) {
    strata::RouterSpec spec;
    spec.selection = strata::RouterSelectionKind::TopK;
    spec.scoring = strata::RouterScoreKind::Sigmoid;
    spec.routed_experts = experts;
    spec.experts_per_token = k;
    spec.normalize_topk = normalize != 0;
    spec.selection_bias = true;
    auto r = strata::laguna_route_sigmoid_topk({logits, experts}, {bias, experts}, spec, softcap);
    if (!r.ok()) return 1;
    std::copy(r.value.experts.begin(), r.value.experts.end(), ids);
    std::copy(r.value.weights.begin(), r.value.weights.end(), weights);
    return 0;
}

// kimi_route_topk, src/models/kimi_k3/kimi_k3_ops.cpp:192-237
REF_API int ref_kimi_route(const float* logits, const float* bias, uint32_t experts, uint32_t k,
                           float routed_scale, uint32_t* ids, float* weights) {
    std::vector<strata::KimiRoutedExpert> sel(k);
    auto r = strata::kimi_route_topk(sel, {logits, experts}, {bias, experts}, routed_scale);
    if (!r.ok()) return 1;
    for (uint32_t i = 0; i < k; ++i) {
        ids[i] = sel[i].expert;
        weights[i] = sel[i].weight;
    }
    return 0;
}

// dsv4_route_sqrtsoftplus_f32, src/models/dsv4/deepseek_ops.cpp:356-388
REF_API int ref_dsv4_route(const float* logits, const float* bias, uint32_t experts, uint32_t k,
                           float routed_scale, uint32_t* ids, float* weights) {
    strata::RouterSpec spec;
    spec.selection = strata::RouterSelectionKind::NoAuxTc;
    spec.scoring = strata::RouterScoreKind::SqrtSoftplus;
    spec.routed_experts = experts;
    spec.experts_per_token = k;
    spec.normalize_topk = true;
    spec.selection_bias = true;
    spec.routed_scale = routed_scale;
    auto r = strata::dsv4_route_sqrtsoftplus_f32({logits, experts}, {bias, experts}, spec);
    if (!r.ok()) return 1;
    std::copy(r.value.experts.begin(), r.value.experts.end(), ids);
    std::copy(r.value.weights.begin(), r.value.weights.end(), weights);
    return 0;
}

// dsv4_route_hash_sqrtsoftplus_f32_into, src/models/dsv4/deepseek_ops.cpp:414-461.
REF_API int ref_dsv4_route_hash(const float* logits, const uint32_t* token_experts, uint32_t experts, uint32_t k,
                                float routed_scale, uint32_t* ids, float* weights) {
    strata::RouterSpec spec;
    spec.selection = strata::RouterSelectionKind::NoAuxTc;
    spec.scoring = strata::RouterScoreKind::SqrtSoftplus;
    spec.routed_experts = experts;
    spec.experts_per_token = k;
    spec.normalize_topk = true;
    spec.selection_bias = true;
    spec.routed_scale = routed_scale;
    return strata::dsv4_route_hash_sqrtsoftplus_f32_into({logits, experts}, {token_experts, k}, spec, {ids, k},
                                                          {weights, k})
                   .ok()
               ? 0
               : 1;
}

// ---- quantized matvecs --------------------------------------------------------
// kimi_mxfp4_matvec, src/models/kimi_k3/kimi_k3_layer.cpp:237-301 (AVX2 when the CPU has it)
REF_API int ref_kimi_mxfp4_matvec(float* out, const float* in, const uint8_t* packed,
                                  const uint8_t* scales, uint32_t rows, uint32_t cols) {
    strata::KimiExpertModuleView m;
    m.packed = {packed, static_cast<std::size_t>(rows) * (cols / 2U)};
    m.scales = {scales, static_cast<std::size_t>(rows) * (cols / 32U)};
    m.rows = rows;
    m.columns = cols;
    return strata::kimi_mxfp4_matvec({out, rows}, {in, cols}, m, nullptr).ok() ? 0 : 1;
}

// dsv4_fp4_e2m1_matvec_f32, src/models/dsv4/deepseek_ops.cpp:488-521 (double accumulate)
REF_API int ref_dsv4_fp4_matvec(float* out, const float* in, const uint8_t* packed,
                                const uint8_t* scales, uint32_t rows, uint32_t cols) {
    return strata::dsv4_fp4_e2m1_matvec_f32(
               {out, rows}, {in, cols}, bytes(packed, static_cast<std::size_t>(rows) * cols / 2U),
               bytes(scales, static_cast<std::size_t>(rows) * cols / 32U), rows, cols)
                   .ok()
               ? 0
               : 1;
}

// laguna_nvfp4_matvec_rows, src/models/laguna/laguna_ops.cpp:41-94
REF_API int ref_laguna_nvfp4_matvec(float* out, const float* in, const uint8_t* packed,
                                    const uint8_t* scales, float global_scale, uint32_t rows,
                                    uint32_t cols, uint32_t row_begin, uint32_t row_end) {
    strata::LagunaNvfp4MatrixView m;
    m.packed = bytes(packed, static_cast<std::size_t>(rows) * (cols / 2U));
    m.scales = bytes(scales, static_cast<std::size_t>(rows) * (cols / 16U));
    m.global_scale = global_scale;
    m.rows = rows;
    m.columns = cols;
    m.packed_columns = cols / 2U;
    m.scale_columns = cols / 16U;
    m.group_size = 16U;
    return strata::laguna_nvfp4_matvec_rows(m, {in, cols}, {out, rows}, row_begin, row_end).ok() ? 0
                                                                                                 : 1;
}

namespace {
strata::GlmInt4MatrixView int4_view(const uint8_t* packed, const uint8_t* scales, uint32_t rows,
                                    uint32_t cols) {
    strata::GlmInt4MatrixView m;
    m.packed = bytes(packed, static_cast<std::size_t>(rows) * (cols / 8U) * 4U);
    m.scales = bytes(scales, static_cast<std::size_t>(rows) * (cols / 128U) * 2U);
    m.rows = rows;
    m.columns = cols;
    m.packed_columns = cols / 8U;
    m.scale_columns = cols / 128U;
    m.group_size = 128U;
    return m;
}
}  // namespace

// glm_int4_group128_matvec_reference, kernels/cpu/glm_int4.cpp:140-160 (scalar)
REF_API int ref_glm_int4_matvec_scalar(float* out, const float* in, const uint8_t* packed,
                                       const uint8_t* scales, uint32_t rows, uint32_t cols) {
    return strata::glm_int4_group128_matvec_reference(int4_view(packed, scales, rows, cols),
                                                      {in, cols}, {out, rows})
                   .ok()
               ? 0
               : 1;
}

// glm_int4_group128_matvec_rows, kernels/cpu/glm_int4.cpp:176-206 (AVX2/FMA when available)
REF_API int ref_glm_int4_matvec_rows(float* out, const float* in, const uint8_t* packed,
                                     const uint8_t* scales, uint32_t rows, uint32_t cols,
                                     uint32_t row_begin, uint32_t row_end) {
    return strata::glm_int4_group128_matvec_rows(int4_view(packed, scales, rows, cols), {in, cols},
                                                 {out, rows}, row_begin, row_end)
                   .ok()
               ? 0
               : 1;
}

// dsv4_host_expert_fp4, kernels/cpu/dsv4_fp4_expert.cpp:864-884: the bit-exact DSV4 expert
// (E4M3 activation quantisation, BF16 rounding points, clamp, table SiLU).
REF_API int ref_dsv4_host_expert(float* out, const float* in, const uint8_t* w1, const uint8_t* s1,
                                 const uint8_t* w3, const uint8_t* s3, const uint8_t* w2,
                                 const uint8_t* s2, uint32_t hidden, uint32_t intermediate,
                                 float coefficient, float swiglu_limit, int use_avx2) {
    strata::Dsv4HostExpertWeights w;
    const std::size_t up = static_cast<std::size_t>(intermediate) * hidden;
    w.w1_packed = bytes(w1, up / 2U);
    w.w1_scales = bytes(s1, up / 32U);
    w.w3_packed = bytes(w3, up / 2U);
    w.w3_scales = bytes(s3, up / 32U);
    w.w2_packed = bytes(w2, up / 2U);
    w.w2_scales = bytes(s2, up / 32U);
    std::vector<float> scratch(intermediate);
    return strata::dsv4_host_expert_fp4({out, hidden}, {in, hidden}, w, scratch, hidden,
                                        intermediate, coefficient, swiglu_limit, use_avx2 != 0)
                   .ok()
               ? 0
               : 1;
}

// dsv4_host_expert_quantize, kernels/cpu/dsv4_fp4_expert.cpp:826-836 (in place, one row).
REF_API int ref_dsv4_quantize(float* values, uint32_t columns) {
    return strata::dsv4_host_expert_quantize({values, columns}, columns).ok() ? 0 : 1;
}

// kimi_situ_glu, src/models/kimi_k3/kimi_k3_ops.cpp:39-62.
REF_API int ref_kimi_situ_glu(float* out, const float* gate, const float* up, uint32_t n, float gate_beta,
                              float linear_beta) {
    return strata::kimi_situ_glu({out, n}, {gate, n}, {up, n}, gate_beta, linear_beta).ok() ? 0 : 1;
}

// ---- timed CPU arm ------------------------------------------------------------------
// One MoE layer's routed experts on the host cores through the reference's own matvec
// kernels, scheduled the way the reference schedules its host experts: one parallel region
// per MoE block with one task per (expert, row block), tasks stolen freely
// (src/models/kimi_k3/kimi_k3_layer.cpp:876-953, src/models/glm52/glm_runtime.cpp:1247-1288).
// fmt: 0 MXFP4 (kimi_mxfp4_matvec), 1 NVFP4 (laguna_nvfp4_matvec_rows, scalar -- the
// reference has no vectorised NVFP4 host kernel), 2 INT4 (glm_int4_group128_matvec_rows).
// Pairs are laid out expert-major: expert e owns pair positions [offsets[e], offsets[e+1]),
// pair_token[pos] is the token row.  y receives [pairs, H] un-combined rows.  Returns the
// elapsed nanoseconds of the parallel region, or -1 on error.
struct RefExpertPtrs {
    const uint8_t* gate_packed;
    const uint8_t* gate_scales;
    const uint8_t* up_packed;
    const uint8_t* up_scales;
    const uint8_t* down_packed;
    const uint8_t* down_scales;
    float gate_global, up_global, down_global;
};

namespace {
int one_matvec(int fmt, float* out, const float* in, const uint8_t* packed, const uint8_t* scales,
               float global, uint32_t rows, uint32_t cols) {
    if (fmt == 0) return ref_kimi_mxfp4_matvec(out, in, packed, scales, rows, cols);
    if (fmt == 1) return ref_laguna_nvfp4_matvec(out, in, packed, scales, global, rows, cols, 0, rows);
    if (fmt == 2) return ref_glm_int4_matvec_rows(out, in, packed, scales, rows, cols, 0, rows);
    return 1;
}
}  // namespace

REF_API int64_t ref_cpu_experts(int fmt, uint32_t hidden, uint32_t intermediate, uint32_t experts,
                                const RefExpertPtrs* weights, const float* x /*[T,H] fp32*/,
                                const uint32_t* offsets, const uint32_t* pair_token,
                                float* y /*[pairs,H]*/, uint32_t threads) {
    strata::HostWorkerPool pool(static_cast<std::size_t>(threads));
    std::vector<uint32_t> task_pos;
    std::vector<uint32_t> task_expert;
    for (uint32_t e = 0; e < experts; ++e) {
        for (uint32_t pos = offsets[e]; pos < offsets[e + 1]; ++pos) {
            task_pos.push_back(pos);
            task_expert.push_back(e);
        }
    }
    std::atomic<int> failed{0};
    const auto started = std::chrono::steady_clock::now();
    auto status = pool.parallel_for(task_pos.size(), [&](std::size_t task) {
        const uint32_t pos = task_pos[task];
        const auto& w = weights[task_expert[task]];
        const float* in = x + static_cast<std::size_t>(pair_token[pos]) * hidden;
        std::vector<float> gate(intermediate), up(intermediate);
        int rc = one_matvec(fmt, gate.data(), in, w.gate_packed, w.gate_scales, w.gate_global,
                            intermediate, hidden);
        rc |= one_matvec(fmt, up.data(), in, w.up_packed, w.up_scales, w.up_global, intermediate,
                         hidden);
        for (uint32_t i = 0; i < intermediate; ++i) gate[i] = strata::silu_f32(gate[i]) * up[i];
        rc |= one_matvec(fmt, y + static_cast<std::size_t>(pos) * hidden, gate.data(), w.down_packed,
                         w.down_scales, w.down_global, hidden, intermediate);
        if (rc != 0) failed.store(1);
    });
    const auto elapsed = std::chrono::duration_cast<std::chrono::nanoseconds>(
                             std::chrono::steady_clock::now() - started)
                             .count();
    if (!status.ok() || failed.load() != 0) return -1;
    return static_cast<int64_t>(elapsed);
}
