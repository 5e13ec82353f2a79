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
#include "strata/diagnostics.hpp"
#include "strata/glm_int4.hpp"
#include "strata/glm_ops.hpp"
#include "strata/inkling_ops.hpp"
#include "strata/kimi_k3_layer.hpp"
#include "strata/kimi_k3_ops.hpp"
#include "strata/laguna_ops.hpp"
#include "strata/model.hpp"
#include "strata/numerics.hpp"
#include "strata/trace.hpp"
#include "strata/worker_pool.hpp"

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {
std::span<const std::byte> bytes(const void* p, std::size_t n) {
    return {static_cast<const std::byte*>(p), n};
}
std::span<const std::byte> bytes_of(const void* p, std::size_t n) { return bytes(p, n); }
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

// stable_bf16_hash, src/platform/diagnostics.cpp:84-88
REF_API uint64_t ref_stable_bf16_hash(const float* values, size_t n) { return strata::stable_bf16_hash({values, n}); }

// inkling_route_sigmoid_sink, src/models/inkling/inkling_ops.cpp:184-275
REF_API int ref_inkling_route_sink(const float* logits, const float* bias, uint32_t experts, uint32_t sinks, uint32_t k,
                                   float routed_scale, float global_scale, uint32_t* ids, float* weights) {
    strata::RouterSpec spec;
    spec.selection = strata::RouterSelectionKind::TopK;
    spec.scoring = strata::RouterScoreKind::Sigmoid;
    spec.routed_experts = experts;
    spec.experts_per_token = k;
    spec.normalize_topk = true;
    spec.selection_bias = true;
    spec.routed_scale = routed_scale;
    auto r = strata::inkling_route_sigmoid_sink({logits, (size_t)experts + sinks}, {bias, experts}, spec, sinks, global_scale);
    if (!r.ok()) return 1;
    std::copy(r.value.experts.begin(), r.value.experts.end(), ids);
    std::copy(r.value.weights.begin(), r.value.weights.end(), weights);
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

// inkling_nvfp4_matvec_rows, src/models/inkling/inkling_ops.cpp:16-69 (block scale = e4m3 * global: the
// multiply convention of ModelOpt checkpoints, where Laguna's compressed-tensors form divides)
REF_API int ref_inkling_nvfp4_matvec(float* out, const float* in, const uint8_t* packed,
                                     const uint8_t* scales, float global_scale, uint32_t rows, uint32_t cols) {
    strata::InklingNvfp4MatrixView m;
    m.packed = bytes(packed, static_cast<std::size_t>(rows) * (cols / 2U));
    m.scales = bytes(scales, static_cast<std::size_t>(rows) * (cols / 16U));
    m.global_scale = global_scale;
    m.rows = rows;
    m.columns = cols;
    m.packed_columns = cols / 2U;
    m.scale_columns = cols / 16U;
    m.group_size = 16U;
    return strata::inkling_nvfp4_matvec_rows(m, {in, cols}, {out, rows}, 0U, rows).ok() ? 0 : 1;
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

// ---- the whole LatentMoE block ------------------------------------------------------------
// kimi_latent_moe_layer, src/models/kimi_k3/kimi_k3_layer.cpp:781-1001, at the shape its contract
// fixes (hidden 7168, latent 3584, 896 experts of width 3072, top-16, two shared experts).
// expert_ptrs[e * 6 + {0..5}] = gate packed, gate scales, up packed, up scales, down packed, down
// scales of expert e (null for experts no token routes to).  selection receives the routed experts
// and weights of every token ([tokens, 16]) as the reference computed them.
namespace {
struct PointerExpertSource final : strata::KimiExpertSource {
    const uint8_t* const* ptrs{};
    strata::ValidationResult prepare(std::uint32_t, std::span<const std::uint32_t>) override { return {}; }
    strata::ValidationResult fetch(std::uint32_t, std::uint32_t expert, strata::KimiExpertWeights& w) override {
        const auto& c = strata::kKimiK3ExecutionContract;
        const uint8_t* const* e = ptrs + static_cast<std::size_t>(expert) * 6U;
        strata::ValidationResult result;
        if (e[0] == nullptr) {
            result.errors.emplace_back("expert was not provided to the fixture");
            return result;
        }
        const auto view = [](const uint8_t* p, const uint8_t* s, std::uint32_t rows, std::uint32_t cols) {
            strata::KimiExpertModuleView v;
            v.packed = {p, static_cast<std::size_t>(rows) * cols / 2U};
            v.scales = {s, static_cast<std::size_t>(rows) * cols / 32U};
            v.rows = rows;
            v.columns = cols;
            return v;
        };
        w.gate = view(e[0], e[1], c.expert_intermediate_size, c.routed_expert_hidden_size);
        w.up = view(e[2], e[3], c.expert_intermediate_size, c.routed_expert_hidden_size);
        w.down = view(e[4], e[5], c.routed_expert_hidden_size, c.expert_intermediate_size);
        return result;
    }
};
}  // namespace

REF_API int ref_kimi_latent_moe(float* out, const float* in, uint32_t tokens, const uint16_t* router,
                                const float* router_bias, const uint16_t* latent_down, const uint16_t* latent_up,
                                const float* latent_norm, const uint16_t* shared_gate, const uint16_t* shared_up,
                                const uint16_t* shared_down, const uint8_t* const* expert_ptrs, uint32_t* ids,
                                float* weights) {
    const auto& c = strata::kKimiK3ExecutionContract;
    const std::size_t H = c.hidden_size, HL = c.routed_expert_hidden_size;
    const std::size_t Is = static_cast<std::size_t>(c.expert_intermediate_size) * c.shared_experts;
    strata::KimiMoeWeights w;
    w.router = {{router, static_cast<std::size_t>(c.routed_experts) * H}, c.routed_experts, c.hidden_size};
    w.router_bias = {router_bias, c.routed_experts};
    w.latent_down = {{latent_down, HL * H}, c.routed_expert_hidden_size, c.hidden_size};
    w.latent_up = {{latent_up, H * HL}, c.hidden_size, c.routed_expert_hidden_size};
    w.latent_norm = {latent_norm, HL};
    w.shared_gate = {{shared_gate, Is * H}, static_cast<std::uint32_t>(Is), c.hidden_size};
    w.shared_up = {{shared_up, Is * H}, static_cast<std::uint32_t>(Is), c.hidden_size};
    w.shared_down = {{shared_down, H * Is}, c.hidden_size, static_cast<std::uint32_t>(Is)};
    PointerExpertSource source;
    source.ptrs = expert_ptrs;
    strata::KimiLayerScratch scratch;
    const auto r = strata::kimi_latent_moe_layer({out, tokens * H}, {in, tokens * H}, w, source, 1U, tokens, scratch,
                                                 nullptr);
    if (ids != nullptr && weights != nullptr && scratch.selection.size() == static_cast<std::size_t>(tokens) * c.experts_per_token)
        for (std::size_t i = 0; i < scratch.selection.size(); ++i) {
            ids[i] = scratch.selection[i].expert;
            weights[i] = scratch.selection[i].weight;
        }
    return r.ok() ? 0 : 1;
}


// ---- host decode layout and route traces (checkers of include/strata_moe_loader.hpp) --------
// dsv4_transform_tiled_expert_shard, kernels/cpu/dsv4_fp4_expert.cpp:360-434.  Returns the shard's byte count
// (0 on error); destination may be null to ask for the size only.
REF_API uint64_t ref_dsv4_tile_shard(uint8_t* destination, const uint8_t* w1, const uint8_t* s1, const uint8_t* w3,
                                     const uint8_t* s3, const uint8_t* w2, const uint8_t* s2, uint64_t hidden,
                                     uint64_t intermediate, uint64_t shard, uint64_t shards) {
    const auto bytes = strata::dsv4_tiled_expert_shard_bytes(hidden, intermediate, shards);
    if (bytes == 0U || destination == nullptr) return bytes;
    strata::Dsv4HostExpertWeights canonical;
    canonical.w1_packed = bytes_of(w1, intermediate * (hidden / 2U));
    canonical.w1_scales = bytes_of(s1, intermediate * (hidden / 32U));
    canonical.w3_packed = bytes_of(w3, intermediate * (hidden / 2U));
    canonical.w3_scales = bytes_of(s3, intermediate * (hidden / 32U));
    canonical.w2_packed = bytes_of(w2, hidden * (intermediate / 2U));
    canonical.w2_scales = bytes_of(s2, hidden * (intermediate / 32U));
    const auto r = strata::dsv4_transform_tiled_expert_shard({reinterpret_cast<std::byte*>(destination), bytes}, canonical,
                                                             hidden, intermediate, shard, shards);
    return r.ok() ? bytes : 0U;
}

// parse_route_trace, src/platform/trace.cpp.  Fills up to `capacity` events (request, position, layer, phase,
// expert count) and the flattened experts / coefficients; returns the event count or -1 on a parse error.
REF_API int64_t ref_parse_route_trace(const char* path, uint64_t* header5, uint32_t* experts, float* coefficients,
                                      uint64_t capacity_events, uint64_t capacity_values) {
    const auto parsed = strata::parse_route_trace(path);
    if (!parsed.ok()) return -1;
    uint64_t values = 0;
    for (std::size_t i = 0; i < parsed.events.size() && i < capacity_events; ++i) {
        const auto& e = parsed.events[i];
        header5[i * 5 + 0] = e.request;
        header5[i * 5 + 1] = e.token_position;
        header5[i * 5 + 2] = e.layer;
        header5[i * 5 + 3] = static_cast<uint64_t>(e.phase);
        header5[i * 5 + 4] = e.experts.size() | (static_cast<uint64_t>(e.coefficients.size()) << 32);
        for (std::size_t j = 0; j < e.experts.size() && values < capacity_values; ++j, ++values) {
            experts[values] = e.experts[j];
            coefficients[values] = j < e.coefficients.size() ? e.coefficients[j] : 0.0F;
        }
    }
    return static_cast<int64_t>(parsed.events.size());
}
