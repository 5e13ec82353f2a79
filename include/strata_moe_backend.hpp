// Header-only C++ shim over the C ABI with the call shapes of the reference backend's MoE
// commands, so that a model runtime written against
//   CudaBackend::enqueue_moe / collect_moe   (include/strata/cuda_backend.hpp:1147-1153)
// can be pointed at this library.  Errors follow the reference's convention: no exceptions, a
// result object whose `ok()` is true when `errors` is empty (include/strata/result.hpp:8-12).
#pragma once
#include <cstdint>
#include <span>
#include <string>
#include <vector>

#include "strata_moe.h"

namespace strata_b200 {

struct ValidationResult {
    std::vector<std::string> errors;
    [[nodiscard]] bool ok() const noexcept { return errors.empty(); }
};

// One routed expert of a dense command (ref: struct CudaMoeExpert, cuda_backend.hpp:740-745).
struct MoeExpert {
    std::uint32_t expert{};   // global expert index registered with strata_moe_set_expert
    float coefficient{1.0F};  // folded before the down projection for INT4, must be 1 otherwise
};

class MoeBackend {
public:
    MoeBackend() = default;
    MoeBackend(const MoeBackend&) = delete;
    MoeBackend& operator=(const MoeBackend&) = delete;
    ~MoeBackend() {
        if (layer_ != nullptr) strata_moe_layer_destroy(layer_);
        if (ctx_ != nullptr) strata_moe_destroy(ctx_);
    }

    // ref: CudaBackend::initialize (cuda_backend.hpp:787)
    [[nodiscard]] ValidationResult initialize(int device, const strata_moe_layer_desc& desc) {
        if (const int rc = strata_moe_create(device, nullptr, &ctx_); rc != 0)
            return {{"strata_moe_create failed: no usable sm_100 device (code " + std::to_string(rc) + ")"}};
        return check(strata_moe_layer_create(ctx_, &desc, &layer_));
    }
    // ref: CudaBackend::upload (cuda_backend.hpp:819-823)
    [[nodiscard]] ValidationResult upload_expert(std::uint32_t expert, int role,
                                                 std::span<const std::byte> weights,
                                                 std::span<const std::byte> scales, float global_scale) {
        return check(strata_moe_set_expert(layer_, expert, role, weights.data(), scales.data(), global_scale,
                                           STRATA_MOE_SRC_HOST));
    }
    [[nodiscard]] ValidationResult upload_router(std::span<const std::byte> gate_bf16, const float* bias) {
        return check(strata_moe_set_router(layer_, gate_bf16.data(), bias, STRATA_MOE_SRC_HOST));
    }
    [[nodiscard]] ValidationResult upload_shared(int role, std::span<const std::byte> weights_bf16) {
        return check(strata_moe_set_shared(layer_, role, weights_bf16.data(), STRATA_MOE_SRC_HOST));
    }

    // ref: CudaBackend::enqueue_moe(device, hidden, rows, routed, shared) (cuda_backend.hpp:1147-1150)
    [[nodiscard]] ValidationResult enqueue_moe(std::span<const float> hidden, std::uint32_t rows,
                                               std::span<const MoeExpert> routed, bool with_shared) {
        std::vector<std::uint32_t> ids(routed.size());
        std::vector<float> coefficients(routed.size());
        for (std::size_t i = 0; i < routed.size(); ++i) {
            ids[i] = routed[i].expert;
            coefficients[i] = routed[i].coefficient;
        }
        return check(strata_moe_enqueue_dense(layer_, hidden.data(), rows, ids.data(), coefficients.data(),
                                              static_cast<std::uint32_t>(routed.size()), with_shared ? 1 : 0));
    }
    // ref: CudaBackend::collect_moe(device, routed_output, shared_output) (cuda_backend.hpp:1151-1153)
    [[nodiscard]] ValidationResult collect_moe(std::span<float> routed_output, std::span<float> shared_output) {
        return check(strata_moe_collect_dense(layer_, routed_output.empty() ? nullptr : routed_output.data(),
                                              shared_output.empty() ? nullptr : shared_output.data()));
    }
    // Whole layer on host buffers: what sparse_mlp() computes around the command in the reference
    // (src/models/glm52/glm_runtime.cpp:1487-1618).
    [[nodiscard]] ValidationResult forward(std::span<const std::uint16_t> x_bf16, std::uint32_t tokens,
                                           std::span<float> out) {
        return check(strata_moe_forward_host(layer_, x_bf16.data(), tokens, out.data()));
    }

    [[nodiscard]] strata_moe_ctx* context() const noexcept { return ctx_; }
    [[nodiscard]] strata_moe_layer* layer() const noexcept { return layer_; }

private:
    [[nodiscard]] ValidationResult check(int rc) const {
        if (rc == 0) return {};
        return {{std::string(strata_moe_last_error(ctx_))}};
    }
    strata_moe_ctx* ctx_{nullptr};
    strata_moe_layer* layer_{nullptr};
};

}  // namespace strata_b200
