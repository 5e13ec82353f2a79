// Header-only C++20 shim over the C ABI (strata_moe.h) with the MoE-command surface of the
// reference backend, signature for signature, so that a model runtime written against
//
//   strata::CudaBackend::upload / enqueue_moe / collect_moe / enqueue_deepseek_moe /
//   collect_deepseek_moe / enqueue_deepseek_moe_rows / collect_deepseek_moe_rows / synchronize
//   (include/strata/cuda_backend.hpp:819-823, 1059-1062, 1123-1125, 1139-1153)
//
// compiles against this library by switching the namespace (namespace strata = strata_b200;).
// Types keep the reference's names and fields: CudaWeightEncoding / CudaWeightDescriptor (:18-51),
// CudaWeight (move-only handle), CudaMoeExpert (:740-745), CudaDeepSeekMoeExpert,
// CudaDeepSeekMoeRowGroup (:724-736, canonical w1/w3/w2 form), ValidationResult
// (include/strata/result.hpp:8-12: no exceptions, ok() <=> no errors).
//
// Protocol kept from the reference: one MoE command in flight per device; upload and synchronize
// are rejected meanwhile; every collect consumes or drains its command; caller spans are written
// only after completion and a clean device status are confirmed.
#pragma once
#include <array>
#include <cstddef>
#include <cstdint>
#include <map>
#include <span>
#include <string>
#include <utility>
#include <vector>

#include "strata_moe.h"

namespace strata_b200 {

struct ValidationResult {
    std::vector<std::string> errors;
    [[nodiscard]] bool ok() const noexcept { return errors.empty(); }
};

enum class SafetensorsDtype : std::uint8_t { Other, Bf16, F32, I32, I8, U8, F8E4M3, F8E8M0 };

enum class CudaWeightEncoding : std::uint8_t {
    Plain,
    OffsetPackedInt4,
    OffsetPackedInt8,   // not an expert format of this library: upload rejects it
    Fp8E4m3Block128,
    Fp4E2m1Group32,
    Nvfp4Group16,
    Fp4E2m1Tiled32,     // host decode layout: not accepted on the device path of this library
};

struct CudaWeightDescriptor {
    CudaWeightEncoding encoding{CudaWeightEncoding::Plain};
    SafetensorsDtype dtype{SafetensorsDtype::Other};
    std::uint64_t rows{};
    std::uint64_t columns{};
    std::uint64_t packed_columns{};
    std::uint64_t scale_columns{};
    std::uint32_t group_size{};
    float global_scale{1.0F};
};

class CudaBackend;

// Move-only handle over one uploaded matrix (ref: class CudaWeight, shared_ptr<Impl> in the reference).
class CudaWeight {
public:
    CudaWeight() = default;
    CudaWeight(const CudaWeight&) = delete;
    CudaWeight& operator=(const CudaWeight&) = delete;
    CudaWeight(CudaWeight&& other) noexcept { swap(other); }
    CudaWeight& operator=(CudaWeight&& other) noexcept {
        if (this != &other) {
            reset();
            swap(other);
        }
        return *this;
    }
    ~CudaWeight() { reset(); }
    [[nodiscard]] bool valid() const noexcept { return handle_ != nullptr; }
    [[nodiscard]] int device() const noexcept { return device_; }
    [[nodiscard]] const CudaWeightDescriptor& descriptor() const noexcept { return descriptor_; }
    void reset() noexcept {
        if (handle_ != nullptr) strata_moe_weight_release(handle_);
        handle_ = nullptr;
    }

private:
    friend class CudaBackend;
    void swap(CudaWeight& other) noexcept {
        std::swap(handle_, other.handle_);
        std::swap(device_, other.device_);
        std::swap(descriptor_, other.descriptor_);
    }
    strata_moe_weight* handle_{nullptr};
    int device_{-1};
    CudaWeightDescriptor descriptor_{};
};

struct CudaMoeExpert {
    const CudaWeight* gate{};
    const CudaWeight* up{};
    const CudaWeight* down{};
    float coefficient{1.0F};
};

struct CudaDeepSeekMoeExpert {
    const CudaWeight* w1{};
    const CudaWeight* w3{};
    const CudaWeight* w2{};
    float coefficient{1.0F};
};

inline constexpr std::size_t kCudaDsv4TiledShards = 2U;

struct CudaDeepSeekMoeRowGroup {
    const CudaWeight* w1{};
    const CudaWeight* w3{};
    const CudaWeight* w2{};
    // The reference's transformed alternative to w1/w3/w2 (include/strata/cuda_backend.hpp:728-733).  This backend
    // keeps the canonical layout only (include/strata_moe_loader.hpp converts tiled shards back): a group that sets
    // a shard is rejected.
    std::array<const CudaWeight*, kCudaDsv4TiledShards> tiled_shards{};
    std::span<const std::uint32_t> rows;
    std::span<const float> coefficients;
};

// The counters of the reference's CudaBackendStats that its MoE command tests read
// (include/strata/cuda_backend.hpp:71-262).
struct CudaBackendStats {
    std::uint64_t deepseek_moe_calls{};
    std::uint64_t deepseek_moe_kernel_launches{};
    std::uint64_t deepseek_moe_h2d_bytes{};
    std::uint64_t deepseek_moe_d2h_bytes{};
    std::uint64_t workspace_allocation_calls{};
};

class CudaBackend {
public:
    CudaBackend() = default;
    CudaBackend(const CudaBackend&) = delete;
    CudaBackend& operator=(const CudaBackend&) = delete;
    ~CudaBackend() {
        for (auto& [device, state] : devices_)
            if (state.ctx != nullptr) strata_moe_destroy(state.ctx);
    }

    [[nodiscard]] static bool compiled() noexcept { return true; }
    [[nodiscard]] static std::vector<int> available_devices() {
        std::vector<int> out;
        const int n = strata_moe_device_count();
        for (int i = 0; i < n; ++i) out.push_back(i);
        return out;
    }

    enum class UploadCompletion : std::uint8_t { Synchronous, Deferred };

    [[nodiscard]] ValidationResult initialize(std::span<const int> devices, bool detailed_timing = false) {
        ValidationResult result;
        for (const int device : devices) {
            if (devices_.count(device) != 0U) continue;
            strata_moe_ctx* ctx = nullptr;
            if (const int rc = strata_moe_create(device, nullptr, &ctx); rc != 0) {
                result.errors.emplace_back("CUDA device " + std::to_string(device) +
                                           " is not usable by the MoE backend (code " + std::to_string(rc) + ")");
                return result;
            }
            strata_moe_set_timing(ctx, detailed_timing ? 1 : 0);
            devices_[device].ctx = ctx;
        }
        return result;
    }

    [[nodiscard]] ValidationResult upload(int device, const CudaWeightDescriptor& descriptor,
                                          std::span<const std::byte> weights, std::span<const std::byte> scales,
                                          CudaWeight& output,
                                          UploadCompletion completion = UploadCompletion::Synchronous) {
        (void)completion;   // the copy is complete when this returns in either mode
        State* state = find(device);
        if (state == nullptr) return error("upload targets an uninitialized CUDA device");
        if (state->in_flight != 0) return error("upload is not allowed while a MoE command is in flight");
        strata_moe_weight_desc d{};
        d.rows = static_cast<std::uint32_t>(descriptor.rows);
        d.cols = static_cast<std::uint32_t>(descriptor.columns);
        d.global_scale = 1.0F;
        switch (descriptor.encoding) {
            case CudaWeightEncoding::Plain:
                if (descriptor.dtype != SafetensorsDtype::Bf16) return error("plain expert weights must be BF16");
                d.format = STRATA_MOE_FMT_BF16;
                break;
            case CudaWeightEncoding::OffsetPackedInt4:
                if (descriptor.group_size != 128U) return error("INT4 expert weights need group size 128");
                d.format = STRATA_MOE_FMT_INT4G128;
                break;
            case CudaWeightEncoding::Fp4E2m1Group32: d.format = STRATA_MOE_FMT_MXFP4; break;
            case CudaWeightEncoding::Nvfp4Group16:
                d.format = STRATA_MOE_FMT_NVFP4;
                d.global_scale = descriptor.global_scale;
                break;
            case CudaWeightEncoding::Fp8E4m3Block128: d.format = STRATA_MOE_FMT_FP8B128; break;
            default: return error("weight encoding is not an expert format of this backend");
        }
        strata_moe_weight* handle = nullptr;
        const int rc = strata_moe_weight_upload(state->ctx, &d, weights.data(), weights.size(),
                                                scales.empty() ? nullptr : scales.data(), scales.size(), &handle);
        if (rc != 0) return last(state);
        output.reset();
        output.handle_ = handle;
        output.device_ = device;
        output.descriptor_ = descriptor;
        return {};
    }
    [[nodiscard]] ValidationResult synchronize_uploads(int device) {
        return find(device) != nullptr ? ValidationResult{} : error("device is not initialized");
    }

    // ---- the model-neutral dense command --------------------------------------------------------
    [[nodiscard]] ValidationResult enqueue_moe(int device, std::span<const float> hidden, std::uint32_t rows,
                                               std::span<const CudaMoeExpert> routed,
                                               const CudaMoeExpert* shared = nullptr) {
        State* state = find(device);
        if (state == nullptr) return error("MoE command targets an uninitialized CUDA device");
        if (state->in_flight != 0) return error("MoE workspace already has an in-flight command");
        std::vector<strata_moe_expert_ref> refs;
        for (const auto& e : routed) {
            if (!usable(e.gate, device) || !usable(e.up, device) || !usable(e.down, device))
                return error("MoE command contains an incompatible CUDA weight");
            refs.push_back({e.gate->handle_, e.up->handle_, e.down->handle_, e.coefficient});
        }
        strata_moe_expert_ref shared_ref{};
        if (shared != nullptr) {
            if (!usable(shared->gate, device) || !usable(shared->up, device) || !usable(shared->down, device))
                return error("MoE command contains an incompatible CUDA weight");
            shared_ref = {shared->gate->handle_, shared->up->handle_, shared->down->handle_, shared->coefficient};
        }
        const int rc = strata_moe_command_enqueue(state->ctx, hidden.data(), hidden.size(), rows, refs.data(),
                                                  static_cast<std::uint32_t>(refs.size()),
                                                  shared != nullptr ? &shared_ref : nullptr);
        if (rc != 0) return last(state);
        state->in_flight = 1;
        return {};
    }
    [[nodiscard]] ValidationResult collect_moe(int device, std::span<float> routed_output,
                                               std::span<float> shared_output = {}) {
        State* state = find(device);
        if (state == nullptr || state->in_flight != 1) return error("no MoE command is in flight");
        state->in_flight = 0;
        const int rc = strata_moe_command_collect(state->ctx, routed_output.data(), routed_output.size(),
                                                  shared_output.data(), shared_output.size());
        return rc == 0 ? ValidationResult{} : last(state);
    }

    // ---- DeepSeek-V4 commands (exact numerical mode) --------------------------------------------
    [[nodiscard]] ValidationResult enqueue_deepseek_moe(int device, std::span<const float> hidden,
                                                        std::span<const CudaDeepSeekMoeExpert> routed,
                                                        const CudaDeepSeekMoeExpert* shared, float swiglu_limit) {
        // one row, every routed expert applied to it with its coefficient: the row-grouped command with
        // one-row groups (the reference's limit of six routed experts is kept)
        if (routed.size() > 6U) return error("DeepSeek MoE command has too many routed experts");
        static constexpr std::uint32_t kRowZero = 0U;
        std::vector<CudaDeepSeekMoeRowGroup> groups;
        std::vector<float> coefficients(routed.size());
        for (std::size_t i = 0; i < routed.size(); ++i) {
            coefficients[i] = routed[i].coefficient;
            groups.push_back({routed[i].w1, routed[i].w3, routed[i].w2, {}, std::span<const std::uint32_t>(&kRowZero, 1),
                              std::span<const float>(&coefficients[i], 1)});
        }
        return enqueue_rows(device, hidden, 1U, groups, shared,
                            shared != nullptr ? std::span<const std::uint32_t>(&kRowZero, 1)
                                              : std::span<const std::uint32_t>{},
                            swiglu_limit, 2);
    }
    [[nodiscard]] ValidationResult collect_deepseek_moe(int device, std::span<float> routed_output,
                                                        std::span<float> shared_output) {
        return collect_rows(device, routed_output, shared_output, 2);
    }
    [[nodiscard]] ValidationResult enqueue_deepseek_moe_rows(int device, std::span<const float> hidden,
                                                             std::uint32_t hidden_rows,
                                                             std::span<const CudaDeepSeekMoeRowGroup> groups,
                                                             const CudaDeepSeekMoeExpert* shared,
                                                             std::span<const std::uint32_t> shared_rows,
                                                             float swiglu_limit) {
        return enqueue_rows(device, hidden, hidden_rows, groups, shared, shared_rows, swiglu_limit, 3);
    }
    [[nodiscard]] ValidationResult collect_deepseek_moe_rows(int device, std::span<float> routed_output,
                                                             std::span<float> shared_output) {
        return collect_rows(device, routed_output, shared_output, 3);
    }

    [[nodiscard]] ValidationResult synchronize(int device) {
        State* state = find(device);
        if (state == nullptr) return error("synchronize targets an uninitialized CUDA device");
        if (state->in_flight != 0) return error("synchronize is not allowed while a MoE command is in flight");
        return strata_moe_synchronize(state->ctx) == 0 ? ValidationResult{} : last(state);
    }

    [[nodiscard]] CudaBackendStats stats() const noexcept {
        CudaBackendStats out;
        for (const auto& [device, state] : devices_) {
            strata_moe_stats s{};
            if (strata_moe_get_stats(state.ctx, &s) != 0) continue;
            out.deepseek_moe_calls += s.command_calls;
            out.deepseek_moe_kernel_launches += s.kernel_launches;
            out.deepseek_moe_h2d_bytes += s.h2d_bytes;
            out.deepseek_moe_d2h_bytes += s.d2h_bytes;
            out.workspace_allocation_calls += s.workspace_allocations;
        }
        return out;
    }

    [[nodiscard]] strata_moe_ctx* context(int device) noexcept {
        State* state = find(device);
        return state != nullptr ? state->ctx : nullptr;
    }

private:
    struct State {
        strata_moe_ctx* ctx{nullptr};
        int in_flight{0};   // 0 none, 1 dense command, 2 single-row DeepSeek command, 3 DeepSeek row groups
    };
    [[nodiscard]] State* find(int device) {
        const auto it = devices_.find(device);
        return it == devices_.end() ? nullptr : &it->second;
    }
    [[nodiscard]] static ValidationResult error(std::string text) {
        ValidationResult r;
        r.errors.emplace_back(std::move(text));
        return r;
    }
    [[nodiscard]] static ValidationResult last(const State* state) {
        return error(strata_moe_last_error(state->ctx));
    }
    [[nodiscard]] static bool usable(const CudaWeight* w, int device) noexcept {
        return w != nullptr && w->valid() && w->device() == device;
    }
    [[nodiscard]] ValidationResult enqueue_rows(int device, std::span<const float> hidden, std::uint32_t hidden_rows,
                                                std::span<const CudaDeepSeekMoeRowGroup> groups,
                                                const CudaDeepSeekMoeExpert* shared,
                                                std::span<const std::uint32_t> shared_rows, float swiglu_limit,
                                                int kind) {
        State* state = find(device);
        if (state == nullptr) return error("DeepSeek MoE command targets an uninitialized CUDA device");
        if (state->in_flight != 0) return error("MoE workspace already has an in-flight command");
        std::vector<strata_moe_row_group> raw;
        for (const auto& g : groups) {
            if (g.tiled_shards[0] != nullptr || g.tiled_shards[1] != nullptr)
                return error("transformed expert shards are not supported: upload the canonical w1 / w3 / w2");
            if (!usable(g.w1, device) || !usable(g.w3, device) || !usable(g.w2, device))
                return error("DeepSeek MoE command contains an incompatible CUDA weight");
            if (g.rows.size() != g.coefficients.size()) return error("row group rows and coefficients differ in size");
            raw.push_back({g.w1->handle_, g.w3->handle_, g.w2->handle_, g.rows.data(), g.coefficients.data(),
                           static_cast<std::uint32_t>(g.rows.size())});
        }
        strata_moe_expert_ref shared_ref{};
        if (shared != nullptr) {
            if (!usable(shared->w1, device) || !usable(shared->w3, device) || !usable(shared->w2, device))
                return error("DeepSeek MoE command contains an incompatible CUDA weight");
            if (shared->coefficient != 1.0F) return error("the shared expert takes coefficient 1");
            shared_ref = {shared->w1->handle_, shared->w3->handle_, shared->w2->handle_, 1.0F};
        }
        const int rc = strata_moe_command_enqueue_rows_dsv4(
            state->ctx, hidden.data(), hidden.size(), hidden_rows, raw.data(), static_cast<std::uint32_t>(raw.size()),
            shared != nullptr ? &shared_ref : nullptr, shared_rows.data(), static_cast<std::uint32_t>(shared_rows.size()),
            swiglu_limit);
        if (rc != 0) return last(state);
        state->in_flight = kind;
        return {};
    }
    [[nodiscard]] ValidationResult collect_rows(int device, std::span<float> routed_output,
                                                std::span<float> shared_output, int kind) {
        State* state = find(device);
        if (state == nullptr || state->in_flight != kind) return error("no DeepSeek MoE command is in flight");
        state->in_flight = 0;
        const int rc = strata_moe_command_collect_rows_dsv4(state->ctx, routed_output.data(), routed_output.size(),
                                                            shared_output.data(), shared_output.size());
        return rc == 0 ? ValidationResult{} : last(state);
    }

    std::map<int, State> devices_;
};

}  // namespace strata_b200
