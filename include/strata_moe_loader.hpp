// Checkpoint-native loading for the MoE expert block: header-only C++20 over the C ABI.
//
//   SafetensorsFile      memory-maps one .safetensors shard and indexes its tensors
//                        (ref: src/platform/safetensors.cpp; the container format is the public one:
//                        u64 little-endian header length, a JSON object name -> {dtype, shape,
//                        data_offsets}, then the tensor bytes)
//   moe_tensor_names     the tensor names each model family uses for one MoE layer (ref: the call sites
//                        src/models/glm52/glm_runtime.cpp:85, 122-123, 230-240, src/models/laguna/
//                        laguna_checkpoint.cpp:38, 159-161, 212-232, src/models/dsv4/deepseek_runtime.cpp:
//                        133, 2480-2552, 5817-5840, src/models/kimi_k3/kimi_k3_checkpoint.cpp:18, 321-348;
//                        compressed-tensors naming: src/platform/compressed_tensors.cpp:287-313)
//   load_moe_layer       registers router, routed experts and BF16 shared expert of one layer with
//                        strata_moe_set_router / set_expert / set_shared straight from the mapped bytes
//   tiled32_to_canonical inverse of the DeepSeek-V4 host decode layout Fp4E2m1Tiled32
//                        (ref: dsv4_transform_tiled_expert_shard, kernels/cpu/dsv4_fp4_expert.cpp:360-434):
//                        a host that only keeps the tiled shards can still register canonical rows
//   deinterleave_gate_up Inkling stores gate and up rows interleaved in one tensor
//                        (ref: src/models/inkling/inkling_ops.cpp:286-299)
//   RouteTraceWriter     strata.route_trace version 2 (ref: src/platform/trace.cpp:175-229), so that the
//                        reference's simulator and predictor tooling reads routes produced here
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <fstream>
#include <iomanip>
#include <limits>
#include <map>
#include <span>
#include <string>
#include <string_view>
#include <vector>

#include "strata_moe.h"

namespace strata_b200 {

struct LoadResult {
    std::vector<std::string> errors;
    [[nodiscard]] bool ok() const noexcept { return errors.empty(); }
};

struct TensorView {
    std::string dtype;                 // "BF16", "F32", "U8", "I8", "I32", "I64", "F8_E4M3", "F8_E8M0", ...
    std::vector<std::uint64_t> shape;
    const std::byte* data{};
    std::size_t bytes{};
};

class SafetensorsFile {
public:
    SafetensorsFile() = default;
    SafetensorsFile(const SafetensorsFile&) = delete;
    SafetensorsFile& operator=(const SafetensorsFile&) = delete;
    ~SafetensorsFile() { close(); }

    [[nodiscard]] LoadResult open(const std::string& path) {
        close();
        LoadResult r;
        fd_ = ::open(path.c_str(), O_RDONLY);
        if (fd_ < 0) return fail(r, "cannot open " + path);
        struct stat st {};
        if (fstat(fd_, &st) != 0 || st.st_size < 8) return fail(r, path + " is not a safetensors file");
        size_ = static_cast<std::size_t>(st.st_size);
        void* p = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (p == MAP_FAILED) return fail(r, "cannot map " + path);
        base_ = static_cast<const std::byte*>(p);
        std::uint64_t header = 0;
        std::memcpy(&header, base_, 8);
        if (header == 0 || header > size_ - 8) return fail(r, path + " has an implausible header length");
        const std::string_view json(reinterpret_cast<const char*>(base_ + 8), static_cast<std::size_t>(header));
        const std::byte* data = base_ + 8 + header;
        const std::size_t data_bytes = size_ - 8 - static_cast<std::size_t>(header);
        std::size_t at = 0;
        if (!parse_header(json, at, data, data_bytes)) return fail(r, path + " has a malformed header near byte " + std::to_string(at));
        return r;
    }
    void close() noexcept {
        if (base_ != nullptr) munmap(const_cast<std::byte*>(base_), size_);
        if (fd_ >= 0) ::close(fd_);
        base_ = nullptr;
        fd_ = -1;
        tensors_.clear();
    }
    [[nodiscard]] const TensorView* find(const std::string& name) const {
        const auto it = tensors_.find(name);
        return it == tensors_.end() ? nullptr : &it->second;
    }
    [[nodiscard]] const std::map<std::string, TensorView>& tensors() const noexcept { return tensors_; }

private:
    static LoadResult fail(LoadResult& r, std::string text) {
        r.errors.push_back(std::move(text));
        return r;
    }
    static void skip_ws(std::string_view s, std::size_t& at) {
        while (at < s.size() && (s[at] == ' ' || s[at] == '\n' || s[at] == '\t' || s[at] == '\r')) ++at;
    }
    static bool parse_string(std::string_view s, std::size_t& at, std::string& out) {
        skip_ws(s, at);
        if (at >= s.size() || s[at] != '"') return false;
        ++at;
        out.clear();
        while (at < s.size() && s[at] != '"') {
            if (s[at] == '\\' && at + 1 < s.size()) ++at;   // names and dtypes hold no escapes that matter
            out.push_back(s[at++]);
        }
        if (at >= s.size()) return false;
        ++at;
        return true;
    }
    static bool parse_uint(std::string_view s, std::size_t& at, std::uint64_t& out) {
        skip_ws(s, at);
        if (at >= s.size() || s[at] < '0' || s[at] > '9') return false;
        out = 0;
        while (at < s.size() && s[at] >= '0' && s[at] <= '9') out = out * 10 + static_cast<std::uint64_t>(s[at++] - '0');
        return true;
    }
    static bool expect(std::string_view s, std::size_t& at, char c) {
        skip_ws(s, at);
        if (at >= s.size() || s[at] != c) return false;
        ++at;
        return true;
    }
    static bool parse_uint_array(std::string_view s, std::size_t& at, std::vector<std::uint64_t>& out) {
        if (!expect(s, at, '[')) return false;
        out.clear();
        skip_ws(s, at);
        if (at < s.size() && s[at] == ']') { ++at; return true; }
        for (;;) {
            std::uint64_t v = 0;
            if (!parse_uint(s, at, v)) return false;
            out.push_back(v);
            skip_ws(s, at);
            if (at < s.size() && s[at] == ',') { ++at; continue; }
            return expect(s, at, ']');
        }
    }
    // skips any JSON value (used for "__metadata__")
    static bool skip_value(std::string_view s, std::size_t& at) {
        skip_ws(s, at);
        if (at >= s.size()) return false;
        if (s[at] == '"') { std::string t; return parse_string(s, at, t); }
        if (s[at] == '{' || s[at] == '[') {
            const char open = s[at], closec = open == '{' ? '}' : ']';
            ++at;
            skip_ws(s, at);
            if (at < s.size() && s[at] == closec) { ++at; return true; }
            for (;;) {
                if (open == '{') {
                    std::string key;
                    if (!parse_string(s, at, key) || !expect(s, at, ':')) return false;
                }
                if (!skip_value(s, at)) return false;
                skip_ws(s, at);
                if (at < s.size() && s[at] == ',') { ++at; continue; }
                return expect(s, at, closec);
            }
        }
        while (at < s.size() && s[at] != ',' && s[at] != '}' && s[at] != ']') ++at;
        return true;
    }
    bool parse_header(std::string_view s, std::size_t& at, const std::byte* data, std::size_t data_bytes) {
        if (!expect(s, at, '{')) return false;
        skip_ws(s, at);
        if (at < s.size() && s[at] == '}') return true;
        for (;;) {
            std::string name;
            if (!parse_string(s, at, name) || !expect(s, at, ':')) return false;
            if (name == "__metadata__") {
                if (!skip_value(s, at)) return false;
            } else {
                TensorView t;
                std::vector<std::uint64_t> offsets;
                if (!expect(s, at, '{')) return false;
                for (;;) {
                    std::string key;
                    if (!parse_string(s, at, key) || !expect(s, at, ':')) return false;
                    if (key == "dtype") { if (!parse_string(s, at, t.dtype)) return false; }
                    else if (key == "shape") { if (!parse_uint_array(s, at, t.shape)) return false; }
                    else if (key == "data_offsets") { if (!parse_uint_array(s, at, offsets)) return false; }
                    else if (!skip_value(s, at)) return false;
                    skip_ws(s, at);
                    if (at < s.size() && s[at] == ',') { ++at; continue; }
                    if (!expect(s, at, '}')) return false;
                    break;
                }
                if (offsets.size() != 2 || offsets[0] > offsets[1] || offsets[1] > data_bytes) return false;
                t.data = data + offsets[0];
                t.bytes = static_cast<std::size_t>(offsets[1] - offsets[0]);
                tensors_.emplace(std::move(name), std::move(t));
            }
            skip_ws(s, at);
            if (at < s.size() && s[at] == ',') { ++at; continue; }
            return expect(s, at, '}');
        }
    }

    int fd_{-1};
    const std::byte* base_{nullptr};
    std::size_t size_{0};
    std::map<std::string, TensorView> tensors_;
};

enum class MoeFamily { DeepSeekV4, Glm, Laguna, KimiK3 };

struct MoeTensorNames {
    std::string router, router_bias;                 // [E, H] BF16, [E] F32
    std::string expert_prefix;                       // + "<expert>."
    std::string proj[3];                             // gate, up, down projection stems
    std::string packed_suffix, scale_suffix;         // appended to the stem
    std::string global_suffix;                       // NVFP4 per-tensor scale, empty when the format has none
    std::string shared_prefix;                       // BF16 shared expert, + stem + ".weight"; empty = none here
};

[[nodiscard]] inline MoeTensorNames moe_tensor_names(MoeFamily family, std::uint32_t layer) {
    MoeTensorNames n;
    const std::string l = std::to_string(layer);
    switch (family) {
        case MoeFamily::DeepSeekV4: {
            const std::string p = "layers." + l + ".ffn.";
            n = {p + "gate.weight", p + "gate.bias", p + "experts.", {"w1", "w3", "w2"}, ".weight", ".scale", "", ""};
            break;   // the FP8 shared expert goes through strata_moe_weight_upload, not set_shared
        }
        case MoeFamily::Glm: {
            const std::string p = "model.layers." + l + ".mlp.";
            n = {p + "gate.weight", p + "gate.e_score_correction_bias", p + "experts.",
                 {"gate_proj", "up_proj", "down_proj"}, ".weight_packed", ".weight_scale", "", ""};
            break;   // GLM's shared expert is INT4 too and rides the dense command as one more expert
        }
        case MoeFamily::Laguna: {
            const std::string p = "model.layers." + l + ".mlp.";
            n = {p + "gate.weight", p + "experts.e_score_correction_bias", p + "experts.",
                 {"gate_proj", "up_proj", "down_proj"}, ".weight_packed", ".weight_scale", ".weight_global_scale",
                 p + "shared_expert."};
            break;
        }
        case MoeFamily::KimiK3: {
            const std::string p = "model.layers." + l + ".block_sparse_moe.";
            n = {p + "gate.weight", p + "gate.e_score_correction_bias", p + "experts.", {"w1", "w3", "w2"},
                 ".weight_packed", ".weight_scale", "", ""};
            break;   // latent projections and shared experts: strata_moe_latent_set_projections / set_shared
        }
    }
    return n;
}

// First file that holds `name`.
[[nodiscard]] inline const TensorView* find_tensor(std::span<const SafetensorsFile* const> files, const std::string& name) {
    for (const auto* f : files)
        if (const TensorView* t = f->find(name)) return t;
    return nullptr;
}

// Registers one MoE layer from checkpoint shards.  The layer must have been created with the matching
// descriptor (format, shapes, resident expert range); every tensor is checked against it before any
// byte is uploaded.  NVFP4: the checkpoint's weight_global_scale is the divisor (w = e2m1 * e4m3 / global);
// a family that multiplies by its scale instead (Inkling) passes 1 / scale -- set invert_global.
[[nodiscard]] inline LoadResult load_moe_layer(strata_moe_layer* layer, const strata_moe_layer_desc& desc,
                                               std::span<const SafetensorsFile* const> files, MoeFamily family,
                                               std::uint32_t layer_index, bool invert_global = false) {
    LoadResult r;
    const MoeTensorNames n = moe_tensor_names(family, layer_index);
    const std::uint64_t H = desc.hidden, I = desc.intermediate;
    auto need = [&](const std::string& name, std::size_t bytes) -> const TensorView* {
        const TensorView* t = find_tensor(files, name);
        if (t == nullptr) r.errors.push_back("missing tensor " + name);
        else if (t->bytes != bytes) {
            r.errors.push_back(name + " has " + std::to_string(t->bytes) + " bytes, the layer expects " + std::to_string(bytes));
            t = nullptr;
        }
        return t;
    };
    auto packed_bytes = [&](std::uint64_t rows, std::uint64_t cols) -> std::size_t {
        return desc.format == STRATA_MOE_FMT_BF16 ? rows * cols * 2 : rows * cols / 2;
    };
    auto scale_bytes = [&](std::uint64_t rows, std::uint64_t cols) -> std::size_t {
        switch (desc.format) {
            case STRATA_MOE_FMT_MXFP4: return rows * cols / 32;
            case STRATA_MOE_FMT_NVFP4: return rows * cols / 16;
            case STRATA_MOE_FMT_INT4G128: return rows * cols / 128 * 2;
            default: return 0;
        }
    };
    const TensorView* router = need(n.router, static_cast<std::size_t>(desc.experts) * H * 2);
    const TensorView* bias = find_tensor(files, n.router_bias);
    if (bias != nullptr && bias->bytes != static_cast<std::size_t>(desc.experts) * 4) {
        r.errors.push_back(n.router_bias + " does not hold one fp32 per expert");
        bias = nullptr;
    }
    struct Proj { const TensorView *packed, *scale; float global; };
    std::vector<Proj> experts(static_cast<std::size_t>(desc.expert_count) * 3);
    for (std::uint32_t le = 0; le < desc.expert_count && r.errors.size() < 16; ++le) {
        const std::string base = n.expert_prefix + std::to_string(desc.expert_begin + le) + ".";
        for (int role = 0; role < 3; ++role) {
            const std::uint64_t rows = role == 2 ? H : I, cols = role == 2 ? I : H;
            Proj& p = experts[static_cast<std::size_t>(le) * 3 + role];
            const bool plain = desc.format == STRATA_MOE_FMT_BF16;
            p.packed = need(base + n.proj[role] + (plain ? ".weight" : n.packed_suffix), packed_bytes(rows, cols));
            p.scale = plain ? nullptr : need(base + n.proj[role] + n.scale_suffix, scale_bytes(rows, cols));
            p.global = 1.0F;
            if (desc.format == STRATA_MOE_FMT_NVFP4 && !n.global_suffix.empty()) {
                if (const TensorView* g = need(base + n.proj[role] + n.global_suffix, 4)) {
                    std::memcpy(&p.global, g->data, 4);
                    if (invert_global) p.global = 1.0F / p.global;
                }
            }
        }
    }
    const TensorView* shared[3] = {nullptr, nullptr, nullptr};
    if (desc.shared_intermediate != 0 && !n.shared_prefix.empty())
        for (int role = 0; role < 3; ++role)
            shared[role] = need(n.shared_prefix + n.proj[role] + ".weight",
                                static_cast<std::size_t>(desc.shared_intermediate) * H * 2);
    if (!r.ok()) return r;
    auto check = [&](int rc, const std::string& what) {
        if (rc != 0) r.errors.push_back(what + " was rejected by the library (code " + std::to_string(rc) + ")");
    };
    check(strata_moe_set_router(layer, router->data, bias != nullptr ? reinterpret_cast<const float*>(bias->data) : nullptr,
                                STRATA_MOE_SRC_HOST), n.router);
    for (std::uint32_t le = 0; le < desc.expert_count && r.ok(); ++le)
        for (int role = 0; role < 3 && r.ok(); ++role) {
            const Proj& p = experts[static_cast<std::size_t>(le) * 3 + role];
            check(strata_moe_set_expert(layer, desc.expert_begin + le, role, p.packed->data,
                                        p.scale != nullptr ? p.scale->data : nullptr, p.global, STRATA_MOE_SRC_HOST),
                  n.expert_prefix + std::to_string(desc.expert_begin + le) + "." + n.proj[role]);
        }
    for (int role = 0; role < 3 && r.ok(); ++role)
        if (shared[role] != nullptr) check(strata_moe_set_shared(layer, role, shared[role]->data, STRATA_MOE_SRC_HOST),
                                           n.shared_prefix + n.proj[role]);
    return r;
}

// ---- DeepSeek-V4 host decode layout ----------------------------------------------------------
// A tiled shard holds one intermediate-dimension slice of an expert: w13 packed, w13 scales, w2 packed,
// w2 scales, output rows blocked by 32 and stored block-column-major, each group-32 scale duplicated
// over its two group-16 halves.  This rebuilds the canonical row-major tensors from all shards.
struct CanonicalExpert {
    std::vector<std::uint8_t> w1, w3, w2;        // packed [I, H/2], [I, H/2], [H, I/2]
    std::vector<std::uint8_t> s1, s3, s2;        // scales [I, H/32], [I, H/32], [H, I/32]
};

[[nodiscard]] inline std::size_t tiled32_shard_bytes(std::uint64_t hidden, std::uint64_t intermediate, std::uint64_t shards) {
    if (hidden == 0 || intermediate == 0 || shards == 0 || hidden % 32 != 0 || intermediate % (32 * shards) != 0) return 0;
    const std::uint64_t si = intermediate / shards;
    return static_cast<std::size_t>(2 * si * (hidden / 2) + 2 * si * (hidden / 16) + hidden * (si / 2) + hidden * (si / 16));
}

[[nodiscard]] inline LoadResult tiled32_to_canonical(std::span<const std::span<const std::byte>> shard_storage,
                                                     std::uint64_t hidden, std::uint64_t intermediate, CanonicalExpert& out) {
    LoadResult r;
    const std::uint64_t shards = shard_storage.size();
    const std::size_t bytes = tiled32_shard_bytes(hidden, intermediate, shards);
    if (bytes == 0) { r.errors.emplace_back("tiled expert geometry is incompatible"); return r; }
    for (const auto& s : shard_storage)
        if (s.size() != bytes) { r.errors.emplace_back("a tiled shard has the wrong extent"); return r; }
    constexpr std::uint64_t kBlock = 32;
    const std::uint64_t si = intermediate / shards;
    out.w1.assign(intermediate * (hidden / 2), 0);
    out.w3.assign(intermediate * (hidden / 2), 0);
    out.w2.assign(hidden * (intermediate / 2), 0);
    out.s1.assign(intermediate * (hidden / 32), 0);
    out.s3.assign(intermediate * (hidden / 32), 0);
    out.s2.assign(hidden * (intermediate / 32), 0);
    for (std::uint64_t shard = 0; shard < shards; ++shard) {
        const auto* packed13 = reinterpret_cast<const std::uint8_t*>(shard_storage[shard].data());
        const auto* scales13 = packed13 + 2 * si * (hidden / 2);
        const auto* packed2 = scales13 + 2 * si * (hidden / 16);
        const auto* scales2 = packed2 + hidden * (si / 2);
        for (std::uint64_t projection = 0; projection < 2; ++projection) {
            auto& w = projection == 0 ? out.w1 : out.w3;
            auto& s = projection == 0 ? out.s1 : out.s3;
            for (std::uint64_t row = 0; row < si; ++row) {
                const std::uint64_t dst_row = shard * si + row, output = projection * si + row;
                const std::uint64_t block = output / kBlock, within = output % kBlock;
                for (std::uint64_t pair = 0; pair < hidden / 2; ++pair)
                    w[dst_row * (hidden / 2) + pair] = packed13[(block * (hidden / 2) + pair) * kBlock + within];
                for (std::uint64_t g = 0; g < hidden / 32; ++g)
                    s[dst_row * (hidden / 32) + g] = scales13[(block * (hidden / 16) + 2 * g) * kBlock + within];
            }
        }
        for (std::uint64_t row = 0; row < hidden; ++row) {
            const std::uint64_t block = row / kBlock, within = row % kBlock;
            for (std::uint64_t pair = 0; pair < si / 2; ++pair)
                out.w2[row * (intermediate / 2) + shard * (si / 2) + pair] = packed2[(block * (si / 2) + pair) * kBlock + within];
            for (std::uint64_t g = 0; g < si / 32; ++g)
                out.s2[row * (intermediate / 32) + shard * (si / 32) + g] = scales2[(block * (si / 16) + 2 * g) * kBlock + within];
        }
    }
    return r;
}

// Rows 2i of `interleaved` ([2 I, row_bytes]) are gate row i, rows 2i + 1 up row i.
inline void deinterleave_gate_up(std::span<const std::byte> interleaved, std::size_t row_bytes, std::vector<std::byte>& gate,
                                 std::vector<std::byte>& up) {
    const std::size_t rows = row_bytes == 0 ? 0 : interleaved.size() / row_bytes / 2;
    gate.resize(rows * row_bytes);
    up.resize(rows * row_bytes);
    for (std::size_t i = 0; i < rows; ++i) {
        std::memcpy(gate.data() + i * row_bytes, interleaved.data() + (2 * i) * row_bytes, row_bytes);
        std::memcpy(up.data() + i * row_bytes, interleaved.data() + (2 * i + 1) * row_bytes, row_bytes);
    }
}

// ---- strata.route_trace, version 2 ---------------------------------------------------------------
enum class RoutePhase { Unknown, Prefill, Decode };

struct RouteEvent {
    std::uint64_t request{};
    RoutePhase phase{RoutePhase::Unknown};
    std::uint64_t token_position{};
    std::uint32_t layer{};
    std::vector<std::uint32_t> experts;
    std::vector<float> coefficients;
};

class RouteTraceWriter {
public:
    [[nodiscard]] LoadResult open(const std::string& path) {
        LoadResult r;
        if (output_.is_open()) { r.errors.emplace_back("route trace writer is already open"); return r; }
        output_.open(path, std::ios::out | std::ios::trunc);
        if (!output_.is_open()) { r.errors.emplace_back("cannot open route trace: " + path); return r; }
        output_ << "{\"schema\":\"strata.route_trace\",\"version\":2,\"position_base\":0,\"layer_base\":0,"
                   "\"coefficient_encoding\":\"float32-roundtrip-decimal\"}\n";
        if (!output_.good()) r.errors.emplace_back("cannot write route trace header");
        return r;
    }
    [[nodiscard]] LoadResult write(const RouteEvent& event) {
        LoadResult r;
        if (!output_.is_open()) { r.errors.emplace_back("route trace writer is not open"); return r; }
        if (event.experts.empty() || (!event.coefficients.empty() && event.coefficients.size() != event.experts.size())) {
            r.errors.emplace_back("route event has incompatible expert coefficients");
            return r;
        }
        static constexpr const char* kPhase[] = {"unknown", "prefill", "decode"};
        output_ << "{\"request\":" << event.request << ",\"phase\":\"" << kPhase[static_cast<int>(event.phase)]
                << "\",\"token_position\":" << event.token_position << ",\"layer\":" << event.layer << ",\"experts\":[";
        for (std::size_t i = 0; i < event.experts.size(); ++i) output_ << (i ? "," : "") << event.experts[i];
        output_ << "],\"coefficients\":[" << std::setprecision(std::numeric_limits<float>::max_digits10);
        for (std::size_t i = 0; i < event.coefficients.size(); ++i) output_ << (i ? "," : "") << event.coefficients[i];
        output_ << "]}\n";
        if (!output_.good()) r.errors.emplace_back("cannot write route trace event");
        return r;
    }
    // One event per token of a routed page: ids / weights [tokens, k] as strata_moe_route produced them.
    [[nodiscard]] LoadResult write_page(std::uint64_t request, RoutePhase phase, std::uint64_t first_position, std::uint32_t layer,
                                        std::span<const std::uint32_t> ids, std::span<const float> weights, std::uint32_t k) {
        LoadResult r;
        if (k == 0 || ids.size() % k != 0 || weights.size() != ids.size()) {
            r.errors.emplace_back("route page has incompatible extents");
            return r;
        }
        RouteEvent e;
        e.request = request;
        e.phase = phase;
        e.layer = layer;
        for (std::size_t t = 0; t < ids.size() / k && r.ok(); ++t) {
            e.token_position = first_position + t;
            e.experts.assign(ids.begin() + static_cast<std::ptrdiff_t>(t * k), ids.begin() + static_cast<std::ptrdiff_t>((t + 1) * k));
            e.coefficients.assign(weights.begin() + static_cast<std::ptrdiff_t>(t * k),
                                  weights.begin() + static_cast<std::ptrdiff_t>((t + 1) * k));
            r = write(e);
        }
        return r;
    }
    void flush() { if (output_.is_open()) output_.flush(); }
    void close() { if (output_.is_open()) output_.close(); }

private:
    std::ofstream output_;
};

}  // namespace strata_b200
