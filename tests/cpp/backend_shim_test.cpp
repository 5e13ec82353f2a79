// The MoE command cases of the reference's backend test, run against the C++ shim
// (include/strata_moe_backend.hpp) and the CUDA library.  The call sites are the reference's own
// (tests/test_cuda_backend.cpp:1509-1574 "batches reusable target-shape GLM INT4 MoE commands" and
// :1576-1780 "enqueues exact grouped DeepSeek MoE"): same upload helpers, same seeds, same hidden
// patterns, same protocol assertions.  Differences, all stated where they occur:
//   * expected values come from the CPU checker (oracle/libmoe_oracle.so) instead of a second pass
//     through the device matmul;
//   * the DeepSeek case runs at hidden = intermediate = 128 (this library's shapes are multiples of
//     128; the reference case uses 32) and at the DeepSeek-V4 shape 4096 / 2048;
//   * statistics that count the reference's own launches and transfers are not asserted.
// Exit code 0 = all cases passed (or no usable device).
#include <algorithm>
#include <array>
#include <bit>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

// STRATA_TEST_REFERENCE_BACKEND: the same cases against the reference's own CUDA backend (compiled unmodified by
// oracle/build.py), which makes this file a two-way check: both implementations have to meet the CPU checker's values.
#ifdef STRATA_TEST_REFERENCE_BACKEND
#include "strata/cuda_backend.hpp"
#define BACKEND_NAME "reference backend"
#else
#include "strata_moe_backend.hpp"

namespace strata = strata_b200;   // the one line a reference call site changes
#define BACKEND_NAME "backend shim"
#endif

extern "C" {
// CPU checker (test infrastructure): oracle/moe_oracle.c
struct orc_matrix {
    int32_t fmt;
    uint32_t rows, cols;
    const void* packed;
    const void* scales;
    float global_scale;
};
struct orc_expert {
    orc_matrix gate, up, down;
    int32_t activation;
    float gate_beta, linear_beta;
};
int orc_expert_ffn(const orc_expert* ex, const float* x, float coef, int coef_before_down, int accumulate_double,
                   float* act_scratch, float* up_scratch, float* y);
int orc_dsv4_expert(float* out, const float* in, const uint8_t* w1, const uint8_t* s1, const uint8_t* w3,
                    const uint8_t* s3, const uint8_t* w2, const uint8_t* s2, uint32_t hidden, uint32_t intermediate,
                    float coefficient, float swiglu_limit, float* scratch);
void orc_router_logits(const uint16_t* x_bf16, const uint16_t* wg_bf16, uint32_t T, uint32_t H, uint32_t E, float* logits);
int orc_dsv4_fp8_shared(float* out, const float* in, const uint8_t* w1, const uint8_t* s1, const uint8_t* w3,
                        const uint8_t* s3, const uint8_t* w2, const uint8_t* s2, uint32_t hidden, uint32_t intermediate,
                        float swiglu_limit, float* scratch);
}

static int g_failures = 0;
#define REQUIRE(cond)                                                                  \
    do {                                                                               \
        if (!(cond)) {                                                                 \
            std::fprintf(stderr, "%s:%d: REQUIRE(%s) failed\n", __FILE__, __LINE__, #cond); \
            ++g_failures;                                                              \
            return;                                                                    \
        }                                                                              \
    } while (0)

namespace {

struct HostWeight {
    std::vector<std::byte> weights, scales;
};

void store_u32(std::byte* p, std::uint32_t v) { std::memcpy(p, &v, 4); }
std::array<std::byte, 2> bf16(float v) {
    std::uint32_t bits;
    std::memcpy(&bits, &v, 4);
    bits = (bits + 0x7FFFU + ((bits >> 16U) & 1U)) >> 16U;
    return {static_cast<std::byte>(bits & 0xFFU), static_cast<std::byte>(bits >> 8U)};
}

// ref: upload_int4, tests/test_cuda_backend.cpp:128-161
strata::CudaWeight upload_int4(strata::CudaBackend& backend, int device, std::uint64_t rows, std::uint64_t columns,
                               std::uint8_t seed, HostWeight& keep) {
    strata::CudaWeightDescriptor descriptor;
    descriptor.encoding = strata::CudaWeightEncoding::OffsetPackedInt4;
    descriptor.dtype = strata::SafetensorsDtype::I32;
    descriptor.rows = rows;
    descriptor.columns = columns;
    descriptor.packed_columns = (columns + 7U) / 8U;
    descriptor.scale_columns = (columns + 127U) / 128U;
    descriptor.group_size = 128U;
    keep.weights.resize(static_cast<std::size_t>(rows * descriptor.packed_columns * 4U));
    for (std::uint64_t row = 0U; row < rows; ++row) {
        for (std::uint64_t word = 0U; word < descriptor.packed_columns; ++word) {
            std::uint32_t value = 0U;
            for (std::uint32_t lane = 0U; lane < 8U; ++lane)
                value |= static_cast<std::uint32_t>((seed + row * 3U + word * 5U + lane * 7U) & 0x0FU) << (lane * 4U);
            store_u32(keep.weights.data() + (row * descriptor.packed_columns + word) * 4U, value);
        }
    }
    const auto scale = bf16(0.015625F);
    keep.scales.resize(static_cast<std::size_t>(rows * descriptor.scale_columns * 2U));
    for (std::size_t index = 0U; index < keep.scales.size(); index += 2U) {
        keep.scales[index] = scale[0];
        keep.scales[index + 1] = scale[1];
    }
    strata::CudaWeight result;
    if (!backend.upload(device, descriptor, keep.weights, keep.scales, result).ok()) ++g_failures;
    return result;
}

// ref: upload_fp4, tests/test_cuda_backend.cpp:65-100
strata::CudaWeight upload_fp4(strata::CudaBackend& backend, int device, std::uint64_t rows, std::uint64_t columns,
                              std::uint8_t seed, HostWeight& keep, bool nan_scale = false) {
    strata::CudaWeightDescriptor descriptor;
    descriptor.encoding = strata::CudaWeightEncoding::Fp4E2m1Group32;
    descriptor.dtype = strata::SafetensorsDtype::I8;
    descriptor.rows = rows;
    descriptor.columns = columns;
    descriptor.packed_columns = (columns + 1U) / 2U;
    descriptor.scale_columns = (columns + 31U) / 32U;
    descriptor.group_size = 32U;
    keep.weights.resize(static_cast<std::size_t>(rows * descriptor.packed_columns));
    for (std::uint64_t row = 0U; row < rows; ++row)
        for (std::uint64_t packed = 0U; packed < descriptor.packed_columns; ++packed) {
            const auto low = static_cast<std::uint8_t>((seed + row * 3U + packed * 5U) & 0x0FU);
            const auto high = static_cast<std::uint8_t>((seed + row * 7U + packed * 11U + 1U) & 0x0FU);
            keep.weights[row * descriptor.packed_columns + packed] =
                static_cast<std::byte>(low | static_cast<std::uint8_t>(high << 4U));
        }
    keep.scales.resize(static_cast<std::size_t>(rows * descriptor.scale_columns));
    for (std::size_t index = 0U; index < keep.scales.size(); ++index)
        keep.scales[index] = nan_scale ? std::byte{0xFFU}
                                       : static_cast<std::byte>(0x78U + static_cast<std::uint8_t>((index + seed) % 3U));
    strata::CudaWeight result;
    if (!backend.upload(device, descriptor, keep.weights, keep.scales, result).ok()) ++g_failures;
    return result;
}

// ref: upload_fp8, tests/test_cuda_backend.cpp:102-126
strata::CudaWeight upload_fp8(strata::CudaBackend& backend, int device, std::uint64_t rows, std::uint64_t columns,
                              std::uint8_t seed, HostWeight& keep) {
    strata::CudaWeightDescriptor descriptor;
    descriptor.encoding = strata::CudaWeightEncoding::Fp8E4m3Block128;
    descriptor.dtype = strata::SafetensorsDtype::F8E4M3;
    descriptor.rows = rows;
    descriptor.columns = columns;
    descriptor.packed_columns = columns;
    descriptor.scale_columns = (columns + 127U) / 128U;
    descriptor.group_size = 128U;
    constexpr std::array<std::uint8_t, 8> encodings{0x00U, 0x30U, 0xB0U, 0x38U, 0xB8U, 0x40U, 0xC0U, 0x28U};
    keep.weights.resize(static_cast<std::size_t>(rows * columns));
    for (std::size_t index = 0U; index < keep.weights.size(); ++index)
        keep.weights[index] = static_cast<std::byte>(encodings[(index + seed) % encodings.size()]);
    const auto scale_rows = (rows + 127U) / 128U;
    keep.scales.assign(static_cast<std::size_t>(scale_rows * descriptor.scale_columns), std::byte{0x78U});
    strata::CudaWeight result;
    if (!backend.upload(device, descriptor, keep.weights, keep.scales, result).ok()) ++g_failures;
    return result;
}

// compressed-tensors "nvfp4-pack-quantized" (Laguna routed experts): E2M1 nibble pairs, one E4M3 scale per 16 columns,
// one FP32 per-tensor divisor.  Scale bytes stay in the normal range of E4M3 (0x30 .. 0x3F: 0.5 .. 1.875).
strata::CudaWeight upload_nvfp4(strata::CudaBackend& backend, int device, std::uint64_t rows, std::uint64_t columns,
                                std::uint8_t seed, float global_scale, HostWeight& keep) {
    strata::CudaWeightDescriptor descriptor;
    descriptor.encoding = strata::CudaWeightEncoding::Nvfp4Group16;
    descriptor.dtype = strata::SafetensorsDtype::U8;
    descriptor.rows = rows;
    descriptor.columns = columns;
    descriptor.packed_columns = columns / 2U;
    descriptor.scale_columns = columns / 16U;
    descriptor.group_size = 16U;
    descriptor.global_scale = global_scale;
    keep.weights.resize(static_cast<std::size_t>(rows * descriptor.packed_columns));
    for (std::uint64_t row = 0U; row < rows; ++row)
        for (std::uint64_t packed = 0U; packed < descriptor.packed_columns; ++packed) {
            const auto low = static_cast<std::uint8_t>((seed + row * 5U + packed * 3U) & 0x0FU);
            const auto high = static_cast<std::uint8_t>((seed + row * 11U + packed * 7U + 2U) & 0x0FU);
            keep.weights[row * descriptor.packed_columns + packed] =
                static_cast<std::byte>(low | static_cast<std::uint8_t>(high << 4U));
        }
    keep.scales.resize(static_cast<std::size_t>(rows * descriptor.scale_columns));
    for (std::size_t index = 0U; index < keep.scales.size(); ++index)
        keep.scales[index] = static_cast<std::byte>(0x30U + static_cast<std::uint8_t>((index * 7U + seed) % 16U));
    strata::CudaWeight result;
    if (!backend.upload(device, descriptor, keep.weights, keep.scales, result).ok()) ++g_failures;
    return result;
}

const uint8_t* u8(const std::vector<std::byte>& v) { return reinterpret_cast<const uint8_t*>(v.data()); }

std::vector<float> oracle_int4_expert(const HostWeight& gate, const HostWeight& up, const HostWeight& down,
                                      std::span<const float> hidden, std::uint32_t rows, std::uint32_t H,
                                      std::uint32_t I) {
    orc_expert ex{};
    ex.gate = {2, I, H, gate.weights.data(), gate.scales.data(), 1.0F};
    ex.up = {2, I, H, up.weights.data(), up.scales.data(), 1.0F};
    ex.down = {2, H, I, down.weights.data(), down.scales.data(), 1.0F};
    std::vector<float> out(static_cast<std::size_t>(rows) * H), a(I), u(I);
    for (std::uint32_t r = 0; r < rows; ++r)
        if (orc_expert_ffn(&ex, hidden.data() + static_cast<std::size_t>(r) * H, 1.0F, 1, 0, a.data(), u.data(),
                           out.data() + static_cast<std::size_t>(r) * H) != 0)
            ++g_failures;
    return out;
}

// ---------------------------------------------------------------------------------------------
// ref: TEST_CASE("native CUDA backend batches reusable target-shape GLM INT4 MoE commands")
void glm_int4_target_shape_command() {
    const auto devices = strata::CudaBackend::available_devices();
    if (!strata::CudaBackend::compiled() || devices.empty()) return;
    constexpr std::uint32_t rows = 2U;
    constexpr std::uint64_t hidden_columns = 6144U;
    constexpr std::uint64_t intermediate_columns = 2048U;
    const int device = devices.front();
    strata::CudaBackend backend;
    const std::array<int, 1> selected{device};
    REQUIRE(backend.initialize(selected, true).ok());

    HostWeight h[9];
    auto gate0 = upload_int4(backend, device, intermediate_columns, hidden_columns, 1U, h[0]);
    auto up0 = upload_int4(backend, device, intermediate_columns, hidden_columns, 3U, h[1]);
    auto down0 = upload_int4(backend, device, hidden_columns, intermediate_columns, 5U, h[2]);
    auto gate1 = upload_int4(backend, device, intermediate_columns, hidden_columns, 7U, h[3]);
    auto up1 = upload_int4(backend, device, intermediate_columns, hidden_columns, 9U, h[4]);
    auto down1 = upload_int4(backend, device, hidden_columns, intermediate_columns, 11U, h[5]);
    auto shared_gate = upload_int4(backend, device, intermediate_columns, hidden_columns, 13U, h[6]);
    auto shared_up = upload_int4(backend, device, intermediate_columns, hidden_columns, 2U, h[7]);
    auto shared_down = upload_int4(backend, device, hidden_columns, intermediate_columns, 4U, h[8]);
    std::vector<float> hidden(rows * hidden_columns);
    for (std::size_t index = 0U; index < hidden.size(); ++index)
        hidden[index] = static_cast<float>(static_cast<int>(index % 13U) - 6) / 16.0F;
    const auto expected0 = oracle_int4_expert(h[0], h[1], h[2], hidden, rows, hidden_columns, intermediate_columns);
    const auto expected1 = oracle_int4_expert(h[3], h[4], h[5], hidden, rows, hidden_columns, intermediate_columns);
    const auto expected_shared =
        oracle_int4_expert(h[6], h[7], h[8], hidden, rows, hidden_columns, intermediate_columns);
    const std::array<strata::CudaMoeExpert, 2> routed{{
        {&gate0, &up0, &down0, 1.0F},
        {&gate1, &up1, &down1, 1.0F},
    }};
    const strata::CudaMoeExpert shared{&shared_gate, &shared_up, &shared_down, 1.0F};
    std::vector<float> routed_output(2U * rows * hidden_columns), shared_output(rows * hidden_columns);
    REQUIRE(backend.enqueue_moe(device, hidden, rows, routed, &shared).ok());
    REQUIRE(backend.collect_moe(device, routed_output, shared_output).ok());
    // The reference compares two passes through the same device arithmetic within 1e-4 absolute.  Here
    // the expected values come from a CPU FP32 accumulation in another order, so the bound is 1e-4 of
    // the largest expected magnitude plus 1e-4 (the values of this pattern reach a few hundred).
    float scale = 0.0F;
    for (float v : expected0) scale = std::max(scale, std::fabs(v));
    for (float v : expected1) scale = std::max(scale, std::fabs(v));
    for (float v : expected_shared) scale = std::max(scale, std::fabs(v));
    const float tol = 1.0e-4F * scale + 1.0e-4F;
    float worst = 0.0F;
    for (std::size_t index = 0U; index < expected0.size(); ++index) {
        worst = std::max(worst, std::fabs(routed_output[index] - expected0[index]));
        worst = std::max(worst, std::fabs(routed_output[expected0.size() + index] - expected1[index]));
        worst = std::max(worst, std::fabs(shared_output[index] - expected_shared[index]));
    }
    std::printf("glm int4 command: max |difference| %.3e, largest expected %.3e, bound %.3e\n", worst, scale, tol);
    REQUIRE(worst <= tol);
    const auto first = backend.stats();
    REQUIRE(backend.enqueue_moe(device, hidden, rows, routed, &shared).ok());
    REQUIRE(backend.collect_moe(device, routed_output, shared_output).ok());
    const auto second = backend.stats();
    REQUIRE(second.workspace_allocation_calls == first.workspace_allocation_calls);   // the workspace is reused
    REQUIRE(second.deepseek_moe_calls - first.deepseek_moe_calls == 1U);

    // protocol: one command in flight; NVFP4 / plain coefficient rule is INT4-only folding
    REQUIRE(backend.enqueue_moe(device, hidden, rows, routed, &shared).ok());
    REQUIRE(!backend.enqueue_moe(device, hidden, rows, routed, &shared).ok());
    REQUIRE(!backend.synchronize(device).ok());
    REQUIRE(backend.collect_moe(device, routed_output, shared_output).ok());
    REQUIRE(!backend.collect_moe(device, routed_output, shared_output).ok());
    const strata::CudaMoeExpert bad_shared{&shared_gate, &shared_up, &shared_down, 0.5F};
    REQUIRE(!backend.enqueue_moe(device, hidden, rows, routed, &bad_shared).ok());     // shared coefficient must be 1
    std::vector<float> short_hidden(hidden.begin(), hidden.end() - 1);
    REQUIRE(!backend.enqueue_moe(device, short_hidden, rows, routed, &shared).ok());   // hidden span of the wrong size
    std::vector<float> nan_hidden = hidden;
    nan_hidden[5] = std::numeric_limits<float>::quiet_NaN();
    REQUIRE(!backend.enqueue_moe(device, nan_hidden, rows, routed, &shared).ok());      // non-finite hidden rejected
    REQUIRE(backend.synchronize(device).ok());
}

// ---------------------------------------------------------------------------------------------
// The Laguna command: NVFP4 routed experts (hidden 2048, intermediate 1024 here), three rows.  The reference has no
// test of its own for this encoding on the MoE command; the case is this repository's, run on both backends against
// the CPU checker (decode, scale direction = divide by the per-tensor value, FP32 accumulation in another order).
void laguna_nvfp4_command() {
    const auto devices = strata::CudaBackend::available_devices();
    if (!strata::CudaBackend::compiled() || devices.empty()) return;
    constexpr std::uint32_t rows = 3U;
    constexpr std::uint64_t hidden_columns = 2048U, intermediate_columns = 1024U;
    const int device = devices.front();
    strata::CudaBackend backend;
    const std::array<int, 1> selected{device};
    REQUIRE(backend.initialize(selected, false).ok());
    HostWeight h[6];
    const float gs[6] = {384.0F, 448.0F, 512.0F, 320.0F, 640.0F, 416.0F};
    auto gate0 = upload_nvfp4(backend, device, intermediate_columns, hidden_columns, 1U, gs[0], h[0]);
    auto up0 = upload_nvfp4(backend, device, intermediate_columns, hidden_columns, 4U, gs[1], h[1]);
    auto down0 = upload_nvfp4(backend, device, hidden_columns, intermediate_columns, 7U, gs[2], h[2]);
    auto gate1 = upload_nvfp4(backend, device, intermediate_columns, hidden_columns, 10U, gs[3], h[3]);
    auto up1 = upload_nvfp4(backend, device, intermediate_columns, hidden_columns, 13U, gs[4], h[4]);
    auto down1 = upload_nvfp4(backend, device, hidden_columns, intermediate_columns, 2U, gs[5], h[5]);
    std::vector<float> hidden(rows * hidden_columns);
    for (std::size_t index = 0U; index < hidden.size(); ++index)
        hidden[index] = static_cast<float>(static_cast<int>(index % 11U) - 5) / 8.0F;
    std::vector<float> expected[2];
    for (int e = 0; e < 2; ++e) {
        orc_expert ex{};
        ex.gate = {1, (uint32_t)intermediate_columns, (uint32_t)hidden_columns, h[3 * e].weights.data(), h[3 * e].scales.data(), gs[3 * e]};
        ex.up = {1, (uint32_t)intermediate_columns, (uint32_t)hidden_columns, h[3 * e + 1].weights.data(), h[3 * e + 1].scales.data(), gs[3 * e + 1]};
        ex.down = {1, (uint32_t)hidden_columns, (uint32_t)intermediate_columns, h[3 * e + 2].weights.data(), h[3 * e + 2].scales.data(), gs[3 * e + 2]};
        expected[e].resize(static_cast<std::size_t>(rows) * hidden_columns);
        std::vector<float> a(intermediate_columns), u(intermediate_columns);
        for (std::uint32_t r = 0; r < rows; ++r)
            REQUIRE(orc_expert_ffn(&ex, hidden.data() + static_cast<std::size_t>(r) * hidden_columns, 1.0F, 0, 0, a.data(), u.data(),
                                   expected[e].data() + static_cast<std::size_t>(r) * hidden_columns) == 0);
    }
    const std::array<strata::CudaMoeExpert, 2> routed{{
        {&gate0, &up0, &down0, 1.0F},
        {&gate1, &up1, &down1, 1.0F},
    }};
    std::vector<float> routed_output(2U * rows * hidden_columns), none;
    REQUIRE(backend.enqueue_moe(device, hidden, rows, routed, nullptr).ok());
    REQUIRE(backend.collect_moe(device, routed_output, none).ok());
    double num = 0.0, den = 0.0;
    for (int e = 0; e < 2; ++e)
        for (std::size_t index = 0U; index < expected[e].size(); ++index) {
            const double d = static_cast<double>(routed_output[e * expected[e].size() + index]) - expected[e][index];
            num += d * d;
            den += static_cast<double>(expected[e][index]) * expected[e][index];
        }
    const double rel = std::sqrt(num / den);
    std::printf("laguna nvfp4 command: relative L2 difference to the checker %.3e\n", rel);
    REQUIRE(den > 0.0 && rel <= 2.0e-5);
}

// ---------------------------------------------------------------------------------------------
// The Inkling sink command: both always-on sink experts are plain BF16 and run on every row as one dense enqueue_moe
// command beside the routed NVFP4 command (ref: src/models/inkling/inkling_runtime.cpp:870-900).  The reference has no
// command test of its own for plain BF16 experts; the case is this repository's, run on both backends against the CPU
// checker.
strata::CudaWeight upload_bf16(strata::CudaBackend& backend, int device, std::uint64_t rows, std::uint64_t columns,
                               std::uint32_t seed, HostWeight& keep) {
    strata::CudaWeightDescriptor descriptor;
    descriptor.encoding = strata::CudaWeightEncoding::Plain;
    descriptor.dtype = strata::SafetensorsDtype::Bf16;
    descriptor.rows = rows;
    descriptor.columns = columns;
    keep.weights.resize(static_cast<std::size_t>(rows * columns * 2U));
    for (std::uint64_t index = 0U; index < rows * columns; ++index) {
        // small exactly representable values: multiples of 1/64 in [-15/64, 15/64]
        const int q = static_cast<int>((index * 7U + seed * 13U + (index >> 9U)) % 31U) - 15;
        const auto b = bf16(static_cast<float>(q) / 64.0F);
        keep.weights[2U * index] = b[0];
        keep.weights[2U * index + 1U] = b[1];
    }
    keep.scales.clear();
    strata::CudaWeight result;
    if (!backend.upload(device, descriptor, keep.weights, keep.scales, result).ok()) ++g_failures;
    return result;
}

void inkling_bf16_sink_command() {
    const auto devices = strata::CudaBackend::available_devices();
    if (!strata::CudaBackend::compiled() || devices.empty()) return;
    constexpr std::uint32_t rows = 5U;
    constexpr std::uint64_t hidden_columns = 1024U, intermediate_columns = 512U;
    const int device = devices.front();
    strata::CudaBackend backend;
    const std::array<int, 1> selected{device};
    REQUIRE(backend.initialize(selected, false).ok());
    HostWeight h[6];
    auto gate0 = upload_bf16(backend, device, intermediate_columns, hidden_columns, 1U, h[0]);
    auto up0 = upload_bf16(backend, device, intermediate_columns, hidden_columns, 2U, h[1]);
    auto down0 = upload_bf16(backend, device, hidden_columns, intermediate_columns, 3U, h[2]);
    auto gate1 = upload_bf16(backend, device, intermediate_columns, hidden_columns, 4U, h[3]);
    auto up1 = upload_bf16(backend, device, intermediate_columns, hidden_columns, 5U, h[4]);
    auto down1 = upload_bf16(backend, device, hidden_columns, intermediate_columns, 6U, h[5]);
    std::vector<float> hidden(rows * hidden_columns);
    for (std::size_t index = 0U; index < hidden.size(); ++index)
        hidden[index] = static_cast<float>(static_cast<int>(index % 17U) - 8) / 32.0F;
    std::vector<float> expected[2];
    for (int e = 0; e < 2; ++e) {
        orc_expert ex{};
        ex.gate = {3, (uint32_t)intermediate_columns, (uint32_t)hidden_columns, h[3 * e].weights.data(), nullptr, 1.0F};
        ex.up = {3, (uint32_t)intermediate_columns, (uint32_t)hidden_columns, h[3 * e + 1].weights.data(), nullptr, 1.0F};
        ex.down = {3, (uint32_t)hidden_columns, (uint32_t)intermediate_columns, h[3 * e + 2].weights.data(), nullptr, 1.0F};
        expected[e].resize(static_cast<std::size_t>(rows) * hidden_columns);
        std::vector<float> a(intermediate_columns), u(intermediate_columns);
        for (std::uint32_t r = 0; r < rows; ++r)
            REQUIRE(orc_expert_ffn(&ex, hidden.data() + static_cast<std::size_t>(r) * hidden_columns, 1.0F, 0, 0, a.data(), u.data(),
                                   expected[e].data() + static_cast<std::size_t>(r) * hidden_columns) == 0);
    }
    const std::array<strata::CudaMoeExpert, 2> sinks{{
        {&gate0, &up0, &down0, 1.0F},
        {&gate1, &up1, &down1, 1.0F},
    }};
    std::vector<float> output(2U * rows * hidden_columns), none;
    REQUIRE(backend.enqueue_moe(device, hidden, rows, sinks, nullptr).ok());
    REQUIRE(backend.collect_moe(device, output, none).ok());
    double num = 0.0, den = 0.0;
    for (int e = 0; e < 2; ++e)
        for (std::size_t index = 0U; index < expected[e].size(); ++index) {
            const double d = static_cast<double>(output[e * expected[e].size() + index]) - expected[e][index];
            num += d * d;
            den += static_cast<double>(expected[e][index]) * expected[e][index];
        }
    const double rel = std::sqrt(num / den);
    std::printf("inkling bf16 sink command: relative L2 difference to the checker %.3e\n", rel);
    REQUIRE(den > 0.0 && rel <= 2.0e-5);
}

// ---------------------------------------------------------------------------------------------
// ref: TEST_CASE("native CUDA backend enqueues exact grouped DeepSeek MoE when available")
// Run at hidden = intermediate = 128 (the reference case uses 32; this library's shapes are multiples of 128) and at the
// DeepSeek-V4 shape 4096 / 2048, the shape of the reference's host-versus-device exactness test
// (tests/test_deepseek_host_expert.cpp:456-496).
template <std::uint64_t hidden_columns, std::uint64_t intermediate_columns>
void deepseek_exact_commands() {
    const auto devices = strata::CudaBackend::available_devices();
    if (!strata::CudaBackend::compiled() || devices.empty()) return;
    const int device = devices.front();
    strata::CudaBackend backend;
    const std::array<int, 1> selected{device};
    REQUIRE(backend.initialize(selected, true).ok());

    HostWeight h[9];
    auto routed0_w1 = upload_fp4(backend, device, intermediate_columns, hidden_columns, 1U, h[0]);
    auto routed0_w3 = upload_fp4(backend, device, intermediate_columns, hidden_columns, 6U, h[1]);
    auto routed0_w2 = upload_fp4(backend, device, hidden_columns, intermediate_columns, 11U, h[2]);
    auto routed1_w1 = upload_fp4(backend, device, intermediate_columns, hidden_columns, 3U, h[3]);
    auto routed1_w3 = upload_fp4(backend, device, intermediate_columns, hidden_columns, 9U, h[4]);
    auto routed1_w2 = upload_fp4(backend, device, hidden_columns, intermediate_columns, 14U, h[5]);
    auto shared_w1 = upload_fp8(backend, device, intermediate_columns, hidden_columns, 1U, h[6]);
    auto shared_w3 = upload_fp8(backend, device, intermediate_columns, hidden_columns, 4U, h[7]);
    auto shared_w2 = upload_fp8(backend, device, hidden_columns, intermediate_columns, 7U, h[8]);

    std::array<float, hidden_columns> hidden{};
    for (std::size_t index = 0U; index < hidden.size(); ++index)
        hidden[index] = static_cast<float>(static_cast<int>(index % 9U) - 4) * 0.125F;
    constexpr float coefficient0 = 0.75F;
    constexpr float coefficient1 = 0.3125F;
    std::vector<float> expected0(hidden_columns), expected1(hidden_columns), expected_shared(hidden_columns),
        scratch(intermediate_columns);
    REQUIRE(orc_dsv4_expert(expected0.data(), hidden.data(), u8(h[0].weights), u8(h[0].scales), u8(h[1].weights),
                            u8(h[1].scales), u8(h[2].weights), u8(h[2].scales), hidden_columns, intermediate_columns,
                            coefficient0, 10.0F, scratch.data()) == 0);
    REQUIRE(orc_dsv4_expert(expected1.data(), hidden.data(), u8(h[3].weights), u8(h[3].scales), u8(h[4].weights),
                            u8(h[4].scales), u8(h[5].weights), u8(h[5].scales), hidden_columns, intermediate_columns,
                            coefficient1, 10.0F, scratch.data()) == 0);
    REQUIRE(orc_dsv4_fp8_shared(expected_shared.data(), hidden.data(), u8(h[6].weights), u8(h[6].scales),
                                u8(h[7].weights), u8(h[7].scales), u8(h[8].weights), u8(h[8].scales), hidden_columns,
                                intermediate_columns, 10.0F, scratch.data()) == 0);

    const std::array<strata::CudaDeepSeekMoeExpert, 2> routed{{
        {&routed0_w1, &routed0_w3, &routed0_w2, coefficient0},
        {&routed1_w1, &routed1_w3, &routed1_w2, coefficient1},
    }};
    const strata::CudaDeepSeekMoeExpert shared{&shared_w1, &shared_w3, &shared_w2, 1.0F};
    REQUIRE(backend.enqueue_deepseek_moe(device, hidden, routed, &shared, 10.0F).ok());
    REQUIRE(!backend.enqueue_deepseek_moe(device, hidden, routed, &shared, 10.0F).ok());
    REQUIRE(!backend.synchronize(device).ok());

    std::array<float, 2U * hidden_columns> routed_output{};
    std::array<float, hidden_columns> shared_output{};
    REQUIRE(backend.collect_deepseek_moe(device, routed_output, shared_output).ok());
    for (std::size_t column = 0U; column < hidden_columns; ++column) {
        REQUIRE(std::bit_cast<std::uint32_t>(routed_output[column]) == std::bit_cast<std::uint32_t>(expected0[column]));
        REQUIRE(std::bit_cast<std::uint32_t>(routed_output[hidden_columns + column]) ==
                std::bit_cast<std::uint32_t>(expected1[column]));
        REQUIRE(std::bit_cast<std::uint32_t>(shared_output[column]) ==
                std::bit_cast<std::uint32_t>(expected_shared[column]));
        REQUIRE((std::bit_cast<std::uint32_t>(routed_output[column]) & 0xFFFFU) == 0U);   // BF16-rounded outputs
        REQUIRE((std::bit_cast<std::uint32_t>(shared_output[column]) & 0xFFFFU) == 0U);
    }

    // the row-grouped form: two rows, expert 0 serves both, expert 1 only the second; the shared expert both
    std::array<float, 2U * hidden_columns> page{};
    for (std::size_t index = 0U; index < page.size(); ++index)
        page[index] = index < hidden_columns ? hidden[index] : static_cast<float>(static_cast<int>(index % 7U) - 3) * 0.25F;
    const std::array<std::uint32_t, 2> rows0{0U, 1U};
    const std::array<float, 2> coefs0{coefficient0, 0.5F};
    const std::array<std::uint32_t, 1> rows1{1U};
    const std::array<float, 1> coefs1{coefficient1};
    const std::array<strata::CudaDeepSeekMoeRowGroup, 2> groups{{
        {&routed0_w1, &routed0_w3, &routed0_w2, {}, rows0, coefs0},
        {&routed1_w1, &routed1_w3, &routed1_w2, {}, rows1, coefs1},
    }};
    const std::array<std::uint32_t, 2> shared_rows{0U, 1U};
    std::array<float, 3U * hidden_columns> grouped_output{};
    std::array<float, 2U * hidden_columns> grouped_shared{};
    REQUIRE(backend.enqueue_deepseek_moe_rows(device, page, 2U, groups, &shared, shared_rows, 10.0F).ok());
    REQUIRE(backend.collect_deepseek_moe_rows(device, grouped_output, grouped_shared).ok());
    std::vector<float> e01(hidden_columns), e11(hidden_columns), es1(hidden_columns);
    REQUIRE(orc_dsv4_expert(e01.data(), page.data() + hidden_columns, u8(h[0].weights), u8(h[0].scales),
                            u8(h[1].weights), u8(h[1].scales), u8(h[2].weights), u8(h[2].scales), hidden_columns,
                            intermediate_columns, 0.5F, 10.0F, scratch.data()) == 0);
    REQUIRE(orc_dsv4_expert(e11.data(), page.data() + hidden_columns, u8(h[3].weights), u8(h[3].scales),
                            u8(h[4].weights), u8(h[4].scales), u8(h[5].weights), u8(h[5].scales), hidden_columns,
                            intermediate_columns, coefficient1, 10.0F, scratch.data()) == 0);
    REQUIRE(orc_dsv4_fp8_shared(es1.data(), page.data() + hidden_columns, u8(h[6].weights), u8(h[6].scales),
                                u8(h[7].weights), u8(h[7].scales), u8(h[8].weights), u8(h[8].scales), hidden_columns,
                                intermediate_columns, 10.0F, scratch.data()) == 0);
    for (std::size_t column = 0U; column < hidden_columns; ++column) {
        // group-major, inside a group in the group's own row order
        REQUIRE(std::bit_cast<std::uint32_t>(grouped_output[column]) == std::bit_cast<std::uint32_t>(expected0[column]));
        REQUIRE(std::bit_cast<std::uint32_t>(grouped_output[hidden_columns + column]) ==
                std::bit_cast<std::uint32_t>(e01[column]));
        REQUIRE(std::bit_cast<std::uint32_t>(grouped_output[2U * hidden_columns + column]) ==
                std::bit_cast<std::uint32_t>(e11[column]));
        REQUIRE(std::bit_cast<std::uint32_t>(grouped_shared[column]) ==
                std::bit_cast<std::uint32_t>(expected_shared[column]));
        REQUIRE(std::bit_cast<std::uint32_t>(grouped_shared[hidden_columns + column]) ==
                std::bit_cast<std::uint32_t>(es1[column]));
    }

    // Non-finite W1/W3 output is an explicit failure and never reaches the caller.
    HostWeight bad;
    auto invalid_w1 = upload_fp4(backend, device, intermediate_columns, hidden_columns, 2U, bad, true);
    const std::array<strata::CudaDeepSeekMoeExpert, 1> invalid_routed{{
        {&invalid_w1, &routed0_w3, &routed0_w2, coefficient0},
    }};
    std::array<float, hidden_columns> invalid_output{};
    invalid_output.fill(123.0F);
    REQUIRE(backend.enqueue_deepseek_moe(device, hidden, invalid_routed, nullptr, 10.0F).ok());
    REQUIRE(!backend.collect_deepseek_moe(device, invalid_output, {}).ok());
    REQUIRE(std::all_of(invalid_output.begin(), invalid_output.end(), [](float value) { return value == 123.0F; }));

    // A failed collect drains the command so that the workspace can be reused.
    REQUIRE(backend.enqueue_deepseek_moe(device, hidden, routed, &shared, 10.0F).ok());
    REQUIRE(!backend.collect_deepseek_moe(device, {}, {}).ok());
    REQUIRE(backend.enqueue_deepseek_moe(device, hidden, routed, &shared, 10.0F).ok());
    REQUIRE(backend.collect_deepseek_moe(device, routed_output, shared_output).ok());
}

}  // namespace

#ifdef STRATA_TEST_REFERENCE_BACKEND
// ---------------------------------------------------------------------------------------------
// The router projection's summation order: the reference runs the gate through CudaBackend::matmul on a plain BF16
// weight (bf16_matvec_kernel / bf16_matvec_rows_kernel, kernels/cuda/backend.cu:651-728).  The CPU checker's
// orc_router_logits restates that order; here the reference's own kernels have to reproduce it bit for bit, for one row
// (the matvec kernel), a few rows and more rows than one tile of the rows kernel (16).  This library's logits are
// compared with the same checker function in the GPU parity tests.
void reference_router_projection_order() {
    const auto devices = strata::CudaBackend::available_devices();
    if (!strata::CudaBackend::compiled() || devices.empty()) return;
    constexpr std::uint32_t experts = 256U, hidden_columns = 4096U;
    const int device = devices.front();
    strata::CudaBackend backend;
    const std::array<int, 1> selected{device};
    REQUIRE(backend.initialize(selected, false).ok());
    std::vector<std::uint16_t> w(static_cast<std::size_t>(experts) * hidden_columns);
    std::uint32_t state = 12345U;
    auto next_bf16 = [&](float scale) {
        state = state * 1664525U + 1013904223U;
        const float v = (static_cast<float>((state >> 8) & 0xFFFFU) / 65535.0F - 0.5F) * scale;
        const auto b = bf16(v);
        return static_cast<std::uint16_t>(static_cast<unsigned>(b[0]) | (static_cast<unsigned>(b[1]) << 8));
    };
    for (auto& v : w) v = next_bf16(0.08F);
    strata::CudaWeightDescriptor descriptor;
    descriptor.encoding = strata::CudaWeightEncoding::Plain;
    descriptor.dtype = strata::SafetensorsDtype::Bf16;
    descriptor.rows = experts;
    descriptor.columns = hidden_columns;
    strata::CudaWeight gate;
    const std::span<const std::byte> bytes(reinterpret_cast<const std::byte*>(w.data()), w.size() * 2U);
    REQUIRE(backend.upload(device, descriptor, bytes, {}, gate).ok());
    for (std::uint32_t rows : {1U, 3U, 20U}) {
        std::vector<std::uint16_t> x(static_cast<std::size_t>(rows) * hidden_columns);
        for (auto& v : x) v = next_bf16(6.0F);
        std::vector<float> xf(x.size());
        for (std::size_t i = 0; i < x.size(); ++i) xf[i] = std::bit_cast<float>(static_cast<std::uint32_t>(x[i]) << 16);
        std::vector<float> got(static_cast<std::size_t>(rows) * experts), want(got.size());
        REQUIRE(backend.matmul(gate, xf, rows, got).ok());
        orc_router_logits(x.data(), w.data(), rows, hidden_columns, experts, want.data());
        std::size_t differ = 0;
        for (std::size_t i = 0; i < got.size(); ++i)
            differ += std::bit_cast<std::uint32_t>(got[i]) != std::bit_cast<std::uint32_t>(want[i]);
        std::printf("reference router projection, %u row(s): %zu of %zu logits differ from the checker\n", rows, differ,
                    got.size());
        REQUIRE(differ == 0U);
    }
}
#endif

// ---------------------------------------------------------------------------------------------
// Timing of one command shape through whichever backend this file was compiled against: the GLM INT4 command at the
// target shape (hidden 6144, intermediate 2048) with `experts` routed experts over `rows` rows, host buffers in and
// out (the reference command's contract), wall clock around enqueue + collect, best of `repeats` after two warm-ups.
void time_glm_command(std::uint32_t rows, std::uint32_t experts, int repeats) {
    const auto devices = strata::CudaBackend::available_devices();
    if (!strata::CudaBackend::compiled() || devices.empty()) return;
    constexpr std::uint64_t hidden_columns = 6144U, intermediate_columns = 2048U;
    const int device = devices.front();
    strata::CudaBackend backend;
    const std::array<int, 1> selected{device};
    REQUIRE(backend.initialize(selected, false).ok());
    std::vector<HostWeight> keep(3U * experts);
    std::vector<strata::CudaWeight> w(3U * experts);
    for (std::uint32_t e = 0; e < experts; ++e) {
        w[3U * e] = upload_int4(backend, device, intermediate_columns, hidden_columns, (std::uint8_t)(1U + e), keep[3U * e]);
        w[3U * e + 1U] = upload_int4(backend, device, intermediate_columns, hidden_columns, (std::uint8_t)(3U + e), keep[3U * e + 1U]);
        w[3U * e + 2U] = upload_int4(backend, device, hidden_columns, intermediate_columns, (std::uint8_t)(5U + e), keep[3U * e + 2U]);
    }
    std::vector<strata::CudaMoeExpert> routed;
    for (std::uint32_t e = 0; e < experts; ++e) routed.push_back({&w[3U * e], &w[3U * e + 1U], &w[3U * e + 2U], 1.0F});
    std::vector<float> hidden(static_cast<std::size_t>(rows) * hidden_columns);
    for (std::size_t index = 0U; index < hidden.size(); ++index)
        hidden[index] = static_cast<float>(static_cast<int>(index % 13U) - 6) / 16.0F;
    std::vector<float> routed_output(static_cast<std::size_t>(experts) * rows * hidden_columns), none;
    double best = 1.0e30;
    for (int it = 0; it < repeats + 2; ++it) {
        const auto t0 = std::chrono::steady_clock::now();
        REQUIRE(backend.enqueue_moe(device, hidden, rows, routed, nullptr).ok());
        REQUIRE(backend.collect_moe(device, routed_output, none).ok());
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        if (it >= 2) best = std::min(best, ms);
    }
    double checksum = 0.0;
    for (float v : routed_output) checksum += v;
    std::printf("%s: glm int4 command, %u experts x %u rows: %.3f ms per command (checksum %.6e)\n", BACKEND_NAME, experts, rows,
                best, checksum);
}

int main(int argc, char** argv) {
    if (argc > 1 && std::strcmp(argv[1], "--compile-check") == 0) return 0;
    if (argc > 1 && std::strcmp(argv[1], "--time") == 0) {
        for (std::uint32_t rows : {1U, 2U, 16U, 128U, 512U}) time_glm_command(rows, 8U, 5);
        return g_failures == 0 ? 0 : 1;
    }
    glm_int4_target_shape_command();
    laguna_nvfp4_command();
    inkling_bf16_sink_command();
    deepseek_exact_commands<128U, 128U>();
    deepseek_exact_commands<4096U, 2048U>();
#ifdef STRATA_TEST_REFERENCE_BACKEND
    reference_router_projection_order();
#endif
    if (g_failures != 0) {
        std::fprintf(stderr, "%d case(s) failed\n", g_failures);
        return 1;
    }
    std::printf(BACKEND_NAME " cases passed\n");
    return 0;
}
