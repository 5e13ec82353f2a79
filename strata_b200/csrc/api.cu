// Host side of the C ABI declared in include/strata_moe.h: contexts, resident weights,
// workspaces and the launch sequence of one MoE layer.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <nvtx3/nvToolsExt.h>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

using namespace smoe;

struct strata_moe_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    std::string err;
    uint32_t* d_status = nullptr;
    uint32_t* h_status = nullptr;  // pinned
    strata_moe_stats stats{};
    bool timing = false;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    cudaStream_t side = nullptr;                  // shared expert runs here, beside the routed experts
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    // host-buffer calls in chunks: copies in and out run on their own streams beside the compute stream
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t ev_in[4] = {}, ev_done[4] = {};
    cudaEvent_t pev[STRATA_MOE_PHASES + 1] = {};  // phase boundaries of the last timed forward
    bool pev_valid = false;
    unsigned long long launches_at_create = 0;
    unsigned long long* d_router_rechecks = nullptr;   // tokens the fast router handed to the canonical kernels
    uint64_t router_fast_tokens = 0;                    // tokens routed through the fast path
    // handle-based commands (strata_moe_command_*): an internal layer whose expert slots borrow the
    // uploaded weights named by the command in flight
    strata_moe_layer* cmd_layer = nullptr;
    uint32_t cmd_slots = 0;
    int cmd_kind = 0;                  // 0 none, 1 dense command, 2 DSV4 row groups
    uint32_t cmd_n = 0, cmd_rows = 0, cmd_pairs = 0, cmd_shared_rows = 0;
    bool cmd_shared = false;
    std::vector<void*> cmd_scratch;    // device buffers of the command in flight (row lists, gathered rows)
    uint64_t workspace_allocations = 0;
    // Activation workspaces shared by every layer of the context (a model has tens of MoE layers that run one
    // after the other on the context's stream; sizing them per layer would multiply gigabytes by the layer
    // count).  Grown to the largest request; a layer picks the current pointers up at every call.
    void* ws[16] = {};
    void* ws_raw[16] = {};    // the allocations behind ws[]: guard zone, body, guard zone
    strata_moe_layer* ws_owner = nullptr;   // layer whose command holds results in the pool until collected
    size_t ws_bytes[16] = {};
};

enum WsSlot { kWsXg, kWsXgLo, kWsActHi, kWsActLo, kWsY, kWsActF32, kWsXRow, kWsActRow, kWsShActHi, kWsShActLo, kWsShY,
              kWsXStage, kWsOutStage, kWsCount };

struct DeviceTable {
    std::vector<const uint8_t*> packed, scales;
    std::vector<float> global;
    const uint8_t** d_packed = nullptr;
    const uint8_t** d_scales = nullptr;
    float* d_global = nullptr;
    uint32_t* d_emin = nullptr;   // f16 path tables
    float* d_post = nullptr;
};

// Tuning and test switches, read from the environment ONCE when a layer is created (never on the
// per-call path).  -1 / 0 = built-in default.
struct LayerKnobs {
    bool no_f16_path = false;       // STRATA_MOE_NO_F16_PATH: FP4 formats use the general BF16 decoders
    bool no_prefill_path = false;   // STRATA_MOE_NO_PREFILL_PATH: never use the tensor-core tile path
    bool no_stream_ring = false;    // STRATA_MOE_NO_STREAM_RING: small batches use the register-streaming kernels
    bool no_half_y = false;         // STRATA_MOE_NO_HALF_Y: the tensor-core down kernel always stores fp32 expert rows
    bool no_small_front = false;    // STRATA_MOE_NO_SMALL_FRONT: decode batches keep the separate route / group / convert kernels
    int prefill_min_rows = -1;      // STRATA_MOE_PREFILL_MIN_ROWS: average rows per expert for the tensor-core path
    int prefill_down_min_rows = -1; // STRATA_MOE_PREFILL_DOWN_MIN_ROWS
    int prefill_ntile = 0;          // STRATA_MOE_PREFILL_NTILE: 128, 160 or 192
    int mixed_min_rows = -1;        // STRATA_MOE_MIXED_MIN_ROWS
    int mixed_min_tokens = -1;      // STRATA_MOE_MIXED_MIN_TOKENS
    int fast_router_min_tokens = 0; // STRATA_MOE_FAST_ROUTER_MIN_TOKENS: 0 = default (512), negative = never
    int no_spread = 0;              // STRATA_MOE_NO_SPREAD=1: operand conversion per grouped row instead of per source row
    int host_chunks = 0;            // STRATA_MOE_HOST_CHUNKS: token chunks of a host-buffer call (0 = chosen from the rows per expert)
    int stream_ring_max_rows = 8;   // STRATA_MOE_STREAM_RING_MAX_ROWS: largest token tile (8 or 16) given to the ring kernels
};

static LayerKnobs read_knobs() {
    LayerKnobs k;
    auto num = [](const char* name, int dflt) {
        const char* e = getenv(name);
        return e ? atoi(e) : dflt;
    };
    k.no_f16_path = getenv("STRATA_MOE_NO_F16_PATH") != nullptr;
    k.no_prefill_path = getenv("STRATA_MOE_NO_PREFILL_PATH") != nullptr;
    k.no_stream_ring = getenv("STRATA_MOE_NO_STREAM_RING") != nullptr;
    k.prefill_min_rows = num("STRATA_MOE_PREFILL_MIN_ROWS", -1);
    k.prefill_down_min_rows = num("STRATA_MOE_PREFILL_DOWN_MIN_ROWS", -1);
    k.prefill_ntile = num("STRATA_MOE_PREFILL_NTILE", 0);
    k.mixed_min_rows = num("STRATA_MOE_MIXED_MIN_ROWS", -1);
    k.mixed_min_tokens = num("STRATA_MOE_MIXED_MIN_TOKENS", -1);
    k.no_small_front = getenv("STRATA_MOE_NO_SMALL_FRONT") != nullptr;
    k.no_half_y = getenv("STRATA_MOE_NO_HALF_Y") != nullptr;
    k.fast_router_min_tokens = num("STRATA_MOE_FAST_ROUTER_MIN_TOKENS", 0);
    k.stream_ring_max_rows = num("STRATA_MOE_STREAM_RING_MAX_ROWS", 8);
    k.host_chunks = num("STRATA_MOE_HOST_CHUNKS", 0);
    k.no_spread = num("STRATA_MOE_NO_SPREAD", 0);
    return k;
}

struct strata_moe_layer {
    strata_moe_ctx* ctx = nullptr;
    LayerKnobs knobs;
    strata_moe_layer_desc d{};
    uint32_t max_pairs = 0;
    __nv_bfloat16* router = nullptr;
    float* bias = nullptr;
    bool has_bias = false;
    DeviceTable tab[3];
    bool tables_dirty = true;
    __nv_bfloat16* shared_w[3] = {nullptr, nullptr, nullptr};
    const uint8_t** d_shared_ptr[3] = {nullptr, nullptr, nullptr};  // 1-entry tables
    std::vector<void*> owned;
    // workspaces
    float* logits = nullptr;
    uint32_t *ids = nullptr, *counts = nullptr, *offsets = nullptr, *perm = nullptr, *inv = nullptr;
    uint32_t *active = nullptr, *n_active = nullptr;
    float* weights = nullptr;
    void* group_scratch = nullptr;
    __nv_bfloat16 *xg = nullptr, *xg_lo = nullptr, *act_hi = nullptr, *act_lo = nullptr;
    float* y = nullptr;
    __nv_bfloat16 *sh_act_hi = nullptr, *sh_act_lo = nullptr;
    float* sh_y = nullptr;
    __nv_bfloat16* x_stage = nullptr;
    float* out_stage = nullptr;
    void* prefill_scratch = nullptr;
    uint32_t* shared_tiles = nullptr;  // tile list of the shared expert's grouped GEMM
    uint32_t* router_tiles = nullptr;  // tile list of the tensor-core router projection
    uint32_t* router_off2 = nullptr;   // {0, T} for it
    uint32_t* recheck_list = nullptr;  // [max_tokens] tokens the fast router hands to the canonical kernels
    uint32_t* recheck_count = nullptr;
    float* one_global = nullptr;  // device float 1.0 for the shared expert table
    void* d_wmaps = nullptr;      // [3][n_local] tensor-map descriptors of the packed weights
    bool wmaps_ok = false;
    // f16 decode path for the FP4 formats
    bool f16_ok = false;
    bool stream_ok = false;   // shapes and alignments allow the TMA ring kernels
    uint8_t* arena_cur = nullptr;   // weight arena: next free byte of the newest chunk (chunks are in `owned`)
    size_t arena_left = 0, arena_next = 4u << 20;
    void* d_smaps = nullptr;  // [3][n_local][3] tensor maps of the ring kernels
    uint32_t* d_not_ok = nullptr;
    float *act_f32 = nullptr, *x_rowscale = nullptr, *act_rowscale = nullptr;
    // dense command state
    bool dense_in_flight = false;
    uint32_t dense_rows = 0, dense_n = 0;
    bool dense_shared = false;
    float* dense_hidden = nullptr;  // device fp32 [rows, H]
    float* dense_coef = nullptr;
    const uint8_t** dense_ptrs = nullptr;  // device: 6 * n pointers
    float* dense_globals = nullptr;        // device: 3 * n
    void* dense_pinned = nullptr;          // host staging for the tables above
};

namespace {

int fail(strata_moe_ctx* c, int code, const std::string& msg) {
    if (c) c->err = msg;
    return code;
}

// phase boundary i of a timed forward (no-op unless timing is on)
// NVTX range over a host-side scope (the launches of one phase): shows up in a timeline profiler, costs a few
// nanoseconds when none is attached.
struct Range {
    explicit Range(const char* name) { nvtxRangePushA(name); }
    ~Range() { nvtxRangePop(); }
    Range(const Range&) = delete;
    Range& operator=(const Range&) = delete;
};

void mark(strata_moe_ctx* c, int i) {
    if (c->timing) cudaEventRecord(c->pev[i], c->stream);
}

#define CK(call)                                                                             \
    do {                                                                                     \
        cudaError_t e_ = (call);                                                             \
        if (e_ != cudaSuccess)                                                               \
            return fail(ctx, STRATA_MOE_E_CUDA,                                              \
                        std::string(#call) + ": " + cudaGetErrorString(e_));                 \
    } while (0)

template <typename T>
cudaError_t dalloc(strata_moe_layer* L, T** p, size_t n) {
    void* v = nullptr;
    cudaError_t e = cudaMalloc(&v, n ? n * sizeof(T) : sizeof(T));
    if (e == cudaSuccess) {
        L->owned.push_back(v);
        *p = static_cast<T*>(v);
    }
    return e;
}

// Every workspace sits between two 256-byte guard zones filled with a canary byte; strata_moe_check_canaries compares
// them (the device-side check that stands in for a memory checker: a kernel that writes past its buffer is found by the
// tests that call it, without a trap).
constexpr size_t kGuard = 256;
constexpr int kCanary = 0xA5;

cudaError_t ws_reserve(strata_moe_ctx* ctx, int slot, size_t bytes) {
    if (bytes <= ctx->ws_bytes[slot]) return cudaSuccess;
    // nothing enqueued may still use the old buffer
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess && ctx->side) e = cudaStreamSynchronize(ctx->side);
    if (e != cudaSuccess) return e;
    if (ctx->ws_raw[slot]) cudaFree(ctx->ws_raw[slot]);
    ctx->ws[slot] = ctx->ws_raw[slot] = nullptr;
    ctx->ws_bytes[slot] = 0;
    const size_t body = (bytes + kGuard - 1) / kGuard * kGuard;
    e = cudaMalloc(&ctx->ws_raw[slot], body + 2 * kGuard);
    if (e != cudaSuccess) return e;
    uint8_t* raw = static_cast<uint8_t*>(ctx->ws_raw[slot]);
    ctx->ws[slot] = raw + kGuard;
    ctx->ws_bytes[slot] = bytes;
    e = cudaMemset(raw, kCanary, kGuard);
    if (e == cudaSuccess) e = cudaMemset(raw + kGuard + body, kCanary, kGuard);
    // rows the tensor-core path owns are still swept by the f32 -> f16 conversion pass: keep them finite
    if (e == cudaSuccess && slot == kWsActF32) e = cudaMemset(ctx->ws[slot], 0, bytes);
    return e;
}

// The context's current workspaces as this layer's pointers (they may have been regrown by another layer).
void bind_ws(strata_moe_layer* L) {
    strata_moe_ctx* c = L->ctx;
    L->xg = static_cast<__nv_bfloat16*>(c->ws[kWsXg]);
    L->xg_lo = static_cast<__nv_bfloat16*>(c->ws[kWsXgLo]);
    L->act_hi = static_cast<__nv_bfloat16*>(c->ws[kWsActHi]);
    L->act_lo = static_cast<__nv_bfloat16*>(c->ws[kWsActLo]);
    L->y = static_cast<float*>(c->ws[kWsY]);
    L->act_f32 = static_cast<float*>(c->ws[kWsActF32]);
    L->x_rowscale = static_cast<float*>(c->ws[kWsXRow]);
    L->act_rowscale = static_cast<float*>(c->ws[kWsActRow]);
    L->sh_act_hi = static_cast<__nv_bfloat16*>(c->ws[kWsShActHi]);
    L->sh_act_lo = static_cast<__nv_bfloat16*>(c->ws[kWsShActLo]);
    L->sh_y = static_cast<float*>(c->ws[kWsShY]);
    L->x_stage = static_cast<__nv_bfloat16*>(c->ws[kWsXStage]);
    L->out_stage = static_cast<float*>(c->ws[kWsOutStage]);
}

size_t packed_bytes(int fmt, uint32_t rows, uint32_t cols) {
    return fmt == STRATA_MOE_FMT_BF16 ? (size_t)rows * cols * 2 : (size_t)rows * cols / 2;
}
size_t scale_bytes(int fmt, uint32_t rows, uint32_t cols) {
    if (fmt == STRATA_MOE_FMT_BF16) return 0;
    if (fmt == STRATA_MOE_FMT_MXFP4) return (size_t)rows * cols / 32;
    if (fmt == STRATA_MOE_FMT_NVFP4) return (size_t)rows * cols / 16;
    return (size_t)rows * cols / 128 * 2;
}

bool tensor_path_ok(const strata_moe_layer* L, int fmt, uint32_t I) {
    return !L->knobs.no_prefill_path && prefill_supported(fmt, L->d.hidden, I);
}

int sync_tables(strata_moe_layer* L) {
    strata_moe_ctx* ctx = L->ctx;
    if (ctx->ws_owner && ctx->ws_owner != L)
        return fail(ctx, STRATA_MOE_E_BUSY, "a MoE command of another layer of this context is in flight");
    bind_ws(L);
    if (!L->tables_dirty) return 0;
    const uint32_t n = L->d.expert_count;
    for (int r = 0; r < 3; ++r) {
        DeviceTable& t = L->tab[r];
        CK(cudaMemcpyAsync(t.d_packed, t.packed.data(), n * sizeof(void*), cudaMemcpyHostToDevice,
                           ctx->stream));
        CK(cudaMemcpyAsync(t.d_scales, t.scales.data(), n * sizeof(void*), cudaMemcpyHostToDevice,
                           ctx->stream));
        CK(cudaMemcpyAsync(t.d_global, t.global.data(), n * sizeof(float), cudaMemcpyHostToDevice,
                           ctx->stream));
    }
    CK(cudaStreamSynchronize(ctx->stream));  // the host vectors may change after this returns
    // f16 weight-streaming path: NVFP4 always qualifies; MXFP4 when every projection's scale
    // bytes fit one exponent window
    L->f16_ok = false;
    if (L->d.format == STRATA_MOE_FMT_NVFP4) {
        for (int r = 0; r < 3; ++r) {
            std::vector<float> post(n);
            for (uint32_t e = 0; e < n; ++e) post[e] = 1.0f / L->tab[r].global[e];
            CK(cudaMemcpy(L->tab[r].d_post, post.data(), n * sizeof(float), cudaMemcpyHostToDevice));
        }
        L->f16_ok = true;
    } else if (L->d.format == STRATA_MOE_FMT_MXFP4) {
        bool complete = true;
        for (int r = 0; r < 3; ++r)
            for (uint32_t e = 0; e < n; ++e) complete &= L->tab[r].scales[e] != nullptr;
        if (complete) {
            CK(cudaMemsetAsync(L->d_not_ok, 0, sizeof(uint32_t), ctx->stream));
            for (int r = 0; r < 3; ++r) {
                const uint32_t rows = r == STRATA_MOE_ROLE_DOWN ? L->d.hidden : L->d.intermediate;
                const uint32_t cols = r == STRATA_MOE_ROLE_DOWN ? L->d.intermediate : L->d.hidden;
                launch_mx_scale_range(L->tab[r].d_scales, n, scale_bytes(L->d.format, rows, cols),
                                      L->tab[r].d_emin, L->tab[r].d_post, L->d_not_ok, ctx->stream);
            }
            uint32_t not_ok = 1;
            CK(cudaMemcpyAsync(&not_ok, L->d_not_ok, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
            CK(cudaStreamSynchronize(ctx->stream));
            L->f16_ok = not_ok == 0;
        }
    }
    if (L->knobs.no_f16_path) L->f16_ok = false;
    // the bulk-copy ring needs 16-byte aligned packed rows and scale rows
    L->stream_ok = L->f16_ok && !L->knobs.no_stream_ring &&
                   decode_stream_supported(L->d.format, L->d.hidden, L->d.intermediate);
    for (int r = 0; r < 3 && L->stream_ok; ++r)
        for (uint32_t e = 0; e < n && L->stream_ok; ++e)
            L->stream_ok = (((uintptr_t)L->tab[r].packed[e] | (uintptr_t)L->tab[r].scales[e]) & 15u) == 0;
    if (L->stream_ok) {
        struct alignas(64) Blob3 { unsigned char b[3 * 128]; };
        std::vector<Blob3> maps((size_t)3 * n);
        for (int r = 0; r < 3 && L->stream_ok; ++r) {
            const uint32_t rows = r == STRATA_MOE_ROLE_DOWN ? L->d.hidden : L->d.intermediate;
            const uint32_t cols = r == STRATA_MOE_ROLE_DOWN ? L->d.intermediate : L->d.hidden;
            for (uint32_t e = 0; e < n && L->stream_ok; ++e)
                L->stream_ok = decode_stream_encode_maps(&maps[(size_t)r * n + e], L->d.format, L->tab[r].packed[e],
                                                         L->tab[r].scales[e], rows, cols) == 0;
        }
        if (L->stream_ok) CK(cudaMemcpy(L->d_smaps, maps.data(), maps.size() * sizeof(Blob3), cudaMemcpyHostToDevice));
    }
    // tensor maps of the packed weights for the tensor-core path's TMA producer
    L->wmaps_ok = false;
    if (L->d.format != STRATA_MOE_FMT_BF16 && tensor_path_ok(L, L->d.format, L->d.intermediate)) {
        struct alignas(64) Blob { unsigned char b[128]; };
        std::vector<Blob> maps((size_t)3 * n);
        bool ok = true;
        for (int r = 0; r < 3 && ok; ++r) {
            const uint32_t rows = r == STRATA_MOE_ROLE_DOWN ? L->d.hidden : L->d.intermediate;
            const uint32_t cols = r == STRATA_MOE_ROLE_DOWN ? L->d.intermediate : L->d.hidden;
            for (uint32_t e = 0; e < n && ok; ++e)
                ok = L->tab[r].packed[e] && ((uintptr_t)L->tab[r].packed[e] & 15u) == 0 &&
                     prefill_encode_weight_map(&maps[(size_t)r * n + e], L->tab[r].packed[e], rows, cols) == 0;
        }
        if (ok) {
            CK(cudaMemcpy(L->d_wmaps, maps.data(), maps.size() * sizeof(Blob), cudaMemcpyHostToDevice));
            L->wmaps_ok = true;
        }
    }
    L->tables_dirty = false;
    return 0;
}

WeightTable wt(const DeviceTable& t) {
    WeightTable w;
    w.packed = t.d_packed;
    w.scales = t.d_scales;
    w.global_scale = t.d_global;
    w.emin = t.d_emin;
    w.post_scale = t.d_post;
    return w;
}

bool all_registered(const strata_moe_layer* L, std::string* why) {
    for (int r = 0; r < 3; ++r)
        for (uint32_t e = 0; e < L->d.expert_count; ++e)
            if (!L->tab[r].packed[e] || !L->tab[r].scales[e]) {
                *why = "expert " + std::to_string(L->d.expert_begin + e) + " role " + std::to_string(r) +
                       " has no weights";
                return false;
            }
    if (!L->router) {
        *why = "router weights were never set";
        return false;
    }
    if (L->d.shared_intermediate)
        for (int r = 0; r < 3; ++r)
            if (!L->shared_w[r]) {
                *why = "shared expert weights were never set";
                return false;
            }
    return true;
}

// rows-per-expert threshold between the weight-streaming path and the tensor-core tile path
bool use_prefill(const strata_moe_layer* L, uint32_t pairs, uint32_t n_groups) {
    if (!tensor_path_ok(L, L->d.format, L->d.intermediate)) return false;
    if (L->d.format == STRATA_MOE_FMT_MXFP4 && !L->f16_ok) return false;  // needs the f16 weight window
    if (!L->wmaps_ok) return false;
    // average rows per expert from which the tensor-core path wins (measured: FP4 formats cross over
    // at 11-12 rows, INT4, whose streaming kernel is slower, at about 8)
    const int thr = L->knobs.prefill_min_rows >= 0 ? L->knobs.prefill_min_rows
                                                   : (L->d.format == STRATA_MOE_FMT_INT4G128 ? 8 : 12);
    return (uint64_t)pairs >= (uint64_t)n_groups * (uint64_t)thr;
}

bool use_prefill_down(const strata_moe_layer* L, uint32_t pairs, uint32_t n_groups) {
    if (!tensor_path_ok(L, L->d.format, L->d.intermediate) || !L->f16_ok || !L->wmaps_ok) return false;
    const int thr = L->knobs.prefill_down_min_rows >= 0 ? L->knobs.prefill_down_min_rows : 8;
    return (uint64_t)pairs >= (uint64_t)n_groups * (uint64_t)thr;
}

// Token tile of the tensor-core path: 192 when groups are large (an expert with up to 192 rows is decoded
// once), 128 with its deeper weight ring when they are small, 160 (three weight stages) for groups of about 128
// rows, nearly all of which still fit one tile (c2, 128 rows per expert on average: 2.99 -> 2.96 ms per step).
uint32_t prefill_ntile(const strata_moe_layer* L, uint64_t pairs, uint64_t n_groups) {
    if (L->knobs.prefill_ntile) return L->knobs.prefill_ntile == 128 ? 128u : (L->knobs.prefill_ntile == 160 ? 160u : 192u);
    if (pairs <= 96u * n_groups) return 128u;
    return pairs <= 140u * n_groups ? 160u : 192u;
}

// Row count from which a single group is handed to the tensor-core path inside an otherwise
// weight-streaming step; 0 = mixed dispatch off.
uint32_t mixed_min_rows(const strata_moe_layer* L, uint32_t max_rows_per_group) {
    if (!tensor_path_ok(L, L->d.format, L->d.intermediate) || !L->f16_ok || !L->wmaps_ok) return 0;
    const int thr = L->knobs.mixed_min_rows >= 0 ? L->knobs.mixed_min_rows : 24;   // above what one or two passes of the streaming kernel cover
    if (thr <= 0) return 0;
    // The two extra launches cost about 10 us even when no group qualifies: worth it only for steps
    // long enough that a hot expert's repeated passes would dominate.
    const uint32_t min_tokens = L->knobs.mixed_min_tokens >= 0 ? (uint32_t)L->knobs.mixed_min_tokens : 128u;
    return max_rows_per_group >= (uint32_t)thr && max_rows_per_group >= min_tokens ? (uint32_t)thr : 0u;
}

__global__ void set_pair_kernel(uint32_t* p, uint32_t a, uint32_t b) {
    p[0] = a;
    p[1] = b;
}

// Router projection, scores, top-k and weights for T tokens.  `logits_out` non-null means the caller
// wants the canonical logits of every (token, expert): that always takes the canonical projection.
// Otherwise large batches take the fast path: tensor-core projection into the layer's workspace, exact
// selection and weights by route_fast_kernel, canonical recomputation of the tokens it does not trust.
int run_router(strata_moe_layer* L, const __nv_bfloat16* x, uint32_t T, float* logits_out, uint32_t* ids, float* w) {
    Range range("strata_moe.router");
    strata_moe_ctx* ctx = L->ctx;
    cudaStream_t s = ctx->stream;
    const strata_moe_layer_desc& d = L->d;
    RouterParams rp{d.experts, d.top_k, d.score_kind, d.normalize, d.norm_init, d.weight_scale, d.softcap};
    const int thr = L->knobs.fast_router_min_tokens == 0 ? 512 : L->knobs.fast_router_min_tokens;
    const bool fast = logits_out == nullptr && thr > 0 && T >= (uint32_t)thr && route_fast_supported(rp, d.hidden) &&
                      tensor_path_ok(L, 3, d.intermediate) && (((uintptr_t)x | (uintptr_t)L->router) & 15u) == 0;
    if (fast) {
        set_pair_kernel<<<1, 1, 0, s>>>(L->router_off2, 0u, T);
        ++g_kernel_launches;
        if (launch_router_tc(x, T, L->router, d.experts, d.hidden, L->logits, L->router_tiles, L->router_off2,
                             ctx->d_status, s) != 0)
            return fail(ctx, STRATA_MOE_E_CUDA, "tensor-core router projection launch failed");
        mark(ctx, 1);
        launch_route_fast(rp, L->logits, L->bias, x, L->router, T, d.hidden, ids, w, L->recheck_list, L->recheck_count,
                          ctx->d_router_rechecks, ctx->d_status, s);
        ctx->router_fast_tokens += T;
        return 0;
    }
    float* lg = logits_out ? logits_out : L->logits;
    launch_router_logits(x, L->router, T, d.hidden, d.experts, lg, s, L->knobs.no_small_front ? nullptr : ctx->d_status);
    mark(ctx, 1);
    launch_route(rp, lg, L->bias, T, ids, w, ctx->d_status, s);
    return 0;
}

// Source rows that each feed k grouped rows: dest[t * k + j] is the grouped row of source row t's j-th use
// (0xFFFFFFFF = none).  Lets the operand conversion of the tensor-core path read and convert a row once.
struct SpreadRows {
    const uint32_t* dest;
    uint32_t rows, k;
    const uint32_t* rows_dev;   // device-side count of source rows, or null
};

// Expert FFN over grouped rows.  x_nat: rows in natural column order (group order).
// If x_kperm is non-null it already holds the K-permuted copy.
int run_experts(strata_moe_layer* L, const __nv_bfloat16* x_src, const uint32_t* perm, uint32_t k_div,
                uint32_t pairs, uint32_t n_groups, const uint32_t* offsets, const uint32_t* active,
                const uint32_t* n_active, uint32_t max_rows, float* y, uint32_t expected_pairs = 0,
                const uint32_t* pairs_dev = nullptr, bool x_ready = false, bool* y_half = nullptr,
                float* y_rowscale_out = nullptr, const SpreadRows* spread = nullptr) {
    // `pairs` bounds the row count.  When the exact count exists only on the device (rows received
    // from other ranks) pairs_dev points at it and expected_pairs steers the host-side heuristics.
    Range range("strata_moe.experts");
    strata_moe_ctx* ctx = L->ctx;
    cudaStream_t s = ctx->stream;
    if (pairs == 0) return 0;
    const uint32_t bound = pairs;
    if (pairs_dev && expected_pairs) pairs = expected_pairs < bound ? expected_pairs : bound;
    // x_ready: the caller's front-end kernel already left the f16 rows and their factors in the workspace
    if (use_prefill(L, pairs, n_groups)) {
        if (!x_ready) {
            if (spread && !L->knobs.no_spread)
                launch_rows_to_f16_spread(x_src, spread->dest, spread->k, spread->rows, spread->rows_dev, bound,
                                          L->d.hidden, L->xg, L->x_rowscale, s);
            else
                launch_rows_to_f16_bf16(x_src, perm, k_div, bound, L->d.hidden, L->xg, L->x_rowscale, s, pairs_dev);
        }
        mark(ctx, 4);
        PrefillArgs p{};
        p.fmt = L->d.format;
        p.H = L->d.hidden;
        p.I = L->d.intermediate;
        p.n_groups = n_groups;
        p.pairs = pairs;
        p.offsets = offsets;
        p.gate = wt(L->tab[0]);
        p.up = wt(L->tab[1]);
        p.down = wt(L->tab[2]);
        p.y = y;
        p.tile_table = static_cast<uint32_t*>(L->prefill_scratch);
        p.status = ctx->d_status;
        p.glu = GluParams{L->d.activation, L->d.gate_beta, L->d.linear_beta};
        p.ntile = prefill_ntile(L, pairs, n_groups);
        // the caller combines right away and can take the expert rows as f16: half the bytes written here and read
        // by the combine pass, which is bound by exactly those bytes
        p.y_half = (y_half && *y_half && !L->knobs.no_half_y) ? 1u : 0u;
        if (y_half) *y_half = p.y_half != 0u;
        p.y_rowscale_out = p.y_half ? y_rowscale_out : nullptr;
        if (launch_prefill(p, L->xg, L->x_rowscale, L->act_hi, L->max_pairs, L->d_wmaps, s,
                           ctx->timing ? ctx->pev[5] : nullptr) != 0)
            return fail(ctx, STRATA_MOE_E_CUDA, "prefill launch failed");
        mark(ctx, 6);
        CK(cudaGetLastError());
        return 0;
    }
    // only the all-tensor-core path above stores f16 rows; a caller that pointed y at an f16-sized buffer must have
    // predicted that path with the same test
    if (y_half && *y_half && y != L->y) return fail(ctx, STRATA_MOE_E_INVALID, "f16 output buffer offered to a path that writes fp32");
    if (y_half) *y_half = false;
    DecodeArgs a{};
    a.fmt = L->d.format;
    a.H = L->d.hidden;
    a.I = L->d.intermediate;
    a.n_groups = n_groups;
    a.offsets = offsets;
    a.active_list = active;
    a.n_active = n_active;
    // token tile of the streaming kernels: sized for the typical group (1.5 x the average rows per
    // expert), not the worst case -- a larger group just takes another pass over its weights
    {
        const uint64_t avg15 = ((uint64_t)pairs * 3u) / ((uint64_t)n_groups * 2u);
        uint32_t hint = (uint32_t)(avg15 < 1u ? 1u : avg15);
        a.max_rows_per_group = hint < max_rows ? hint : max_rows;
    }
    a.gate = wt(L->tab[0]);
    a.up = wt(L->tab[1]);
    a.down = wt(L->tab[2]);
    a.x_hi = L->xg;
    a.x_lo = nullptr;
    a.coef = nullptr;
    a.act_hi = L->act_hi;
    a.act_lo = L->act_lo;
    a.y = y;
    a.status = ctx->d_status;
    a.glu = GluParams{L->d.activation, L->d.gate_beta, L->d.linear_beta};
    if (L->f16_ok) {
        a.x_rowscale = L->x_rowscale;
        a.act_f32 = L->act_f32;
        a.act_rowscale = L->act_rowscale;
        a.x_rows = (uint32_t)L->max_pairs;
        // Mixed dispatch for uneven loads: groups with many rows (a hot expert under a skewed router) go
        // to the tensor-core path, the rest stay on the weight-streaming kernels.  An expert receives at
        // most one row per token, so nothing qualifies while max_rows is below the threshold.
        const uint32_t big = mixed_min_rows(L, max_rows);
        const bool down_all_tensor = use_prefill_down(L, pairs, n_groups);
        PrefillArgs p{};
        p.fmt = L->d.format;
        p.H = L->d.hidden;
        p.I = L->d.intermediate;
        p.n_groups = n_groups;
        p.pairs = pairs;
        p.offsets = offsets;
        p.gate = wt(L->tab[0]);
        p.up = wt(L->tab[1]);
        p.down = wt(L->tab[2]);
        p.y = y;
        p.tile_table = static_cast<uint32_t*>(L->prefill_scratch);
        p.status = ctx->d_status;
        p.glu = GluParams{L->d.activation, L->d.gate_beta, L->d.linear_beta};
        p.ntile = 128;   // hybrid down: few rows per expert
        a.skip_from = big;
        if (!x_ready) launch_rows_to_f16_bf16(x_src, perm, k_div, bound, L->d.hidden, L->xg, L->x_rowscale, s, pairs_dev);
        mark(ctx, 4);
        // the ring kernels win while a group fits one 8-row token tile (measured: 8 tokens of c0 99 us against 114 us;
        // 256 tokens of c1, 16-row tiles and several passes per group: 419 us against 339 us)
        // ... and only for decode-sized calls (at most 32 rows per call can reach one expert: an expert gets at most one
        // row per token).  With more tokens a skewed router makes groups of many rows, whose weights the 8-row ring tile
        // would stream again for every 8 rows: measured at the c4 shape (896 experts, Zipf, 256 tokens) 1.13 ms per step
        // with the ring kernels for the small groups against 0.96 ms with the register-streaming kernels for all; at 64
        // uniformly routed tokens of c1 the two are equal (0.405 / 0.408 ms).
        const uint32_t ring_rows = (uint32_t)L->knobs.stream_ring_max_rows;
        const bool ring = L->stream_ok && a.max_rows_per_group <= ring_rows && max_rows <= 4u * ring_rows;
        // ring kernels, no group on the tensor-core path: the gate/up epilogue writes the down kernel's f16 operand itself
        // and the separate conversion pass is skipped
        const bool act_direct = ring && !big && !down_all_tensor;
        a.act_direct = act_direct ? 1u : 0u;
        a.act_rowscale_out = L->act_rowscale;
        if (ring) {
            if (launch_decode_stream_gate_up(a, L->d_smaps, s) != 0) return fail(ctx, STRATA_MOE_E_CUDA, "stream gate/up launch failed");
        } else {
            launch_decode_fp4_gate_up(a, s);
        }
        if (!big) mark(ctx, 5);     // the gate/up phase is the kernel alone; the f16 split below belongs to the down phase
        if (!act_direct)
            launch_rows_to_f16_f32(L->act_f32, 0, bound, L->d.intermediate, L->act_hi, L->act_lo,
                                   L->act_rowscale, s, pairs_dev);
        if (big) {   // after the conversion above: these rows' f16 activations and unit row factors overwrite it
            p.min_rows = big;
            p.ntile = 128;   // measured at the c4 shape: 407 us with 128-token tiles, 439 us with 192
            p.act_rowscale_out = L->act_rowscale;
            if (launch_prefill_gate_up(p, L->xg, L->x_rowscale, L->act_hi, L->max_pairs, L->d_wmaps, s) != 0)
                return fail(ctx, STRATA_MOE_E_CUDA, "prefill gate/up launch failed");
            mark(ctx, 5);
        }
        // Medium batches: the down projection (short K, many output tiles) is faster on the tensor-core
        // path from about 8 rows per expert, the gate/up projection only from about 12.
        p.act_rowscale_out = nullptr;
        if (down_all_tensor) {
            p.min_rows = 0;
            p.ntile = 128;
            if (launch_prefill_down(p, L->act_hi, L->act_rowscale, L->max_pairs, L->d_wmaps, s) != 0)
                return fail(ctx, STRATA_MOE_E_CUDA, "prefill down launch failed");
        } else {
            if (ring) {
                if (launch_decode_stream_down(a, L->d_smaps, s) != 0) return fail(ctx, STRATA_MOE_E_CUDA, "stream down launch failed");
            } else {
                launch_decode_fp4_down(a, s);
            }
            if (big) {
                p.min_rows = big;
                p.reuse_tiles = 1;   // same groups as the gate/up launch above
                if (launch_prefill_down(p, L->act_hi, L->act_rowscale, L->max_pairs, L->d_wmaps, s) != 0)
                    return fail(ctx, STRATA_MOE_E_CUDA, "prefill down launch failed");
            }
        }
        mark(ctx, 6);
        CK(cudaGetLastError());
        return 0;
    }
    if (L->d.format == STRATA_MOE_FMT_BF16)   // BF16 weights read the activations in natural column order
        launch_gather_rows_plain(x_src, perm, k_div, bound, L->d.hidden, L->xg, s);
    else
        launch_gather_rows_kperm(x_src, perm, k_div, bound, L->d.hidden, L->xg, s, pairs_dev);
    mark(ctx, 4);
    launch_decode_gate_up(a, s);
    mark(ctx, 5);
    launch_decode_down(a, s);
    mark(ctx, 6);
    CK(cudaGetLastError());
    return 0;
}

// shared expert over T rows in natural order; offsets table = {0, T} in L->offsets scratch tail
int run_shared(strata_moe_layer* L, const __nv_bfloat16* x, const __nv_bfloat16* x_lo, uint32_t T,
               const uint32_t* offsets2, cudaStream_t st = nullptr) {
    strata_moe_ctx* ctx = L->ctx;
    if (!st) st = ctx->stream;
    // enough rows to fill tensor-core tiles (and BF16 inputs): grouped-GEMM path with one group
    const uint32_t thr = L->knobs.prefill_min_rows >= 0 ? (uint32_t)L->knobs.prefill_min_rows : 24u;
    if (!x_lo && T >= thr && tensor_path_ok(L, 3, L->d.shared_intermediate)) {
        PrefillArgs p{};
        p.fmt = 3;
        p.H = L->d.hidden;
        p.I = L->d.shared_intermediate;
        p.n_groups = 1;
        p.pairs = T;
        p.ntile = prefill_ntile(L, T, 1);
        p.offsets = offsets2;
        p.y = L->sh_y;
        p.tile_table = L->shared_tiles;
        p.status = ctx->d_status;
        p.glu = GluParams{L->d.activation, L->d.gate_beta, L->d.linear_beta};
        if (launch_prefill_bf16(p, x, T, L->shared_w[0], L->shared_w[1], L->shared_w[2], L->sh_act_hi,
                                L->d.max_tokens, st) != 0)
            return fail(ctx, STRATA_MOE_E_CUDA, "shared expert prefill launch failed");
        CK(cudaGetLastError());
        return 0;
    }
    DecodeArgs a{};
    a.fmt = 3;
    a.H = L->d.hidden;
    a.I = L->d.shared_intermediate;
    a.n_groups = 1;
    a.offsets = offsets2;
    a.max_rows_per_group = T;
    WeightTable g{L->d_shared_ptr[0], L->d_shared_ptr[0], L->one_global, nullptr, nullptr};
    WeightTable u{L->d_shared_ptr[1], L->d_shared_ptr[1], L->one_global, nullptr, nullptr};
    WeightTable dn{L->d_shared_ptr[2], L->d_shared_ptr[2], L->one_global, nullptr, nullptr};
    a.gate = g;
    a.up = u;
    a.down = dn;
    a.x_hi = x;
    a.x_lo = x_lo;
    a.act_hi = L->sh_act_hi;
    a.act_lo = L->sh_act_lo;
    a.y = L->sh_y;
    a.status = ctx->d_status;
    a.glu = GluParams{L->d.activation, L->d.gate_beta, L->d.linear_beta};
    launch_decode_gate_up(a, st);
    launch_decode_down(a, st);
    CK(cudaGetLastError());
    return 0;
}

__global__ void uniform_offsets_kernel(uint32_t* p, uint32_t n, uint32_t rows) {
    for (uint32_t i = threadIdx.x; i <= n; i += blockDim.x) p[i] = i * rows;
}
__global__ void widen_bf16_kernel(const __nv_bfloat16* x, size_t n, float* out) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __bfloat162float(x[i]);
}
__global__ void split_f32_kernel(const float* x, size_t n, __nv_bfloat16* hi, __nv_bfloat16* lo) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        const __nv_bfloat16 h = __float2bfloat16_rn(x[i]);
        hi[i] = h;
        lo[i] = __float2bfloat16_rn(x[i] - __bfloat162float(h));
    }
}

}  // namespace

// =========================================================================================
extern "C" {

int strata_moe_create(int device, void* stream, strata_moe_ctx** out) {
    if (!out) return STRATA_MOE_E_INVALID;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0 || device < 0 || device >= n)
        return STRATA_MOE_E_NO_DEVICE;
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return STRATA_MOE_E_NO_DEVICE;
    if (prop.major != 10) return STRATA_MOE_E_NO_DEVICE;  // kernels are built for sm_100a only
    strata_moe_ctx* ctx = new (std::nothrow) strata_moe_ctx();
    if (!ctx) return STRATA_MOE_E_INVALID;
    ctx->device = device;
    if (cudaSetDevice(device) != cudaSuccess) { delete ctx; return STRATA_MOE_E_CUDA; }
    if (stream) {
        ctx->stream = static_cast<cudaStream_t>(stream);
    } else {
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete ctx;
            return STRATA_MOE_E_CUDA;
        }
        ctx->own_stream = true;
    }
    if (cudaMalloc(&ctx->d_status, sizeof(uint32_t)) != cudaSuccess ||
        cudaMemset(ctx->d_status, 0, sizeof(uint32_t)) != cudaSuccess ||
        cudaMallocHost(&ctx->h_status, sizeof(uint32_t)) != cudaSuccess ||
        cudaEventCreate(&ctx->ev0) != cudaSuccess || cudaEventCreate(&ctx->ev1) != cudaSuccess) {
        strata_moe_destroy(ctx);
        return STRATA_MOE_E_CUDA;
    }
    for (int i = 0; i <= STRATA_MOE_PHASES; ++i)
        if (cudaEventCreate(&ctx->pev[i]) != cudaSuccess) {
            strata_moe_destroy(ctx);
            return STRATA_MOE_E_CUDA;
        }
    if (cudaStreamCreateWithFlags(&ctx->side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&ctx->ev_join, cudaEventDisableTiming) != cudaSuccess) {
        strata_moe_destroy(ctx);
        return STRATA_MOE_E_CUDA;
    }
    if (cudaMalloc(&ctx->d_router_rechecks, 2 * sizeof(unsigned long long)) != cudaSuccess ||
        cudaMemset(ctx->d_router_rechecks, 0, 2 * sizeof(unsigned long long)) != cudaSuccess) {
        strata_moe_destroy(ctx);
        return STRATA_MOE_E_CUDA;
    }
    ctx->launches_at_create = g_kernel_launches;
    *out = ctx;
    return 0;
}

int strata_moe_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) return 0;
    int usable = 0;
    for (int i = 0; i < n; ++i) {
        cudaDeviceProp prop{};
        if (cudaGetDeviceProperties(&prop, i) != cudaSuccess || prop.major != 10) break;   // ordinals stay contiguous
        ++usable;
    }
    return usable;
}

void strata_moe_destroy(strata_moe_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->cmd_layer) strata_moe_layer_destroy(ctx->cmd_layer);
    for (void* p : ctx->cmd_scratch) cudaFree(p);
    for (void*& p : ctx->ws_raw) {
        if (p) cudaFree(p);
        p = nullptr;
    }
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->d_router_rechecks) cudaFree(ctx->d_router_rechecks);
    if (ctx->h_status) cudaFreeHost(ctx->h_status);
    if (ctx->ev0) cudaEventDestroy(ctx->ev0);
    if (ctx->ev1) cudaEventDestroy(ctx->ev1);
    if (ctx->side) { cudaStreamSynchronize(ctx->side); cudaStreamDestroy(ctx->side); }
    if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
    if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
    for (cudaEvent_t e : ctx->ev_in)
        if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : ctx->ev_done)
        if (e) cudaEventDestroy(e);
    if (ctx->ev_fork) cudaEventDestroy(ctx->ev_fork);
    if (ctx->ev_join) cudaEventDestroy(ctx->ev_join);
    for (int i = 0; i <= STRATA_MOE_PHASES; ++i)
        if (ctx->pev[i]) cudaEventDestroy(ctx->pev[i]);
    if (ctx->own_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char* strata_moe_last_error(const strata_moe_ctx* ctx) { return ctx ? ctx->err.c_str() : "no context"; }

int strata_moe_synchronize(strata_moe_ctx* ctx) {
    if (!ctx) return STRATA_MOE_E_INVALID;
    CK(cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    CK(cudaMemsetAsync(ctx->d_status, 0, sizeof(uint32_t), ctx->stream));
    CK(cudaStreamSynchronize(ctx->stream));
    const uint32_t st = *ctx->h_status;
    if (st) {
        std::string m = "device status:";
        if (st & kStatusNonFiniteLogit) m += " non-finite router logit or bias;";
        if (st & kStatusBadNormaliser) m += " router normaliser not positive;";
        if (st & kStatusNonFiniteOutput) m += " non-finite expert output;";
        if (st & kStatusWaitTimeout) m += " bounded wait timed out;";
        if (st & kStatusBadGroup) m += " inconsistent group table;";
        return fail(ctx, STRATA_MOE_E_NUMERIC, m);
    }
    return 0;
}

int strata_moe_get_stats(const strata_moe_ctx* ctx, strata_moe_stats* out) {
    if (!ctx || !out) return STRATA_MOE_E_INVALID;
    *out = ctx->stats;
    out->kernel_launches = g_kernel_launches - ctx->launches_at_create;
    out->router_fast_tokens = ctx->router_fast_tokens;
    out->workspace_allocations = ctx->workspace_allocations;
    out->router_rechecked_tokens = 0;
    out->router_worst_error = 0.0f;
    if (ctx->d_router_rechecks) {   // waits for the work enqueued so far
        unsigned long long v[2] = {0, 0};    // [0] rechecked tokens, [1] float bits of the worst error fraction
        if (cudaMemcpy(v, ctx->d_router_rechecks, sizeof(v), cudaMemcpyDeviceToHost) == cudaSuccess) {
            out->router_rechecked_tokens = v[0];
            const uint32_t bits = (uint32_t)v[1];
            memcpy(&out->router_worst_error, &bits, sizeof(bits));
        }
    }
    return 0;
}

void strata_moe_set_timing(strata_moe_ctx* ctx, int enabled) {
    if (ctx) ctx->timing = enabled != 0;
}

int strata_moe_get_phase_ms(strata_moe_ctx* ctx, float* out) {
    if (!ctx || !out) return STRATA_MOE_E_INVALID;
    if (!ctx->pev_valid) return fail(ctx, STRATA_MOE_E_INVALID, "no timed forward has completed");
    for (int i = 0; i < STRATA_MOE_PHASES; ++i) CK(cudaEventElapsedTime(&out[i], ctx->pev[i], ctx->pev[i + 1]));
    return 0;
}

int strata_moe_layer_create(strata_moe_ctx* ctx, const strata_moe_layer_desc* desc, strata_moe_layer** out) {
    if (!ctx || !desc || !out) return STRATA_MOE_E_INVALID;
    *out = nullptr;
    const strata_moe_layer_desc& d = *desc;
    if (d.hidden == 0 || d.hidden % 128 || d.intermediate == 0 || d.intermediate % 128)
        return fail(ctx, STRATA_MOE_E_INVALID, "hidden and intermediate must be positive multiples of 128");
    if (d.experts == 0 || d.experts > 1024 || d.top_k == 0 || d.top_k > 32 || d.top_k > d.experts)
        return fail(ctx, STRATA_MOE_E_INVALID, "experts must be in 1..1024 and top_k in 1..min(32, experts)");
    if (d.format < 0 || d.format > STRATA_MOE_FMT_BF16)
        return fail(ctx, STRATA_MOE_E_INVALID, "unknown weight format");
    if (d.score_kind < 0 || d.score_kind > STRATA_MOE_SCORE_SQRTSOFTPLUS)
        return fail(ctx, STRATA_MOE_E_INVALID, "unknown router score kind");
    if (d.expert_count == 0 || (uint64_t)d.expert_begin + d.expert_count > d.experts)
        return fail(ctx, STRATA_MOE_E_INVALID, "resident expert range is outside the layer");
    if (d.shared_intermediate % 128)
        return fail(ctx, STRATA_MOE_E_INVALID, "shared intermediate must be a multiple of 128");
    if (d.max_tokens == 0) return fail(ctx, STRATA_MOE_E_INVALID, "max_tokens must be positive");
    if (d.activation != STRATA_MOE_ACT_SWIGLU && d.activation != STRATA_MOE_ACT_SITU_GLU)
        return fail(ctx, STRATA_MOE_E_INVALID, "unknown activation");
    if (d.activation == STRATA_MOE_ACT_SITU_GLU && !(d.gate_beta > 0.0f && d.linear_beta > 0.0f))
        return fail(ctx, STRATA_MOE_E_INVALID, "SiTU-GLU betas must be positive");
    if (!(d.weight_scale == d.weight_scale) || !(d.output_scale == d.output_scale))
        return fail(ctx, STRATA_MOE_E_INVALID, "router scales must be finite");
    CK(cudaSetDevice(ctx->device));
    strata_moe_layer* L = new (std::nothrow) strata_moe_layer();
    if (!L) return fail(ctx, STRATA_MOE_E_INVALID, "out of host memory");
    L->ctx = ctx;
    L->d = d;
    L->knobs = read_knobs();
    const uint64_t mp = d.max_pairs ? d.max_pairs : (uint64_t)d.max_tokens * d.top_k;
    if (mp > 0x7FFFFFFFull) { delete L; return fail(ctx, STRATA_MOE_E_INVALID, "max_pairs too large"); }
    L->max_pairs = (uint32_t)mp;
    const uint32_t P = L->max_pairs, T = d.max_tokens, H = d.hidden, I = d.intermediate, E = d.experts;
    const uint32_t n = d.expert_count;
    cudaError_t e = cudaSuccess;
    auto A = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
    for (int r = 0; r < 3; ++r) {
        DeviceTable& t = L->tab[r];
        t.packed.assign(n, nullptr);
        t.scales.assign(n, nullptr);
        t.global.assign(n, 1.0f);
        A(dalloc(L, &t.d_packed, n));
        A(dalloc(L, &t.d_scales, n));
        A(dalloc(L, &t.d_global, n));
        A(dalloc(L, &t.d_emin, n));
        A(dalloc(L, &t.d_post, n));
        A(dalloc(L, &L->d_shared_ptr[r], 1));
    }
    A(dalloc(L, &L->logits, (size_t)T * E));
    A(dalloc(L, &L->ids, (size_t)T * d.top_k));
    A(dalloc(L, &L->weights, (size_t)T * d.top_k));
    A(dalloc(L, &L->counts, (size_t)E));
    A(dalloc(L, &L->offsets, (size_t)E + 1 + 2 + 12));
    A(dalloc(L, &L->perm, (size_t)P));
    A(dalloc(L, &L->inv, (size_t)T * d.top_k > P ? (size_t)T * d.top_k : (size_t)P));
    A(dalloc(L, &L->active, (size_t)E));
    A(dalloc(L, &L->n_active, 1));
    {
        void* gs = nullptr;
        size_t gb = group_scratch_bytes((uint32_t)((size_t)T * d.top_k > P ? (size_t)T * d.top_k : P), E);
        A(cudaMalloc(&gs, gb));
        if (gs) L->owned.push_back(gs);
        L->group_scratch = gs;
        void* ps = nullptr;
        A(cudaMalloc(&ps, prefill_scratch_bytes(n, P) + 16));
        if (ps) L->owned.push_back(ps);
        L->prefill_scratch = ps;
    }
    A(ws_reserve(ctx, kWsXg, (size_t)P * H * 2));
    A(ws_reserve(ctx, kWsXgLo, 16));
    A(ws_reserve(ctx, kWsActHi, (size_t)P * I * 2));
    A(ws_reserve(ctx, kWsActLo, (size_t)P * I * 2));
    A(ws_reserve(ctx, kWsY, (size_t)P * H * 4));
    A(dalloc(L, &L->one_global, 1));
    A(dalloc(L, &L->d_not_ok, 1));
    {
        void* wm = nullptr;
        A(cudaMalloc(&wm, (size_t)3 * n * 128 + 128));
        if (wm) L->owned.push_back(wm);
        L->d_wmaps = wm;
        void* sm = nullptr;
        A(cudaMalloc(&sm, (size_t)9 * n * 128 + 128));
        if (sm) L->owned.push_back(sm);
        L->d_smaps = sm;
    }
    A(ws_reserve(ctx, kWsActF32, (size_t)P * I * 4));
    A(ws_reserve(ctx, kWsXRow, (size_t)P * 4));
    A(ws_reserve(ctx, kWsActRow, (size_t)P * 4));
    if (d.shared_intermediate) {
        A(dalloc(L, &L->shared_tiles, prefill_scratch_bytes(1, T) / sizeof(uint32_t) + 4));
        A(ws_reserve(ctx, kWsShActHi, (size_t)T * d.shared_intermediate * 2));
        A(ws_reserve(ctx, kWsShActLo, (size_t)T * d.shared_intermediate * 2));
        A(ws_reserve(ctx, kWsShY, (size_t)T * H * 4));
    }
    A(dalloc(L, &L->router_tiles, prefill_scratch_bytes(1, T) / sizeof(uint32_t) + 4));
    A(dalloc(L, &L->router_off2, 2));
    A(dalloc(L, &L->recheck_list, (size_t)T));
    A(dalloc(L, &L->recheck_count, 1));
    A(ws_reserve(ctx, kWsXStage, (size_t)T * H * 2));
    A(ws_reserve(ctx, kWsOutStage, (size_t)T * H * 4));
    bind_ws(L);
    if (e == cudaSuccess) {
        const float one = 1.0f;
        e = cudaMemcpy(L->one_global, &one, sizeof(float), cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) {
        strata_moe_layer_destroy(L);
        return fail(ctx, STRATA_MOE_E_CUDA, std::string("layer allocation: ") + cudaGetErrorString(e));
    }
    *out = L;
    return 0;
}

void strata_moe_layer_destroy(strata_moe_layer* L) {
    if (!L) return;
    cudaSetDevice(L->ctx->device);
    cudaStreamSynchronize(L->ctx->stream);
    if (L->ctx->ws_owner == L) L->ctx->ws_owner = nullptr;
    for (void* p : L->owned) cudaFree(p);
    if (L->dense_pinned) cudaFreeHost(L->dense_pinned);
    delete L;
}

constexpr size_t kArenaChunk = 256u << 20;

static int put(strata_moe_layer* L, const void* src, size_t bytes, int source, const void** dev) {
    strata_moe_ctx* ctx = L->ctx;
    if (!src) return fail(ctx, STRATA_MOE_E_INVALID, "null weight pointer");
    if (source == STRATA_MOE_SRC_DEVICE_BORROW) {
        *dev = src;
        return 0;
    }
    if (source != STRATA_MOE_SRC_HOST && source != STRATA_MOE_SRC_DEVICE_COPY)
        return fail(ctx, STRATA_MOE_E_INVALID, "unknown source kind");
    // Layer-owned copies are carved out of large chunks at 256-byte granularity, like the reference's weight arena
    // (kernels/cuda/backend.cu:4889-4890): a few allocations per layer instead of six per expert.  Space is only
    // returned when the layer is destroyed (a tensor registered twice keeps both copies until then).
    const size_t need = (bytes + 255) / 256 * 256;
    if (need > L->arena_left) {
        const size_t chunk = need > L->arena_next ? need : L->arena_next;     // 4 MB, doubling up to 256 MB
        if (L->arena_next < kArenaChunk) L->arena_next *= 2;
        void* c = nullptr;
        CK(cudaMalloc(&c, chunk));
        L->owned.push_back(c);
        L->arena_cur = static_cast<uint8_t*>(c);
        L->arena_left = chunk;
    }
    void* p = L->arena_cur;
    L->arena_cur += need;
    L->arena_left -= need;
    CK(cudaMemcpyAsync(p, src, bytes,
                       source == STRATA_MOE_SRC_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice,
                       ctx->stream));
    CK(cudaStreamSynchronize(ctx->stream));
    if (source == STRATA_MOE_SRC_HOST) ctx->stats.h2d_bytes += bytes;
    ctx->stats.weight_bytes += bytes;
    *dev = p;
    return 0;
}

int strata_moe_set_router(strata_moe_layer* L, const void* gate_bf16, const float* bias, int source) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    CK(cudaSetDevice(ctx->device));
    const void* p = nullptr;
    int rc = put(L, gate_bf16, (size_t)L->d.experts * L->d.hidden * 2, source, &p);
    if (rc) return rc;
    L->router = (__nv_bfloat16*)p;
    L->has_bias = bias != nullptr;
    if (bias) {
        rc = put(L, bias, (size_t)L->d.experts * 4, source, &p);
        if (rc) return rc;
        L->bias = (float*)p;
    } else {
        L->bias = nullptr;
    }
    return 0;
}

int strata_moe_set_expert(strata_moe_layer* L, uint32_t expert, int role, const void* packed,
                          const void* scales, float global_scale, int source) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (role < 0 || role > 2) return fail(ctx, STRATA_MOE_E_INVALID, "role must be gate, up or down");
    if (expert < L->d.expert_begin || expert >= L->d.expert_begin + L->d.expert_count)
        return fail(ctx, STRATA_MOE_E_INVALID, "expert is not resident on this device");
    if (L->d.format == STRATA_MOE_FMT_NVFP4 && !(global_scale > 0.0f && global_scale < 3.0e38f))
        return fail(ctx, STRATA_MOE_E_INVALID, "NVFP4 global scale must be finite and positive");
    if (((uintptr_t)packed & 15u) && source == STRATA_MOE_SRC_DEVICE_BORROW)
        return fail(ctx, STRATA_MOE_E_INVALID, "borrowed weights must be 16-byte aligned");
    CK(cudaSetDevice(ctx->device));
    const uint32_t rows = role == STRATA_MOE_ROLE_DOWN ? L->d.hidden : L->d.intermediate;
    const uint32_t cols = role == STRATA_MOE_ROLE_DOWN ? L->d.intermediate : L->d.hidden;
    const void *pp = nullptr, *ps = nullptr;
    int rc = put(L, packed, packed_bytes(L->d.format, rows, cols), source, &pp);
    if (rc) return rc;
    if (L->d.format == STRATA_MOE_FMT_BF16) {
        ps = pp;   // no scales: the table entry only has to be non-null
    } else {
        rc = put(L, scales, scale_bytes(L->d.format, rows, cols), source, &ps);
        if (rc) return rc;
    }
    const uint32_t le = expert - L->d.expert_begin;
    L->tab[role].packed[le] = (const uint8_t*)pp;
    L->tab[role].scales[le] = (const uint8_t*)ps;
    L->tab[role].global[le] = L->d.format == STRATA_MOE_FMT_NVFP4 ? global_scale : 1.0f;
    L->tables_dirty = true;
    return 0;
}

int strata_moe_set_shared(strata_moe_layer* L, int role, const void* w, int source) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (role < 0 || role > 2) return fail(ctx, STRATA_MOE_E_INVALID, "role must be gate, up or down");
    if (!L->d.shared_intermediate) return fail(ctx, STRATA_MOE_E_INVALID, "layer has no shared expert");
    CK(cudaSetDevice(ctx->device));
    const void* p = nullptr;
    int rc = put(L, w, (size_t)L->d.shared_intermediate * L->d.hidden * 2, source, &p);
    if (rc) return rc;
    L->shared_w[role] = (__nv_bfloat16*)p;
    CK(cudaMemcpy(L->d_shared_ptr[role], &p, sizeof(void*), cudaMemcpyHostToDevice));
    return 0;
}

int strata_moe_route(strata_moe_layer* L, const void* x, uint32_t T, float* logits, uint32_t* ids,
                     float* weights) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!x || !ids || !weights) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (T > L->d.max_tokens) return fail(ctx, STRATA_MOE_E_INVALID, "tokens exceed max_tokens");
    if (!L->router) return fail(ctx, STRATA_MOE_E_INVALID, "router weights were never set");
    CK(cudaSetDevice(ctx->device));
    int rc = run_router(L, (const __nv_bfloat16*)x, T, logits, ids, weights);
    if (rc) return rc;
    CK(cudaGetLastError());
    return 0;
}

int strata_moe_route_hash(strata_moe_layer* L, const void* x, uint32_t T, const uint32_t* token_experts,
                          float* logits, uint32_t* ids, float* weights) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!x || !token_experts || !ids || !weights) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (T > L->d.max_tokens) return fail(ctx, STRATA_MOE_E_INVALID, "tokens exceed max_tokens");
    if (!L->router) return fail(ctx, STRATA_MOE_E_INVALID, "router weights were never set");
    CK(cudaSetDevice(ctx->device));
    float* lg = logits ? logits : L->logits;
    launch_router_logits((const __nv_bfloat16*)x, L->router, T, L->d.hidden, L->d.experts, lg, ctx->stream, ctx->d_status);
    RouterParams p{L->d.experts, L->d.top_k, L->d.score_kind, L->d.normalize, L->d.norm_init,
                   L->d.weight_scale, L->d.softcap};
    // an expert id outside the layer raises the status word (kStatusNonFiniteLogit's neighbour: bad route)
    launch_route(p, lg, nullptr, T, ids, weights, ctx->d_status, ctx->stream, token_experts);
    CK(cudaGetLastError());
    return 0;
}

int strata_moe_check_canaries(strata_moe_ctx* ctx) {
    if (!ctx) return STRATA_MOE_E_INVALID;
    CK(cudaSetDevice(ctx->device));
    CK(cudaStreamSynchronize(ctx->stream));
    if (ctx->side) CK(cudaStreamSynchronize(ctx->side));
    uint8_t guard[2 * kGuard];
    for (int slot = 0; slot < 16; ++slot) {
        if (!ctx->ws_raw[slot]) continue;
        const uint8_t* raw = static_cast<const uint8_t*>(ctx->ws_raw[slot]);
        const size_t body = (ctx->ws_bytes[slot] + kGuard - 1) / kGuard * kGuard;
        CK(cudaMemcpy(guard, raw, kGuard, cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(guard + kGuard, raw + kGuard + body, kGuard, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < 2 * kGuard; ++i)
            if (guard[i] != (uint8_t)kCanary)
                return fail(ctx, STRATA_MOE_E_CUDA, "workspace " + std::to_string(slot) + ": guard zone " +
                                                        (i < kGuard ? "before" : "after") + " the buffer was overwritten");
    }
    return 0;
}

int strata_moe_stable_bf16_hash(strata_moe_ctx* ctx, const float* values, size_t n, uint64_t* hash) {
    if (!ctx) return STRATA_MOE_E_INVALID;
    if (!hash || (!values && n)) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    CK(cudaSetDevice(ctx->device));
    std::vector<float> host(n);
    if (n) CK(cudaMemcpyAsync(host.data(), values, n * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    CK(cudaStreamSynchronize(ctx->stream));
    ctx->stats.d2h_bytes += n * sizeof(float);
    uint64_t h = 14695981039346656037ull;
    for (size_t i = 0; i < n; ++i) {
        uint32_t b;
        memcpy(&b, &host[i], 4);
        if ((b & 0x7F800000u) != 0x7F800000u) b += 0x7FFFu + ((b >> 16) & 1u);   // infinities and NaNs are truncated
        const uint32_t v = b >> 16;
        h = (h ^ (v & 0xFFu)) * 1099511628211ull;
        h = (h ^ (v >> 8)) * 1099511628211ull;
    }
    *hash = h;
    return 0;
}

int strata_moe_project_rows(strata_moe_ctx* ctx, const void* x, uint32_t T, uint32_t H, const void* w, uint32_t rows,
                            float* logits) {
    if (!ctx) return STRATA_MOE_E_INVALID;
    if (!x || !w || !logits) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (H == 0 || H % 32u || rows == 0) return fail(ctx, STRATA_MOE_E_INVALID, "hidden must be a positive multiple of 32 and rows positive");
    if ((((uintptr_t)x | (uintptr_t)w) & 15u) != 0) return fail(ctx, STRATA_MOE_E_INVALID, "x and w must be 16-byte aligned");
    CK(cudaSetDevice(ctx->device));
    launch_router_logits((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, T, H, rows, logits, ctx->stream, ctx->d_status);
    CK(cudaGetLastError());
    return 0;
}

int strata_moe_route_sink(strata_moe_ctx* ctx, const float* logits, const float* bias, uint32_t T, uint32_t E, uint32_t S,
                          uint32_t k, float scale, uint32_t* ids, float* weights, float* sink_weights) {
    if (!ctx) return STRATA_MOE_E_INVALID;
    if (!logits || !bias || !ids || !weights || (S && !sink_weights)) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (k == 0 || k > E) return fail(ctx, STRATA_MOE_E_INVALID, "Inkling router selection is out of range");
    if (k + S > 32u) return fail(ctx, STRATA_MOE_E_INVALID, "top_k + sinks exceed 32");
    if ((size_t)E * 4u * sizeof(float) > 48u * 1024u) return fail(ctx, STRATA_MOE_E_INVALID, "too many routed experts");
    if (!std::isfinite(scale)) return fail(ctx, STRATA_MOE_E_INVALID, "Inkling router global scale must be finite");
    CK(cudaSetDevice(ctx->device));
    launch_route_sink(logits, bias, T, E, S, k, scale, ids, weights, sink_weights, ctx->d_status, ctx->stream);
    CK(cudaGetLastError());
    return 0;
}

int strata_moe_group(strata_moe_layer* L, const uint32_t* ids, uint32_t pairs, uint32_t expert_begin,
                     uint32_t n_experts, uint32_t* counts, uint32_t* offsets, uint32_t* perm,
                     uint32_t* inv) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!ids || !counts || !offsets || !perm) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (n_experts == 0 || n_experts > L->d.experts) return fail(ctx, STRATA_MOE_E_INVALID, "bad expert range");
    if ((uint64_t)pairs > (uint64_t)L->d.max_tokens * L->d.top_k && pairs > L->max_pairs)
        return fail(ctx, STRATA_MOE_E_INVALID, "pairs exceed the layer's workspace");
    CK(cudaSetDevice(ctx->device));
    launch_group(ids, pairs, expert_begin, n_experts, counts, offsets, perm, inv, nullptr, nullptr,
                 L->group_scratch, ctx->stream);
    CK(cudaGetLastError());
    return 0;
}

int strata_moe_experts_grouped(strata_moe_layer* L, const void* rows, uint32_t pairs,
                               const uint32_t* offsets, float* y) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!rows || !offsets || !y) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (pairs > L->max_pairs) return fail(ctx, STRATA_MOE_E_INVALID, "pairs exceed max_pairs");
    std::string why;
    for (int r = 0; r < 3; ++r)
        for (uint32_t e = 0; e < L->d.expert_count; ++e)
            if (!L->tab[r].packed[e]) return fail(ctx, STRATA_MOE_E_INVALID, "an expert has no weights");
    CK(cudaSetDevice(ctx->device));
    int rc = sync_tables(L);
    if (rc) return rc;
    return run_experts(L, (const __nv_bfloat16*)rows, nullptr, 1, pairs, L->d.expert_count, offsets,
                       nullptr, nullptr, pairs, y);
}

int strata_moe_gather_rows(strata_moe_layer* L, const void* src, uint32_t row_bytes,
                           const uint32_t* index, uint32_t index_div, uint32_t n, void* dst) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!src || !dst || !index) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (row_bytes == 0 || row_bytes % 16u || index_div == 0)
        return fail(ctx, STRATA_MOE_E_INVALID, "rows must be a multiple of 16 bytes");
    CK(cudaSetDevice(ctx->device));
    // a row of row_bytes is copied as row_bytes / 16 sixteen-byte vectors
    launch_gather_rows_plain(static_cast<const __nv_bfloat16*>(src), index, index_div, n, row_bytes / 2u,
                             static_cast<__nv_bfloat16*>(dst), ctx->stream);
    CK(cudaGetLastError());
    return 0;
}

int strata_moe_combine(strata_moe_layer* L, const float* y, const uint32_t* inv, const float* weights,
                       const void* x_shared, uint32_t T, float* out) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!y || !inv || !weights || !out) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (T > L->d.max_tokens) return fail(ctx, STRATA_MOE_E_INVALID, "tokens exceed max_tokens");
    if (T == 0) return 0;
    CK(cudaSetDevice(ctx->device));
    bind_ws(L);
    const float* shared = nullptr;
    if (x_shared && L->d.shared_intermediate) {
        for (int r = 0; r < 3; ++r)
            if (!L->shared_w[r]) return fail(ctx, STRATA_MOE_E_INVALID, "shared expert weights were never set");
        uint32_t* off2 = L->offsets + L->d.experts + 1 + 2;
        set_pair_kernel<<<1, 1, 0, ctx->stream>>>(off2, 0u, T);
        ++g_kernel_launches;
        int rc = run_shared(L, static_cast<const __nv_bfloat16*>(x_shared), nullptr, T, off2);
        if (rc) return rc;
        shared = L->sh_y;
    }
    launch_combine(y, inv, weights, shared, T, L->d.top_k, L->d.hidden, L->d.output_scale, out,
                   ctx->d_status, ctx->stream);
    CK(cudaGetLastError());
    return 0;
}

int strata_moe_forward(strata_moe_layer* L, const void* x, uint32_t T, float* out,
                       const strata_moe_aux* aux) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!x || !out) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (T > L->d.max_tokens) return fail(ctx, STRATA_MOE_E_INVALID, "tokens exceed max_tokens");
    if (L->d.expert_count != L->d.experts)
        return fail(ctx, STRATA_MOE_E_INVALID, "forward needs every expert resident; use the stage calls for expert parallelism");
    if (L->dense_in_flight) return fail(ctx, STRATA_MOE_E_BUSY, "a dense command is in flight");
    if ((uint64_t)T * L->d.top_k > L->max_pairs)
        return fail(ctx, STRATA_MOE_E_INVALID, "tokens * top_k exceed the layer's max_pairs");
    std::string why;
    if (!all_registered(L, &why)) return fail(ctx, STRATA_MOE_E_INVALID, why);
    if (T == 0) return 0;
    CK(cudaSetDevice(ctx->device));
    int rc = sync_tables(L);
    if (rc) return rc;
    cudaStream_t s = ctx->stream;
    const strata_moe_layer_desc& d = L->d;
    if (ctx->timing) CK(cudaEventRecord(ctx->ev0, s));
    mark(ctx, 0);
    const bool fork_shared = d.shared_intermediate != 0 && !ctx->timing;
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    uint32_t* ids = (aux && aux->ids) ? aux->ids : L->ids;
    float* w = (aux && aux->weights) ? aux->weights : L->weights;
    uint32_t* counts = (aux && aux->counts) ? aux->counts : L->counts;
    uint32_t* offsets = (aux && aux->offsets) ? aux->offsets : L->offsets;
    uint32_t* perm = (aux && aux->perm) ? aux->perm : L->perm;
    const uint32_t P = T * d.top_k;
    if (fork_shared) {
        // the shared expert needs only x: it runs on the side stream while the routed path runs here
        uint32_t* off2 = L->offsets + d.experts + 1 + 2;
        set_pair_kernel<<<1, 1, 0, s>>>(off2, 0u, T);
        ++g_kernel_launches;
        CK(cudaEventRecord(ctx->ev_fork, s));
        CK(cudaStreamWaitEvent(ctx->side, ctx->ev_fork, 0));
        rc = run_shared(L, xb, nullptr, T, off2, ctx->side);
        if (rc) return rc;
        CK(cudaEventRecord(ctx->ev_join, ctx->side));
    }
    // Decode batches (<= 16 tokens): canonical logits, then ONE kernel for scores / top-k / weights, grouping and the
    // gather + f16 conversion of the routed rows (when the expert kernels read f16 rows at all).
    bool x_ready = false, front_done = false;
    if (T <= 16 && !L->knobs.no_small_front) {
        float* lg = (aux && aux->logits) ? aux->logits : L->logits;
        const bool convert = use_prefill(L, P, d.experts) || L->f16_ok;
        RouterParams rp{d.experts, d.top_k, d.score_kind, d.normalize, d.norm_init, d.weight_scale, d.softcap};
        launch_router_logits(xb, L->router, T, d.hidden, d.experts, lg, s, ctx->d_status);
        mark(ctx, 1);
        front_done = launch_front_small(rp, lg, L->bias, T, ids, w, counts, offsets, perm, L->inv, L->active, L->n_active,
                                        xb, d.hidden, convert ? L->xg : nullptr, L->x_rowscale, ctx->d_status, s);
        if (front_done) {
            x_ready = convert;
            mark(ctx, 2);
            mark(ctx, 3);
        } else {
            launch_route(rp, lg, L->bias, T, ids, w, ctx->d_status, s);
        }
    } else {
        rc = run_router(L, xb, T, (aux && aux->logits) ? aux->logits : nullptr, ids, w);
        if (rc) return rc;
    }
    if (!front_done) {
        Range range("strata_moe.group");
        mark(ctx, 2);
        launch_group(ids, P, 0, d.experts, counts, offsets, perm, L->inv, L->active, L->n_active,
                     L->group_scratch, s);
        mark(ctx, 3);
    }
    bool y_half = true;
    const SpreadRows spread{L->inv, T, d.top_k, nullptr};
    rc = run_experts(L, xb, perm, d.top_k, P, d.experts, offsets, L->active, L->n_active, T, L->y, 0, nullptr, x_ready,
                     &y_half, nullptr, d.top_k <= 32u ? &spread : nullptr);
    if (rc) return rc;
    const float* shared = nullptr;
    if (fork_shared) {
        CK(cudaStreamWaitEvent(s, ctx->ev_join, 0));
        shared = L->sh_y;
    } else if (d.shared_intermediate) {   // timed run: keep the phases serial so they can be told apart
        uint32_t* off2 = L->offsets + d.experts + 1 + 2;
        set_pair_kernel<<<1, 1, 0, s>>>(off2, 0u, T);
        ++g_kernel_launches;
        rc = run_shared(L, xb, nullptr, T, off2);
        if (rc) return rc;
        shared = L->sh_y;
    }
    mark(ctx, 7);
    {
        Range range("strata_moe.combine");
        launch_combine(L->y, L->inv, w, shared, T, d.top_k, d.hidden, d.output_scale, out, ctx->d_status, s, y_half);
    }
    mark(ctx, 8);
    CK(cudaGetLastError());
    if (ctx->timing) {
        CK(cudaEventRecord(ctx->ev1, s));
        CK(cudaEventSynchronize(ctx->ev1));
        CK(cudaEventElapsedTime(&ctx->stats.last_forward_ms, ctx->ev0, ctx->ev1));
        ctx->pev_valid = true;
    }
    ctx->stats.forward_calls++;
    return 0;
}

// The layer after routing: ids / weights given (device, [T, k], selection-rank order).
int strata_moe_forward_routed(strata_moe_layer* L, const void* x, uint32_t T, const uint32_t* ids, const float* w,
                              float* out) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!x || !out || !ids || !w) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (T > L->d.max_tokens) return fail(ctx, STRATA_MOE_E_INVALID, "tokens exceed max_tokens");
    if (L->d.expert_count != L->d.experts)
        return fail(ctx, STRATA_MOE_E_INVALID, "forward needs every expert resident; use the stage calls for expert parallelism");
    if (L->dense_in_flight) return fail(ctx, STRATA_MOE_E_BUSY, "a dense command is in flight");
    if ((uint64_t)T * L->d.top_k > L->max_pairs)
        return fail(ctx, STRATA_MOE_E_INVALID, "tokens * top_k exceed the layer's max_pairs");
    for (int r = 0; r < 3; ++r)
        for (uint32_t e = 0; e < L->d.expert_count; ++e)
            if (!L->tab[r].packed[e] || !L->tab[r].scales[e]) return fail(ctx, STRATA_MOE_E_INVALID, "an expert has no weights");
    if (T == 0) return 0;
    CK(cudaSetDevice(ctx->device));
    int rc = sync_tables(L);
    if (rc) return rc;
    cudaStream_t s = ctx->stream;
    const strata_moe_layer_desc& d = L->d;
    const uint32_t P = T * d.top_k;
    launch_group(ids, P, 0, d.experts, L->counts, L->offsets, L->perm, L->inv, L->active, L->n_active, L->group_scratch, s);
    rc = run_experts(L, (const __nv_bfloat16*)x, L->perm, d.top_k, P, d.experts, L->offsets, L->active, L->n_active, T, L->y);
    if (rc) return rc;
    launch_combine(L->y, L->inv, w, nullptr, T, d.top_k, d.hidden, d.output_scale, out, ctx->d_status, s);
    CK(cudaGetLastError());
    ctx->stats.forward_calls++;
    return 0;
}

int strata_moe_forward_host(strata_moe_layer* L, const void* x_host, uint32_t T, float* out_host) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!x_host || !out_host) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (T > L->d.max_tokens) return fail(ctx, STRATA_MOE_E_INVALID, "tokens exceed max_tokens");
    if (T == 0) return 0;
    CK(cudaSetDevice(ctx->device));
    bind_ws(L);
    const size_t H = L->d.hidden;
    const size_t in_bytes = (size_t)T * H * 2, out_bytes = (size_t)T * H * 4;
    ctx->stats.h2d_bytes += in_bytes;
    ctx->stats.d2h_bytes += out_bytes;
    // Large batches go through in token chunks: the copy of chunk i + 1 into the device and the copy of chunk i - 1
    // back to the host run on their own streams while chunk i computes.  Tokens are independent, so the result is
    // bit-identical to the one-piece call; the expert GEMMs see fewer rows per expert per chunk, which costs less than
    // the copies it hides (16384 tokens of c3: 235 MB in, 470 MB out, about 14 ms of PCIe time beside 12 ms of compute).
    // by default up to three chunks, and only while a chunk still brings every expert most of a 192-token tile on
    // average: with fewer rows per expert the GEMMs lose more than the copies hide (4096 tokens of c2 in two chunks:
    // 606 k tokens/s end to end against 685 k in one piece; 16384 tokens of c3: 680 k in one piece, 851 k in two
    // chunks, 981 k in three -- 171 rows per expert, still one tile each -- and 935 k in four)
    uint32_t parts = 1u;
    if (L->knobs.host_chunks > 0) {
        parts = (uint32_t)L->knobs.host_chunks;
    } else if (T >= 4096u) {
        for (uint32_t p = 3u; p >= 2u; --p)
            if ((uint64_t)(T / p) * L->d.top_k >= 160ull * L->d.experts) {
                parts = p;
                break;
            }
    }
    if (parts > 4u) parts = 4u;
    if (parts > T) parts = T;
    // only while every chunk stays on the expert path the whole batch would take (the tensor-core path): the paths
    // round the SwiGLU output differently, and the chunked call must return the one-piece call's bits
    while (parts > 1u && !(use_prefill(L, T * L->d.top_k, L->d.experts) &&
                           use_prefill(L, (T / parts) * L->d.top_k, L->d.experts)))
        --parts;
    if (parts <= 1u) {
        CK(cudaMemcpyAsync(L->x_stage, x_host, in_bytes, cudaMemcpyHostToDevice, ctx->stream));
        int rc = strata_moe_forward(L, L->x_stage, T, L->out_stage, nullptr);
        if (rc) return rc;
        CK(cudaMemcpyAsync(out_host, L->out_stage, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        return strata_moe_synchronize(ctx);
    }
    if (!ctx->copy_in) {
        CK(cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
        CK(cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
        for (int i = 0; i < 4; ++i) {
            CK(cudaEventCreateWithFlags(&ctx->ev_in[i], cudaEventDisableTiming));
            CK(cudaEventCreateWithFlags(&ctx->ev_done[i], cudaEventDisableTiming));
        }
    }
    // whatever the caller enqueued on the context's stream comes first
    CK(cudaEventRecord(ctx->ev_done[0], ctx->stream));
    CK(cudaStreamWaitEvent(ctx->copy_in, ctx->ev_done[0], 0));
    uint32_t begin[5];
    for (uint32_t i = 0; i <= parts; ++i) begin[i] = (uint32_t)((uint64_t)T * i / parts);
    const uint8_t* xh = static_cast<const uint8_t*>(x_host);
    for (uint32_t i = 0; i < parts; ++i) {
        const size_t off = (size_t)begin[i] * H, n = (size_t)(begin[i + 1] - begin[i]) * H;
        CK(cudaMemcpyAsync(L->x_stage + off, xh + off * 2, n * 2, cudaMemcpyHostToDevice, ctx->copy_in));
        CK(cudaEventRecord(ctx->ev_in[i], ctx->copy_in));
    }
    for (uint32_t i = 0; i < parts; ++i) {
        const size_t off = (size_t)begin[i] * H, n = (size_t)(begin[i + 1] - begin[i]) * H;
        CK(cudaStreamWaitEvent(ctx->stream, ctx->ev_in[i], 0));
        int rc = strata_moe_forward(L, L->x_stage + off, begin[i + 1] - begin[i], L->out_stage + off, nullptr);
        if (rc) {
            cudaStreamSynchronize(ctx->copy_in);
            cudaStreamSynchronize(ctx->copy_out);
            return rc;
        }
        bind_ws(L);
        CK(cudaEventRecord(ctx->ev_done[i], ctx->stream));
        CK(cudaStreamWaitEvent(ctx->copy_out, ctx->ev_done[i], 0));
        CK(cudaMemcpyAsync(out_host + off, L->out_stage + off, n * 4, cudaMemcpyDeviceToHost, ctx->copy_out));
    }
    CK(cudaStreamSynchronize(ctx->copy_out));
    return strata_moe_synchronize(ctx);
}

int strata_moe_dequant_export(strata_moe_layer* L, uint32_t expert, int role, float* out_host) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!out_host || role < 0 || role > 2) return fail(ctx, STRATA_MOE_E_INVALID, "bad argument");
    if (expert < L->d.expert_begin || expert >= L->d.expert_begin + L->d.expert_count)
        return fail(ctx, STRATA_MOE_E_INVALID, "expert is not resident on this device");
    const uint32_t le = expert - L->d.expert_begin;
    if (!L->tab[role].packed[le]) return fail(ctx, STRATA_MOE_E_INVALID, "expert has no weights");
    CK(cudaSetDevice(ctx->device));
    const uint32_t rows = role == STRATA_MOE_ROLE_DOWN ? L->d.hidden : L->d.intermediate;
    const uint32_t cols = role == STRATA_MOE_ROLE_DOWN ? L->d.intermediate : L->d.hidden;
    int rc0 = sync_tables(L);
    if (rc0) return rc0;
    float* tmp = nullptr;
    CK(cudaMalloc(&tmp, (size_t)rows * cols * 4));
    if (L->d.format == STRATA_MOE_FMT_BF16) {
        widen_bf16_kernel<<<148 * 4, 256, 0, ctx->stream>>>(
            reinterpret_cast<const __nv_bfloat16*>(L->tab[role].packed[le]), (size_t)rows * cols, tmp);
        ++g_kernel_launches;
    } else if (L->f16_ok) {
        // export what the f16 weight-streaming kernels consume
        uint32_t emin = 0;
        float post = 1.0f;
        CK(cudaMemcpy(&emin, L->tab[role].d_emin + le, sizeof(uint32_t), cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(&post, L->tab[role].d_post + le, sizeof(float), cudaMemcpyDeviceToHost));
        launch_dequant_export_f16(L->d.format, L->tab[role].packed[le], L->tab[role].scales[le], emin, post,
                                  rows, cols, tmp, ctx->stream);
    } else {
        launch_dequant_export(L->d.format, L->tab[role].packed[le], L->tab[role].scales[le],
                              L->tab[role].global[le], rows, cols, tmp, ctx->stream);
    }
    cudaError_t e = cudaMemcpyAsync(out_host, tmp, (size_t)rows * cols * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(tmp);
    if (e != cudaSuccess) return fail(ctx, STRATA_MOE_E_CUDA, cudaGetErrorString(e));
    return 0;
}

int strata_moe_enqueue_dense(strata_moe_layer* L, const float* hidden_host, uint32_t rows,
                             const uint32_t* experts, const float* coefficients, uint32_t n, int with_shared) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    const strata_moe_layer_desc& d = L->d;
    if (L->dense_in_flight)
        return fail(ctx, STRATA_MOE_E_BUSY, "a MoE command is already in flight on this layer");
    if (ctx->ws_owner && ctx->ws_owner != L)
        return fail(ctx, STRATA_MOE_E_BUSY, "a MoE command of another layer of this context is in flight");
    if (!hidden_host || rows == 0) return fail(ctx, STRATA_MOE_E_INVALID, "hidden rows are required");
    if (n == 0 && !with_shared) return fail(ctx, STRATA_MOE_E_INVALID, "command has no experts");
    if (n && (!experts || !coefficients)) return fail(ctx, STRATA_MOE_E_INVALID, "null expert list");
    // the pointer tables of a command hold one slot per resident expert (the reference bounds its
    // list the same way, kernels/cuda/backend.cu:1209-1213)
    if (n > d.expert_count) return fail(ctx, STRATA_MOE_E_INVALID, "more experts listed than are resident");
    if ((uint64_t)n * rows > L->max_pairs) return fail(ctx, STRATA_MOE_E_INVALID, "experts * rows exceed max_pairs");
    if (rows > d.max_tokens) return fail(ctx, STRATA_MOE_E_INVALID, "rows exceed max_tokens");
    if (with_shared && !d.shared_intermediate) return fail(ctx, STRATA_MOE_E_INVALID, "layer has no shared expert");
    for (uint32_t i = 0; i < n; ++i) {
        if (experts[i] < d.expert_begin || experts[i] >= d.expert_begin + d.expert_count)
            return fail(ctx, STRATA_MOE_E_INVALID, "expert is not resident on this device");
        const uint32_t le = experts[i] - d.expert_begin;
        for (int r = 0; r < 3; ++r)
            if (!L->tab[r].packed[le]) return fail(ctx, STRATA_MOE_E_INVALID, "expert has no weights");
        if (!(coefficients[i] == coefficients[i]) || !(fabsf(coefficients[i]) <= 3.0e38f))
            return fail(ctx, STRATA_MOE_E_INVALID, "coefficient is not finite");
        if (d.format != STRATA_MOE_FMT_INT4G128 && coefficients[i] != 1.0f)
            return fail(ctx, STRATA_MOE_E_INVALID, "only INT4 experts fold a coefficient; pass 1.0");
    }
    CK(cudaSetDevice(ctx->device));
    bind_ws(L);
    cudaStream_t s = ctx->stream;
    const uint32_t H = d.hidden;
    if (!L->dense_hidden) {
        CK(dalloc(L, &L->dense_hidden, (size_t)d.max_tokens * H));
        CK(dalloc(L, &L->dense_coef, (size_t)L->max_pairs));
        CK(dalloc(L, &L->dense_ptrs, (size_t)6 * d.expert_count));
        CK(dalloc(L, &L->dense_globals, (size_t)3 * d.expert_count));
        CK(ws_reserve(ctx, kWsXgLo, (size_t)L->max_pairs * H * 2));
        bind_ws(L);
        CK(cudaMallocHost(&L->dense_pinned, (size_t)d.expert_count * (6 * sizeof(void*) + 3 * sizeof(float)) +
                                                (size_t)L->max_pairs * sizeof(float)));
    }
    CK(cudaMemcpyAsync(L->dense_hidden, hidden_host, (size_t)rows * H * 4, cudaMemcpyHostToDevice, s));
    ctx->stats.h2d_bytes += (size_t)rows * H * 4;
    const uint32_t ne = d.expert_count;
    const uint8_t** hp = static_cast<const uint8_t**>(L->dense_pinned);
    float* hg = reinterpret_cast<float*>(hp + 6 * ne);
    float* hc = hg + 3 * ne;
    for (uint32_t i = 0; i < n; ++i) {
        const uint32_t le = experts[i] - d.expert_begin;
        for (int r = 0; r < 3; ++r) {
            hp[(2 * r) * ne + i] = L->tab[r].packed[le];
            hp[(2 * r + 1) * ne + i] = L->tab[r].scales[le];
            hg[r * ne + i] = L->tab[r].global[le];
        }
        for (uint32_t rrow = 0; rrow < rows; ++rrow) hc[(size_t)i * rows + rrow] = coefficients[i];
    }
    uint32_t* off = L->offsets;
    if (n) {
        CK(cudaMemcpyAsync(L->dense_ptrs, hp, 6 * ne * sizeof(void*), cudaMemcpyHostToDevice, s));
        CK(cudaMemcpyAsync(L->dense_globals, hg, 3 * ne * sizeof(float), cudaMemcpyHostToDevice, s));
        CK(cudaMemcpyAsync(L->dense_coef, hc, (size_t)n * rows * sizeof(float), cudaMemcpyHostToDevice, s));
        uniform_offsets_kernel<<<1, 256, 0, s>>>(off, n, rows);
        ++g_kernel_launches;
        launch_gather_rows_kperm_f32(L->dense_hidden, rows, n, H, L->xg, L->xg_lo, s, d.format == STRATA_MOE_FMT_BF16);
        DecodeArgs a{};
        a.fmt = d.format;
        a.H = H;
        a.I = d.intermediate;
        a.n_groups = n;
        a.offsets = off;
        a.max_rows_per_group = rows;
        a.gate = WeightTable{L->dense_ptrs + 0 * ne, L->dense_ptrs + 1 * ne, L->dense_globals + 0 * ne};
        a.up = WeightTable{L->dense_ptrs + 2 * ne, L->dense_ptrs + 3 * ne, L->dense_globals + 1 * ne};
        a.down = WeightTable{L->dense_ptrs + 4 * ne, L->dense_ptrs + 5 * ne, L->dense_globals + 2 * ne};
        a.x_hi = L->xg;
        a.x_lo = L->xg_lo;
        a.coef = d.format == STRATA_MOE_FMT_INT4G128 ? L->dense_coef : nullptr;
        a.act_hi = L->act_hi;
        a.act_lo = L->act_lo;
        a.y = L->y;
        a.status = ctx->d_status;
        a.glu = GluParams{L->d.activation, L->d.gate_beta, L->d.linear_beta};
        launch_decode_gate_up(a, s);
        launch_decode_down(a, s);
    }
    if (with_shared) {
        for (int r = 0; r < 3; ++r)
            if (!L->shared_w[r]) return fail(ctx, STRATA_MOE_E_INVALID, "shared expert weights were never set");
        uint32_t* off2 = L->offsets + d.experts + 1 + 2;
        set_pair_kernel<<<1, 1, 0, s>>>(off2, 0u, rows);
        // natural-layout hi/lo split of the fp32 rows for the BF16 shared expert
        __nv_bfloat16* sh_hi = L->x_stage;
        __nv_bfloat16* sh_lo = reinterpret_cast<__nv_bfloat16*>(L->out_stage);
        split_f32_kernel<<<148, 256, 0, s>>>(L->dense_hidden, (size_t)rows * H, sh_hi, sh_lo);
        g_kernel_launches += 2;
        int rc = run_shared(L, sh_hi, sh_lo, rows, off2);
        if (rc) return rc;
    }
    CK(cudaGetLastError());
    L->dense_in_flight = true;
    ctx->ws_owner = L;
    L->dense_rows = rows;
    L->dense_n = n;
    L->dense_shared = with_shared != 0;
    return 0;
}

int strata_moe_collect_dense(strata_moe_layer* L, float* routed_output, float* shared_output) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!L->dense_in_flight) return fail(ctx, STRATA_MOE_E_INVALID, "no MoE command is in flight");
    CK(cudaSetDevice(ctx->device));
    bind_ws(L);
    // results reach the caller only after completion and a clean status are confirmed
    int rc = strata_moe_synchronize(ctx);
    L->dense_in_flight = false;
    ctx->ws_owner = nullptr;
    if (rc) return rc;
    const size_t H = L->d.hidden;
    if (L->dense_n) {
        if (!routed_output) return fail(ctx, STRATA_MOE_E_INVALID, "routed output buffer is required");
        CK(cudaMemcpyAsync(routed_output, L->y, (size_t)L->dense_n * L->dense_rows * H * 4,
                           cudaMemcpyDeviceToHost, ctx->stream));
        ctx->stats.d2h_bytes += (size_t)L->dense_n * L->dense_rows * H * 4;
    }
    if (L->dense_shared) {
        if (!shared_output) return fail(ctx, STRATA_MOE_E_INVALID, "shared output buffer is required");
        CK(cudaMemcpyAsync(shared_output, L->sh_y, (size_t)L->dense_rows * H * 4, cudaMemcpyDeviceToHost,
                           ctx->stream));
        ctx->stats.d2h_bytes += (size_t)L->dense_rows * H * 4;
    }
    CK(cudaStreamSynchronize(ctx->stream));
    return 0;
}

// ------------------------------------------------------------------------- DSV4-exact mode
int strata_moe_quantize_e4m3(strata_moe_ctx* ctx, float* values, uint32_t rows, uint32_t cols) {
    if (!ctx) return STRATA_MOE_E_INVALID;
    if (!values && rows && cols) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    CK(cudaSetDevice(ctx->device));
    launch_dsv4_quantize(values, nullptr, 1, rows, cols, values, ctx->stream);
    CK(cudaGetLastError());
    return 0;
}

// rows_f32 [*, H] fp32; row_index (device, or nullptr = rows already in group order) names the source row of
// every grouped row.
static int dsv4_grouped_core(strata_moe_layer* L, const float* rows_f32, const uint32_t* row_index, uint32_t pairs,
                             const uint32_t* offsets, const float* coefficients, float swiglu_limit, float* y) {
    strata_moe_ctx* ctx = L->ctx;
    if (!rows_f32 || !offsets || !y) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (L->d.format != STRATA_MOE_FMT_MXFP4)
        return fail(ctx, STRATA_MOE_E_INVALID, "the DSV4-exact mode needs FP4 E2M1 weights with E8M0 block scales");
    if (pairs > L->max_pairs) return fail(ctx, STRATA_MOE_E_INVALID, "pairs exceed max_pairs");
    if (!(swiglu_limit > 0.0f && swiglu_limit < 3.0e38f))
        return fail(ctx, STRATA_MOE_E_INVALID, "SwiGLU limit must be finite and positive");
    for (int r = 0; r < 3; ++r)
        for (uint32_t e = 0; e < L->d.expert_count; ++e)
            if (!L->tab[r].packed[e] || !L->tab[r].scales[e]) return fail(ctx, STRATA_MOE_E_INVALID, "an expert has no weights");
    if (pairs == 0) return 0;
    CK(cudaSetDevice(ctx->device));
    int rc = sync_tables(L);
    if (rc) return rc;
    cudaStream_t s = ctx->stream;
    const uint32_t H = L->d.hidden, I = L->d.intermediate, n = L->d.expert_count;
    float* xq = L->y;            // [pairs, H] scratch: the E4M3-quantised input rows
    float* act = L->act_f32;     // [pairs, I]
    launch_dsv4_quantize(rows_f32, row_index, 1, pairs, H, xq, s);
    launch_dsv4_gate_up(n, offsets, H, I, wt(L->tab[0]), wt(L->tab[1]), xq, coefficients, swiglu_limit, act,
                        ctx->d_status, s);
    launch_dsv4_quantize(act, nullptr, 1, pairs, I, act, s);
    launch_dsv4_down(n, offsets, H, I, wt(L->tab[2]), act, y, ctx->d_status, s);
    CK(cudaGetLastError());
    return 0;
}

int strata_moe_experts_grouped_dsv4(strata_moe_layer* L, const float* rows_f32, uint32_t pairs,
                                    const uint32_t* offsets, const float* coefficients, float swiglu_limit,
                                    float* y) {
    if (!L) return STRATA_MOE_E_INVALID;
    return dsv4_grouped_core(L, rows_f32, nullptr, pairs, offsets, coefficients, swiglu_limit, y);
}

int strata_moe_combine_dsv4(strata_moe_layer* L, const float* y, const uint32_t* inv, const float* shared_rows,
                            uint32_t T, float* out) {
    if (!L) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    if (!y || !inv || !out) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (T > L->d.max_tokens) return fail(ctx, STRATA_MOE_E_INVALID, "tokens exceed max_tokens");
    CK(cudaSetDevice(ctx->device));
    launch_dsv4_join(y, inv, shared_rows, T, L->d.top_k, L->d.hidden, out, ctx->d_status, ctx->stream);
    CK(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------------- LatentMoE wrapper
struct strata_moe_latent {
    strata_moe_ctx* ctx = nullptr;
    strata_moe_layer* route = nullptr;     // router + shared experts on the raw hidden state
    strata_moe_layer* experts = nullptr;   // routed experts on the latent
    uint32_t H = 0, HL = 0, max_tokens = 0;
    float eps = 0.0f;
    const __nv_bfloat16 *down = nullptr, *up = nullptr;
    const float* norm = nullptr;
    std::vector<void*> owned;
    float *latent_f32 = nullptr, *mix = nullptr, *w = nullptr;
    __nv_bfloat16 *latent_bf16 = nullptr, *mixn = nullptr;
    uint32_t *tiles = nullptr, *off2 = nullptr, *ids = nullptr;
};

int strata_moe_latent_create(strata_moe_ctx* ctx, const strata_moe_layer_desc* desc, uint32_t model_hidden,
                             float rms_epsilon, strata_moe_latent** out) {
    if (!ctx || !desc || !out) return STRATA_MOE_E_INVALID;
    *out = nullptr;
    if (model_hidden == 0 || model_hidden % 128u) return fail(ctx, STRATA_MOE_E_INVALID, "model hidden must be a positive multiple of 128");
    if (desc->expert_count != desc->experts || desc->expert_begin != 0)
        return fail(ctx, STRATA_MOE_E_INVALID, "the LatentMoE wrapper needs every expert resident");
    if (!(rms_epsilon >= 0.0f) || !(rms_epsilon < 1.0f)) return fail(ctx, STRATA_MOE_E_INVALID, "RMS epsilon out of range");
    if (desc->score_kind == STRATA_MOE_SCORE_SOFTMAX && false) return STRATA_MOE_E_INVALID;
    CK(cudaSetDevice(ctx->device));
    strata_moe_latent* lat = new (std::nothrow) strata_moe_latent();
    if (!lat) return fail(ctx, STRATA_MOE_E_INVALID, "out of host memory");
    lat->ctx = ctx;
    lat->H = model_hidden;
    lat->HL = desc->hidden;
    lat->eps = rms_epsilon;
    lat->max_tokens = desc->max_tokens;
    strata_moe_layer_desc ed = *desc;
    ed.shared_intermediate = 0;
    strata_moe_layer_desc rd = *desc;      // router + shared experts: no routed weights, minimal pair workspaces
    rd.hidden = model_hidden;
    rd.intermediate = 128;
    rd.format = STRATA_MOE_FMT_BF16;
    rd.max_pairs = 1;
    int rc = strata_moe_layer_create(ctx, &ed, &lat->experts);
    if (rc == 0) rc = strata_moe_layer_create(ctx, &rd, &lat->route);
    const size_t T = desc->max_tokens;
    cudaError_t e = cudaSuccess;
    auto alloc = [&](void** p, size_t bytes) {
        if (rc != 0 || e != cudaSuccess) return;
        e = cudaMalloc(p, bytes ? bytes : 16);
        if (e == cudaSuccess) lat->owned.push_back(*p);
    };
    alloc((void**)&lat->latent_f32, T * lat->HL * 4);
    alloc((void**)&lat->mix, T * lat->HL * 4);
    alloc((void**)&lat->latent_bf16, T * lat->HL * 2);
    alloc((void**)&lat->mixn, T * lat->HL * 2);
    alloc((void**)&lat->tiles, prefill_scratch_bytes(1, (uint32_t)T) + 16);
    alloc((void**)&lat->off2, 16);
    alloc((void**)&lat->ids, T * desc->top_k * 4);
    alloc((void**)&lat->w, T * desc->top_k * 4);
    if (rc != 0 || e != cudaSuccess) {
        const std::string msg = rc != 0 ? ctx->err : std::string("LatentMoE allocation: ") + cudaGetErrorString(e);
        strata_moe_latent_destroy(lat);
        return fail(ctx, rc != 0 ? rc : STRATA_MOE_E_CUDA, msg);
    }
    *out = lat;
    return 0;
}

void strata_moe_latent_destroy(strata_moe_latent* lat) {
    if (!lat) return;
    cudaSetDevice(lat->ctx->device);
    cudaStreamSynchronize(lat->ctx->stream);
    if (lat->experts) strata_moe_layer_destroy(lat->experts);
    if (lat->route) strata_moe_layer_destroy(lat->route);
    for (void* p : lat->owned) cudaFree(p);
    delete lat;
}

strata_moe_layer* strata_moe_latent_experts(strata_moe_latent* lat) { return lat ? lat->experts : nullptr; }

int strata_moe_latent_set_router(strata_moe_latent* lat, const void* gate_bf16, const float* bias, int source) {
    if (!lat) return STRATA_MOE_E_INVALID;
    return strata_moe_set_router(lat->route, gate_bf16, bias, source);
}

int strata_moe_latent_set_shared(strata_moe_latent* lat, int role, const void* w, int source) {
    if (!lat) return STRATA_MOE_E_INVALID;
    return strata_moe_set_shared(lat->route, role, w, source);
}

int strata_moe_latent_set_projections(strata_moe_latent* lat, const void* down, const void* up, const float* norm,
                                      int source) {
    if (!lat) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = lat->ctx;
    if (!down || !up || !norm) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    CK(cudaSetDevice(ctx->device));
    const void* p = nullptr;
    int rc = put(lat->route, down, (size_t)lat->HL * lat->H * 2, source, &p);   // storage owned by the routing layer
    if (rc) return rc;
    lat->down = static_cast<const __nv_bfloat16*>(p);
    rc = put(lat->route, up, (size_t)lat->H * lat->HL * 2, source, &p);
    if (rc) return rc;
    lat->up = static_cast<const __nv_bfloat16*>(p);
    rc = put(lat->route, norm, (size_t)lat->HL * 4, source, &p);
    if (rc) return rc;
    lat->norm = static_cast<const float*>(p);
    if ((((uintptr_t)lat->down | (uintptr_t)lat->up) & 15u) != 0)
        return fail(ctx, STRATA_MOE_E_INVALID, "projection weights must be 16-byte aligned");
    return 0;
}

int strata_moe_latent_forward(strata_moe_latent* lat, const void* x, uint32_t T, float* out, uint32_t* ids_out,
                              float* weights_out) {
    if (!lat) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = lat->ctx;
    if (!x || !out) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (T > lat->max_tokens) return fail(ctx, STRATA_MOE_E_INVALID, "tokens exceed max_tokens");
    if (!lat->down || !lat->up || !lat->norm) return fail(ctx, STRATA_MOE_E_INVALID, "latent projections were never set");
    if (((uintptr_t)x & 15u) != 0) return fail(ctx, STRATA_MOE_E_INVALID, "activations must be 16-byte aligned");
    if (T == 0) return 0;
    CK(cudaSetDevice(ctx->device));
    cudaStream_t s = ctx->stream;
    strata_moe_layer* R = lat->route;
    bind_ws(R);
    const strata_moe_layer_desc& rd = R->d;
    if (!tensor_path_ok(R, 3, 128)) return fail(ctx, STRATA_MOE_E_INVALID, "the LatentMoE projections need the tensor-core path");
    uint32_t* ids = ids_out ? ids_out : lat->ids;
    float* w = weights_out ? weights_out : lat->w;
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    const bool shared = rd.shared_intermediate != 0;
    if (shared) {   // the shared experts need only x: side stream, joined before the final add
        for (int r = 0; r < 3; ++r)
            if (!R->shared_w[r]) return fail(ctx, STRATA_MOE_E_INVALID, "shared expert weights were never set");
        uint32_t* off2 = R->offsets + rd.experts + 1 + 2;
        set_pair_kernel<<<1, 1, 0, s>>>(off2, 0u, T);
        ++g_kernel_launches;
        CK(cudaEventRecord(ctx->ev_fork, s));
        CK(cudaStreamWaitEvent(ctx->side, ctx->ev_fork, 0));
        int rc = run_shared(R, xb, nullptr, T, off2, ctx->side);
        if (rc) return rc;
        CK(cudaEventRecord(ctx->ev_join, ctx->side));
    }
    int rc = strata_moe_route(R, x, T, nullptr, ids, w);      // routing reads the raw hidden state
    if (rc) return rc;
    set_pair_kernel<<<1, 1, 0, s>>>(lat->off2, 0u, T);
    ++g_kernel_launches;
    if (launch_router_tc(x, T, lat->down, lat->HL, lat->H, lat->latent_f32, lat->tiles, lat->off2, ctx->d_status, s) != 0)
        return fail(ctx, STRATA_MOE_E_CUDA, "latent down projection launch failed");
    launch_f32_to_bf16(lat->latent_f32, (size_t)T * lat->HL, lat->latent_bf16, s);
    rc = strata_moe_forward_routed(lat->experts, lat->latent_bf16, T, ids, w, lat->mix);
    if (rc) return rc;
    launch_rmsnorm_bf16(lat->mix, lat->norm, T, lat->HL, lat->eps, lat->mixn, ctx->d_status, s);
    if (launch_router_tc(lat->mixn, T, lat->up, lat->H, lat->HL, out, lat->tiles, lat->off2, ctx->d_status, s) != 0)
        return fail(ctx, STRATA_MOE_E_CUDA, "latent up projection launch failed");
    if (shared) {
        CK(cudaStreamWaitEvent(s, ctx->ev_join, 0));
        bind_ws(R);
        launch_add_rows(out, R->sh_y, (size_t)T * lat->H, s);
    }
    CK(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------------- weight handles + commands
struct strata_moe_weight {
    strata_moe_ctx* ctx = nullptr;
    int fmt = 0;
    uint32_t rows = 0, cols = 0;
    float global_scale = 1.0f;
    uint8_t* packed = nullptr;   // one allocation: packed bytes, then the scales at a 256-byte aligned offset
    uint8_t* scales = nullptr;
};

static size_t handle_packed_bytes(int fmt, uint32_t rows, uint32_t cols) {
    if (fmt == STRATA_MOE_FMT_FP8B128) return (size_t)rows * cols;
    return packed_bytes(fmt, rows, cols);
}
static size_t handle_scale_bytes(int fmt, uint32_t rows, uint32_t cols) {
    if (fmt == STRATA_MOE_FMT_FP8B128) return (size_t)((rows + 127u) / 128u) * ((cols + 127u) / 128u);
    return scale_bytes(fmt, rows, cols);
}

int strata_moe_weight_upload(strata_moe_ctx* ctx, const strata_moe_weight_desc* desc, const void* weights_host,
                             size_t weight_bytes, const void* scales_host, size_t scale_bytes_in,
                             strata_moe_weight** out) {
    if (!ctx || !desc || !out) return STRATA_MOE_E_INVALID;
    *out = nullptr;
    if (desc->format < 0 || desc->format > STRATA_MOE_FMT_FP8B128)
        return fail(ctx, STRATA_MOE_E_INVALID, "unknown weight encoding");
    if (desc->rows == 0 || desc->cols == 0 || desc->rows % 128u || desc->cols % 128u)
        return fail(ctx, STRATA_MOE_E_INVALID, "weight rows and columns must be positive multiples of 128");
    const size_t pb = handle_packed_bytes(desc->format, desc->rows, desc->cols);
    const size_t sb = handle_scale_bytes(desc->format, desc->rows, desc->cols);
    if (!weights_host || weight_bytes != pb) return fail(ctx, STRATA_MOE_E_INVALID, "weight payload size does not match the descriptor");
    if (sb && (!scales_host || scale_bytes_in != sb))
        return fail(ctx, STRATA_MOE_E_INVALID, "scale payload size does not match the descriptor");
    if (desc->format == STRATA_MOE_FMT_NVFP4 && !(desc->global_scale > 0.0f && desc->global_scale < 3.0e38f))
        return fail(ctx, STRATA_MOE_E_INVALID, "NVFP4 global scale must be finite and positive");
    CK(cudaSetDevice(ctx->device));
    strata_moe_weight* w = new (std::nothrow) strata_moe_weight();
    if (!w) return fail(ctx, STRATA_MOE_E_INVALID, "out of host memory");
    const size_t soff = (pb + 255) / 256 * 256;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, soff + (sb ? sb : 16));
    if (e == cudaSuccess) e = cudaMemcpyAsync(p, weights_host, pb, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess && sb)
        e = cudaMemcpyAsync(static_cast<uint8_t*>(p) + soff, scales_host, sb, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);   // the host spans may go away when this returns
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        delete w;
        return fail(ctx, STRATA_MOE_E_CUDA, std::string("weight upload: ") + cudaGetErrorString(e));
    }
    w->ctx = ctx;
    w->fmt = desc->format;
    w->rows = desc->rows;
    w->cols = desc->cols;
    w->global_scale = desc->format == STRATA_MOE_FMT_NVFP4 ? desc->global_scale : 1.0f;
    w->packed = static_cast<uint8_t*>(p);
    w->scales = sb ? w->packed + soff : w->packed;
    ctx->stats.h2d_bytes += pb + sb;
    ctx->stats.weight_bytes += pb + sb;
    *out = w;
    return 0;
}

void strata_moe_weight_release(strata_moe_weight* w) {
    if (!w) return;
    cudaSetDevice(w->ctx->device);
    cudaStreamSynchronize(w->ctx->stream);   // nothing enqueued may still read it
    cudaFree(w->packed);
    delete w;
}

}  // extern "C"

namespace {

// The internal layer of the handle-based commands: its expert slots borrow the weights of the command in
// flight.  Rebuilt (and counted) only when the shape changes or a command needs more room.
int ensure_cmd_layer(strata_moe_ctx* ctx, int fmt, uint32_t H, uint32_t I, uint32_t slots, uint32_t rows, uint32_t pairs) {
    strata_moe_layer* L = ctx->cmd_layer;
    if (L && L->d.format == fmt && L->d.hidden == H && L->d.intermediate == I && L->d.expert_count >= slots &&
        L->d.max_tokens >= rows && L->max_pairs >= pairs)
        return 0;
    if (L) {
        strata_moe_layer_destroy(L);
        ctx->cmd_layer = nullptr;
    }
    strata_moe_layer_desc d{};
    d.hidden = H;
    d.intermediate = I;
    d.experts = d.expert_count = slots < 16u ? 16u : (slots + 15u) / 16u * 16u;
    d.top_k = 1;
    d.format = fmt;
    d.score_kind = STRATA_MOE_SCORE_SIGMOID;
    d.weight_scale = d.output_scale = 1.0f;
    d.max_tokens = rows < 64u ? 64u : rows + rows / 2u;
    d.max_pairs = pairs < 256u ? 256u : pairs + pairs / 2u;
    if (d.max_pairs < d.max_tokens) d.max_pairs = d.max_tokens;
    d.activation = STRATA_MOE_ACT_SWIGLU;
    int rc = strata_moe_layer_create(ctx, &d, &ctx->cmd_layer);
    if (rc == 0) ++ctx->workspace_allocations;
    return rc;
}

void cmd_release_scratch(strata_moe_ctx* ctx) {
    for (void* p : ctx->cmd_scratch) cudaFree(p);
    ctx->cmd_scratch.clear();
}

template <typename T>
cudaError_t cmd_alloc(strata_moe_ctx* ctx, T** p, size_t n) {
    void* v = nullptr;
    cudaError_t e = cudaMalloc(&v, (n ? n : 1) * sizeof(T));
    if (e == cudaSuccess) {
        ctx->cmd_scratch.push_back(v);
        *p = static_cast<T*>(v);
    }
    return e;
}

bool same_device(const strata_moe_ctx* ctx, const strata_moe_weight* w) { return w && w->ctx == ctx; }

}  // namespace

extern "C" {

int strata_moe_command_enqueue(strata_moe_ctx* ctx, const float* hidden, size_t hidden_floats, uint32_t rows,
                               const strata_moe_expert_ref* routed, uint32_t n, const strata_moe_expert_ref* shared) {
    if (!ctx) return STRATA_MOE_E_INVALID;
    if (ctx->cmd_kind != 0) return fail(ctx, STRATA_MOE_E_BUSY, "MoE workspace already has an in-flight command");
    const uint32_t total = n + (shared ? 1u : 0u);
    // limits of the reference command: at most 10 routed experts, 11 with the shared one
    if (rows == 0 || total == 0 || total > 11u || n > 10u || (n && !routed))
        return fail(ctx, STRATA_MOE_E_INVALID, "MoE command has an unsupported row or expert count");
    const strata_moe_weight* first = n ? routed[0].gate : shared->gate;
    if (!same_device(ctx, first)) return fail(ctx, STRATA_MOE_E_INVALID, "MoE command has no valid leading expert");
    const int fmt = first->fmt;
    if (fmt != STRATA_MOE_FMT_INT4G128 && fmt != STRATA_MOE_FMT_NVFP4 && fmt != STRATA_MOE_FMT_BF16)
        return fail(ctx, STRATA_MOE_E_INVALID, "MoE command has an unsupported weight encoding");
    const uint32_t H = first->cols, I = first->rows;
    for (uint32_t i = 0; i < total; ++i) {
        const strata_moe_expert_ref& e = i < n ? routed[i] : *shared;
        const strata_moe_weight* ws[3] = {e.gate, e.up, e.down};
        for (const strata_moe_weight* w : ws)
            if (!same_device(ctx, w) || w->fmt != fmt)
                return fail(ctx, STRATA_MOE_E_INVALID, "MoE command contains an incompatible CUDA weight");
        if (e.gate->rows != I || e.gate->cols != H || e.up->rows != I || e.up->cols != H || e.down->rows != H ||
            e.down->cols != I)
            return fail(ctx, STRATA_MOE_E_INVALID, i == 0 ? "MoE gate/up/down shapes are incompatible"
                                                          : "MoE experts do not share one activation shape");
        if (!(e.coefficient == e.coefficient) || !(fabsf(e.coefficient) <= 3.0e38f) ||
            ((i >= n || fmt != STRATA_MOE_FMT_INT4G128) && e.coefficient != 1.0f))
            return fail(ctx, STRATA_MOE_E_INVALID, "MoE expert coefficient is invalid");
    }
    if (!hidden || hidden_floats != (size_t)rows * H) return fail(ctx, STRATA_MOE_E_INVALID, "MoE hidden rows are incompatible");
    for (size_t i = 0; i < hidden_floats; ++i)
        if (!(fabsf(hidden[i]) <= 3.0e38f)) return fail(ctx, STRATA_MOE_E_INVALID, "MoE hidden rows are incompatible");
    CK(cudaSetDevice(ctx->device));
    int rc = ensure_cmd_layer(ctx, fmt, H, I, total, rows, total * rows);
    if (rc) return rc;
    strata_moe_layer* L = ctx->cmd_layer;
    uint32_t ids[11];
    float coefs[11];
    for (uint32_t i = 0; i < total; ++i) {
        const strata_moe_expert_ref& e = i < n ? routed[i] : *shared;
        const strata_moe_weight* ws[3] = {e.gate, e.up, e.down};
        for (int r = 0; r < 3; ++r) {
            L->tab[r].packed[i] = ws[r]->packed;
            L->tab[r].scales[i] = ws[r]->scales;
            L->tab[r].global[i] = ws[r]->global_scale;
        }
        ids[i] = i;
        coefs[i] = e.coefficient;
    }
    L->tables_dirty = true;
    rc = strata_moe_enqueue_dense(L, hidden, rows, ids, coefs, total, 0);
    if (rc) return rc;
    ctx->cmd_kind = 1;
    ctx->cmd_n = n;
    ctx->cmd_rows = rows;
    ctx->cmd_shared = shared != nullptr;
    return 0;
}

int strata_moe_command_collect(strata_moe_ctx* ctx, float* routed_out, size_t routed_floats, float* shared_out,
                               size_t shared_floats) {
    if (!ctx) return STRATA_MOE_E_INVALID;
    if (ctx->cmd_kind != 1) return fail(ctx, STRATA_MOE_E_INVALID, "no MoE command is in flight");
    strata_moe_layer* L = ctx->cmd_layer;
    CK(cudaSetDevice(ctx->device));
    bind_ws(L);
    // every return consumes or drains the command; results reach the caller only after completion and a
    // clean status word are confirmed
    const int rc = strata_moe_synchronize(ctx);
    ctx->cmd_kind = 0;
    L->dense_in_flight = false;
    ctx->ws_owner = nullptr;
    if (rc) return rc;
    const size_t H = L->d.hidden, row_floats = (size_t)ctx->cmd_rows * H;
    if (routed_floats != (size_t)ctx->cmd_n * row_floats || (ctx->cmd_n && !routed_out))
        return fail(ctx, STRATA_MOE_E_INVALID, "routed output span does not match the command");
    if (shared_floats != (ctx->cmd_shared ? row_floats : 0u) || (ctx->cmd_shared && !shared_out))
        return fail(ctx, STRATA_MOE_E_INVALID, "shared output span does not match the command");
    if (ctx->cmd_n)
        CK(cudaMemcpyAsync(routed_out, L->y, routed_floats * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (ctx->cmd_shared)
        CK(cudaMemcpyAsync(shared_out, L->y + (size_t)ctx->cmd_n * row_floats, shared_floats * 4,
                           cudaMemcpyDeviceToHost, ctx->stream));
    CK(cudaStreamSynchronize(ctx->stream));
    ctx->stats.d2h_bytes += (routed_floats + shared_floats) * 4;
    ++ctx->stats.command_calls;
    return 0;
}

int strata_moe_command_enqueue_rows_dsv4(strata_moe_ctx* ctx, const float* hidden, size_t hidden_floats,
                                         uint32_t hidden_rows, const strata_moe_row_group* groups, uint32_t n_groups,
                                         const strata_moe_expert_ref* shared, const uint32_t* shared_rows,
                                         uint32_t n_shared_rows, float swiglu_limit) {
    if (!ctx) return STRATA_MOE_E_INVALID;
    if (ctx->cmd_kind != 0) return fail(ctx, STRATA_MOE_E_BUSY, "MoE workspace already has an in-flight command");
    if (hidden_rows == 0 || (n_groups == 0 && !shared) || (n_groups && !groups))
        return fail(ctx, STRATA_MOE_E_INVALID, "DeepSeek MoE command has no rows or no experts");
    if (!(swiglu_limit > 0.0f && swiglu_limit < 3.0e38f))
        return fail(ctx, STRATA_MOE_E_INVALID, "SwiGLU limit must be finite and positive");
    const strata_moe_weight* first = n_groups ? groups[0].w1 : shared->gate;
    if (!same_device(ctx, first)) return fail(ctx, STRATA_MOE_E_INVALID, "DeepSeek MoE command has no valid leading expert");
    const uint32_t H = first->cols, I = first->rows;
    uint64_t pairs64 = 0;
    for (uint32_t g = 0; g < n_groups; ++g) {
        const strata_moe_row_group& gr = groups[g];
        const strata_moe_weight* ws[3] = {gr.w1, gr.w3, gr.w2};
        for (const strata_moe_weight* w : ws)
            if (!same_device(ctx, w) || w->fmt != STRATA_MOE_FMT_MXFP4)
                return fail(ctx, STRATA_MOE_E_INVALID, "DeepSeek routed experts need FP4 E2M1 group-32 weights");
        if (gr.w1->rows != I || gr.w1->cols != H || gr.w3->rows != I || gr.w3->cols != H || gr.w2->rows != H ||
            gr.w2->cols != I)
            return fail(ctx, STRATA_MOE_E_INVALID, "DeepSeek expert shapes are incompatible");
        if (gr.n_rows == 0 || !gr.rows || !gr.coefficients)
            return fail(ctx, STRATA_MOE_E_INVALID, "a row group is empty");
        for (uint32_t i = 0; i < gr.n_rows; ++i) {
            if (gr.rows[i] >= hidden_rows) return fail(ctx, STRATA_MOE_E_INVALID, "a row group names a row outside the page");
            if (!(fabsf(gr.coefficients[i]) <= 3.0e38f)) return fail(ctx, STRATA_MOE_E_INVALID, "a coefficient is not finite");
        }
        pairs64 += gr.n_rows;
    }
    if (pairs64 > 0x3FFFFFFFull) return fail(ctx, STRATA_MOE_E_INVALID, "too many rows");
    const uint32_t pairs = (uint32_t)pairs64;
    if (shared) {
        const strata_moe_weight* ws[3] = {shared->gate, shared->up, shared->down};
        for (const strata_moe_weight* w : ws)
            if (!same_device(ctx, w) || w->fmt != STRATA_MOE_FMT_FP8B128)
                return fail(ctx, STRATA_MOE_E_INVALID, "the DeepSeek shared expert needs FP8 E4M3 block-128 weights");
        if (shared->gate->rows != I || shared->gate->cols != H || shared->up->rows != I || shared->up->cols != H ||
            shared->down->rows != H || shared->down->cols != I)
            return fail(ctx, STRATA_MOE_E_INVALID, "DeepSeek shared expert shapes are incompatible");
        if (n_shared_rows == 0 || !shared_rows) return fail(ctx, STRATA_MOE_E_INVALID, "the shared expert has no rows");
        for (uint32_t i = 0; i < n_shared_rows; ++i)
            if (shared_rows[i] >= hidden_rows) return fail(ctx, STRATA_MOE_E_INVALID, "a shared row lies outside the page");
    } else {
        n_shared_rows = 0;
    }
    if (!hidden || hidden_floats != (size_t)hidden_rows * H) return fail(ctx, STRATA_MOE_E_INVALID, "DeepSeek hidden rows are incompatible");
    for (size_t i = 0; i < hidden_floats; ++i)
        if (!(fabsf(hidden[i]) <= 3.0e38f)) return fail(ctx, STRATA_MOE_E_INVALID, "DeepSeek hidden rows are incompatible");
    CK(cudaSetDevice(ctx->device));
    const uint32_t slots = n_groups ? n_groups : 1u;
    int rc = ensure_cmd_layer(ctx, STRATA_MOE_FMT_MXFP4, H, I, slots, hidden_rows > n_shared_rows ? hidden_rows : n_shared_rows,
                              pairs > n_shared_rows ? pairs : n_shared_rows);
    if (rc) return rc;
    strata_moe_layer* L = ctx->cmd_layer;
    cudaStream_t s = ctx->stream;
    const uint32_t n_slots = L->d.expert_count;
    // host staging of the row lists, coefficients and the group table
    std::vector<uint32_t> h_rows(pairs + n_shared_rows), h_off(n_slots + 1 + 2);
    std::vector<float> h_coef(pairs ? pairs : 1);
    uint32_t at = 0;
    for (uint32_t g = 0; g < n_slots; ++g) {
        h_off[g] = at;
        if (g < n_groups) {
            const strata_moe_row_group& gr = groups[g];
            const strata_moe_weight* ws[3] = {gr.w1, gr.w3, gr.w2};
            for (int r = 0; r < 3; ++r) {
                L->tab[r].packed[g] = ws[r]->packed;
                L->tab[r].scales[g] = ws[r]->scales;
                L->tab[r].global[g] = 1.0f;
            }
            for (uint32_t i = 0; i < gr.n_rows; ++i) {
                h_rows[at + i] = gr.rows[i];
                h_coef[at + i] = gr.coefficients[i];
            }
            at += gr.n_rows;
        } else if (n_groups) {
            for (int r = 0; r < 3; ++r) {   // unused slots: any valid pointers, zero rows
                L->tab[r].packed[g] = L->tab[r].packed[0];
                L->tab[r].scales[g] = L->tab[r].scales[0];
                L->tab[r].global[g] = 1.0f;
            }
        }
    }
    h_off[n_slots] = at;
    h_off[n_slots + 1] = 0;                 // the shared expert's one-group table {0, n_shared_rows}
    h_off[n_slots + 2] = n_shared_rows;
    for (uint32_t i = 0; i < n_shared_rows; ++i) h_rows[pairs + i] = shared_rows[i];
    L->tables_dirty = true;
    cmd_release_scratch(ctx);
    float *d_hidden = nullptr, *d_coef = nullptr, *d_y = nullptr, *d_sx = nullptr, *d_sact = nullptr, *d_sy = nullptr;
    uint32_t *d_rows = nullptr, *d_off = nullptr;
    const uint8_t** d_sp = nullptr;
    cudaError_t e = cmd_alloc(ctx, &d_hidden, hidden_floats);
    if (e == cudaSuccess) e = cmd_alloc(ctx, &d_coef, h_coef.size());
    if (e == cudaSuccess) e = cmd_alloc(ctx, &d_rows, h_rows.size());
    if (e == cudaSuccess) e = cmd_alloc(ctx, &d_off, h_off.size());
    if (e == cudaSuccess) e = cmd_alloc(ctx, &d_y, (size_t)(pairs + n_shared_rows) * H);
    if (e == cudaSuccess && shared) e = cmd_alloc(ctx, &d_sx, (size_t)n_shared_rows * H);
    if (e == cudaSuccess && shared) e = cmd_alloc(ctx, &d_sact, (size_t)n_shared_rows * I);
    if (e == cudaSuccess && shared) e = cmd_alloc(ctx, &d_sp, 6);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_hidden, hidden, hidden_floats * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_coef, h_coef.data(), h_coef.size() * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess && !h_rows.empty())
        e = cudaMemcpyAsync(d_rows, h_rows.data(), h_rows.size() * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_off, h_off.data(), h_off.size() * 4, cudaMemcpyHostToDevice, s);
    const uint8_t* sp[6] = {};
    if (e == cudaSuccess && shared) {
        sp[0] = shared->gate->packed; sp[1] = shared->gate->scales;
        sp[2] = shared->up->packed;   sp[3] = shared->up->scales;
        sp[4] = shared->down->packed; sp[5] = shared->down->scales;
        e = cudaMemcpyAsync(d_sp, sp, sizeof(sp), cudaMemcpyHostToDevice, s);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);   // the host vectors above go out of scope
    if (e != cudaSuccess) {
        cmd_release_scratch(ctx);
        return fail(ctx, STRATA_MOE_E_CUDA, std::string("DeepSeek MoE command set-up: ") + cudaGetErrorString(e));
    }
    ctx->stats.h2d_bytes += hidden_floats * 4;
    if (pairs) {
        rc = dsv4_grouped_core(L, d_hidden, d_rows, pairs, d_off, d_coef, swiglu_limit, d_y);
        if (rc) { cmd_release_scratch(ctx); return rc; }
    }
    if (shared) {
        d_sy = d_y + (size_t)pairs * H;
        const uint32_t* off2 = d_off + n_slots + 1;
        WeightTable g{d_sp + 0, d_sp + 1, nullptr, nullptr, nullptr}, u{d_sp + 2, d_sp + 3, nullptr, nullptr, nullptr},
            dn{d_sp + 4, d_sp + 5, nullptr, nullptr, nullptr};
        launch_dsv4_quantize(d_hidden, d_rows + pairs, 1, n_shared_rows, H, d_sx, s);
        launch_dsv4_gate_up(1, off2, H, I, g, u, d_sx, nullptr, swiglu_limit, d_sact, ctx->d_status, s, true);
        launch_dsv4_quantize(d_sact, nullptr, 1, n_shared_rows, I, d_sact, s);
        launch_dsv4_down(1, off2, H, I, dn, d_sact, d_sy, ctx->d_status, s, true);
        CK(cudaGetLastError());
    }
    ctx->cmd_kind = 2;
    ctx->cmd_pairs = pairs;
    ctx->cmd_shared_rows = n_shared_rows;
    ctx->cmd_rows = hidden_rows;
    ctx->cmd_shared = shared != nullptr;
    return 0;
}

int strata_moe_command_collect_rows_dsv4(strata_moe_ctx* ctx, float* routed_out, size_t routed_floats, float* shared_out,
                                         size_t shared_floats) {
    if (!ctx) return STRATA_MOE_E_INVALID;
    if (ctx->cmd_kind != 2) return fail(ctx, STRATA_MOE_E_INVALID, "no DeepSeek MoE row command is in flight");
    strata_moe_layer* L = ctx->cmd_layer;
    CK(cudaSetDevice(ctx->device));
    const int rc = strata_moe_synchronize(ctx);
    ctx->cmd_kind = 0;
    const size_t H = L->d.hidden;
    const float* d_y = ctx->cmd_scratch.size() > 4 ? static_cast<const float*>(ctx->cmd_scratch[4]) : nullptr;
    int out_rc = rc;
    if (rc == 0) {
        if (routed_floats != (size_t)ctx->cmd_pairs * H || (ctx->cmd_pairs && !routed_out))
            out_rc = fail(ctx, STRATA_MOE_E_INVALID, "routed output span does not match the command");
        else if (shared_floats != (size_t)ctx->cmd_shared_rows * H || (ctx->cmd_shared_rows && !shared_out))
            out_rc = fail(ctx, STRATA_MOE_E_INVALID, "shared output span does not match the command");
    }
    if (out_rc == 0 && d_y) {
        cudaError_t e = cudaSuccess;
        if (ctx->cmd_pairs) e = cudaMemcpyAsync(routed_out, d_y, routed_floats * 4, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess && ctx->cmd_shared_rows)
            e = cudaMemcpyAsync(shared_out, d_y + (size_t)ctx->cmd_pairs * H, shared_floats * 4, cudaMemcpyDeviceToHost,
                                ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) out_rc = fail(ctx, STRATA_MOE_E_CUDA, cudaGetErrorString(e));
        else {
            ctx->stats.d2h_bytes += (routed_floats + shared_floats) * 4;
            ++ctx->stats.command_calls;
        }
    }
    cmd_release_scratch(ctx);
    return out_rc;
}

// ------------------------------------------------------------------------- expert parallelism
struct strata_moe_ep {
    strata_moe_layer* L = nullptr;
    EpWindows w{};
    EpPlan pl{};                    // device tables of the step (layer scratch)
    const __nv_bfloat16* x = nullptr;   // inputs of the step in progress
    uint32_t T = 0;
    int stage = 0;                  // 0 idle, 1 counts published, 2 rows sent, 3 experts done
    bool forked = false;
};

size_t strata_moe_ep_window_bytes(const strata_moe_layer_desc* desc, uint32_t world, uint32_t row_capacity) {
    if (!desc || world == 0 || world > kEpMaxWorld || row_capacity == 0) return 0;
    if (desc->top_k == 0 || desc->top_k > 32u) return 0;
    return ep_window_bytes(world, desc->experts, desc->hidden, row_capacity, desc->top_k);
}

int strata_moe_ep_window_alloc(strata_moe_ctx* ctx, size_t bytes, void** window, void* handle64) {
    if (!ctx || !window || bytes == 0) return STRATA_MOE_E_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    CK(cudaSetDevice(ctx->device));
    void* p = nullptr;
    CK(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess && handle64) {
        cudaIpcMemHandle_t h;
        e = cudaIpcGetMemHandle(&h, p);
        if (e == cudaSuccess) memcpy(handle64, &h, sizeof(h));
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(ctx, STRATA_MOE_E_CUDA, std::string("window allocation: ") + cudaGetErrorString(e));
    }
    *window = p;
    return 0;
}

int strata_moe_ep_window_open(strata_moe_ctx* ctx, const void* handle64, void** window) {
    if (!ctx || !handle64 || !window) return STRATA_MOE_E_INVALID;
    CK(cudaSetDevice(ctx->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    CK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *window = p;
    return 0;
}

int strata_moe_ep_window_close(strata_moe_ctx* ctx, void* window) {
    if (!ctx || !window) return STRATA_MOE_E_INVALID;
    CK(cudaSetDevice(ctx->device));
    CK(cudaIpcCloseMemHandle(window));
    return 0;
}

int strata_moe_ep_window_free(strata_moe_ctx* ctx, void* window) {
    if (!ctx || !window) return STRATA_MOE_E_INVALID;
    CK(cudaSetDevice(ctx->device));
    CK(cudaDeviceSynchronize());
    CK(cudaFree(window));
    return 0;
}

int strata_moe_ep_create(strata_moe_layer* L, uint32_t rank, uint32_t world, uint32_t row_capacity,
                         void* const* windows, uint32_t wait_ms, strata_moe_ep** out) {
    if (!L || !out) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = L->ctx;
    *out = nullptr;
    const strata_moe_layer_desc& d = L->d;
    if (!windows) return fail(ctx, STRATA_MOE_E_INVALID, "null window table");
    if (world == 0 || world > kEpMaxWorld || rank >= world)
        return fail(ctx, STRATA_MOE_E_INVALID, "world must be 1..16 and rank below it");
    if (d.experts % world) return fail(ctx, STRATA_MOE_E_INVALID, "experts must divide evenly over the ranks");
    if (d.experts > 1024u) return fail(ctx, STRATA_MOE_E_INVALID, "expert parallelism supports at most 1024 experts");
    if (d.top_k > 32u) return fail(ctx, STRATA_MOE_E_INVALID, "expert parallelism supports top_k up to 32");
    const uint32_t B = d.experts / world;
    if (d.expert_count != B || d.expert_begin != rank * B)
        return fail(ctx, STRATA_MOE_E_INVALID, "layer must hold exactly this rank's block of experts");
    if (row_capacity == 0 || row_capacity > L->max_pairs)
        return fail(ctx, STRATA_MOE_E_INVALID, "row capacity must be in 1..max_pairs of the layer");
    if ((uint64_t)d.max_tokens * d.top_k > L->max_pairs)
        return fail(ctx, STRATA_MOE_E_INVALID, "max_pairs must cover max_tokens * top_k");
    for (uint32_t r = 0; r < world; ++r)
        if (!windows[r] || ((uintptr_t)windows[r] & 255u))
            return fail(ctx, STRATA_MOE_E_INVALID, "windows must be non-null and 256-byte aligned");
    CK(cudaSetDevice(ctx->device));
    strata_moe_ep* ep = new (std::nothrow) strata_moe_ep();
    if (!ep) return fail(ctx, STRATA_MOE_E_INVALID, "out of host memory");
    ep->L = L;
    for (uint32_t r = 0; r < world; ++r) ep->w.win[r] = static_cast<uint8_t*>(windows[r]);
    ep->w.world = world;
    ep->w.rank = rank;
    ep->w.E = d.experts;
    ep->w.H = d.hidden;
    ep->w.cap = row_capacity;
    ep->w.step = 0;
    ep->w.k = d.top_k;
    ep->w.wait_ns = (unsigned long long)(wait_ms ? wait_ms : 10000u) * 1000000ull;
    EpPlan& pl = ep->pl;
    pl.stride = d.max_tokens;
    cudaError_t e = dalloc(L, &pl.dst_row, (size_t)d.experts);
    if (e == cudaSuccess) e = dalloc(L, &pl.loffsets, (size_t)B + 1);
    if (e == cudaSuccess) e = dalloc(L, &pl.vis_idx, (size_t)world * d.max_tokens);
    if (e == cudaSuccess) e = dalloc(L, &pl.nvis, (size_t)kEpMaxWorld);
    if (e == cudaSuccess) e = dalloc(L, &pl.tok_base, (size_t)kEpMaxWorld);
    if (e == cudaSuccess) e = dalloc(L, &pl.vis_total, 1);
    if (e == cudaSuccess) e = dalloc(L, &pl.abort_word, 1);
    if (e == cudaSuccess) e = dalloc(L, &pl.done, 1);
    if (e == cudaSuccess) e = cudaMemset(pl.done, 0, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(pl.abort_word, 0, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(pl.nvis, 0, kEpMaxWorld * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(pl.vis_total, 0, sizeof(uint32_t));
    if (e != cudaSuccess) {
        delete ep;
        return fail(ctx, STRATA_MOE_E_CUDA, std::string("ep allocation: ") + cudaGetErrorString(e));
    }
    *out = ep;
    return 0;
}

void strata_moe_ep_destroy(strata_moe_ep* ep) {
    if (!ep) return;
    cudaSetDevice(ep->L->ctx->device);
    cudaStreamSynchronize(ep->L->ctx->stream);
    delete ep;   // device scratch belongs to the layer
}

// Stage 1: route this rank's tokens, group the pairs by global expert, publish the counts.
int strata_moe_ep_begin(strata_moe_ep* ep, const void* x, uint32_t T) {
    if (!ep) return STRATA_MOE_E_INVALID;
    strata_moe_layer* L = ep->L;
    strata_moe_ctx* ctx = L->ctx;
    const strata_moe_layer_desc& d = L->d;
    if (ep->stage != 0) return fail(ctx, STRATA_MOE_E_BUSY, "an expert-parallel step is in progress");
    if (!x && T) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    if (T > d.max_tokens) return fail(ctx, STRATA_MOE_E_INVALID, "tokens exceed max_tokens");
    std::string why;
    if (!all_registered(L, &why)) return fail(ctx, STRATA_MOE_E_INVALID, why);
    CK(cudaSetDevice(ctx->device));
    int rc = sync_tables(L);
    if (rc) return rc;
    cudaStream_t s = ctx->stream;
    ep->x = static_cast<const __nv_bfloat16*>(x);
    ep->T = T;
    ep->forked = false;
    if (d.shared_intermediate && T) {
        uint32_t* off2 = L->offsets + d.experts + 1 + 2;
        set_pair_kernel<<<1, 1, 0, s>>>(off2, 0u, T);
        ++g_kernel_launches;
        CK(cudaEventRecord(ctx->ev_fork, s));
        CK(cudaStreamWaitEvent(ctx->side, ctx->ev_fork, 0));
        rc = run_shared(L, ep->x, nullptr, T, off2, ctx->side);
        if (rc) return rc;
        CK(cudaEventRecord(ctx->ev_join, ctx->side));
        ep->forked = true;
    }
    if (T) {
        rc = run_router(L, ep->x, T, nullptr, L->ids, L->weights);
        if (rc) return rc;
        launch_group(L->ids, T * d.top_k, 0, d.experts, L->counts, L->offsets, L->perm, L->inv, nullptr, nullptr,
                     L->group_scratch, s);
    } else {
        CK(cudaMemsetAsync(L->counts, 0, (size_t)d.experts * sizeof(uint32_t), s));
        CK(cudaMemsetAsync(L->offsets, 0, ((size_t)d.experts + 1) * sizeof(uint32_t), s));
    }
    // The step number advances only once nothing on the host can fail any more: a begin that
    // returned an error must leave this rank in step with its peers.
    launch_ep_visits(ep->w, ep->pl, L->ids, T, s);
    ep->w.step += 1;
    launch_ep_publish(ep->w, ep->pl, L->counts, s);
    if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) {
        ep->w.step -= 1;
        return fail(ctx, STRATA_MOE_E_CUDA, std::string("ep publish launch: ") + cudaGetErrorString(e));
    }
    ep->stage = 1;
    return 0;
}

// Stage 2: wait for every rank's counts, lay out the owners' buffers, store the rows there.
int strata_moe_ep_dispatch(strata_moe_ep* ep) {
    if (!ep) return STRATA_MOE_E_INVALID;
    Range range("strata_moe.ep.dispatch");
    strata_moe_layer* L = ep->L;
    strata_moe_ctx* ctx = L->ctx;
    if (ep->stage != 1) return fail(ctx, STRATA_MOE_E_INVALID, "ep_dispatch must follow ep_begin");
    CK(cudaSetDevice(ctx->device));
    bind_ws(L);
    cudaStream_t s = ctx->stream;
    launch_ep_plan(ep->w, ep->pl, ctx->d_status, s);
    launch_ep_dispatch(ep->w, ep->pl, ep->x, L->ids, L->inv, L->offsets, L->weights, ep->T, s);
    CK(cudaGetLastError());
    ep->stage = 2;
    return 0;
}

// Stage 3: wait for every rank's rows, run this rank's experts over them, announce the outputs.
int strata_moe_ep_experts(strata_moe_ep* ep, uint32_t expected_rows) {
    if (!ep) return STRATA_MOE_E_INVALID;
    strata_moe_layer* L = ep->L;
    strata_moe_ctx* ctx = L->ctx;
    if (ep->stage != 2) return fail(ctx, STRATA_MOE_E_INVALID, "ep_experts must follow ep_dispatch");
    CK(cudaSetDevice(ctx->device));
    bind_ws(L);
    cudaStream_t s = ctx->stream;
    const uint32_t par = ep->w.step & 1u, B = L->d.expert_count;
    launch_ep_wait(ep->w, 1, ep->pl.abort_word, ctx->d_status, s);
    if (expected_rows == 0) expected_rows = ep->T != 0u ? ep->T * L->d.top_k : 1u;
    // The experts read their grouped rows out of the received token rows through the slot table the
    // sources filled (one token row serves all of the token's experts here); the tensor-core path
    // leaves its outputs as f16 rows, the others as fp32, and the partial-sum pass takes either.
    const uint32_t* total = ep->pl.loffsets + B;
    const SpreadRows spread{ep->w.vis_pos(ep->w.rank, par), ep->w.cap, L->d.top_k, ep->pl.vis_total};
    bool half = true;
    int rc = run_experts(L, ep->w.rows(ep->w.rank, par), ep->w.src_of(ep->w.rank, par), 1, ep->w.cap, B,
                         ep->pl.loffsets, nullptr, nullptr, ep->w.cap, L->y, expected_rows, total, false, &half,
                         nullptr, &spread);
    if (rc) return rc;
    launch_ep_partial(ep->w, ep->pl, L->y, half, ctx->d_status, s);
    launch_ep_signal(ep->w, 2, s);
    CK(cudaGetLastError());
    ep->stage = 3;
    return 0;
}

// Stage 4: wait for every owner's outputs and form this rank's tokens from them.
int strata_moe_ep_finish(strata_moe_ep* ep, float* out) {
    if (!ep) return STRATA_MOE_E_INVALID;
    Range range("strata_moe.ep.combine");
    strata_moe_layer* L = ep->L;
    strata_moe_ctx* ctx = L->ctx;
    if (ep->stage != 3) return fail(ctx, STRATA_MOE_E_INVALID, "ep_finish must follow ep_experts");
    if (!out && ep->T) return fail(ctx, STRATA_MOE_E_INVALID, "null pointer");
    CK(cudaSetDevice(ctx->device));
    bind_ws(L);
    cudaStream_t s = ctx->stream;
    const float* shared = nullptr;
    if (ep->forked) {
        CK(cudaStreamWaitEvent(s, ctx->ev_join, 0));
        shared = L->sh_y;
    }
    // one CTA waits for the peers' results; the combine kernel's own check then passes at once, so its CTAs never sit
    // on SMs spinning (a second step in flight on another stream may need them for its GEMMs)
    launch_ep_wait(ep->w, 2, ep->pl.abort_word, ctx->d_status, s);
    launch_ep_combine(ep->w, ep->pl, shared, ep->T, L->d.output_scale, out, ctx->d_status, s);
    CK(cudaGetLastError());
    ep->stage = 0;
    ctx->stats.forward_calls++;
    return 0;
}

int strata_moe_ep_abandon(strata_moe_ep* ep) {
    if (!ep) return STRATA_MOE_E_INVALID;
    strata_moe_ctx* ctx = ep->L->ctx;
    if (ep->forked) {
        CK(cudaStreamWaitEvent(ctx->stream, ctx->ev_join, 0));
        ep->forked = false;
    }
    ep->stage = 0;
    return 0;
}

int strata_moe_ep_last_counts(strata_moe_ep* ep, uint32_t* sent_rows, uint32_t* received_rows,
                              uint32_t* received_pairs) {
    if (!ep) return STRATA_MOE_E_INVALID;
    strata_moe_layer* L = ep->L;
    strata_moe_ctx* ctx = L->ctx;
    if (ep->stage != 0) return fail(ctx, STRATA_MOE_E_BUSY, "an expert-parallel step is in progress");
    CK(cudaSetDevice(ctx->device));
    CK(cudaStreamSynchronize(ctx->stream));
    if (sent_rows)
        CK(cudaMemcpy(sent_rows, ep->pl.nvis, ep->w.world * sizeof(uint32_t), cudaMemcpyDeviceToHost));
    if (received_rows) CK(cudaMemcpy(received_rows, ep->pl.vis_total, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    if (received_pairs)
        CK(cudaMemcpy(received_pairs, ep->pl.loffsets + L->d.expert_count, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    return 0;
}

int strata_moe_ep_forward(strata_moe_ep* ep, const void* x, uint32_t T, float* out, uint32_t expected_rows) {
    int rc = strata_moe_ep_begin(ep, x, T);
    if (rc == 0) rc = strata_moe_ep_dispatch(ep);
    if (rc == 0) rc = strata_moe_ep_experts(ep, expected_rows);
    if (rc == 0) rc = strata_moe_ep_finish(ep, out);
    return rc;
}

}  // extern "C"
