// Shared declarations of the MoE expert-block kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/strata_moe.h"

namespace smoe {

constexpr int kNumSMs = 148;

// Device status word bits (never a trap: kernels record and carry on).
enum : uint32_t {
    kStatusNonFiniteLogit = 1u,   // router saw a non-finite logit or bias
    kStatusBadNormaliser = 2u,    // selected scores do not sum to a positive finite value
    kStatusNonFiniteOutput = 4u,  // an expert produced a non-finite value
    kStatusWaitTimeout = 8u,      // a bounded mbarrier wait gave up
    kStatusBadGroup = 16u         // group table inconsistent with the pair count
};

struct RouterParams {
    uint32_t experts, top_k;
    int32_t score_kind, normalize;
    float norm_init, weight_scale, softcap;
};

// Gated activation of the expert FFN (STRATA_MOE_ACT_*); SwiGLU is evaluated by each kernel's own
// fast path, the other kinds through glu_other().
struct GluParams {
    int32_t kind;
    float gate_beta, linear_beta;
};
__device__ __forceinline__ float glu_other(float g, float u, const GluParams& p) {
    // SiTU-GLU: the tanh bounds the gate, the plain sigmoid gates it, the up projection is bounded too
    const float sig = __fdividef(1.0f, 1.0f + __expf(-g));
    return p.gate_beta * tanhf(g / p.gate_beta) * sig * (p.linear_beta * tanhf(u / p.linear_beta));
}

// One projection of every local expert: base pointers per expert.
struct WeightTable {
    const uint8_t* const* packed;  // [n_local] device array of device pointers
    const uint8_t* const* scales;  // [n_local]
    const float* global_scale;     // [n_local] NVFP4 divisor (1 otherwise)
    const uint32_t* emin;          // [n_local] MXFP4 f16 path: smallest E8M0 byte of the projection
    const float* post_scale;       // [n_local] f16 path: factor applied to the fp32 accumulator
};

// ---- launch wrappers (definitions in the .cu files) ---------------------------------
// router.cu
void launch_router_logits(const __nv_bfloat16* x, const __nv_bfloat16* wg, uint32_t T, uint32_t H,
                          uint32_t E, float* logits, cudaStream_t s, uint32_t* status = nullptr);
void launch_route(const RouterParams& p, const float* logits, const float* bias, uint32_t T,
                  uint32_t* ids, float* weights, uint32_t* status, cudaStream_t s,
                  const uint32_t* forced_ids = nullptr);
// Fast router (tensor-core projection + exact recheck), see router.cu.
bool launch_front_small(const RouterParams& p, const float* logits, const float* bias, uint32_t T, uint32_t* ids,
                        float* weights, uint32_t* counts, uint32_t* offsets, uint32_t* perm, uint32_t* inv,
                        uint32_t* active_list, uint32_t* n_active, const __nv_bfloat16* x, uint32_t H, void* xg,
                        float* x_rowscale, uint32_t* status, cudaStream_t s);
void launch_route_sink(const float* logits, const float* bias, uint32_t T, uint32_t E, uint32_t S, uint32_t k, float scale,
                       uint32_t* ids, float* w_routed, float* w_sinks, uint32_t* status, cudaStream_t s);
bool route_fast_supported(const RouterParams& p, uint32_t H);
void launch_route_fast(const RouterParams& p, float* logits, const float* bias, const __nv_bfloat16* x,
                       const __nv_bfloat16* wg, uint32_t T, uint32_t H, uint32_t* ids, float* weights,
                       uint32_t* list, uint32_t* count, unsigned long long* recheck_total, uint32_t* status,
                       cudaStream_t s);
// group.cu
size_t group_scratch_bytes(uint32_t pairs, uint32_t n_experts);
void launch_group(const uint32_t* ids, uint32_t pairs, uint32_t expert_begin, uint32_t n_experts,
                  uint32_t* counts, uint32_t* offsets, uint32_t* perm, uint32_t* inv,
                  uint32_t* active_list, uint32_t* n_active, void* scratch, cudaStream_t s);
// K-permuted copy of activation rows (layout the decode kernel's B operand reads).
// src_row[pos] = perm[pos] / k_div when perm != nullptr, else pos.
void launch_gather_rows_kperm(const __nv_bfloat16* x, const uint32_t* perm, uint32_t k_div,
                              uint32_t pairs, uint32_t H, __nv_bfloat16* dst, cudaStream_t s,
                              const uint32_t* pairs_dev = nullptr);
void launch_gather_rows_kperm_f32(const float* x, uint32_t rows, uint32_t reps, uint32_t H,
                                  __nv_bfloat16* hi, __nv_bfloat16* lo, cudaStream_t s, bool natural = false);
void launch_gather_rows_plain(const __nv_bfloat16* x, const uint32_t* perm, uint32_t k_div,
                              uint32_t pairs, uint32_t H, __nv_bfloat16* dst, cudaStream_t s);
// decode.cu : small-batch expert FFN (warp-level MMA GEMV path)
struct DecodeArgs {
    int fmt;                       // STRATA_MOE_FMT_* or 3 = BF16 (shared expert)
    uint32_t H, I;
    uint32_t n_groups;             // size of the offsets table - 1
    const uint32_t* offsets;       // [n_groups + 1] rows of group g = [offsets[g], offsets[g+1])
    const uint32_t* active_list;   // [n_active] groups with rows, or nullptr = all groups
    const uint32_t* n_active;      // device scalar (nullptr when active_list is nullptr)
    uint32_t max_rows_per_group;   // upper bound used to pick the token tile
    uint32_t ksplit;               // decode.cu: 1 = the four warps of a CTA split K of one tile (few tiles)
    GluParams glu;                 // activation between gate/up and down
    uint32_t skip_from;            // groups with at least this many rows are left to another kernel (0 = none)
    WeightTable gate, up, down;
    const __nv_bfloat16* x_hi;     // [pairs, H] K-permuted (or natural for BF16 weights)
    const __nv_bfloat16* x_lo;     // optional low part (fp32 inputs), nullptr otherwise
    const float* coef;             // optional [pairs] multiplied into the activation, or nullptr
    __nv_bfloat16* act_hi;         // [pairs, I] scratch, K-permuted
    __nv_bfloat16* act_lo;
    float* y;                      // [pairs, H]
    uint32_t* status;
    // f16 path (decode_fp4.cu): activations as f16 with a per-row power-of-two pre-scale
    const float* x_rowscale;       // [pairs] factor that undoes the pre-scale of x
    float* act_f32;                // [pairs, I] SwiGLU output before its f16 split
    const float* act_rowscale;     // [pairs]
    uint32_t x_rows;               // decode_stream.cu: rows allocated in x_hi / act_hi / act_lo (bounds of the row boxes)
    uint32_t act_direct;           // decode_stream.cu gate/up: write act_hi / act_lo (f16 hi + lo) and unit row factors, not act_f32
    float* act_rowscale_out;       // [pairs], written when act_direct
};
void launch_decode_fp4_gate_up(const DecodeArgs& a, cudaStream_t s);
void launch_decode_fp4_down(const DecodeArgs& a, cudaStream_t s);
void launch_rows_to_f16_bf16(const __nv_bfloat16* x, const uint32_t* perm, uint32_t k_div, uint32_t rows,
                             uint32_t C, void* hi, float* rowscale, cudaStream_t s,
                             const uint32_t* rows_dev = nullptr);
void launch_rows_to_f16_spread(const __nv_bfloat16* x, const uint32_t* dest, uint32_t k, uint32_t rows,
                               const uint32_t* rows_dev, uint32_t dst_bound, uint32_t C, void* hi, float* rowscale,
                               cudaStream_t s);
void launch_rows_to_f16_f32(const float* x, uint32_t src_rows, uint32_t rows, uint32_t C, void* hi, void* lo,
                            float* rowscale, cudaStream_t s, const uint32_t* rows_dev = nullptr);
void launch_mx_scale_range(const uint8_t* const* scales, uint32_t n, size_t bytes, uint32_t* emin,
                           float* post_scale, uint32_t* not_ok, cudaStream_t s);
void launch_dequant_export_f16(int fmt, const uint8_t* packed, const uint8_t* scales, uint32_t emin,
                               float post_scale, uint32_t rows, uint32_t cols, float* out, cudaStream_t s);
// decode_stream.cu : the same two GEMMs with the weights streamed through a shared-memory ring by bulk copies
bool decode_stream_supported(int fmt, uint32_t H, uint32_t I);
// maps: device array [3 roles][n_groups][3] of 128-byte tensor maps made by decode_stream_encode_maps
int decode_stream_encode_maps(void* out3x128, int fmt, const void* packed, const void* scales, uint32_t rows, uint32_t K);
int launch_decode_stream_gate_up(const DecodeArgs& a, const void* maps, cudaStream_t s);
int launch_decode_stream_down(const DecodeArgs& a, const void* maps, cudaStream_t s);
void launch_decode_gate_up(const DecodeArgs& a, cudaStream_t s);
void launch_decode_down(const DecodeArgs& a, cudaStream_t s);
// prefill.cu : large-batch expert FFN (tcgen05 grouped GEMM path)
struct PrefillArgs {
    int fmt;
    uint32_t H, I, n_groups, pairs;
    const uint32_t* offsets;       // [n_groups + 1]
    WeightTable gate, up, down;
    float* y;                      // [pairs, H] fp32
    uint32_t y_half;               // down: store y as f16 [pairs, H] into the same buffer (values beyond the f16 range are reported)
    float* y_rowscale_out;         // down with y_half: receives 1.0 for every row written (rows are not scaled), or nullptr
    uint32_t* tile_table;          // scratch of prefill_scratch_bytes()
    uint32_t* status;
    GluParams glu;                 // activation of the gate/up epilogue
    uint32_t ntile;                // tokens per tile: 128, or anything else for 192 (large groups)
    uint32_t min_rows;             // only groups with at least this many rows get tiles (0 = all)
    uint32_t reuse_tiles;          // down-only launch: the tile list of the preceding gate/up launch is still valid
    float* act_rowscale_out;       // gate/up: receives 1.0 for every row written (the activation is not pre-scaled), or nullptr
};
bool prefill_supported(int fmt, uint32_t H, uint32_t I);
size_t prefill_scratch_bytes(uint32_t n_groups, uint32_t pairs);
// x16: [pairs_cap, H] f16 rows (pre-scaled, group order), x_rowscale [pairs_cap], act16:
// [pairs_cap, I] f16 scratch.  mid, when non-null, is recorded between the two GEMMs.
// wmaps: device array [3][n_groups] of 128-byte tensor-map descriptors made by
// prefill_encode_weight_map (gate, up, down of every local expert).
int launch_prefill(const PrefillArgs& a, const void* x16, const float* x_rowscale, void* act16,
                   uint32_t pairs_cap, const void* wmaps, cudaStream_t s, cudaEvent_t mid);
// Down projection alone on the tensor-core path: act16 [pairs_cap, I] f16 rows pre-scaled per row,
// act_rowscale [pairs_cap] the factors that undo it.
// Gate/up + SwiGLU alone (tile list + one kernel): act16 rows of the listed groups are written.
int launch_prefill_gate_up(const PrefillArgs& a, const void* x16, const float* x_rowscale, void* act16,
                           uint32_t pairs_cap, const void* wmaps, cudaStream_t s);
int launch_prefill_down(const PrefillArgs& a, const void* act16, const float* act_rowscale, uint32_t pairs_cap,
                        const void* wmaps, cudaStream_t s);
int prefill_encode_weight_map(void* out128, const void* packed, uint32_t rows, uint32_t K);
int launch_prefill_bf16(const PrefillArgs& a, const void* x, uint32_t rows, const void* w_gate, const void* w_up,
                        const void* w_down, void* act, uint32_t rows_cap, cudaStream_t s);
// Router projection on the tensor cores (approximate summation order; see router.cu for its use).
// tile_table: scratch of prefill_scratch_bytes(1, T); offsets2: device {0, T}.
int launch_router_tc(const void* x_bf16, uint32_t T, const void* wg_bf16, uint32_t E, uint32_t H, float* logits,
                     uint32_t* tile_table, const uint32_t* offsets2, uint32_t* status, cudaStream_t s);
// latent.cu : row kernels of the LatentMoE wrapper
void launch_f32_to_bf16(const float* src, size_t n, __nv_bfloat16* dst, cudaStream_t s);
void launch_rmsnorm_bf16(const float* x, const float* weight, uint32_t rows, uint32_t cols, float eps,
                         __nv_bfloat16* y, uint32_t* status, cudaStream_t s);
void launch_add_rows(float* out, const float* a, size_t n, cudaStream_t s);
// combine.cu
void launch_combine(const void* y, const uint32_t* inv, const float* weights, const float* shared,
                    uint32_t T, uint32_t k, uint32_t H, float output_scale, float* out,
                    uint32_t* status, cudaStream_t s, bool y_half = false);
void launch_dequant_export(int fmt, const uint8_t* packed, const uint8_t* scales, float global_scale,
                           uint32_t rows, uint32_t cols, float* out, cudaStream_t s);

// ep.cu : expert-parallel exchange over peer memory
constexpr uint32_t kEpMaxWorld = 16;
// The windows of all ranks as mapped into this process, plus the step being executed.  Passed to
// the kernels by value.  Layout of one window (byte offsets, every region 256-byte aligned):
// flags | counts [2][world][E] u32 | rows [2][cap][H] bf16 | y [2][cap][H] f16 | yscale [2][cap] f32.
// Expert outputs cross NVLink as f16 rows with an exact power-of-two scale per row (11 significant
// bits, half the bytes of fp32); the home rank widens them back while it forms the weighted sum.
struct EpWindows {
    uint8_t* win[kEpMaxWorld];
    uint32_t world, rank, E, H, cap, step, k;
    unsigned long long wait_ns;
    __host__ __device__ static size_t up256(size_t v) { return (v + 255u) / 256u * 256u; }
    __host__ __device__ size_t flags_bytes() const { return up256((size_t)3 * kEpMaxWorld * 4u); }
    __host__ __device__ size_t counts_bytes() const { return up256((size_t)2 * world * E * 4u); }
    __host__ __device__ size_t visits_bytes() const { return up256((size_t)2 * kEpMaxWorld * kEpMaxWorld * 4u); }
    __host__ __device__ size_t rows_bytes() const { return up256((size_t)2 * cap * H * 2u); }
    __host__ __device__ size_t y_bytes() const { return up256((size_t)2 * cap * H * 2u); }
    __host__ __device__ size_t yscale_bytes() const { return up256((size_t)2 * cap * 4u); }
    __host__ __device__ size_t src_of_bytes() const { return up256((size_t)2 * cap * 4u); }
    __host__ __device__ size_t vis_bytes() const { return up256((size_t)2 * cap * k * 4u); }
    __host__ __device__ size_t total_bytes() const {
        return flags_bytes() + counts_bytes() + visits_bytes() + rows_bytes() + y_bytes() + yscale_bytes() +
               src_of_bytes() + 2u * vis_bytes();
    }
    __host__ __device__ uint32_t* flag(uint32_t r, uint32_t kind, uint32_t src) const {
        return reinterpret_cast<uint32_t*>(win[r]) + kind * kEpMaxWorld + src;
    }
    __host__ __device__ uint32_t* counts(uint32_t r, uint32_t parity, uint32_t src) const {
        return reinterpret_cast<uint32_t*>(win[r] + flags_bytes()) + ((size_t)parity * world + src) * E;
    }
    // visits(r, p, s)[o] = token rows rank s sends to owner o in a step of parity p (every rank holds the full matrix)
    __host__ __device__ uint32_t* visits(uint32_t r, uint32_t parity, uint32_t src) const {
        return reinterpret_cast<uint32_t*>(win[r] + flags_bytes() + counts_bytes()) +
               ((size_t)parity * kEpMaxWorld + src) * kEpMaxWorld;
    }
    __host__ __device__ size_t rows_at() const { return flags_bytes() + counts_bytes() + visits_bytes(); }
    __host__ __device__ __nv_bfloat16* rows(uint32_t r, uint32_t parity) const {
        return reinterpret_cast<__nv_bfloat16*>(win[r] + rows_at()) + (size_t)parity * cap * H;
    }
    __host__ __device__ unsigned short* y(uint32_t r, uint32_t parity) const {   // f16 bit patterns
        return reinterpret_cast<unsigned short*>(win[r] + rows_at() + rows_bytes()) + (size_t)parity * cap * H;
    }
    __host__ __device__ float* yscale(uint32_t r, uint32_t parity) const {
        return reinterpret_cast<float*>(win[r] + rows_at() + rows_bytes() + y_bytes()) + (size_t)parity * cap;
    }
    __host__ __device__ uint32_t* src_of(uint32_t r, uint32_t parity) const {
        return reinterpret_cast<uint32_t*>(win[r] + rows_at() + rows_bytes() + y_bytes() + yscale_bytes()) +
               (size_t)parity * cap;
    }
    __host__ __device__ uint32_t* vis_pos(uint32_t r, uint32_t parity) const {
        return reinterpret_cast<uint32_t*>(win[r] + rows_at() + rows_bytes() + y_bytes() + yscale_bytes() +
                                           src_of_bytes()) + (size_t)parity * cap * k;
    }
    __host__ __device__ float* vis_w(uint32_t r, uint32_t parity) const {
        return reinterpret_cast<float*>(win[r] + rows_at() + rows_bytes() + y_bytes() + yscale_bytes() +
                                        src_of_bytes() + vis_bytes()) + (size_t)parity * cap * k;
    }
};
// Device-side tables of one rank's step (all in the layer's scratch).
struct EpPlan {
    uint32_t* dst_row;     // [E]      first row, in the owner's grouped order, of this rank's pairs for expert e
    uint32_t* loffsets;    // [B + 1]  row ranges of this rank's local experts over all sources
    uint32_t* vis_idx;     // [world][stride]  index of token t among the rows this rank sends to owner o, or ~0
    uint32_t* nvis;        // [world]  rows this rank sends to owner o
    uint32_t* tok_base;    // [world]  first slot, in owner o's window, of this rank's token rows
    uint32_t* vis_total;   // [1]      token rows this rank received as an owner
    uint32_t* abort_word;
    uint32_t* done;
    uint32_t stride;       // tokens per row of vis_idx
};
size_t ep_window_bytes(uint32_t world, uint32_t E, uint32_t H, uint32_t cap, uint32_t k);
void launch_ep_visits(const EpWindows& w, const EpPlan& pl, const uint32_t* ids, uint32_t T, cudaStream_t s);
void launch_ep_publish(const EpWindows& w, const EpPlan& pl, const uint32_t* counts, cudaStream_t s);
void launch_ep_plan(const EpWindows& w, const EpPlan& pl, uint32_t* status, cudaStream_t s);
void launch_ep_dispatch(const EpWindows& w, const EpPlan& pl, const __nv_bfloat16* x, const uint32_t* ids,
                        const uint32_t* inv, const uint32_t* offsets, const float* weights, uint32_t T,
                        cudaStream_t s);
void launch_ep_wait(const EpWindows& w, uint32_t kind, uint32_t* abort_word, uint32_t* status, cudaStream_t s);
void launch_ep_signal(const EpWindows& w, uint32_t kind, cudaStream_t s);
void launch_ep_partial(const EpWindows& w, const EpPlan& pl, const void* y, bool y_half, uint32_t* status,
                       cudaStream_t s);
void launch_ep_combine(const EpWindows& w, const EpPlan& pl, const float* shared, uint32_t T, float output_scale,
                       float* out, uint32_t* status, cudaStream_t s);

// dsv4_exact.cu : bit-exact DeepSeek-V4 numerical mode (CUDA-core kernels, reference summation order)
void launch_dsv4_quantize(const float* src, const uint32_t* perm, uint32_t k_div, uint32_t rows, uint32_t cols,
                          float* dst, cudaStream_t s);
void launch_dsv4_gate_up(uint32_t n_groups, const uint32_t* offsets, uint32_t H, uint32_t I, const WeightTable& gate,
                         const WeightTable& up, const float* xq, const float* coef, float limit, float* act,
                         uint32_t* status, cudaStream_t s, bool fp8 = false);
void launch_dsv4_join(const float* y, const uint32_t* inv, const float* shared, uint32_t T, uint32_t k, uint32_t H,
                      float* out, uint32_t* status, cudaStream_t s);
void launch_dsv4_down(uint32_t n_groups, const uint32_t* offsets, uint32_t H, uint32_t I, const WeightTable& down,
                      const float* actq, float* y, uint32_t* status, cudaStream_t s, bool fp8 = false);

// Launch counter (every wrapper above bumps it once per kernel launch; host threads of several
// contexts share it).
extern std::atomic<unsigned long long> g_kernel_launches;

}  // namespace smoe
