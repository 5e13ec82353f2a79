/*
 * strata_moe.h -- C ABI of the B200-native MoE expert block.
 *
 * One hot path of ro99/strata behind plain-C entry points: router scoring with top-k,
 * token->expert permutation with per-expert offsets, grouped quantized expert GEMMs
 * (gate/up + SwiGLU, down) on MXFP4 / NVFP4 / INT4-g128 weights, and the top-k-weighted
 * combine plus shared expert.  All compute runs in hand-written sm_100a CUDA kernels;
 * there is no CPU fallback: every entry point fails with an error when no CUDA device
 * is usable.
 *
 * Citations "ref:" name the file:line of the reference interface an entry point
 * replaces (paths within the reference project).
 *
 * Conventions
 *   - every function returns 0 on success or a negative STRATA_MOE_E_* code; the text of
 *     the last failure is available from strata_moe_last_error() (the reference's
 *     ValidationResult, include/strata/result.hpp:8-20, flattened to code + message);
 *   - work is enqueued on the context's stream and is asynchronous unless stated;
 *   - device kernels never trap: data-dependent failures (non-finite logits or results)
 *     raise a status word that strata_moe_synchronize()/strata_moe_status() report, as the
 *     reference's moe_error flag does (ref: kernels/cuda/backend.cu:1922-1924);
 *   - pointers are plain device or host addresses as each parameter states.
 */
#ifndef STRATA_MOE_H
#define STRATA_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct strata_moe_ctx strata_moe_ctx;     /* one per process and device */
typedef struct strata_moe_layer strata_moe_layer; /* one MoE layer's resident weights + workspaces */

enum {
    STRATA_MOE_OK = 0,
    STRATA_MOE_E_INVALID = -1,  /* bad argument / shape / state */
    STRATA_MOE_E_CUDA = -2,     /* a CUDA call failed */
    STRATA_MOE_E_NUMERIC = -3,  /* device status word: non-finite value or bad route */
    STRATA_MOE_E_BUSY = -4,     /* a dense command is already in flight */
    STRATA_MOE_E_NO_DEVICE = -5
};

/* Weight encodings (ref: include/strata/cuda_backend.hpp:18-39 CudaWeightEncoding).
 *   MXFP4    u8 [rows, cols/2], low nibble = even column; E8M0 u8 [rows, cols/32]
 *   NVFP4    u8 [rows, cols/2]; E4M3 u8 [rows, cols/16]; fp32 global scale;
 *            w = e2m1 * (e4m3 / global)   (ref: include/strata/cuda_backend.hpp:24-29)
 *   INT4G128 little-endian u32 [rows, cols/8], nibble j = column 8w+j, value raw-8;
 *            BF16 scale [rows, cols/128]  (ref: kernels/cuda/backend.cu:1908-1916)
 *   BF16     plain BF16 [rows, cols] row-major, no scales (scales pointer ignored, may be NULL)
 *            (ref: the plain-BF16 expert layers, kernels/cuda/backend.cu:2075-2152) */
enum { STRATA_MOE_FMT_MXFP4 = 0, STRATA_MOE_FMT_NVFP4 = 1, STRATA_MOE_FMT_INT4G128 = 2, STRATA_MOE_FMT_BF16 = 3 };

/* Router score functions (ref: include/strata/model.hpp:43-48 RouterScoreKind). */
enum {
    STRATA_MOE_SCORE_SIGMOID = 0,       /* ref: src/platform/numerics.cpp:44-48 */
    STRATA_MOE_SCORE_SIGMOID_PLAIN = 1, /* ref: src/models/kimi_k3/kimi_k3_ops.cpp:12-14 */
    STRATA_MOE_SCORE_SOFTMAX = 2,       /* no reference implementation exists */
    STRATA_MOE_SCORE_SQRTSOFTPLUS = 3   /* ref: src/models/dsv4/deepseek_ops.cpp:82-133 */
};

enum { STRATA_MOE_ROLE_GATE = 0, STRATA_MOE_ROLE_UP = 1, STRATA_MOE_ROLE_DOWN = 2 };

/* Gated activations between the gate/up and the down projection.
 *   SWIGLU    silu(gate) * up                    (ref: kernels/cuda/backend.cu:2016-2032)
 *   SITU_GLU  gate_beta * tanh(gate / gate_beta) * sigmoid(gate) * linear_beta * tanh(up / linear_beta)
 *             (ref: kimi_situ_glu, src/models/kimi_k3/kimi_k3_ops.cpp:39-62) */
enum { STRATA_MOE_ACT_SWIGLU = 0, STRATA_MOE_ACT_SITU_GLU = 1 };

/* Where a source pointer lives and what registration does with it. */
enum {
    STRATA_MOE_SRC_HOST = 0,          /* host memory: copied to the device */
    STRATA_MOE_SRC_DEVICE_COPY = 1,   /* device memory: copied into layer-owned storage */
    STRATA_MOE_SRC_DEVICE_BORROW = 2  /* device memory: used in place, caller keeps it alive */
};

/* One MoE layer (ref: include/strata/model.hpp:50-60 RouterSpec plus the shape constants
 * each runtime hard-codes, e.g. src/models/glm52/glm_runtime.cpp kHidden/kExperts/kTopK). */
typedef struct strata_moe_layer_desc {
    uint32_t hidden;              /* H, multiple of 128 */
    uint32_t intermediate;        /* I, multiple of 128 */
    uint32_t experts;             /* E routed experts in the whole model layer (<= 1024) */
    uint32_t top_k;               /* k (<= 32) */
    int32_t format;               /* STRATA_MOE_FMT_* of the routed experts */
    int32_t score_kind;           /* STRATA_MOE_SCORE_* */
    int32_t normalize;            /* divide the selected scores by their sum */
    float norm_init;              /* start value of that sum (GLM: 1e-20, others 0) */
    float weight_scale;           /* multiplied into every routing weight (GLM 2.5, DSV4 1.5) */
    float output_scale;           /* multiplied into the summed routed output (Laguna 2.5) */
    float softcap;                /* Laguna tanh logit soft-cap, 0 = off */
    uint32_t shared_intermediate; /* width of the always-on BF16 shared expert, 0 = none */
    uint32_t expert_begin;        /* first routed expert resident on this device */
    uint32_t expert_count;        /* number resident here (experts for a single GPU) */
    uint32_t max_tokens;          /* largest T of a forward call (sizes the workspaces) */
    uint32_t max_pairs;           /* largest number of (token, expert) rows the local experts
                                     receive in one call; 0 = max_tokens * top_k */
    int32_t activation;           /* STRATA_MOE_ACT_*, routed and shared experts alike */
    float gate_beta;              /* SITU_GLU only, > 0 */
    float linear_beta;            /* SITU_GLU only, > 0 */
} strata_moe_layer_desc;

/* Optional device outputs of strata_moe_forward (any may be NULL). */
typedef struct strata_moe_aux {
    float* logits;     /* [T, E] fp32 */
    uint32_t* ids;     /* [T, k] expert ids in selection-rank order */
    float* weights;    /* [T, k] routing weights */
    uint32_t* counts;  /* [E] */
    uint32_t* offsets; /* [E + 1] exclusive prefix of counts */
    uint32_t* perm;    /* [T * k]: position -> token * k + rank, stable by (expert, token, rank) */
} strata_moe_aux;

typedef struct strata_moe_stats {
    uint64_t forward_calls;
    uint64_t kernel_launches; /* kernels of this library launched since creation */
    uint64_t h2d_bytes, d2h_bytes;
    uint64_t weight_bytes;    /* resident expert + router + shared bytes */
    float last_forward_ms;    /* CUDA-event time of the last forward when timing is on */
    uint64_t router_fast_tokens;      /* tokens routed through the tensor-core projection + exact recheck */
    uint64_t router_rechecked_tokens; /* of those, tokens recomputed completely by the canonical kernels */
    uint64_t command_calls;           /* handle-based commands collected */
    uint64_t workspace_allocations;   /* times a command had to (re)build its workspace */
    float router_worst_error;         /* fast router: largest |canonical - tensor-core logit| seen on a selected expert,
                                         as a fraction of the bound delta the selection assumes (trusted up to 0.5) */
} strata_moe_stats;

/* ---- context ------------------------------------------------------------------------
 * ref: CudaBackend::initialize, include/strata/cuda_backend.hpp:787 (one stream per device,
 * kernels/cuda/backend.cu:5854-5895).  stream = an existing cudaStream_t to run on, or NULL
 * to create a non-blocking stream owned by the context. */
int strata_moe_create(int device, void* stream, strata_moe_ctx** out);
/* Number of CUDA devices this library can run on (compute capability 10.x), 0 when there is none.
 * ref: CudaBackend::available_devices, include/strata/cuda_backend.hpp:783. */
int strata_moe_device_count(void);
void strata_moe_destroy(strata_moe_ctx* ctx);
const char* strata_moe_last_error(const strata_moe_ctx* ctx);
/* Waits for the stream, then reports and clears the device status word.
 * ref: CudaBackend::synchronize + the moe_error read-back, kernels/cuda/backend.cu:16927-16943 */
int strata_moe_synchronize(strata_moe_ctx* ctx);
int strata_moe_get_stats(const strata_moe_ctx* ctx, strata_moe_stats* out);
void strata_moe_set_timing(strata_moe_ctx* ctx, int enabled);
/* With timing on, strata_moe_forward brackets its phases with CUDA events on the context's
 * stream and waits for the call to finish (ref: the per-command event timing in
 * kernels/cuda/backend.cu:16294-16380, read back at 16927-16943).  out receives
 * STRATA_MOE_PHASES durations in ms: router projection, score/top-k, grouping, row gather,
 * gate/up + SwiGLU, down, shared expert, combine. */
#define STRATA_MOE_PHASES 8
int strata_moe_get_phase_ms(strata_moe_ctx* ctx, float* out);

/* ---- layer + weights ------------------------------------------------------------------
 * ref: CudaBackend::upload(device, CudaWeightDescriptor, weights, scales, CudaWeight&),
 * include/strata/cuda_backend.hpp:819-823; descriptor include/strata/cuda_backend.hpp:41-51. */
int strata_moe_layer_create(strata_moe_ctx* ctx, const strata_moe_layer_desc* desc,
                            strata_moe_layer** out);
void strata_moe_layer_destroy(strata_moe_layer* layer);
/* gate_bf16 [E, H] BF16 row-major; bias [E] fp32 or NULL (selection bias only). */
int strata_moe_set_router(strata_moe_layer* layer, const void* gate_bf16, const float* bias,
                          int source);
/* One projection of one routed expert (global expert index, must be resident here).
 * gate/up are [I, H], down is [H, I]; packed and scales as the format defines. */
int strata_moe_set_expert(strata_moe_layer* layer, uint32_t expert, int role, const void* packed,
                          const void* scales, float global_scale, int source);
/* BF16 shared expert projection: gate/up [Is, H], down [H, Is]. */
int strata_moe_set_shared(strata_moe_layer* layer, int role, const void* weights_bf16, int source);

/* ---- the layer ------------------------------------------------------------------------
 * out[t] = output_scale * sum_r w[t,r] * expert_{id[t,r]}(x[t]) + shared(x[t]), r in rank order.
 * Replaces the sparse_mlp bodies of the model runtimes (ref: src/models/glm52/glm_runtime.cpp:
 * 1487-1618, src/models/laguna/laguna_runtime.cpp:907-1158, src/models/dsv4/deepseek_runtime.cpp:
 * 6070-6096) including the host-side routing, grouping and combine they wrap around
 * CudaBackend::enqueue_moe.  x_bf16 [T, H] BF16 and out [T, H] fp32 are device pointers.
 * Requires expert_count == experts (single-GPU layer). */
int strata_moe_forward(strata_moe_layer* layer, const void* x_bf16, uint32_t tokens, float* out,
                       const strata_moe_aux* aux);
/* The same layer AFTER routing: the experts of every token and their routing weights are given
 * (device, [T, k], selection-rank order), e.g. by a router that runs on other features than the
 * experts (Kimi-K3 routes on the hidden state and runs the experts on a latent, see
 * strata_moe_latent_*) or by a token-id table.  No shared expert term.
 * ref: the part of sparse_mlp after the route call, src/models/glm52/glm_runtime.cpp:1521-1618. */
int strata_moe_forward_routed(strata_moe_layer* layer, const void* x_bf16, uint32_t tokens, const uint32_t* ids,
                              const float* weights, float* out);
/* Same call with HOST buffers (pageable or pinned): copies x in, runs, copies out back and
 * waits.  This is the call shape of the reference, whose commands take host spans
 * (ref: include/strata/cuda_backend.hpp:1147-1153). */
int strata_moe_forward_host(strata_moe_layer* layer, const void* x_bf16_host, uint32_t tokens,
                            float* out_host);

/* Diagnostics: every activation workspace of the context lies between two guard zones filled with a canary byte;
 * this waits for the context's streams and compares them.  0, or STRATA_MOE_E_CUDA with the workspace named in the
 * error text when a kernel wrote outside its buffer.  (The reference relies on host-side shape validation and a
 * device error flag, kernels/cuda/backend.cu:1922-1924, 16045-16142; a memory checker is not available to the tests.) */
int strata_moe_check_canaries(strata_moe_ctx* ctx);

/* Diagnostics: FNV-1a hash of n fp32 values (device memory) after round-to-nearest-even to BF16, the reference's
 * per-layer state hash ("[state]" lines, src/models/glm52/glm_runtime.cpp:1592-1598).  Waits for the context's
 * stream, copies the values to the host and hashes them there.
 * ref: stable_bf16_hash, include/strata/diagnostics.hpp:38-41, src/platform/diagnostics.cpp:84-88. */
int strata_moe_stable_bf16_hash(strata_moe_ctx* ctx, const float* values, size_t n, uint64_t* hash);

/* ---- stages (used by the expert-parallel driver and by the parity tests) ---------------- */
/* ref: linear(gate) + glm_route_logits_noaux_tc / laguna_route_sigmoid_topk / kimi_route_topk /
 * dsv4_route_sqrtsoftplus_f32 (src/models/glm52/glm_ops.cpp:176-233, src/models/laguna/
 * laguna_ops.cpp:182-243, src/models/kimi_k3/kimi_k3_ops.cpp:192-237, src/models/dsv4/
 * deepseek_ops.cpp:82-133); projection order as kernels/cuda/backend.cu:651-728. */
int strata_moe_route(strata_moe_layer* layer, const void* x_bf16, uint32_t tokens, float* logits,
                     uint32_t* ids, float* weights);
/* Hash routing: the experts of every token are given (token_experts [T, k], device, e.g. looked up from the
 * checkpoint's token-id table); the weights are the layer's scores of those experts, summed in rank order,
 * normalised and scaled exactly as strata_moe_route does.  ids receives a copy of token_experts.
 * ref: dsv4_route_hash_sqrtsoftplus_f32(_into), src/models/dsv4/deepseek_ops.cpp:390-461. */
int strata_moe_route_hash(strata_moe_layer* layer, const void* x_bf16, uint32_t tokens,
                          const uint32_t* token_experts, float* logits, uint32_t* ids, float* weights);
/* Inkling's router with shared "sink" experts.  Two stage calls, all pointers device memory:
 *   strata_moe_project_rows   logits[t, r] = x[t, :] . w[r, :] in the router's canonical summation order, for any
 *                             BF16 matrix w [rows, hidden] (here the gate over routed_experts + sinks rows);
 *   strata_moe_route_sink     logits [tokens, routed_experts + sinks] -> ids [tokens, top_k] (top-k of
 *                             sigmoid(logit) + bias over the routed range), their weights [tokens, top_k] and the
 *                             sinks' weights [tokens, sinks]: softmax over the log-sigmoid of the raw logits of the
 *                             selected experts and every sink, times scale (= routed_scale * global_scale).
 * top_k + sinks <= 32.  The routed part then runs through strata_moe_forward_routed, the sinks as a dense command.
 * ref: inkling_route_sigmoid_sink, src/models/inkling/inkling_ops.cpp:184-275; call site
 * src/models/inkling/inkling_runtime.cpp:524-560. */
int strata_moe_project_rows(strata_moe_ctx* ctx, const void* x_bf16, uint32_t tokens, uint32_t hidden,
                            const void* w_bf16, uint32_t rows, float* logits);
int strata_moe_route_sink(strata_moe_ctx* ctx, const float* logits, const float* bias, uint32_t tokens,
                          uint32_t routed_experts, uint32_t sinks, uint32_t top_k, float scale, uint32_t* ids,
                          float* weights, float* sink_weights);
/* ref: job building in sparse_mlp (src/models/glm52/glm_runtime.cpp:1521-1541) and the page
 * group table (src/models/dsv4/deepseek_runtime.cpp:6216-6321).  Groups pairs whose expert lies
 * in [expert_begin, expert_begin + n_experts); counts/offsets are indexed from expert_begin.
 * pairs = number of entries of ids; perm[pos] = index into ids. */
int strata_moe_group(strata_moe_layer* layer, const uint32_t* ids, uint32_t pairs,
                     uint32_t expert_begin, uint32_t n_experts, uint32_t* counts,
                     uint32_t* offsets, uint32_t* perm, uint32_t* inv /* [pairs] or NULL: entry ->
                     position, 0xFFFFFFFF for an entry outside the expert range */);
/* Allocation-free variant of strata_moe_group.  It has no counterpart in the reference.
 * For hosts that must not let a library allocate device memory -- a runtime that gave the
 * whole GPU to its own arena at start-up, or a caller in a section where cudaMalloc's implicit
 * device synchronisation is unacceptable.  It needs no context or layer (creating those
 * allocates): inputs and outputs are caller memory, `stream` is a cudaStream_t (NULL = default
 * stream), and the scratch is a fixed 520 KiB device array inside the library, resident on every
 * GPU that loads it.  Limits: pairs <= 65536, n_experts <= 256; larger calls are rejected with a
 * message in `err`.  The first call on a device resolves the array's address: issue it before
 * any stream capture on that device.  All calls share the array, so calls that overlap on the
 * GPU race; serialise them.  The call runs on the CURRENT CUDA device: `stream` and every pointer
 * must belong to it.  Returns 0 or a negative STRATA_MOE_E_* and a message in err. */
int strata_moe_group_static(void* stream, const uint32_t* ids, uint32_t pairs, uint32_t expert_begin,
                            uint32_t n_experts, uint32_t* counts, uint32_t* offsets, uint32_t* perm,
                            uint32_t* inv /* or NULL */, char* err, size_t err_cap);
/* dst row i = src row (index[i] / index_div); rows are row_bytes long (multiple of 16).
 * ref: the hidden-row and row-list upload of the grouped command,
 * kernels/cuda/backend.cu:15346-15996, and the placement-driven copies the runtimes do on the
 * host around it (src/models/dsv4/deepseek_runtime.cpp:6364-6387).  Used to pack the rows an
 * expert-parallel rank sends and to restore received order. */
int strata_moe_gather_rows(strata_moe_layer* layer, const void* src, uint32_t row_bytes,
                           const uint32_t* index, uint32_t index_div, uint32_t n, void* dst);
/* out[t] = output_scale * sum_r weights[t,r] * y[inv[t*k+r]] + shared(x_shared[t]), rank order.
 * x_shared may be NULL (no shared expert term).
 * ref: the host combine loops, src/models/glm52/glm_runtime.cpp:1586-1617,
 * src/models/laguna/laguna_runtime.cpp:1129-1156, src/models/dsv4/deepseek_runtime.cpp:5897-5914. */
int strata_moe_combine(strata_moe_layer* layer, const float* y, const uint32_t* inv,
                       const float* weights, const void* x_shared_bf16, uint32_t tokens, float* out);
/* Grouped expert FFN on rows already sorted by local expert.
 * ref: CudaBackend::enqueue_deepseek_moe_rows (the grouped command),
 * include/strata/cuda_backend.hpp:1139-1146, kernels/cuda/backend.cu:15346-15996.
 * rows_bf16 [pairs, H] BF16 in group order; offsets [expert_count + 1] device;
 * y [pairs, H] fp32 un-combined expert outputs. */
int strata_moe_experts_grouped(strata_moe_layer* layer, const void* rows_bf16, uint32_t pairs,
                               const uint32_t* offsets, float* y);
/* Exact fp32 dequantisation of one resident projection into host memory [rows, cols]
 * (the NVFP4 value includes the division by the global scale).  Synchronous. */
int strata_moe_dequant_export(strata_moe_layer* layer, uint32_t expert, int role, float* out_host);

/* ---- dense command, call-compatible with the reference backend --------------------------
 * ref: CudaBackend::enqueue_moe / collect_moe, include/strata/cuda_backend.hpp:1147-1153,
 * kernels/cuda/backend.cu:16003-16396, 17199-17203.  Every listed expert is applied to all
 * `rows` rows; routed_output is [expert][row][H] fp32, shared_output [row][H] (NULL = skip).
 * hidden_host is fp32 [rows, H] on the host.  coefficients[i] multiplies expert i's
 * activation before the down projection for INT4 (ref: kernels/cuda/backend.cu:1933) and must
 * be 1.0 for the other formats (ref: kernels/cuda/backend.cu:16088-16096).
 * One command may be in flight per layer; collect waits for it. */
int strata_moe_enqueue_dense(strata_moe_layer* layer, const float* hidden_host, uint32_t rows,
                             const uint32_t* experts, const float* coefficients, uint32_t n_experts,
                             int with_shared);
int strata_moe_collect_dense(strata_moe_layer* layer, float* routed_output, float* shared_output);

/* ---- LatentMoE wrapper (Kimi-K3) ------------------------------------------------------------
 * ref: kimi_latent_moe_layer, include/strata/kimi_k3_layer.hpp:257-261,
 * src/models/kimi_k3/kimi_k3_layer.cpp:781-1001.  Routing reads the raw hidden state [T, H]; the routed
 * experts run on latent = x * down^T (BF16 [HL, H]); their routing-weighted mixture is RMS-normalised
 * in the latent space (weight fp32 [HL], kimi_rms_norm) and projected back with up (BF16 [H, HL]); the
 * BF16 shared experts (concatenated: gate / up [Is, H], down [H, Is]) run on the raw hidden state
 * and add in.  desc describes the EXPERT side: desc->hidden = HL, desc->shared_intermediate = Is
 * (0 = none), every expert resident; model_hidden = H.  Expert weights are registered on
 * strata_moe_latent_experts() with strata_moe_set_expert (gate / up [I, HL], down [HL, I]).
 * The mixture is summed in selection-rank order (the reference sums in ascending expert order per
 * worker: a reassociation, inside the layer tolerance); the latent and the normalised mixture are
 * rounded to BF16 before the expert and the output GEMMs. */
typedef struct strata_moe_latent strata_moe_latent;
int strata_moe_latent_create(strata_moe_ctx* ctx, const strata_moe_layer_desc* desc, uint32_t model_hidden,
                             float rms_epsilon, strata_moe_latent** out);
void strata_moe_latent_destroy(strata_moe_latent* lat);
strata_moe_layer* strata_moe_latent_experts(strata_moe_latent* lat);
int strata_moe_latent_set_router(strata_moe_latent* lat, const void* gate_bf16 /* [E, H] */, const float* bias,
                                 int source);
int strata_moe_latent_set_projections(strata_moe_latent* lat, const void* down_bf16 /* [HL, H] */,
                                      const void* up_bf16 /* [H, HL] */, const float* norm_f32 /* [HL] */, int source);
int strata_moe_latent_set_shared(strata_moe_latent* lat, int role, const void* weights_bf16, int source);
/* x_bf16 [T, H] and out [T, H] fp32 are device pointers; ids / weights (device, [T, k]) may be NULL. */
int strata_moe_latent_forward(strata_moe_latent* lat, const void* x_bf16, uint32_t tokens, float* out,
                              uint32_t* ids, float* weights);

/* ---- weight handles and handle-based commands: the reference backend's own call shape -----
 * ref: CudaBackend::upload(device, CudaWeightDescriptor, weights, scales, CudaWeight&),
 * include/strata/cuda_backend.hpp:819-823 (descriptor :41-51).  One uploaded matrix [rows, cols] in one
 * of the STRATA_MOE_FMT_* encodings, or FP8 E4M3 with one E8M0 scale per 128 x 128 block
 * (STRATA_MOE_FMT_FP8B128: weights u8 [rows, cols], scales u8 [ceil(rows/128), ceil(cols/128)];
 * ref: CudaWeightEncoding::Fp8E4m3Block128, the DeepSeek-V4 shared expert).  The bytes are copied
 * to the device; the handle owns them until strata_moe_weight_release. */
#define STRATA_MOE_FMT_FP8B128 4
typedef struct strata_moe_weight strata_moe_weight;
typedef struct strata_moe_weight_desc {
    int32_t format;      /* STRATA_MOE_FMT_* */
    uint32_t rows, cols;
    float global_scale;  /* NVFP4 divisor, 1 otherwise */
} strata_moe_weight_desc;
int strata_moe_weight_upload(strata_moe_ctx* ctx, const strata_moe_weight_desc* desc, const void* weights_host,
                             size_t weight_bytes, const void* scales_host, size_t scale_bytes,
                             strata_moe_weight** out);
void strata_moe_weight_release(strata_moe_weight* w);
/* ref: struct CudaMoeExpert, include/strata/cuda_backend.hpp:740-745. */
typedef struct strata_moe_expert_ref {
    const strata_moe_weight* gate; /* [I, H] */
    const strata_moe_weight* up;   /* [I, H] */
    const strata_moe_weight* down; /* [H, I] */
    float coefficient;
} strata_moe_expert_ref;
/* ref: CudaBackend::enqueue_moe / collect_moe, include/strata/cuda_backend.hpp:1147-1153 and the
 * validation in kernels/cuda/backend.cu:16003-16145.  Every routed expert (at most 10, plus the
 * optional shared one) is applied to all `rows` fp32 rows of hidden_host; one encoding per
 * command (INT4-g128, NVFP4 or plain BF16); the coefficient is folded before the down projection
 * for INT4 and must be 1 otherwise and for the shared expert; non-finite hidden values are
 * rejected.  One command may be in flight per context.  collect waits, checks the device status
 * word and only then writes routed_out [n][rows][H] and shared_out [rows][H] (span sizes are
 * checked); a failed collect leaves the buffers untouched and drains the command. */
int strata_moe_command_enqueue(strata_moe_ctx* ctx, const float* hidden_host, size_t hidden_floats, uint32_t rows,
                               const strata_moe_expert_ref* routed, uint32_t n_routed,
                               const strata_moe_expert_ref* shared /* or NULL */);
int strata_moe_command_collect(strata_moe_ctx* ctx, float* routed_out, size_t routed_floats, float* shared_out,
                               size_t shared_floats);
/* ref: struct CudaDeepSeekMoeRowGroup, include/strata/cuda_backend.hpp:724-736 (canonical w1/w3/w2 form). */
typedef struct strata_moe_row_group {
    const strata_moe_weight* w1; /* gate [I, H], MXFP4 encoding with DSV4 scale edges */
    const strata_moe_weight* w3; /* up   [I, H] */
    const strata_moe_weight* w2; /* down [H, I] */
    const uint32_t* rows;        /* indices into the hidden rows this expert serves */
    const float* coefficients;   /* that row's router coefficient, same order */
    uint32_t n_rows;
} strata_moe_row_group;
/* ref: CudaBackend::enqueue_deepseek_moe_rows / collect_deepseek_moe_rows,
 * include/strata/cuda_backend.hpp:1139-1146, kernels/cuda/backend.cu:15346-15996.  The row-grouped
 * DSV4 command in the exact numerical mode described below; routed results are flattened group-major
 * and, inside a group, in the group's own row order.  `shared` (FP8B128 weights, or NULL) runs over
 * shared_rows and its results are flattened in that order. */
int strata_moe_command_enqueue_rows_dsv4(strata_moe_ctx* ctx, const float* hidden_host, size_t hidden_floats,
                                         uint32_t hidden_rows, const strata_moe_row_group* groups, uint32_t n_groups,
                                         const strata_moe_expert_ref* shared, const uint32_t* shared_rows,
                                         uint32_t n_shared_rows, float swiglu_limit);
int strata_moe_command_collect_rows_dsv4(strata_moe_ctx* ctx, float* routed_out, size_t routed_floats,
                                         float* shared_out, size_t shared_floats);

/* ---- DSV4-exact numerical mode ---------------------------------------------------------
 * Bit-exact DeepSeek-V4 routed-expert arithmetic (ref: enqueue_deepseek_moe_rows, the grouped
 * command, include/strata/cuda_backend.hpp:1139-1146; kernels deepseek_fp4_gate_up_kernel /
 * deepseek_fp4_down_kernel / quantize_activation_e4m3_kernel, kernels/cuda/backend.cu:2308-2413,
 * 247-272; CPU replay kernels/cpu/dsv4_fp4_expert.cpp:774-884): the input rows and the SwiGLU
 * output are quantised to E4M3 with one power-of-two scale per 128 columns, every dot product is
 * summed in the reference's order (256 strided partial sums, fixed tree), gate and up are rounded
 * to BF16, clamped (gate from above, up on both sides) to swiglu_limit, SiLU is taken of the
 * BF16 gate, the coefficient (route weight) multiplies the activation before its BF16 rounding,
 * and the output rows are BF16-rounded fp32.  Needs MXFP4-format weights (E2M1 + E8M0/32; scale
 * byte 0 means 2^-127 and 0xFF NaN, as in DSV4).  rows_f32 [pairs, H] fp32 in group order (device),
 * offsets [expert_count + 1], coefficients [pairs] or NULL (= 1), y [pairs, H] fp32: un-combined
 * expert outputs, to be summed in selection-rank order (weights already applied). */
int strata_moe_experts_grouped_dsv4(strata_moe_layer* layer, const float* rows_f32, uint32_t pairs,
                                    const uint32_t* offsets, const float* coefficients, float swiglu_limit,
                                    float* y);
/* The DSV4 join: out[t] = bf16(sum over the token's k rows of y, in selection-rank order, + bf16(shared[t])).
 * y are the rows strata_moe_experts_grouped_dsv4 produced (route weights already applied), inv the
 * entry -> row map of strata_moe_group, shared_rows [tokens, H] fp32 the shared expert's output (or NULL).
 * ref: src/models/dsv4/deepseek_runtime.cpp:5897-5914, kernels/cuda/backend.cu:2868-2880. */
int strata_moe_combine_dsv4(strata_moe_layer* layer, const float* y, const uint32_t* inv,
                            const float* shared_rows, uint32_t tokens, float* out);
/* The activation quantisation alone, in place on fp32 [rows, cols] (device memory).
 * ref: quantize_activation_e4m3_kernel, kernels/cuda/backend.cu:247-272. */
int strata_moe_quantize_e4m3(strata_moe_ctx* ctx, float* values, uint32_t rows, uint32_t cols);

/* ---- expert parallelism over peer memory (one process per GPU) ---------------------------
 * ref: the reference shards experts over the GPUs of ONE process and carries activations
 * through host memory (src/models/glm52/glm_runtime.cpp:650-652 placement, 1561-1576 per-device
 * enqueue/collect); these calls replace that transport for one rank per GPU.  Rank r holds the
 * experts [r * E / world, (r + 1) * E / world) (a layer created with that expert_begin /
 * expert_count) and its own tokens.  Each rank owns a "window" of device memory that all peers
 * map; the dispatch kernel stores a token's row straight into the window of every rank that owns
 * one of its selected experts (once per owner, however many of that owner's experts were selected),
 * the owner forms the routing-weighted sum of its experts' outputs for the token, and the combine
 * kernel loads those partial sums straight from the owners' windows and adds them in rank order
 * (NVLink peer loads and stores, flags with release/acquire at system scope, every wait bounded by
 * wait_ms).  The partial sums travel as f16 rows with an exact power-of-two factor per row, so a
 * step agrees with the single-GPU forward to f16 rounding of the partial sums, not bit for bit.
 * Limits: experts <= 1024, top_k <= 32.
 *
 * Set-up: every rank calls ep_window_bytes (same arguments everywhere), ep_window_alloc, sends
 * the 64-byte handle to its peers by any host channel, opens the peers' handles with
 * ep_window_open, passes the `world` window pointers (its own at index rank) to ep_create, and
 * the ranks synchronise on the host once before the first step.  row_capacity bounds the (token,
 * expert) pairs a rank can receive in one step; a step that would exceed it on any rank stores nothing, computes
 * nothing and reports STRATA_MOE_E_NUMERIC ("inconsistent group table") at the next synchronize
 * on every rank.  A rank that stops taking part makes its peers' waits run out after wait_ms
 * (0 = 10 s): "bounded wait timed out" from synchronize, context still usable. */
typedef struct strata_moe_ep strata_moe_ep;
size_t strata_moe_ep_window_bytes(const strata_moe_layer_desc* desc, uint32_t world, uint32_t row_capacity);
int strata_moe_ep_window_alloc(strata_moe_ctx* ctx, size_t bytes, void** window, void* handle64 /* or NULL */);
int strata_moe_ep_window_open(strata_moe_ctx* ctx, const void* handle64, void** window);
int strata_moe_ep_window_close(strata_moe_ctx* ctx, void* window);
int strata_moe_ep_window_free(strata_moe_ctx* ctx, void* window);
int strata_moe_ep_create(strata_moe_layer* layer, uint32_t rank, uint32_t world, uint32_t row_capacity,
                         void* const* windows /* [world] */, uint32_t wait_ms, strata_moe_ep** out);
void strata_moe_ep_destroy(strata_moe_ep* ep);
/* One step = begin, dispatch, experts, finish, each only enqueueing work on the context's stream.
 * x_bf16 [tokens, H] are this rank's tokens, out [tokens, H] fp32 its results.  expected_rows is
 * a hint for the number of rows this rank will receive (0 = as many as it sends); the exact
 * number never reaches the host.  ep_forward runs the four stages back to back.  The stages are
 * separate entry points so that a host can interleave other work, and so that several ranks can
 * be stepped by one process in tests. */
int strata_moe_ep_begin(strata_moe_ep* ep, const void* x_bf16, uint32_t tokens);
int strata_moe_ep_dispatch(strata_moe_ep* ep);
int strata_moe_ep_experts(strata_moe_ep* ep, uint32_t expected_rows);
int strata_moe_ep_finish(strata_moe_ep* ep, float* out);
int strata_moe_ep_forward(strata_moe_ep* ep, const void* x_bf16, uint32_t tokens, float* out,
                          uint32_t expected_rows);
/* Drops a step that failed between stages so that the next ep_begin is accepted. */
int strata_moe_ep_abandon(strata_moe_ep* ep);
/* Row counts of the last completed step, read back from the device (waits for the context's stream):
 * sent_rows [world] = token rows this rank stored into each owner's window (its own included),
 * received_rows = token rows it received as an owner, received_pairs = (token, expert) rows its experts
 * computed.  A token counts once per owner, so sum(sent_rows) <= tokens * min(top_k, world).
 * Any pointer may be NULL.  Diagnostics; ref: the per-command counters of CudaBackendStats,
 * include/strata/cuda_backend.hpp:71-262. */
int strata_moe_ep_last_counts(strata_moe_ep* ep, uint32_t* sent_rows, uint32_t* received_rows,
                              uint32_t* received_pairs);

#ifdef __cplusplus
}
#endif
#endif /* STRATA_MOE_H */
