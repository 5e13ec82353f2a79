// Large-batch ("prefill") expert FFN: grouped GEMMs on the 5th-generation tensor cores.
//
// Orientation: the WEIGHTS are the M operand (128 output features per tile) and the expert's
// token rows are the N operand (up to 128 per tile, any multiple of 16), so ragged expert
// groups cost at most 15 padded rows instead of a padded 128-row tile.  D (FP32) lives in
// tensor memory: lane = output feature, column = token.
//
//   warp 0        TMA producer: activation tiles [N x 64] f16 -> shared memory (128-byte swizzle)
//   warps 1, 3    MMA issuers: one thread each issues tcgen05.mma (kind::f16, M=128, K=16) per k-slice,
//                 warp 1 for the first weight tile of a stage, warp 3 for the second.  An issuing
//                 thread is serial (barrier polls, descriptor arithmetic, commits) and the tensor
//                 pipe drains whenever it is not issuing; two issuers cover each other's gaps
//   warp 2        TMA producer for the packed 4-bit weights: [128 rows x 128 B] blocks (256 columns,
//                 four pipeline stages) land in a double-buffered, 128-byte-swizzled staging area
//   warps 4..19   decoders: each lane owns one weight row (= one tensor-memory lane) and reads 16
//                 packed bytes (32 columns) of it per stage from the staging area, decodes exactly
//                 to f16 (hardware E2M1 conversion / INT4 magic-number trick), applies the block
//                 scale and writes the 16 f16x2 words straight into TENSOR MEMORY (tcgen05.st):
//                 the decoded weights are the A operand of a tensor-memory-sourced MMA and never
//                 touch shared memory, which halves the shared-memory traffic per MMA
//   warps 20..27  epilogue: tcgen05.ld the accumulators, fuse SwiGLU (gate/up) or the output
//                 scale (down), store
// Tensor memory (512 columns): accumulators in columns 0..255 (two tiles x up to 128 tokens),
// a four-stage ring of decoded weight slices in columns 256..511 (2 tiles x 32 columns per
// stage).  BF16 weights (the shared expert) need no decode and keep the shared-memory A operand.
// CTAs are persistent (one per SM) and walk a tile list built on the device from the
// per-expert offsets.
//
// Every wait is bounded: on expiry the kernel raises kStatusWaitTimeout, all roles leave their
// loops, tensor memory is released and the kernel returns normally.
//
// Replaces the reference's per-row page kernels (kernels/cuda/backend.cu:2439-2582, 2600-2779)
// and the per-expert matmul fallbacks (kernels/cuda/backend.cu:1140-1207).
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstddef>
#include <cstdlib>

#include "common.cuh"

namespace smoe {

// Tokens per tile: 192 (an expert with up to 192 rows is decoded once; two tensor-memory weight stages) when
// groups are large, 128 (four weight stages: shorter handshakes for small tiles) when they are small, and 160
// (three weight stages) for groups of about 128 rows, which a 128-token tile would split in two half the time.
template <int NT>
struct Geo {
    static_assert(NT == 128 || NT == 160 || NT == 192, "tile sizes");
    static constexpr uint32_t kNTile = NT;
    static constexpr uint32_t kAccCols = 2u * NT;                    // accumulator columns (2 tiles x NT)
    static constexpr uint32_t kAStages = (512u - 2u * NT) / 64u;     // tensor-memory ring of decoded weight slices
    static constexpr uint32_t kBStages = NT == 128 ? 8u : 6u;        // activation tiles in flight
    static constexpr uint32_t kBTile = NT * 64u * 2u;                // bytes of one activation tile stage
};
constexpr uint32_t kMaxAStages = 4;
constexpr uint32_t kMTile = 128;    // output features per tile
constexpr uint32_t kBK = 64;        // K per pipeline stage (128 bytes of f16 per row)
// Two rings: decoded weight tiles only have to bridge decode -> MMA (on-chip, short), while
// the activation tiles arrive by TMA and need enough stages in flight to cover its latency.
constexpr uint32_t kPkBufs = 2;      // packed-weight staging blocks (256 columns each) in flight
constexpr uint32_t kAStageCols = 64;                    // tensor-memory columns per A stage: 2 tiles x (kBK / 2)
constexpr uint32_t kATile = kMTile * kBK * 2;  // 16 KiB
constexpr uint32_t kDecodeWarps = 16;  // each lane decodes 32 columns of one row per stage
constexpr uint32_t kEpilogueWarps = 8;   // two per tensor-memory lane quarter: even / odd 16-token chunks
constexpr uint32_t kThreads = (4 + kDecodeWarps + kEpilogueWarps) * 32;
constexpr uint32_t kPkCols = 256;                       // columns per packed staging block (4 stages)
constexpr uint32_t kPkTile = kMTile * (kPkCols / 2);    // 16 KiB of 4-bit weights: 128 rows x 128 B
constexpr uint32_t kFirstDecodeWarp = 4, kFirstEpilogueWarp = kFirstDecodeWarp + kDecodeWarps;
constexpr uint32_t kSpinLimit = 1u << 19;   // x up to kWaitHintNs each: about two seconds
constexpr int kFmtBf16W = 3;  // plain BF16 weights (shared expert): tiles arrive by TMA, no decode

// ------------------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// Bounded wait: false when the phase did not complete within the spin limit.  Each try_wait
// carries a suspend-time hint: the hardware parks the thread until the phase completes or the
// hint expires, so waiting warps (the epilogue during a main loop, producers on a full ring) do
// not burn issue slots that the decode warps need.
constexpr uint32_t kWaitHintNs = 4096;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile uint32_t* abort_flag) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(kWaitHintNs)
            : "memory");
        if (done) return true;
        if ((spin & 63u) == 63u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint32_t x, uint32_t y,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);       // start address
    d |= (uint64_t)1 << 16;                         // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024u >> 4) << 32;              // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                         // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                         // 128-byte swizzle
    return d;
}
// Instruction descriptor, kind::f16: F16 x F16 (or BF16 x BF16) -> F32, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t umma_idesc_f16(uint32_t n, uint32_t ab_format /* 0 = F16, 1 = BF16 */) {
    uint32_t d = 0;
    d |= 1u << 4;               // D format F32
    d |= ab_format << 7;        // A format
    d |= ab_format << 10;       // B format
    d |= (n >> 3) << 17;        // N
    d |= (kMTile >> 4) << 24;   // M
    return d;
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same MMA with the A operand read from tensor memory (lane = row, 32-bit column = two K values).
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// This thread's 16 words -> 16 consecutive columns of its tensor-memory lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t v[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t v[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
        "%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t v[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint4 ldg_stream16_c(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// ------------------------------------------------------------------------------ decoders (f16)
__device__ __forceinline__ void p_e2m1x8_f16(uint32_t w, uint32_t r[4]) {
    asm("{\n .reg .b8 b0, b1, b2, b3;\n mov.b32 {b0, b1, b2, b3}, %4;\n"
        " cvt.rn.f16x2.e2m1x2 %0, b0;\n cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        " cvt.rn.f16x2.e2m1x2 %2, b2;\n cvt.rn.f16x2.e2m1x2 %3, b3;\n}"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
        : "r"(w));
}
__device__ __forceinline__ uint32_t p_mul_f16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t p_sub_f16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// 8 offset-binary INT4 nibbles -> 4 f16x2 of (q - 8) in natural column order.
// Byte permutes gather adjacent nibbles and splice in the high byte 0x64: 0x6400 | q is the f16
// number 1024 + q, and subtracting 1032 leaves q - 8 exactly.
__device__ __forceinline__ uint32_t p_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void p_int4x8_f16(uint32_t w, uint32_t r[4]) {
    const uint32_t lo = w & 0x0F0F0F0Fu;          // nibbles 0,2,4,6
    const uint32_t hi = (w >> 4) & 0x0F0F0F0Fu;   // nibbles 1,3,5,7
    const uint32_t n03 = p_prmt(lo, hi, 0x5140u);  // bytes n0,n1,n2,n3
    const uint32_t n47 = p_prmt(lo, hi, 0x7362u);  // bytes n4,n5,n6,n7
    const uint32_t k64 = 0x00000064u, k1032 = 0x64086408u;
    r[0] = p_sub_f16x2(p_prmt(n03, k64, 0x4140u), k1032);
    r[1] = p_sub_f16x2(p_prmt(n03, k64, 0x4342u), k1032);
    r[2] = p_sub_f16x2(p_prmt(n47, k64, 0x4140u), k1032);
    r[3] = p_sub_f16x2(p_prmt(n47, k64, 0x4342u), k1032);
}

// One row's 16 packed bytes (32 columns) -> 4 x 16-byte f16 chunks, scaled.
// m[c] multiplies chunk c (8 columns).
template <int FMT>
__device__ __forceinline__ void decode16(const uint4& p, const uint32_t m[4], uint4 out[4]) {
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t r[4];
        if (FMT == STRATA_MOE_FMT_INT4G128) p_int4x8_f16(w[c], r);
        else p_e2m1x8_f16(w[c], r);
        out[c] = make_uint4(p_mul_f16x2(r[0], m[c]), p_mul_f16x2(r[1], m[c]), p_mul_f16x2(r[2], m[c]),
                            p_mul_f16x2(r[3], m[c]));
    }
}

// Activation tensor maps with boxes of 16, 32, 64 and 128 rows: a tile with few valid rows
// fetches only the rows the MMA will read (rounded up to the next box size).
struct BMaps {
    CUtensorMap m[4];
};

struct TileInfo {
    uint32_t g, row0, n;  // expert, first row of this n-tile, valid rows (1..kNTile)
    uint32_t m0;          // first output feature
};

template <int NT>
struct __align__(1024) PrefillSmem {
    // 4-bit formats: packed staging [buffer][gate/down, up][kPkTile], then the activation ring.
    // BF16 weights: w and b together are one arena that the kernel cuts into four stages of A tiles
    // [stage][gate/down, up][kATile] followed by the activation stages that still fit.
    uint8_t w[kPkBufs][2][kPkTile];
    uint8_t b[Geo<NT>::kBStages][Geo<NT>::kBTile];   // activation tile
    uint64_t full_a[kMaxAStages], empty_a[kMaxAStages], full_b[Geo<NT>::kBStages], empty_b[Geo<NT>::kBStages];
    uint64_t pk_full[kPkBufs], pk_empty[kPkBufs];
    uint64_t acc_full, acc_empty;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

__device__ __forceinline__ bool tile_lookup(const uint32_t* table, uint32_t tile, uint32_t m_tiles, TileInfo& t,
                                            uint32_t tile_feat = kMTile) {
    const uint32_t total = table[0] * m_tiles;
    if (tile >= total) return false;
    const uint32_t j = tile / m_tiles;
    t.g = table[4 + 3 * j];
    t.row0 = table[4 + 3 * j + 1];
    t.n = table[4 + 3 * j + 2];
    t.m0 = (tile - j * m_tiles) * tile_feat;
    return true;
}

// MODE 0: gate + up tiles of the same 128 features, SwiGLU, act (16-bit) out.  K = H, features over I.
// MODE 1: one down tile (128 features), y (fp32) out.                          K = I, features over H.
// MODE 2: two adjacent down tiles (256 features) against the same activation tile -- halves the
//         shared-memory traffic per MMA of MODE 1; needs H % 256 == 0.
// DUAL (two weight tiles and two accumulators per activation tile) = MODE 0 or 2.
template <int FMT, int MODE, int NT>
__global__ void __launch_bounds__(kThreads, 1)
prefill_ffn_kernel(const __grid_constant__ BMaps maps_b, const __grid_constant__ CUtensorMap map_a0,
                   const __grid_constant__ CUtensorMap map_a1, PrefillArgs a, const float* __restrict__ rowscale,
                   void* __restrict__ act_out_v, const CUtensorMap* __restrict__ wmaps /* [3][n_groups] */) {
    extern __shared__ uint8_t smem_raw[];
    PrefillSmem<NT>& S =
        *reinterpret_cast<PrefillSmem<NT>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr uint32_t kNTile = Geo<NT>::kNTile, kAccCols = Geo<NT>::kAccCols, kAStages = Geo<NT>::kAStages;
    // BF16 weights arrive as ready A tiles by TMA: the staging blocks and the activation ring are re-cut into four
    // stages of weight tiles (two stages left a K-step waiting for a whole memory round trip: 112 K-steps of a
    // router projection took 0.6 us each) and as many activation stages as the rest holds (4 at 128 tokens, 3 at 192)
    constexpr bool BF = FMT == kFmtBf16W;
    constexpr uint32_t kBfAStages = 4;
    constexpr uint32_t kArena = kPkBufs * 2u * kPkTile + Geo<NT>::kBStages * Geo<NT>::kBTile;
    constexpr uint32_t kBStages = BF ? (kArena - kBfAStages * 2u * kATile) / Geo<NT>::kBTile : Geo<NT>::kBStages;
    static_assert(kBfAStages <= kMaxAStages && kBStages >= 2u && kBStages <= Geo<NT>::kBStages, "ring geometry");
    static_assert(offsetof(PrefillSmem<NT>, b) == kPkBufs * 2u * kPkTile, "staging blocks and activation ring form one arena");
    uint8_t* const arena = &S.w[0][0][0];
    auto a_tile = [&](uint32_t stage, uint32_t which) -> uint8_t* { return arena + (stage * 2u + which) * kATile; };
    auto b_tile = [&](uint32_t stage) -> uint8_t* {
        return BF ? arena + kBfAStages * 2u * kATile + stage * Geo<NT>::kBTile : S.b[stage];
    };
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    constexpr bool DUAL = MODE != 1;
    constexpr bool GU = MODE == 0;
    constexpr uint32_t kTileFeat = MODE == 2 ? 2u * kMTile : kMTile;  // features per tile
    constexpr uint32_t kSecond = MODE == 2 ? kMTile : 0u;              // row offset of the second weight tile
    const uint32_t K = GU ? a.H : a.I;
    const uint32_t R = GU ? a.I : a.H;
    const uint32_t m_tiles = R / kTileFeat;
    const uint32_t k_stages = K / kBK;
    volatile uint32_t* abort_flag = &S.abort_flag;
    if (a.tile_table[0] == 0u) return;   // nothing listed (mixed dispatch with no large group): leave before any set-up

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kMaxAStages; ++s) {
            // one arrival per producer warp, or one TMA transaction group for BF16 weights
            // (a stage is decoded by half of the decode warps: the other half works on the next one)
            mbar_init(&S.full_a[s], FMT == kFmtBf16W ? 1u : (DUAL ? kDecodeWarps / 2u : kDecodeWarps / 4u));
            mbar_init(&S.empty_a[s], DUAL ? 2u : 1u);   // one commit per MMA issuer
        }
        for (uint32_t s = 0; s < Geo<NT>::kBStages; ++s) {
            mbar_init(&S.full_b[s], 1);
            mbar_init(&S.empty_b[s], DUAL ? 2u : 1u);
        }
        mbar_init(&S.acc_full, DUAL ? 2u : 1u);
        mbar_init(&S.acc_empty, kEpilogueWarps);  // one arrival per epilogue warp
        for (uint32_t i = 0; i < kPkBufs; ++i) {
            mbar_init(&S.pk_full[i], 1);
            mbar_init(&S.pk_empty[i], DUAL ? kDecodeWarps : kDecodeWarps / 2u);
        }
        S.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // tensor-memory allocation: all 512 columns (one CTA per SM)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&S.tmem_base)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = S.tmem_base;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok; tile += gridDim.x) {
                TileInfo t;
                if (!tile_lookup(a.tile_table, tile, m_tiles, t, kTileFeat)) break;
                for (uint32_t ks = 0; ks < k_stages; ++ks, ++it) {
                    const uint32_t s = it % kBStages, ph = (it / kBStages) & 1u;
                    if (!mbar_wait(&S.empty_b[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t bsel = t.n <= 16u ? 0u : (t.n <= 32u ? 1u : (t.n <= 64u ? 2u : 3u));
                    const bool tail = t.n > 128u;   // rows from 128 on arrive as a second box: 64 rows (192-token tile) or 32
                    constexpr uint32_t kTailSel = NT == 192 ? 2u : 1u, kTailRows = 16u << kTailSel;
                    mbar_arrive_expect_tx(&S.full_b[s], ((16u << bsel) + (tail ? kTailRows : 0u)) * kBK * 2u);
                    tma_load_2d(b_tile(s), &maps_b.m[bsel], ks * kBK, t.row0, &S.full_b[s]);
                    if (tail) tma_load_2d(b_tile(s) + 128u * kBK * 2u, &maps_b.m[kTailSel], ks * kBK, t.row0 + 128u, &S.full_b[s]);
                    if (FMT == kFmtBf16W) {
                        const uint32_t sa = it % kBfAStages, pa = (it / kBfAStages) & 1u;
                        if (!mbar_wait(&S.empty_a[sa], pa ^ 1u, abort_flag)) { ok = false; break; }
                        mbar_arrive_expect_tx(&S.full_a[sa], DUAL ? 2u * kATile : kATile);
                        tma_load_2d(a_tile(sa, 0), &map_a0, ks * kBK, t.m0, &S.full_a[sa]);
                        if (DUAL) tma_load_2d(a_tile(sa, 1), &map_a1, ks * kBK, t.m0 + kSecond, &S.full_a[sa]);
                    }
                }
            }
            if (!ok) { *abort_flag = 1; atomicOr(a.status, kStatusWaitTimeout); }
            if (*abort_flag) {
                // copies issued but possibly not consumed: give each a bounded chance to land
                // before the CTA's shared memory is released
                const uint32_t pending = it < kBStages ? it : kBStages;
                for (uint32_t q = 0; q < pending; ++q) {
                    const uint32_t j = it - 1u - q;
                    const uint32_t addr = smem_u32(&S.full_b[j % kBStages]);
                    for (uint32_t spin = 0; spin < (1u << 16); ++spin) {
                        uint32_t done;
                        asm volatile(
                            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                            " selp.u32 %0, 1, 0, p;\n}"
                            : "=r"(done)
                            : "r"(addr), "r"((j / kBStages) & 1u)
                            : "memory");
                        if (done) break;
                    }
                }
            }
        }
    } else if (warp == 1 || warp == 3) {
        // ---------------------------------------------------------------- MMA issuers
        const uint32_t mi = warp == 3 ? 1u : 0u;   // which weight tile of the stage this thread feeds
        if (lane == 0 && (DUAL || mi == 0u)) {
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok; tile += gridDim.x, ++tcount) {
                TileInfo t;
                if (!tile_lookup(a.tile_table, tile, m_tiles, t, kTileFeat)) break;
                if (!mbar_wait(&S.acc_empty, (tcount & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t n = (t.n + 15u) & ~15u;
                const uint32_t idesc = umma_idesc_f16(n, FMT == kFmtBf16W ? 1u : 0u);
                const uint32_t d = tmem_base + mi * kNTile;
                constexpr uint32_t kRing = BF ? kBfAStages : kAStages;
                for (uint32_t ks = 0; ks < k_stages; ++ks, ++it) {
                    const uint32_t sa = it % kRing, pa = (it / kRing) & 1u;
                    const uint32_t sb = it % kBStages, pb = (it / kBStages) & 1u;
                    if (!mbar_wait(&S.full_a[sa], pa, abort_flag) || !mbar_wait(&S.full_b[sb], pb, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t b = smem_u32(b_tile(sb));
                    if (FMT == kFmtBf16W) {
                        const uint32_t a0 = smem_u32(a_tile(sa, mi));
#pragma unroll
                        for (uint32_t kk = 0; kk < kBK / 16u; ++kk) {
                            umma_f16(d, umma_desc_sw128(a0 + kk * 32u), umma_desc_sw128(b + kk * 32u), idesc,
                                     (ks | kk) ? 1u : 0u);
                        }
                    } else {
                        // decoded weights of this stage: columns [ta, ta + 32) tile 0, [ta + 32, ta + 64) tile 1;
                        // a K = 16 slice is 8 columns
                        const uint32_t ta = tmem_base + kAccCols + sa * kAStageCols + mi * (kBK / 2u);
#pragma unroll
                        for (uint32_t kk = 0; kk < kBK / 16u; ++kk) {
                            umma_f16_ts(d, ta + kk * 8u, umma_desc_sw128(b + kk * 32u), idesc, (ks | kk) ? 1u : 0u);
                        }
                    }
                    umma_commit(&S.empty_a[sa]);  // a stage is free once both issuers' MMAs have read it
                    umma_commit(&S.empty_b[sb]);
                }
                if (ok) umma_commit(&S.acc_full);
            }
            if (!ok) { *abort_flag = 1; atomicOr(a.status, kStatusWaitTimeout); }
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- packed-weight TMA producer
        if (lane == 0 && FMT != kFmtBf16W) {
            const uint32_t blocks = (K + kPkCols - 1u) / kPkCols;
            uint32_t bi = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok; tile += gridDim.x) {
                TileInfo t;
                if (!tile_lookup(a.tile_table, tile, m_tiles, t, kTileFeat)) break;
                const CUtensorMap* m0 = wmaps + (GU ? 0u : 2u) * a.n_groups + t.g;
                const CUtensorMap* m1 = wmaps + (GU ? 1u : 2u) * a.n_groups + t.g;
                for (uint32_t q = 0; q < blocks; ++q, ++bi) {
                    const uint32_t pb = bi % kPkBufs, ph = (bi / kPkBufs) & 1u;
                    if (!mbar_wait(&S.pk_empty[pb], ph ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(&S.pk_full[pb], DUAL ? 2u * kPkTile : kPkTile);
                    tma_load_2d(S.w[pb][0], m0, q * (kPkCols / 2u), t.m0, &S.pk_full[pb]);
                    if (DUAL) tma_load_2d(S.w[pb][1], m1, q * (kPkCols / 2u), t.m0 + kSecond, &S.pk_full[pb]);
                }
            }
            if (!ok) { *abort_flag = 1; atomicOr(a.status, kStatusWaitTimeout); }
            if (*abort_flag) {
                for (uint32_t q = 0; q < (bi < kPkBufs ? bi : kPkBufs); ++q) {
                    const uint32_t j = bi - 1u - q;
                    const uint32_t addr = smem_u32(&S.pk_full[j % kPkBufs]);
                    for (uint32_t spin = 0; spin < (1u << 16); ++spin) {
                        uint32_t done;
                        asm volatile(
                            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                            " selp.u32 %0, 1, 0, p;\n}"
                            : "=r"(done)
                            : "r"(addr), "r"((j / kPkBufs) & 1u)
                            : "memory");
                        if (done) break;
                    }
                }
            }
        }
    } else if (warp < kFirstEpilogueWarp && FMT == kFmtBf16W) {
        // BF16 weights need no decode: the TMA producer loads their tiles
    } else if (warp < kFirstEpilogueWarp) {
        // ---------------------------------------------------------------- weight producers
        // A warp can only write the tensor-memory lanes 32 * (warp % 4) .. + 31, and a lane holds one
        // weight row: lane i of a decode warp owns row 32 * (warp % 4) + i of one weight tile and
        // decodes all 64 of its columns in EVERY OTHER stage.  The four decode warps that share a lane
        // quarter split into tile 0 / tile 1 and even / odd stages: a warp's chain for one stage (wait for
        // the stage's columns, store, wait for the store, arrive) takes longer than the MMAs of a stage, and
        // with every warp in every stage that chain set the pace of the whole pipeline; now two stages'
        // chains overlap.  (32 consecutive rows reading the same swizzled 16-byte chunk index are free of
        // bank conflicts.)  With one weight tile per stage (MODE 1) only the tile-0 warps work.
        const uint32_t wd = warp - kFirstDecodeWarp;
        const uint32_t which = DUAL ? (wd >> 3) : 0u;
        const uint32_t parity = (wd >> 2) & 1u;
        const uint32_t arow = (warp & 3u) * 32u + lane;
        constexpr uint32_t CH = 2u;  // 16-byte packed chunks per thread per stage
        const bool active = DUAL || wd < kDecodeWarps / 2u;
        // this thread's first column in an A stage: tile, then 16 columns (32 K values) per chunk
        const uint32_t a_col = kAccCols + which * (kBK / 2u);
        const uint32_t a_lane_addr = tmem_base + (((warp & 3u) * 32u) << 16) + a_col;
        uint32_t it = 0, bi = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; ok && active; tile += gridDim.x) {
            TileInfo t;
            if (!tile_lookup(a.tile_table, tile, m_tiles, t, kTileFeat)) break;
            const WeightTable& wt = GU ? (which ? a.up : a.gate) : a.down;
            const uint32_t row = t.m0 + arow + which * kSecond;
            const uint8_t* srow = wt.scales[t.g];
            int32_t mx_off = 0;
            if (FMT == STRATA_MOE_FMT_MXFP4) {
                srow += (size_t)row * (K / 32u);
                mx_off = 2 - (int32_t)wt.emin[t.g];
            } else if (FMT == STRATA_MOE_FMT_NVFP4) {
                srow += (size_t)row * (K / 16u);
            } else {
                srow += (size_t)row * (K / 128u) * 2u;
            }
            // Scale bytes of one 256-column block of this thread's row, fetched one block ahead:
            // MXFP4 8 bytes, NVFP4 16 bytes, INT4 two BF16 values.
            // Vector loads need the row's scale bytes aligned to the vector: true when K % 256 == 0
            // (then every row holds a whole number of blocks); otherwise fall back to narrow loads.
            const bool whole_blocks = (K % kPkCols) == 0u;
            auto load_scales = [&](uint32_t q) -> uint4 {
                const uint32_t nblk = (K + kPkCols - 1u) / kPkCols;
                q = q < nblk ? q : nblk - 1u;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (FMT == STRATA_MOE_FMT_MXFP4) {          // 8 bytes per block, rows 4-byte aligned
                    if (whole_blocks) {
                        const uint2 w = __ldg(reinterpret_cast<const uint2*>(srow + q * 8u));
                        v.x = w.x; v.y = w.y;
                    } else {
                        v.x = __ldg(reinterpret_cast<const uint32_t*>(srow + q * 8u));
                        if ((q + 1u) * 8u <= K / 32u) v.y = __ldg(reinterpret_cast<const uint32_t*>(srow + q * 8u + 4u));
                    }
                } else if (FMT == STRATA_MOE_FMT_NVFP4) {   // 16 bytes per block, rows 8-byte aligned
                    if (whole_blocks) {
                        v = __ldg(reinterpret_cast<const uint4*>(srow + q * 16u));
                    } else {
                        const uint2 w = __ldg(reinterpret_cast<const uint2*>(srow + q * 16u));
                        v.x = w.x; v.y = w.y;
                        if ((q + 1u) * 16u <= K / 16u) {
                            const uint2 w2 = __ldg(reinterpret_cast<const uint2*>(srow + q * 16u + 8u));
                            v.z = w2.x; v.w = w2.y;
                        }
                    }
                } else {                                     // two BF16 per block, rows 2-byte aligned
                    if (whole_blocks) {
                        v.x = __ldg(reinterpret_cast<const uint32_t*>(srow + q * 4u));
                    } else {
                        v.x = __ldg(reinterpret_cast<const unsigned short*>(srow + q * 4u));
                        if ((q + 1u) * 2u <= K / 128u)
                            v.x |= (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(srow + q * 4u + 2u)) << 16;
                    }
                }
                return v;
            };
            const uint32_t blocks = (K + kPkCols - 1u) / kPkCols;
            uint4 sc_next = load_scales(0);
            for (uint32_t q = 0; q < blocks && ok; ++q, ++bi) {
                const uint4 sc = sc_next;
                sc_next = load_scales(q + 1u);
                const uint32_t pb = bi % kPkBufs, pph = (bi / kPkBufs) & 1u;
                if (!mbar_wait(&S.pk_full[pb], pph, abort_flag)) { ok = false; break; }
                const uint8_t* pk_row = S.w[pb][which] + arow * 128u;
                const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
                for (uint32_t j = 0; j < kPkCols / kBK; ++j) {
                    const uint32_t ks = q * (kPkCols / kBK) + j;
                    if (ks >= k_stages) break;
                    const uint32_t s = it % kAStages, ph = (it / kAStages) & 1u;
                    const bool mine = (it & 1u) == parity;
                    ++it;
                    if (!mine) continue;   // the other warp of this lane quarter and tile decodes this stage
                    // this thread's packed bytes of the stage: 16-byte chunks 2j and 2j + 1, swizzled by row
                    uint4 pkv[CH];
#pragma unroll
                    for (uint32_t c = 0; c < CH; ++c) {
                        const uint32_t chunk = 2u * j + c;
                        pkv[c] = *reinterpret_cast<const uint4*>(pk_row + ((chunk ^ (arow & 7u)) << 4));
                    }
                    // block multipliers of this thread's 32-column chunks
                    uint32_t m[CH][4];
#pragma unroll
                    for (uint32_t c = 0; c < CH; ++c) {
                        const uint32_t c32 = 2u * j + c;  // 32-column chunk inside the block
                        if (FMT == STRATA_MOE_FMT_MXFP4) {
                            const uint32_t e = (scw[c32 >> 2] >> (8u * (c32 & 3u))) & 0xFFu;
                            const uint32_t h = (uint32_t)((int32_t)e + mx_off) << 10;
                            m[c][0] = m[c][1] = m[c][2] = m[c][3] = h * 0x00010001u;
                        } else if (FMT == STRATA_MOE_FMT_NVFP4) {
                            const uint32_t sb = (scw[c32 >> 1] >> (16u * (c32 & 1u))) & 0xFFFFu;
                            uint32_t pair;
                            asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"((unsigned short)sb));
                            m[c][0] = m[c][1] = __byte_perm(pair, pair, 0x1010);
                            m[c][2] = m[c][3] = __byte_perm(pair, pair, 0x3232);
                        } else {
                            const uint32_t sb = (scw[0] >> (16u * (c32 >> 2))) & 0xFFFFu;
                            const uint32_t h = __half_as_ushort(__float2half_rn(__uint_as_float(sb << 16)));
                            m[c][0] = m[c][1] = m[c][2] = m[c][3] = h * 0x00010001u;
                        }
                    }
                    if (!mbar_wait(&S.empty_a[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();   // the MMAs that read this stage have completed
#pragma unroll
                    for (uint32_t c = 0; c < CH; ++c) {
                        uint4 o[4];
                        decode16<FMT>(pkv[c], m[c], o);
                        const uint32_t v[16] = {o[0].x, o[0].y, o[0].z, o[0].w, o[1].x, o[1].y, o[1].z, o[1].w,
                                                o[2].x, o[2].y, o[2].z, o[2].w, o[3].x, o[3].y, o[3].z, o[3].w};
                        tmem_st16(a_lane_addr + s * kAStageCols + c * 16u, v);
                    }
                    tmem_st_wait();
                    tc_fence_before();   // order the tensor-memory stores before the MMA issuer's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&S.full_a[s]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&S.pk_empty[pb]);  // this warp is done reading the block
            }
        }
        if (!ok) { *abort_flag = 1; atomicOr(a.status, kStatusWaitTimeout); }
    } else {
        // ---------------------------------------------------------------- epilogue
        const uint32_t ew = warp - kFirstEpilogueWarp;
        const uint32_t lane_base = (warp & 3u) * 32u;
        uint32_t tcount = 0;
        bool ok = true, bad = false;
        (void)ew;
        for (uint32_t tile = blockIdx.x; ok; tile += gridDim.x, ++tcount) {
            TileInfo t;
            if (!tile_lookup(a.tile_table, tile, m_tiles, t, kTileFeat)) break;
            if (!mbar_wait(&S.acc_full, tcount & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t feat = t.m0 + lane_base + lane;
            float s0, s1 = 1.0f;
            constexpr bool kNoPost = FMT == STRATA_MOE_FMT_INT4G128 || FMT == kFmtBf16W;
            if (GU) {
                s0 = kNoPost ? 1.0f : a.gate.post_scale[t.g];
                s1 = kNoPost ? 1.0f : a.up.post_scale[t.g];
            } else {
                s0 = s1 = kNoPost ? 1.0f : a.down.post_scale[t.g];
            }
            const uint32_t taddr = tmem_base + (lane_base << 16);
            for (uint32_t c0 = (ew >> 2) * 16u; c0 < t.n; c0 += 16u * (kEpilogueWarps / 4u)) {
                uint32_t g[16], u[16];
                tmem_ld16(taddr + c0, g);
                if (DUAL) tmem_ld16(taddr + kNTile + c0, u);
                tmem_ld_wait();
#pragma unroll
                for (uint32_t j = 0; j < 16u; ++j) {
                    if (c0 + j >= t.n) break;
                    const size_t pos = (size_t)t.row0 + c0 + j;
                    if (GU) {
                        if (a.act_rowscale_out != nullptr && feat == 0u) a.act_rowscale_out[pos] = 1.0f;
                        const float rs = rowscale ? rowscale[pos] : 1.0f;
                        const float gv = __uint_as_float(g[j]) * s0 * rs, uv = __uint_as_float(u[j]) * s1 * rs;
                        float v;
                        if (a.glu.kind == STRATA_MOE_ACT_SWIGLU) {
                            const float e = __expf(-fabsf(gv));
                            const float sig = gv >= 0.0f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
                            v = gv * sig * uv;
                        } else {
                            v = glu_other(gv, uv, a.glu);
                        }
                        if (!(fabsf(v) <= 65504.0f)) bad = true;
                        if (FMT == kFmtBf16W)
                            static_cast<__nv_bfloat16*>(act_out_v)[pos * R + feat] = __float2bfloat16_rn(v);
                        else
                            static_cast<__half*>(act_out_v)[pos * R + feat] = __float2half_rn(v);
                    } else {
                        const float rs = rowscale ? rowscale[pos] : 1.0f;   // pre-scaled activation rows
                        const float v = __uint_as_float(g[j]) * s0 * rs;
                        const float lim = a.y_half ? 65504.0f : 3.0e38f;
                        if (a.y_rowscale_out != nullptr && feat == 0u) a.y_rowscale_out[pos] = 1.0f;
                        if (!(fabsf(v) <= lim)) bad = true;
                        if (a.y_half) reinterpret_cast<__half*>(a.y)[pos * R + feat] = __float2half_rn(v);
                        else a.y[pos * R + feat] = v;
                        if (MODE == 2) {
                            const float v2 = __uint_as_float(u[j]) * s1 * rs;
                            if (!(fabsf(v2) <= lim)) bad = true;
                            if (a.y_half) reinterpret_cast<__half*>(a.y)[pos * R + feat + kMTile] = __float2half_rn(v2);
                            else a.y[pos * R + feat + kMTile] = v2;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&S.acc_empty);
        }
        if (!ok) { *abort_flag = 1; atomicOr(a.status, kStatusWaitTimeout); }
        if (bad) atomicOr(a.status, kStatusNonFiniteOutput);
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------ tile list
// table[0] = number of n-tiles, then (expert, first row, rows) per n-tile, experts ascending.
__global__ void __launch_bounds__(1024) prefill_tiles_kernel(const uint32_t* __restrict__ offsets, uint32_t n_groups,
                                                             uint32_t* __restrict__ table, uint32_t min_rows,
                                                             uint32_t kNTile) {
    __shared__ uint32_t scan[1024];
    const uint32_t tid = threadIdx.x;
    uint32_t cnt = 0, r0 = 0;
    if (tid < n_groups) {
        r0 = offsets[tid];
        cnt = offsets[tid + 1] - r0;
    }
    const uint32_t mine = cnt >= min_rows ? (cnt + kNTile - 1) / kNTile : 0u;   // small groups: weight-streaming path
    scan[tid] = mine;
    __syncthreads();
    for (uint32_t off = 1; off < 1024u; off <<= 1) {
        const uint32_t v = tid >= off ? scan[tid - off] : 0u;
        __syncthreads();
        scan[tid] += v;
        __syncthreads();
    }
    const uint32_t base = scan[tid] - mine;
    for (uint32_t i = 0; i < mine; ++i) {
        table[4 + 3 * (base + i)] = tid;
        table[4 + 3 * (base + i) + 1] = r0 + i * kNTile;
        table[4 + 3 * (base + i) + 2] = min(kNTile, cnt - i * kNTile);
    }
    if (tid == 1023u) table[0] = scan[1023];
}

// ------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 16-bit matrix [rows, cols] row-major; box = 64 columns x box_rows rows, 128-byte swizzle.
static bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {kBK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool prefill_supported(int fmt, uint32_t H, uint32_t I) {
    if (fmt < 0 || fmt > kFmtBf16W) return false;
    return H % 128u == 0 && I % 128u == 0 && encode_fn() != nullptr;
}

size_t prefill_scratch_bytes(uint32_t n_groups, uint32_t pairs) {
    return (4 + 3 * ((size_t)pairs / 128u + n_groups + 1)) * sizeof(uint32_t);   // the smaller tile size bounds it
}

static bool make_bmaps(BMaps* b, const void* base, uint64_t rows, uint64_t cols) {
    for (int i = 0; i < 4; ++i)
        if (!make_map(&b->m[i], base, rows, cols, 16u << i)) return false;
    return true;
}

template <int FMT, int NT>
static int set_smem_attr(size_t smem) {
    // the opt-in to more than 48 KB of dynamic shared memory is a per-device property of the function
    static bool done[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -2;
    if (done[dev]) return 0;
    if (cudaFuncSetAttribute(prefill_ffn_kernel<FMT, 0, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_ffn_kernel<FMT, 1, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_ffn_kernel<FMT, 2, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
        return -2;
    done[dev] = true;
    return 0;
}

// Tensor map over one projection's packed 4-bit rows ([rows, K/2] bytes): 128-byte x 128-row
// boxes, 128-byte swizzle.  `out` receives the 128-byte descriptor (host memory).
int prefill_encode_weight_map(void* out, const void* packed, uint32_t rows, uint32_t K) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return -1;
    const cuuint64_t dims[2] = {K / 2u, rows};
    const cuuint64_t strides[1] = {K / 2u};
    const cuuint32_t box[2] = {kPkCols / 2u, kMTile};
    const cuuint32_t estr[2] = {1, 1};
    static_assert(sizeof(CUtensorMap) == 128, "descriptor size");
    return fn(static_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(packed), dims,
              strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
               ? 0
               : -1;
}

template <int FMT, int NT>
static int launch_fmt(const PrefillArgs& a, const void* x16, const float* x_rowscale, void* act16,
                      uint32_t pairs_cap, const void* wmaps, cudaStream_t s, cudaEvent_t mid) {
    const CUtensorMap* wm = static_cast<const CUtensorMap*>(wmaps);
    BMaps map_x, map_act;
    if (!make_bmaps(&map_x, x16, pairs_cap, a.H) || !make_bmaps(&map_act, act16, pairs_cap, a.I)) return -1;
    const CUtensorMap& dummy = map_x.m[0];
    const size_t smem = sizeof(PrefillSmem<NT>) + 1024;
    if (set_smem_attr<FMT, NT>(smem)) return -2;
    prefill_tiles_kernel<<<1, 1024, 0, s>>>(a.offsets, a.n_groups, a.tile_table, a.min_rows, NT);
    prefill_ffn_kernel<FMT, 0, NT><<<kNumSMs, kThreads, smem, s>>>(map_x, dummy, dummy, a, x_rowscale, act16, wm);
    if (mid) cudaEventRecord(mid, s);
    if (a.H % 256u == 0u)
        prefill_ffn_kernel<FMT, 2, NT><<<kNumSMs, kThreads, smem, s>>>(map_act, dummy, dummy, a, nullptr, nullptr, wm);
    else
        prefill_ffn_kernel<FMT, 1, NT><<<kNumSMs, kThreads, smem, s>>>(map_act, dummy, dummy, a, nullptr, nullptr, wm);
    g_kernel_launches += 3;
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

template <int FMT, int NT>
static int launch_gate_up_fmt(const PrefillArgs& a, const void* x16, const float* x_rowscale, void* act16,
                              uint32_t pairs_cap, const void* wmaps, cudaStream_t s) {
    const CUtensorMap* wm = static_cast<const CUtensorMap*>(wmaps);
    BMaps map_x;
    if (!make_bmaps(&map_x, x16, pairs_cap, a.H)) return -1;
    const CUtensorMap& dummy = map_x.m[0];
    const size_t smem = sizeof(PrefillSmem<NT>) + 1024;
    if (set_smem_attr<FMT, NT>(smem)) return -2;
    prefill_tiles_kernel<<<1, 1024, 0, s>>>(a.offsets, a.n_groups, a.tile_table, a.min_rows, NT);
    prefill_ffn_kernel<FMT, 0, NT><<<kNumSMs, kThreads, smem, s>>>(map_x, dummy, dummy, a, x_rowscale, act16, wm);
    g_kernel_launches += 2;
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int launch_prefill_gate_up(const PrefillArgs& a, const void* x16, const float* x_rowscale, void* act16,
                           uint32_t pairs_cap, const void* wmaps, cudaStream_t s) {
    const bool wide = a.ntile != 128u;
    switch (a.fmt) {
        case STRATA_MOE_FMT_MXFP4:
            return wide ? launch_gate_up_fmt<STRATA_MOE_FMT_MXFP4, 192>(a, x16, x_rowscale, act16, pairs_cap, wmaps, s)
                        : launch_gate_up_fmt<STRATA_MOE_FMT_MXFP4, 128>(a, x16, x_rowscale, act16, pairs_cap, wmaps, s);
        case STRATA_MOE_FMT_NVFP4:
            return wide ? launch_gate_up_fmt<STRATA_MOE_FMT_NVFP4, 192>(a, x16, x_rowscale, act16, pairs_cap, wmaps, s)
                        : launch_gate_up_fmt<STRATA_MOE_FMT_NVFP4, 128>(a, x16, x_rowscale, act16, pairs_cap, wmaps, s);
        default: return -1;
    }
}

// Down projection only, over f16 activation rows that carry a per-row factor (act_rowscale undoes it).
template <int FMT, int NT>
static int launch_down_fmt(const PrefillArgs& a, const void* act16, const float* act_rowscale, uint32_t pairs_cap,
                           const void* wmaps, cudaStream_t s) {
    const CUtensorMap* wm = static_cast<const CUtensorMap*>(wmaps);
    BMaps map_act;
    if (!make_bmaps(&map_act, act16, pairs_cap, a.I)) return -1;
    const CUtensorMap& dummy = map_act.m[0];
    const size_t smem = sizeof(PrefillSmem<NT>) + 1024;
    if (set_smem_attr<FMT, NT>(smem)) return -2;
    if (!a.reuse_tiles) {
        prefill_tiles_kernel<<<1, 1024, 0, s>>>(a.offsets, a.n_groups, a.tile_table, a.min_rows, NT);
        ++g_kernel_launches;
    }
    if (a.H % 256u == 0u)
        prefill_ffn_kernel<FMT, 2, NT><<<kNumSMs, kThreads, smem, s>>>(map_act, dummy, dummy, a, act_rowscale, nullptr, wm);
    else
        prefill_ffn_kernel<FMT, 1, NT><<<kNumSMs, kThreads, smem, s>>>(map_act, dummy, dummy, a, act_rowscale, nullptr, wm);
    ++g_kernel_launches;
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int launch_prefill_down(const PrefillArgs& a, const void* act16, const float* act_rowscale, uint32_t pairs_cap,
                        const void* wmaps, cudaStream_t s) {
    const bool wide = a.ntile != 128u;
    switch (a.fmt) {
        case STRATA_MOE_FMT_MXFP4:
            return wide ? launch_down_fmt<STRATA_MOE_FMT_MXFP4, 192>(a, act16, act_rowscale, pairs_cap, wmaps, s)
                        : launch_down_fmt<STRATA_MOE_FMT_MXFP4, 128>(a, act16, act_rowscale, pairs_cap, wmaps, s);
        case STRATA_MOE_FMT_NVFP4:
            return wide ? launch_down_fmt<STRATA_MOE_FMT_NVFP4, 192>(a, act16, act_rowscale, pairs_cap, wmaps, s)
                        : launch_down_fmt<STRATA_MOE_FMT_NVFP4, 128>(a, act16, act_rowscale, pairs_cap, wmaps, s);
        default: return -1;
    }
}

int launch_prefill(const PrefillArgs& a, const void* x16, const float* x_rowscale, void* act16,
                   uint32_t pairs_cap, const void* wmaps, cudaStream_t s, cudaEvent_t mid) {
    const bool wide = a.ntile != 128u;
#define STRATA_PREFILL_CASE(F)                                                                              \
    case F:                                                                                                 \
        if (a.ntile == 160u) return launch_fmt<F, 160>(a, x16, x_rowscale, act16, pairs_cap, wmaps, s, mid); \
        return wide ? launch_fmt<F, 192>(a, x16, x_rowscale, act16, pairs_cap, wmaps, s, mid)               \
                    : launch_fmt<F, 128>(a, x16, x_rowscale, act16, pairs_cap, wmaps, s, mid);
    switch (a.fmt) {
        STRATA_PREFILL_CASE(STRATA_MOE_FMT_MXFP4)
        STRATA_PREFILL_CASE(STRATA_MOE_FMT_NVFP4)
        STRATA_PREFILL_CASE(STRATA_MOE_FMT_INT4G128)
        default: return -1;
    }
#undef STRATA_PREFILL_CASE
}

// BF16 expert (the shared expert) over `rows` token rows in natural order: x [rows, H] BF16,
// gate/up [I, H], down [H, I] BF16, act [rows_cap, I] BF16 scratch, y [rows, H] fp32.
// a.offsets must hold {0, rows}; a.n_groups = 1.
template <int NT>
static int launch_bf16_nt(const PrefillArgs& a, const void* x, uint32_t rows, const void* w_gate, const void* w_up,
                          const void* w_down, void* act, uint32_t rows_cap, cudaStream_t s) {
    BMaps map_x, map_act;
    CUtensorMap map_g, map_u, map_d;
    if (!make_bmaps(&map_x, x, rows, a.H) || !make_bmaps(&map_act, act, rows_cap, a.I) ||
        !make_map(&map_g, w_gate, a.I, a.H, kMTile) || !make_map(&map_u, w_up, a.I, a.H, kMTile) ||
        !make_map(&map_d, w_down, a.H, a.I, kMTile))
        return -1;
    const size_t smem = sizeof(PrefillSmem<NT>) + 1024;
    if (set_smem_attr<kFmtBf16W, NT>(smem)) return -2;
    prefill_tiles_kernel<<<1, 1024, 0, s>>>(a.offsets, a.n_groups, a.tile_table, a.min_rows, NT);
    prefill_ffn_kernel<kFmtBf16W, 0, NT><<<kNumSMs, kThreads, smem, s>>>(map_x, map_g, map_u, a, nullptr, act, nullptr);
    if (a.H % 256u == 0u)
        prefill_ffn_kernel<kFmtBf16W, 2, NT><<<kNumSMs, kThreads, smem, s>>>(map_act, map_d, map_d, a, nullptr, nullptr,
                                                                         nullptr);
    else
        prefill_ffn_kernel<kFmtBf16W, 1, NT><<<kNumSMs, kThreads, smem, s>>>(map_act, map_d, map_d, a, nullptr, nullptr,
                                                                         nullptr);
    g_kernel_launches += 3;
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Router projection on the tensor cores: logits[t, e] = sum_h x[t, h] * wg[e, h] for BF16 operands,
// FP32 accumulation in tensor memory.  The expert rows play the 128-feature M tiles and the tokens the
// N tiles of the single-GEMM modes (one group holding all T rows), so the output lands as [T, E] fp32.
// The summation order differs from the canonical lane-strided order: these logits feed the fast
// router, which re-derives everything that reaches the caller in the canonical order.
// a.offsets must hold {0, T}.  Needs E % 128 == 0 and H % 64 == 0.
template <int NT>
static int launch_router_tc_nt(PrefillArgs a, const void* x, uint32_t T, const void* wg, uint32_t E, uint32_t H,
                               cudaStream_t s) {
    BMaps map_x;
    CUtensorMap map_w;
    if (!make_bmaps(&map_x, x, T, H) || !make_map(&map_w, wg, E, H, kMTile)) return -1;
    const size_t smem = sizeof(PrefillSmem<NT>) + 1024;
    if (set_smem_attr<kFmtBf16W, NT>(smem)) return -2;
    a.fmt = kFmtBf16W;
    a.H = E;     // features of the single-GEMM modes
    a.I = H;     // their K
    a.n_groups = 1;
    a.pairs = T;
    a.min_rows = 0;
    prefill_tiles_kernel<<<1, 1024, 0, s>>>(a.offsets, 1, a.tile_table, 0, NT);
    // 256 experts per job while that still gives every other SM a job; with few tokens (a rank's share of an
    // expert-parallel step) 128 per job: twice the jobs, each half as long (2048 tokens: 16 jobs otherwise)
    const uint64_t jobs256 = (uint64_t)((T + NT - 1) / NT) * (E / 256u);
    if (E % 256u == 0u && jobs256 * 2u >= (uint64_t)kNumSMs)
        prefill_ffn_kernel<kFmtBf16W, 2, NT><<<kNumSMs, kThreads, smem, s>>>(map_x, map_w, map_w, a, nullptr, nullptr, nullptr);
    else
        prefill_ffn_kernel<kFmtBf16W, 1, NT><<<kNumSMs, kThreads, smem, s>>>(map_x, map_w, map_w, a, nullptr, nullptr, nullptr);
    g_kernel_launches += 2;
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int launch_router_tc(const void* x, uint32_t T, const void* wg, uint32_t E, uint32_t H, float* logits,
                     uint32_t* tile_table, const uint32_t* offsets2, uint32_t* status, cudaStream_t s) {
    if (E % 128u || H % 64u || T == 0u) return -1;
    PrefillArgs a{};
    a.offsets = offsets2;
    a.y = logits;
    a.tile_table = tile_table;
    a.status = status;
    a.glu = GluParams{STRATA_MOE_ACT_SWIGLU, 1.0f, 1.0f};
    // 128-token tiles: more tiles than the 192-token geometry gives, and a tile is short (E features x H)
    return launch_router_tc_nt<128>(a, x, T, wg, E, H, s);
}

int launch_prefill_bf16(const PrefillArgs& a, const void* x, uint32_t rows, const void* w_gate, const void* w_up,
                        const void* w_down, void* act, uint32_t rows_cap, cudaStream_t s) {
    return a.ntile != 128u ? launch_bf16_nt<192>(a, x, rows, w_gate, w_up, w_down, act, rows_cap, s)
                           : launch_bf16_nt<128>(a, x, rows, w_gate, w_up, w_down, act, rows_cap, s);
}

}  // namespace smoe
