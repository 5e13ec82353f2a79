// Exact 4-bit -> BF16 decoders shared by the expert kernels and the dequant export.
//
// E2M1 (FP4) trick: a nibble s|e1|e0|m placed at bf16 bits 15 | 8 | 7 | 6 is the bf16
// number e2m1(nibble) * 2^-126 (exponent bias 127 against E2M1's bias 1; the E2M1
// subnormal 0.5 lands on the bf16 subnormal 2^-127).  One packed multiply by a power of
// two (or by the block scale times a power of two) then yields the exact dequantised
// value: every product has at most 6 significant bits, so BF16 holds it exactly.
// A nibble times 0x1040 replicates it at bit offsets 6 and 12, so one AND, one IMAD and
// one AND place both nibbles of a 16-bit-strided pair at once.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace smoe {

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Word of 8 E2M1 nibbles (nibble q = column 8w+q) -> r[j] = {low half: nibble j, high half:
// nibble j+4}, each half = e2m1 * 2^-126 as bf16 bits.
__device__ __forceinline__ void e2m1x8_raw(uint32_t w, uint32_t r[4]) {
    const uint32_t w8 = w >> 8;
    r[0] = ((w & 0x000F000Fu) * 0x1040u) & 0x81C081C0u;
    r[1] = ((w & 0x00F000F0u) * 0x0104u) & 0x81C081C0u;
    r[2] = ((w8 & 0x000F000Fu) * 0x1040u) & 0x81C081C0u;
    r[3] = ((w8 & 0x00F000F0u) * 0x0104u) & 0x81C081C0u;
}

// Word of 8 offset-binary INT4 nibbles -> r[j] = {nibble j - 8, nibble j+4 - 8} as exact bf16.
// 0x4300 | q is the bf16 number 128 + q (the mantissa step at 2^7 is 1); minus 136 is q - 8.
__device__ __forceinline__ void int4x8_bf16(uint32_t w, uint32_t r[4]) {
    const uint32_t k136 = 0x43084308u;  // bf16 136.0 twice
    r[0] = sub_bf16x2((w & 0x000F000Fu) | 0x43004300u, k136);
    r[1] = sub_bf16x2(((w >> 4) & 0x000F000Fu) | 0x43004300u, k136);
    r[2] = sub_bf16x2(((w >> 8) & 0x000F000Fu) | 0x43004300u, k136);
    r[3] = sub_bf16x2(((w >> 12) & 0x000F000Fu) | 0x43004300u, k136);
}

// MXFP4 block multiplier.  E8M0 byte e means 2^(e-127); the raw nibble form carries 2^-126,
// so the multiplier is 2^(e-1): bf16 exponent field e + 126.  That field exists only for
// e <= 128; larger scales (block scale >= 4, never seen in checkpoints but legal) take a
// second multiply.  0xFF (reserved, NaN in the reference's device decode) yields NaN.
struct Mx4Mult {
    uint32_t m1, m2;  // packed bf16x2 multipliers; m2 == 0 means "single multiply"
};
__device__ __forceinline__ Mx4Mult mxfp4_mult(uint32_t e) {
    Mx4Mult r;
    if (e <= 128u) {
        const uint32_t m = (e + 126u) << 7;
        r.m1 = m | (m << 16);
        r.m2 = 0u;
    } else {
        r.m1 = 0x7E807E80u;  // 2^126
        const uint32_t m = (e == 0xFFu) ? 0x7FC0u : (e << 7);
        r.m2 = m | (m << 16);
    }
    return r;
}
__device__ __forceinline__ uint32_t apply_mx4(uint32_t raw, const Mx4Mult& m) {
    uint32_t v = mul_bf16x2(raw, m.m1);
    if (m.m2) v = mul_bf16x2(v, m.m2);
    return v;
}

// NVFP4 block multiplier: E4M3 block scale times 2^117 as bf16, so that
// raw * mult = e2m1 * e4m3 * 2^-9 exactly (the 2^9 and the per-tensor divisor are applied
// to the fp32 accumulator).  Normal positive scales are a shift and an add; subnormal or
// negative ones go through the general conversion.
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
    const uint32_t e = (b >> 3) & 0xFu, m = b & 7u;
    float v;
    if (e == 0u) v = ldexpf((float)m * 0.125f, -6);
    else if (e == 0xFu && m == 7u) v = __int_as_float(0x7FC00000);
    else v = ldexpf(1.0f + (float)m * 0.125f, (int)e - 7);
    return (b & 0x80u) ? -v : v;
}
__device__ __forceinline__ uint32_t nvfp4_mult(uint32_t b) {
    uint32_t m;
    if ((b & 0x80u) == 0u && (b & 0x78u) != 0u && b != 0x7Fu) {
        m = ((b & 0x7Fu) << 4) + 0x7680u;
    } else {
        const float v = e4m3_to_f32(b);
        m = (v == v) ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(ldexpf(v, 117))) : 0x7FC0u;
    }
    return m | (m << 16);
}
constexpr float kNvfp4AccScale = 512.0f;  // 2^9 taken out of the block multiplier

// Scalar decoders for the export kernel (same bit construction, one element).
__device__ __forceinline__ float e2m1_raw_to_f32(uint32_t bf16_bits) {
    return __uint_as_float(bf16_bits << 16);
}

}  // namespace smoe
