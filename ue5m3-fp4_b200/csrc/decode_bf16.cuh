// Packed E2M1 codes x raw UE5M3 block scales -> the exact encoded values as bf16 (a 2-bit by a
// 4-bit significand: the product is exact), in registers.  Shared by the recomputation pass's
// in-kernel producers (gemm_fallback.cu) and its decode-once kernel (fallback_workspace.cu).
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

#include "ue5m3_device.cuh"

namespace ue5m3 {
namespace fb {

// prmt.b32 as the hardware defines it: bit 3 of a selector nibble replicates the selected byte's
// top bit over the result byte (the __byte_perm intrinsic promises the low three bits only).
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
    return d;
}

// A UE5M3 scale byte as a bf16 pair (both halves the same).  A normal byte E<<3|M is the bf16
// (E + 112) << 7 | M << 4; the seven subnormal bytes take the slow way; byte 0 (an all-zero
// block, or padding) gives 0.
__device__ __forceinline__ uint32_t scale_pair(uint32_t scale_byte) {
    uint32_t bits = (scale_byte << 4) + 0x3800u;
    if (scale_byte < 8u) bits = __bfloat16_as_ushort(__float2bfloat16_rn(ue5m3_decode(scale_byte)));
    return __byte_perm(bits, bits, 0x1010);
}

// Eight codes (one 32-bit word) x one scale -> eight bf16 values, in registers only.  A byte
// permute is a four-way lookup in an eight-byte table, which is exactly an E2M1 magnitude (3
// bits) -> one byte of its bf16 encoding: two permutes give the high bytes of eight codes, two
// the low bytes.  The sign bit of a code is bit 3 of its nibble, which a permute's selector reads
// as "replicate the selected byte's top bit": over a table of 0x80 bytes that yields 0xFF for a
// negative code and 0x80 otherwise, and bit 6 of that byte, moved up by one, is the bf16 sign.
// The packed multiply by the scale is exact (a 2-bit by a 4-bit significand).
__device__ __forceinline__ uint4 decode_word(uint32_t word, uint32_t scale2_bits) {
    constexpr uint32_t kHighA = 0x3F3F3F00u, kHighB = 0x40404040u;   // 0 .5 1 1.5 | 2 3 4 6
    constexpr uint32_t kLowA = 0xC0800000u, kLowB = 0xC0804000u;
    const uint32_t mag = word & 0x77777777u;
    const uint32_t word_hi = word >> 16, mag_hi = mag >> 16;
    uint32_t high0 = prmt(kHighA, kHighB, mag), low0 = prmt(kLowA, kLowB, mag);
    uint32_t high1 = prmt(kHighA, kHighB, mag_hi), low1 = prmt(kLowA, kLowB, mag_hi);
    const uint32_t neg0 = prmt(0x80808080u, 0x80808080u, word & 0xFFFFu);
    const uint32_t neg1 = prmt(0x80808080u, 0x80808080u, word_hi);
    high0 |= (neg0 << 1) & 0x80808080u;
    high1 |= (neg1 << 1) & 0x80808080u;
    const uint32_t pairs[4] = {__byte_perm(low0, high0, 0x5140), __byte_perm(low0, high0, 0x7362),
                               __byte_perm(low1, high1, 0x5140), __byte_perm(low1, high1, 0x7362)};
    const __nv_bfloat162 scale2 = *reinterpret_cast<const __nv_bfloat162*>(&scale2_bits);
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 product = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&pairs[i]), scale2);
        out[i] = *reinterpret_cast<const uint32_t*>(&product);
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

}  // namespace fb
}  // namespace ue5m3
