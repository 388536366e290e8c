// Device-side numerics shared by the quantize / dequantize kernels.
//
// Every fp32 step uses an explicit round-to-nearest intrinsic so that the
// operation order of the reference (formats.py:390-450,
// backends/triton/quantization.py:77-137) is kept bit for bit; nothing here may
// be contracted into an FMA unless it is written as one.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ue5m3_fp4.h"

namespace ue5m3 {

constexpr float kScaleMax = 61440.0f;     // formats.py:133
constexpr float kInvSix = 0.16666667163372040f;  // fl32(1/6) = 0x3E2AAAAB, formats.py:418-422
constexpr float kFltMax = 3.4028234663852886e38f;

struct TensorScale {
    float enc;   // global encode multiplier      formats.py:399-407
    float dec;   // global decode multiplier      formats.py:408
    float mult;  // enc * fl(1/6)                 formats.py:423
};

// six_t = fl32(6 * T) computed on the host (formats.py:394-398).
__device__ __forceinline__ TensorScale tensor_scale(float amax, float six_t) {
    TensorScale t;
    float raw = __fdiv_rn(six_t, amax);
    t.enc = (amax == 0.0f) ? 1.0f : fminf(raw, kFltMax);
    t.dec = (t.enc == 0.0f) ? 1.0f : __fdiv_rn(1.0f, t.enc);
    t.mult = __fmul_rn(t.enc, kInvSix);
    return t;
}

// UE5M3 ties-to-even encode of v in [0, 61440]  (formats.py:150-205 with
// UE5M3 125-134).  Returns the byte E<<3|M; 0 means the value rounded to zero.
__device__ __forceinline__ uint32_t ue5m3_encode(float v) {
    uint32_t b = __float_as_uint(v);
    if (v >= 6.103515625e-05f) {  // normal range, >= 2^-14
        uint32_t r = b + 0x7FFFFu + ((b >> 20) & 1u);
        uint32_t code = (r >> 20) - (112u << 3);
        return code > 0xF7u ? 0xF7u : code;
    }
    // subnormal range: RNE of v * 2^17 on the integer grid (quantum 2^-17)
    return (uint32_t)__float2int_rn(v * 131072.0f);
}

__device__ __forceinline__ float ue5m3_decode(uint32_t code) {
    if (code >= 8u) return __uint_as_float((code + (112u << 3)) << 20);
    return (float)code * 7.62939453125e-06f;  // M * 2^-17
}

// Block amax -> UE5M3 scale byte with the 0 -> 1.0 rule (formats.py:424-437).
__device__ __forceinline__ uint32_t block_scale_code(float block_amax, const TensorScale& t) {
    float ideal = __fmul_rn(block_amax, t.mult);
    if (block_amax == 0.0f) ideal = 0.0f;
    ideal = fminf(ideal, kScaleMax);
    uint32_t code = ue5m3_encode(ideal);
    return code == 0u ? 0x78u : code;  // 0x78 = 1.0
}

// Reciprocal-then-multiply payload multiplier (formats.py:439-443).
__device__ __forceinline__ float payload_multiplier(float scale, const TensorScale& t) {
    return __frcp_rn(__fmul_rn(scale, t.dec));  // correctly rounded, same bits as 1/d
}

// ---- E2M1 rounding -------------------------------------------------------
// Magnitude index i in {0..7} <-> {0,.5,1,1.5,2,3,4,6}.  All routines take
// a = min(|u|, 6) (anything above 6 rounds to 6 in both modes, formats.py:205).

// ties-to-even, software (formats.py:172-174).
__device__ __forceinline__ uint32_t e2m1_index_tte(float a) {
    uint32_t b = __float_as_uint(a);
    uint32_t hi = ((b + 0x1FFFFFu + ((b >> 22) & 1u)) >> 22) - 0xFCu;
    uint32_t lo = (a > 0.25f ? 1u : 0u) + (a >= 0.75f ? 1u : 0u);
    return b >= 0x3F800000u ? hi : lo;
}

// 8-bit-midpoint stochastic rounding (formats.py:196-200): away from zero iff
// fl(delta + (2r+1)*2^-9) >= 1.  r14 = ((2r+1) << 14) | (4 << 23).
//  * a >= 1: delta = low22/2^22 and the sum is exact, so the rule is the carry
//    of 2*bits + (2r+1)<<14 into bit 23; (2*bits + r14) >> 23 is then
//    0xFC + 4 + index, i.e. the index modulo 8 (the 4 << 23 in r14 supplies the 4).
//  * a <  1: quantum 0.5, significand 2a; z = fl(2a + mid) is the reference's
//    own fp32 add when a < 0.5 (lower = 0) and is exact for a in [0.5, 1);
//    floor(z) is the index, read from the low bits of RZ(z + 2^23).
// Returns a word whose low three bits are the magnitude index.
__device__ __forceinline__ uint32_t e2m1_index_sr(float a, uint32_t r14) {
    uint32_t b = __float_as_uint(a);
    uint32_t hi = (b * 2u + r14) >> 23;
    // bit 25 of r14 is already set in 0x3F800000, so the OR sees only (2r+1) << 14
    float mid = __fadd_rn(__uint_as_float(0x3F800000u | r14), -1.0f);  // (2r+1)*2^-9, exact
    float z = __fmaf_rn(a, 2.0f, mid);
    uint32_t lo = __float_as_uint(__fadd_rz(z, 8388608.0f));
    return b >= 0x3F800000u ? hi : lo;
}

__device__ __forceinline__ float e2m1_magnitude(uint32_t idx) {
    return idx >= 2u ? __uint_as_float((idx + 0xFCu) << 22) : 0.5f * (float)idx;
}

// nibble of the scaled input u: sign of u (signbit convention, formats.py:233-235).
template <bool kStochastic>
__device__ __forceinline__ uint32_t e2m1_nibble(float u, uint32_t r14) {
    float a = fminf(fabsf(u), 6.0f);
    uint32_t idx = kStochastic ? e2m1_index_sr(a, r14) : e2m1_index_tte(a);
    // low three bits from idx, bit 3 from the sign of u (u >> 28 has the sign in bit 3)
    return (idx & 7u) | ((__float_as_uint(u) >> 28) & ~7u);
}

__device__ __forceinline__ float e2m1_value(uint32_t nibble) {
    float m = e2m1_magnitude(nibble & 7u);
    return (nibble & 8u) ? -m : m;
}

// Hardware ties-to-even conversion of 8 floats to 8 packed nibbles (element 0
// in the lowest nibble).  cvt.rn.satfinite.e2m1x2.f32 d, a, b puts a in the
// upper and b in the lower nibble of d.
__device__ __forceinline__ uint32_t e2m1_pack8_hw(const float (&u)[8]) {
    uint32_t out;
    asm volatile(
        "{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
        "mov.b32 %0, {b0, b1, b2, b3};\n"
        "}\n"
        : "=r"(out)
        : "f"(u[0]), "f"(u[1]), "f"(u[2]), "f"(u[3]), "f"(u[4]), "f"(u[5]), "f"(u[6]), "f"(u[7]));
    return out;
}

// Hardware decode of one packed byte (two nibbles) to two floats: lo = low nibble.
__device__ __forceinline__ void e2m1_unpack2_hw(uint32_t byte, float& lo, float& hi) {
    uint32_t h2;
    asm("{\n"
        ".reg .b8 b;\n"
        "cvt.u8.u32 b, %1;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b;\n"
        "}\n"
        : "=r"(h2)
        : "r"(byte));
    __half2 h = *reinterpret_cast<__half2*>(&h2);
    float2 f = __half22float2(h);
    lo = f.x;
    hi = f.y;
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
    return __uint_as_float(bits16 << 16);
}

// fp32 -> bf16 bits, round-to-nearest-even (finite inputs).
__device__ __forceinline__ uint32_t float_to_bf16_bits(float v) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
}

}  // namespace ue5m3
