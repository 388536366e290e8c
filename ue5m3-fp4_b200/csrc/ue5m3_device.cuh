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

// block_scale_code + ue5m3_decode for a CONVERGED warp: the normal range (ideal >= 2^-14) is
// four integer operations whose rounded bits are the decoded scale itself; the subnormal range
// (including the all-zero block -> 1.0 rule) is taken as a warp-uniform branch only when some
// lane needs it.
__device__ __forceinline__ void block_scale_converged(float block_amax, const TensorScale& t,
                                                      uint32_t& code, float& scale) {
    float ideal = fminf(__fmul_rn(block_amax, t.mult), kScaleMax);
    if (block_amax == 0.0f) ideal = 0.0f;
    const uint32_t b = __float_as_uint(ideal);
    const uint32_t r = (b + 0x7FFFFu + ((b >> 20) & 1u)) & 0xFFF00000u;  // RNE to three fraction bits
    code = (r >> 20) - (112u << 3);
    scale = __uint_as_float(r);
    if (__any_sync(0xFFFFFFFFu, ideal < 6.103515625e-05f)) {
        if (ideal < 6.103515625e-05f) {
            code = block_scale_code(block_amax, t);
            scale = ue5m3_decode(code);
        }
    }
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

// ---- stochastic rounding of eight values at once -----------------------------------
// Same rule as e2m1_index_sr, arranged so that the integer pipe does as little as possible
// and nothing is selected per element.  With a = min(|u|, 6) two candidate indices are built:
//  * H, exact for a >= 1: the TOP BYTE of 4*bits(a) + ((2r+1) << 15) + (4 << 24) is the
//    index (2..7, nothing else set).
//  * L = floor(fl(2a + mid)), mid = (2r+1) * 2^-9, exact for a < 2 (for a in [1, 2) the sum is
//    exact and equals the carry rule; for a >= 2 it is >= 4).  Packed fp32 instructions, two
//    elements each; floor() is the low byte of RZ(z + 2^23).
// Four H bytes and four L bytes are gathered into words and the index is, per byte,
// L >= 4 ? H : L.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
    // default mode: a selector nibble with its top bit set replicates the sign bit of the
    // selected byte over the result byte (the __byte_perm intrinsic drops that bit)
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
    return d;
}

// t (top byte = H) and s (low byte = L, upper bytes 0x4B0000) of two elements.  One permute
// per element builds the word 0x4B00rr80, which serves twice: as a float it is
// 2^23 + 128*(2r+1), so mid = word * 2^-16 - 128 in one exact fma; as an integer its multiple
// by 256 is (2r+1) << 15 (the 0x4B falls off the top), the random offset of the a >= 1 path.
__device__ __forceinline__ void e2m1_sr_candidates2(float u0, float u1, uint32_t rword, int k,
                                                    uint32_t& t0, uint32_t& t1, uint32_t& s0,
                                                    uint32_t& s1) {
    const float a0 = fminf(fabsf(u0), 6.0f), a1 = fminf(fabsf(u1), 6.0f);
    // bytes: [0] = 0x80, [1] = r, [2] = 0x00, [3] = 0x4B
    const uint32_t m0 = __byte_perm(rword, 0x4B000080u, 0x7504u | ((uint32_t)k << 4));
    const uint32_t m1 = __byte_perm(rword, 0x4B000080u, 0x7504u | ((uint32_t)(k + 1) << 4));
    t0 = m0 * 256u + (__float_as_uint(a0) * 4u + 0x04000000u);
    t1 = m1 * 256u + (__float_as_uint(a1) * 4u + 0x04000000u);
    asm("{\n"
        ".reg .b64 m, a, z, c8, cm, c2, cb;\n"
        "mov.b64 m, {%2, %3};\n"
        "mov.b64 a, {%4, %5};\n"
        "mov.b64 c8, {%6, %6};\n"
        "mov.b64 cm, {%7, %7};\n"
        "mov.b64 c2, {%8, %8};\n"
        "mov.b64 cb, {%9, %9};\n"
        "fma.rn.f32x2 m, m, c8, cm;\n"   // (2r+1) * 2^-9, exact
        "fma.rn.f32x2 z, a, c2, m;\n"    // fl(2a + mid): the reference's own add where it rounds
        "add.rz.f32x2 z, z, cb;\n"       // 2^23 + floor(z)
        "mov.b64 {%0, %1}, z;\n"
        "}\n"
        : "=r"(s0), "=r"(s1)
        : "r"(m0), "r"(m1), "f"(a0), "f"(a1), "f"(1.52587890625e-05f), "f"(-128.0f), "f"(2.0f),
          "f"(8388608.0f));
}

// top bytes of four words -> one word (w0's in the lowest byte)
__device__ __forceinline__ uint32_t gather_top_bytes(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
    return __byte_perm(__byte_perm(w0, w1, 0x0073u), __byte_perm(w2, w3, 0x0073u), 0x5410u);
}

// low bytes of four words 0x4B0000xx -> one word, by multiply-adds (s0's in the lowest byte)
__device__ __forceinline__ uint32_t gather_low_bytes_of_magic(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t s3) {
    uint32_t acc = s3 * 0x1000000u + 0xB5000000u;  // cancels the 0x4B that s0 leaves in the top byte
    acc = s2 * 0x10000u + acc;
    acc = s1 * 0x100u + acc;
    return acc + s0;
}

// per word 0xFF if its sign bit is set, else 0x00 (w0's in the lowest byte)
__device__ __forceinline__ uint32_t gather_sign_bytes(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
    return prmt(prmt(w0, w1, 0x00FBu), prmt(w2, w3, 0x00FBu), 0x5410u);
}

// per byte: l >= 4 ? h : l   (l <= 12 in every byte)
__device__ __forceinline__ uint32_t select_index_bytes(uint32_t h, uint32_t l) {
    const uint32_t biased = l + 0x7C7C7C7Cu;  // bit 7 of a byte set iff l >= 4
    const uint32_t mask = prmt(biased, biased, 0xBA98u);
    return (h & mask) | (l & ~mask);
}

// Eight scaled inputs -> eight packed nibbles (element 0 lowest), 8-bit-midpoint stochastic
// rounding; r03 / r47 hold the random bytes of elements 0..3 / 4..7.
// `se` / `so`: per byte 0xFF where element 0,2,4,6 / 1,3,5,7 is negative, else 0x00.
__device__ __forceinline__ uint32_t e2m1_pack8_sr_signed(const float (&u)[8], uint32_t r03, uint32_t r47,
                                                         uint32_t se, uint32_t so) {
    uint32_t t[8], s[8];
#pragma unroll
    for (int i = 0; i < 8; i += 2)
        e2m1_sr_candidates2(u[i], u[i + 1], i < 4 ? r03 : r47, i & 3, t[i], t[i + 1], s[i], s[i + 1]);
    const uint32_t even = select_index_bytes(gather_top_bytes(t[0], t[2], t[4], t[6]),
                                             gather_low_bytes_of_magic(s[0], s[2], s[4], s[6]));
    const uint32_t odd = select_index_bytes(gather_top_bytes(t[1], t[3], t[5], t[7]),
                                            gather_low_bytes_of_magic(s[1], s[3], s[5], s[7]));
    const uint32_t magnitude = even + odd * 16u;  // indices <= 7: no carry between nibbles
    return magnitude | (se & 0x08080808u) | (so & 0x80808080u);
}

__device__ __forceinline__ uint32_t e2m1_pack8_sr(const float (&u)[8], uint32_t r03, uint32_t r47) {
    const uint32_t se = gather_sign_bytes(__float_as_uint(u[0]), __float_as_uint(u[2]),
                                          __float_as_uint(u[4]), __float_as_uint(u[6]));
    const uint32_t so = gather_sign_bytes(__float_as_uint(u[1]), __float_as_uint(u[3]),
                                          __float_as_uint(u[5]), __float_as_uint(u[7]));
    return e2m1_pack8_sr_signed(u, r03, r47, se, so);
}

// Sign bytes of eight bf16 elements held in four words (two elements per word, the even one in
// the low half): four sign-replicating permutes.  Valid where the sign of the scaled value is
// the sign of the input (every finite input: the multiplier is positive).
__device__ __forceinline__ void bf16_sign_bytes(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3,
                                                uint32_t& se, uint32_t& so) {
    const uint32_t a = prmt(w0, w1, 0xFBD9u);  // signs of elements 0, 2, 1, 3
    const uint32_t b = prmt(w2, w3, 0xFBD9u);  // signs of elements 4, 6, 5, 7
    se = __byte_perm(a, b, 0x5410u);
    so = __byte_perm(a, b, 0x7632u);
}

// ---- counter-based random bytes (Philox4x32-10) --------------------------------------
// 16 bytes for the 16-element unit `unit` of the stream {seed, stream}: key = seed,
// counter = {unit, stream}.  r[j] holds the bytes of elements 4j..4j+3 (lowest byte first).
__device__ __forceinline__ void philox_unit(uint2 seed, uint2 stream, uint64_t unit, uint32_t (&r)[4]) {
    uint32_t c0 = (uint32_t)unit, c1 = (uint32_t)(unit >> 32), c2 = stream.x, c3 = stream.y;
    uint32_t k0 = seed.x, k1 = seed.y;
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        c0 = hi1 ^ c1 ^ k0;
        c1 = lo1;
        c2 = hi0 ^ c3 ^ k1;
        c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    r[0] = c0; r[1] = c1; r[2] = c2; r[3] = c3;
}

// {seed, stream} as the kernels read them: two uint64 at `bits`
__device__ __forceinline__ void philox_load_key(const void* bits, uint2& seed, uint2& stream) {
    const uint2* p = static_cast<const uint2*>(bits);
    seed = __ldg(p);
    stream = __ldg(p + 1);
}

__device__ __forceinline__ uint32_t philox_byte(const void* bits, int64_t elem) {
    uint2 seed, stream;
    philox_load_key(bits, seed, stream);
    uint32_t r[4];
    philox_unit(seed, stream, (uint64_t)(elem >> 4), r);
    const int i = (int)(elem & 15);
    return (r[i >> 2] >> (8 * (i & 3))) & 0xFFu;
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
    return __uint_as_float(bits16 << 16);
}

// fp32 -> bf16 bits, round-to-nearest-even (finite inputs).
__device__ __forceinline__ uint32_t float_to_bf16_bits(float v) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
}

}  // namespace ue5m3
