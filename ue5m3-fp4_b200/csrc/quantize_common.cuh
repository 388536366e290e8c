// Load / store / random-bit helpers shared by the block quantizer kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "abi_common.cuh"
#include "ue5m3_device.cuh"

namespace ue5m3 {

enum : int { kRoundTteHw = 0, kRoundTteSw = 1, kRoundSr = 2 };

// (2r + 1) << 14 plus the 4 << 23 bias that e2m1_index_sr expects
__device__ __forceinline__ uint32_t r14_from_byte(uint32_t r) { return (r << 15) | 0x02004000u; }

// Load 8 consecutive elements as fp32.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);

template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 w = __ldg(reinterpret_cast<const uint4*>(p));
    v[0] = __uint_as_float(w.x << 16); v[1] = __uint_as_float(w.x & 0xFFFF0000u);
    v[2] = __uint_as_float(w.y << 16); v[3] = __uint_as_float(w.y & 0xFFFF0000u);
    v[4] = __uint_as_float(w.z << 16); v[5] = __uint_as_float(w.z & 0xFFFF0000u);
    v[6] = __uint_as_float(w.w << 16); v[7] = __uint_as_float(w.w & 0xFFFF0000u);
}

template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
    float4 a = __ldg(reinterpret_cast<const float4*>(p));
    float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

template <typename T>
__device__ __forceinline__ float load1(const T* p);
template <>
__device__ __forceinline__ float load1<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat162float(*p);
}
template <>
__device__ __forceinline__ float load1<float>(const float* p) { return *p; }

// 8 random bytes -> 8 r14 words.
template <int BITS>
__device__ __forceinline__ void load_bits8(const void* bits, int64_t elem, uint32_t (&r14)[8]) {
    if (BITS == UE5M3_BITS_PHILOX) {
        uint2 seed, stream;
        philox_load_key(bits, seed, stream);
        uint32_t r[4];
        philox_unit(seed, stream, (uint64_t)(elem >> 4), r);  // elem is a multiple of 8
        const uint32_t lo = (elem & 8) ? r[2] : r[0], hi = (elem & 8) ? r[3] : r[1];
        r14[0] = r14_from_byte(lo & 0xFFu);         r14[1] = r14_from_byte((lo >> 8) & 0xFFu);
        r14[2] = r14_from_byte((lo >> 16) & 0xFFu); r14[3] = r14_from_byte(lo >> 24);
        r14[4] = r14_from_byte(hi & 0xFFu);         r14[5] = r14_from_byte((hi >> 8) & 0xFFu);
        r14[6] = r14_from_byte((hi >> 16) & 0xFFu); r14[7] = r14_from_byte(hi >> 24);
    } else if (BITS == UE5M3_BITS_U8) {
        uint2 w = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(bits) + elem));
        r14[0] = r14_from_byte(w.x & 0xFFu);         r14[1] = r14_from_byte((w.x >> 8) & 0xFFu);
        r14[2] = r14_from_byte((w.x >> 16) & 0xFFu); r14[3] = r14_from_byte(w.x >> 24);
        r14[4] = r14_from_byte(w.y & 0xFFu);         r14[5] = r14_from_byte((w.y >> 8) & 0xFFu);
        r14[6] = r14_from_byte((w.y >> 16) & 0xFFu); r14[7] = r14_from_byte(w.y >> 24);
    } else {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const int32_t*>(bits) + elem);
        uint4 a = __ldg(p), b = __ldg(p + 1);
        r14[0] = r14_from_byte(a.x & 0xFFu); r14[1] = r14_from_byte(a.y & 0xFFu);
        r14[2] = r14_from_byte(a.z & 0xFFu); r14[3] = r14_from_byte(a.w & 0xFFu);
        r14[4] = r14_from_byte(b.x & 0xFFu); r14[5] = r14_from_byte(b.y & 0xFFu);
        r14[6] = r14_from_byte(b.z & 0xFFu); r14[7] = r14_from_byte(b.w & 0xFFu);
    }
}

__device__ __forceinline__ float fake_value(uint32_t nibble, float scale, float scale_dec,
                                            float dec, int domain) {
    float p = e2m1_value(nibble);
    if (domain == UE5M3_FAKE_DEQUANT) return __fmul_rn(p, scale_dec);
    float e = __fmul_rn(p, scale);
    return domain == UE5M3_FAKE_DECODED ? __fmul_rn(e, dec) : e;
}

__device__ __forceinline__ void store_fake8(void* fake, int fake_dtype, int64_t elem,
                                            const float (&f)[8]) {
    if (fake_dtype == UE5M3_DTYPE_BF16) {
        uint4 w;
        w.x = float_to_bf16_bits(f[0]) | (float_to_bf16_bits(f[1]) << 16);
        w.y = float_to_bf16_bits(f[2]) | (float_to_bf16_bits(f[3]) << 16);
        w.z = float_to_bf16_bits(f[4]) | (float_to_bf16_bits(f[5]) << 16);
        w.w = float_to_bf16_bits(f[6]) | (float_to_bf16_bits(f[7]) << 16);
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(fake) + elem) = w;
    } else {
        float4* p = reinterpret_cast<float4*>(static_cast<float*>(fake) + elem);
        p[0] = make_float4(f[0], f[1], f[2], f[3]);
        p[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
}

__device__ __forceinline__ void ldg256(const void* p, uint32_t (&r)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                   "=r"(r[7])
                 : "l"(p));
}

// (a, b) * (s, s) with one packed fp32 instruction, round-to-nearest
__device__ __forceinline__ void mul2_rn(float& a, float& b, float s) {
    asm("{\n"
        ".reg .b64 x, y;\n"
        "mov.b64 x, {%0, %1};\n"
        "mov.b64 y, {%2, %2};\n"
        "mul.rn.f32x2 x, x, y;\n"
        "mov.b64 {%0, %1}, x;\n"
        "}\n"
        : "+f"(a), "+f"(b)
        : "f"(s));
}

template <typename T>
__device__ __forceinline__ void load_unit(const T* x, int64_t unit, float (&v)[16]);

template <>
__device__ __forceinline__ void load_unit<__nv_bfloat16>(const __nv_bfloat16* x, int64_t unit, float (&v)[16]) {
    uint32_t w[8];
    ldg256(x + unit * 16, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}

template <>
__device__ __forceinline__ void load_unit<float>(const float* x, int64_t unit, float (&v)[16]) {
    uint32_t w[8];
    ldg256(x + unit * 16, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(w[i]);
    ldg256(x + unit * 16 + 8, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[8 + i] = __uint_as_float(w[i]);
}

// A 16-element unit as it sits in memory (bf16: 8 words, fp32: 16 words); kept raw until the
// unit is processed so that only one unit's fp32 values are live at a time.
template <typename T>
struct RawUnit {
    uint32_t w[sizeof(T) * 4];
};

template <typename T>
__device__ __forceinline__ void load_raw_unit(const T* x, int64_t unit, RawUnit<T>& r);

template <>
__device__ __forceinline__ void load_raw_unit<__nv_bfloat16>(const __nv_bfloat16* x, int64_t unit,
                                                             RawUnit<__nv_bfloat16>& r) {
    ldg256(x + unit * 16, r.w);
}

template <>
__device__ __forceinline__ void load_raw_unit<float>(const float* x, int64_t unit, RawUnit<float>& r) {
    uint32_t a[8], b[8];
    ldg256(x + unit * 16, a);
    ldg256(x + unit * 16 + 8, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) { r.w[i] = a[i]; r.w[8 + i] = b[i]; }
}

__device__ __forceinline__ void unit_values(const RawUnit<__nv_bfloat16>& r, float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[2 * i] = __uint_as_float(r.w[i] << 16);
        v[2 * i + 1] = __uint_as_float(r.w[i] & 0xFFFF0000u);
    }
}

__device__ __forceinline__ void unit_values(const RawUnit<float>& r, float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r.w[i]);
}

template <typename T>
__device__ __forceinline__ void zero_raw_unit(RawUnit<T>& r) {
#pragma unroll
    for (int i = 0; i < (int)(sizeof(T) * 4); ++i) r.w[i] = 0u;
}

// 16 random bytes of one unit, packed four per word
template <int BITS>
__device__ __forceinline__ void load_unit_bits(const void* bits, int64_t unit, uint32_t (&r)[4]) {
    if (BITS == UE5M3_BITS_PHILOX) {
        uint2 seed, stream;
        philox_load_key(bits, seed, stream);
        philox_unit(seed, stream, (uint64_t)unit, r);
    } else if (BITS == UE5M3_BITS_U8) {
        uint4 w = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(bits) + unit * 16));
        r[0] = w.x; r[1] = w.y; r[2] = w.z; r[3] = w.w;
    } else {
        const int32_t* p = static_cast<const int32_t*>(bits) + unit * 16;
        uint32_t w[8];
        ldg256(p, w);
        r[0] = (w[0] & 0xFFu) | ((w[1] & 0xFFu) << 8) | ((w[2] & 0xFFu) << 16) | (w[3] << 24);
        r[1] = (w[4] & 0xFFu) | ((w[5] & 0xFFu) << 8) | ((w[6] & 0xFFu) << 16) | (w[7] << 24);
        ldg256(p + 8, w);
        r[2] = (w[0] & 0xFFu) | ((w[1] & 0xFFu) << 8) | ((w[2] & 0xFFu) << 16) | (w[3] << 24);
        r[3] = (w[4] & 0xFFu) | ((w[5] & 0xFFu) << 8) | ((w[6] & 0xFFu) << 16) | (w[7] << 24);
    }
}

// r14 = (2r + 1) << 14 of byte k of a packed word
__device__ __forceinline__ uint32_t r14_of(uint32_t word, int k) {
    uint32_t shifted = k == 0 ? (word << 15) : k == 1 ? (word << 7) : k == 2 ? (word >> 1) : (word >> 9);
    return (shifted & 0x7F8000u) | 0x02004000u;
}

// Software-rule TTE is used only when the hardware conversion is disabled by
// UE5M3_E2M1_HW_CVT=0 in the environment.
bool use_hw_cvt();

}  // namespace ue5m3
