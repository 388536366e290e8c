// Fused single-pass UE5M3/E2M1 block quantizers for sm_100a.
//
// Two kernels:
//  * quantize_row_kernel   1 x B blocks along the contiguous axis.  Pure
//    streaming: one 256-bit load per 16 elements (one thread owns a B=16 block;
//    two lanes share a B=32 block through one shuffle), one 64-bit packed-nibble
//    store per thread, one scale byte per block.  HBM bound.
//  * quantize_tile_kernel  B x 1 blocks along the strided axis and B x B tiles.
//    A 128 x 64 tile is staged in shared memory so that the strided-axis blocks
//    are read without bank conflicts and every global access stays coalesced;
//    outputs can be written transposed (reduction axis contiguous), which is
//    the operand layout the GEMM consumes.
//
// Numerics: ue5m3_device.cuh (restates formats.py:350-457 and
// backends/triton/quantization.py:99-142 of the reference).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "quantize_common.cuh"
#include "window_record.cuh"

namespace ue5m3 {

// ---------------------------------------------------------------------------
// 1 x B blocks along the contiguous axis.  The tensor is viewed as a flat run of
// 16-element units (cols % B == 0, so units and blocks never straddle rows); one
// thread owns one unit per step: a 256-bit load of the values, a 128-bit load of
// the random bytes, one 64-bit store of 16 nibbles and one scale byte.  With
// B = 16 a thread owns the whole block (no shuffle); with B = 32 two lanes share.
// ---------------------------------------------------------------------------
template <typename T, int B, int RMODE, int BITS>
__global__ void __launch_bounds__(256, (RMODE == kRoundSr && sizeof(T) == 4) ? 3 : 4)
quantize_row_kernel(const T* __restrict__ x, int64_t nunits, const float* __restrict__ amax_dev,
                    float six_t, const void* __restrict__ bits, uint2* __restrict__ codes,
                    uint8_t* __restrict__ scales, void* __restrict__ fake, int fake_dtype,
                    int fake_domain) {
    constexpr int kLanesPerBlock = B / 16;
    constexpr int kUnroll = 2;
    const TensorScale ts = tensor_scale(__ldg(amax_dev), six_t);
    const int64_t stride = (int64_t)gridDim.x * (256 * kUnroll);
    for (int64_t base = (int64_t)blockIdx.x * (256 * kUnroll); base < nunits; base += stride) {
        RawUnit<T> raw[kUnroll];
        uint32_t rb[kUnroll][4];
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            int64_t unit = base + k * 256 + threadIdx.x;
            if (unit < nunits) {
                load_raw_unit<T>(x, unit, raw[k]);
                if (RMODE == kRoundSr) load_unit_bits<BITS>(bits, unit, rb[k]);
            } else {
                zero_raw_unit(raw[k]);
#pragma unroll
                for (int i = 0; i < 4; ++i) rb[k][i] = 0u;
            }
        }
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            int64_t unit = base + k * 256 + threadIdx.x;
            float v[16];
            unit_values(raw[k], v);
            float m = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
            if (kLanesPerBlock == 2) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
            uint32_t code;
            float scale;
            block_scale_converged(m, ts, code, scale);
            const float rcp = payload_multiplier(scale, ts);
#pragma unroll
            for (int i = 0; i < 16; i += 2) mul2_rn(v[i], v[i + 1], rcp);
            uint32_t packed[2];
            if (RMODE == kRoundTteHw) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float u[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) u[i] = v[h * 8 + i];
                    packed[h] = e2m1_pack8_hw(u);
                }
            } else if (RMODE == kRoundSr) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float u[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) u[i] = v[h * 8 + i];
                    if (sizeof(T) == 2) {
                        // sign bits straight from the stored bf16 words
                        uint32_t se, so;
                        bf16_sign_bytes(raw[k].w[4 * h], raw[k].w[4 * h + 1], raw[k].w[4 * h + 2],
                                        raw[k].w[4 * h + 3], se, so);
                        packed[h] = e2m1_pack8_sr_signed(u, rb[k][2 * h], rb[k][2 * h + 1], se, so);
                    } else {
                        packed[h] = e2m1_pack8_sr(u, rb[k][2 * h], rb[k][2 * h + 1]);
                    }
                }
            } else {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    packed[h] = 0u;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        packed[h] += e2m1_nibble<false>(v[h * 8 + i], 0u) * (1u << (4 * i));
                }
            }
            if (unit < nunits) {
                if (codes) codes[unit] = make_uint2(packed[0], packed[1]);
                if (scales && (kLanesPerBlock == 1 || (threadIdx.x & 1) == 0))
                    scales[unit / kLanesPerBlock] = (uint8_t)code;
                if (fake) {
                    // hardware nibble decode, then the multiplier chain of the requested domain
                    const float sd = __fmul_rn(scale, ts.dec);
                    const float first = fake_domain == UE5M3_FAKE_DEQUANT ? sd : scale;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float f[8];
#pragma unroll
                        for (int i = 0; i < 8; i += 2) {
                            e2m1_unpack2_hw((packed[h] >> (4 * i)) & 0xFFu, f[i], f[i + 1]);
                            mul2_rn(f[i], f[i + 1], first);
                            if (fake_domain == UE5M3_FAKE_DECODED) mul2_rn(f[i], f[i + 1], ts.dec);
                        }
                        store_fake8(fake, fake_dtype, unit * 16 + h * 8, f);
                    }
                }
            }
        }
    }
}

// Any shape / alignment: one thread per block, scalar accesses, zero padding.
template <typename T>
__global__ void quantize_row_generic_kernel(const T* __restrict__ x, int64_t rows, int64_t cols,
                                            int B, const float* __restrict__ amax_dev, float six_t,
                                            int stochastic, const void* __restrict__ bits,
                                            int bits_dtype, uint8_t* __restrict__ codes,
                                            uint8_t* __restrict__ scales, void* __restrict__ fake,
                                            int fake_dtype, int fake_domain) {
    const TensorScale ts = tensor_scale(__ldg(amax_dev), six_t);
    const int64_t nbc = (cols + B - 1) / B;
    const int64_t code_ld = (cols + 1) / 2;
    for (int64_t blk = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; blk < rows * nbc;
         blk += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = blk / nbc, c0 = (blk % nbc) * B;
        int64_t c1 = c0 + B < cols ? c0 + B : cols;
        float m = 0.0f;
        for (int64_t c = c0; c < c1; ++c) m = fmaxf(m, fabsf(load1<T>(x + r * cols + c)));
        uint32_t code = block_scale_code(m, ts);
        float scale = ue5m3_decode(code);
        float rcp = payload_multiplier(scale, ts);
        float sd = __fmul_rn(scale, ts.dec);
        if (scales) scales[blk] = (uint8_t)code;
        for (int64_t c = c0; c < c1; c += 2) {  // c0 is even (B is even)
            uint32_t byte = 0u;
            for (int h = 0; h < 2 && c + h < c1; ++h) {
                int64_t e = r * cols + c + h;
                uint32_t rb = 0u;
                if (stochastic)
                    rb = bits_dtype == UE5M3_BITS_PHILOX ? philox_byte(bits, e)
                         : bits_dtype == UE5M3_BITS_U8
                             ? static_cast<const uint8_t*>(bits)[e]
                             : (uint32_t)static_cast<const int32_t*>(bits)[e] & 0xFFu;
                float u = __fmul_rn(load1<T>(x + e), rcp);
                uint32_t nib = stochastic ? e2m1_nibble<true>(u, r14_from_byte(rb))
                                          : e2m1_nibble<false>(u, 0u);
                byte |= nib << (4 * h);
                if (fake) {
                    float f = fake_value(nib, scale, sd, ts.dec, fake_domain);
                    if (fake_dtype == UE5M3_DTYPE_BF16)
                        static_cast<__nv_bfloat16*>(fake)[e] = __float2bfloat16_rn(f);
                    else
                        static_cast<float*>(fake)[e] = f;
                }
            }
            if (codes) codes[r * code_ld + c / 2] = (uint8_t)byte;
        }
    }
}

// ---------------------------------------------------------------------------
// B x 1 and B x B blocks: 128 x 64 tile in shared memory.
// ---------------------------------------------------------------------------
constexpr int kTileRows = 128;
constexpr int kTileCols = 64;
constexpr int kTilePitch = kTileCols + 1;     // floats; column reads hit 32 distinct banks
constexpr int kStageTPitch = kTileRows / 2 + 4;  // bytes per column of the transposed code stage

struct TileSmem {
    float tile[kTileRows][kTilePitch];
    uint8_t rbits[kTileRows][kTileCols];
    __align__(16) uint8_t stage_t[kTileCols][kStageTPitch];   // codes_t: [col][row/2]
    __align__(16) uint8_t stage_n[kTileRows][kTileCols / 2];  // codes  : [row][col/2]
    __align__(8) uint8_t scale_t[kTileCols][8];               // COL scales_t: [col][row group]
    __align__(8) uint8_t sf_t[kTileCols][8];                  // UE4M3 bytes per 16 rows of the tile
    __align__(8) uint8_t sf_raw_t[kTileCols][8];              // the same blocks' UE5M3 bytes
};

struct TileArgs {
    const void* x;
    int64_t rows, cols;
    const float* amax_dev;
    float six_t;
    const void* bits;
    uint8_t* codes;     // 2D only
    uint8_t* scales;    // 2D only
    uint8_t* codes_t;
    uint8_t* scales_t;
    void* fake;
    void* fake_t;
    int fake_dtype;
    int fake_domain;
    int vec_ok;  // x (and bits) rows start on 16-byte boundaries
    // transposed operand of the FP4 GEMM: scale atoms [ceil(cols/128)][rows/64][128 words]
    uint32_t* sf_t;
    uint32_t* sf_raw_t;  // same layout, unmodified UE5M3 bytes, may be null
    int shift;
    int* window_record;  // see include/ue5m3_fp4.h
};

template <typename T, int B, bool TWO_D, int RMODE, int BITS>
__global__ void __launch_bounds__(256) quantize_tile_kernel(TileArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    TileSmem& s = *reinterpret_cast<TileSmem*>(smem_raw);
    const T* __restrict__ x = static_cast<const T*>(a.x);
    const int tid = threadIdx.x;
    const int64_t r0 = (int64_t)blockIdx.y * kTileRows;
    const int64_t c0 = (int64_t)blockIdx.x * kTileCols;
    const TensorScale ts = tensor_scale(__ldg(a.amax_dev), a.six_t);
    constexpr bool kSr = RMODE == kRoundSr;

    // ---- phase 1: global -> shared (rows coalesced), zero padding at the edges
#pragma unroll
    for (int pass = 0; pass < kTileRows / 32; ++pass) {
        int lr = pass * 32 + tid / 8;
        int lc = (tid % 8) * 8;
        int64_t gr = r0 + lr, gc = c0 + lc;
        float v[8];
        uint32_t rb[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { v[i] = 0.0f; rb[i] = 0u; }
        if (gr < a.rows) {
            if (a.vec_ok && gc + 8 <= a.cols) {
                load8<T>(x + gr * a.cols + gc, v);
                if (kSr) {
                    uint32_t r14[8];
                    load_bits8<BITS>(a.bits, gr * a.cols + gc, r14);
#pragma unroll
                    for (int i = 0; i < 8; ++i) rb[i] = r14[i] >> 15;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (gc + i < a.cols) {
                        int64_t e = gr * a.cols + gc + i;
                        v[i] = load1<T>(x + e);
                        if (kSr)
                            rb[i] = BITS == UE5M3_BITS_PHILOX ? philox_byte(a.bits, e)
                                    : BITS == UE5M3_BITS_U8
                                        ? static_cast<const uint8_t*>(a.bits)[e]
                                        : (uint32_t)static_cast<const int32_t*>(a.bits)[e] & 0xFFu;
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) s.tile[lr][lc + i] = v[i];
        if (kSr) {
#pragma unroll
            for (int i = 0; i < 8; ++i) s.rbits[lr][lc + i] = (uint8_t)rb[i];
        }
    }
    __syncthreads();

    // ---- phase 2: one (column, row group) item per step; lanes = consecutive columns
    constexpr int kGroups = kTileRows / B;
    constexpr int kItems = kTileCols * kGroups;
    const int64_t nbr = (a.rows + B - 1) / B;  // scale rows
    const int64_t nbc = (a.cols + B - 1) / B;  // scale columns (2D)
    const bool want_fake = a.fake != nullptr || a.fake_t != nullptr;
    int bad_units = 0;
#pragma unroll 1
    for (int item = tid; item < kItems; item += 256) {
        const int c = item % kTileCols;
        const int g = item / kTileCols;
        float v[B];
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < B; ++i) {
            v[i] = s.tile[g * B + i][c];
            m = fmaxf(m, fabsf(v[i]));
        }
        if (TWO_D) {
#pragma unroll
            for (int o = 1; o < B; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        }
        const uint32_t code = block_scale_code(m, ts);
        const float scale = ue5m3_decode(code);
        const float rcp = payload_multiplier(scale, ts);
        const float sd = __fmul_rn(scale, ts.dec);
        if (a.sf_t) {
            bool outside;
            const uint32_t code4 = ue4m3_window_byte(code, (8 + a.shift) << 3, outside);
            if (outside && c0 + c < a.cols && r0 + (int64_t)g * B < a.rows) {
                bad_units += B / 16;
                window_record_row(a.window_record, c0 + c);
            }
#pragma unroll
            for (int h = 0; h < B / 16; ++h) {
                s.sf_t[c][g * (B / 16) + h] = (uint8_t)code4;
                s.sf_raw_t[c][g * (B / 16) + h] = m == 0.0f ? (uint8_t)0 : (uint8_t)code;   // 0 marks an all-zero block
            }
        }
        uint32_t nib[B];
        if (RMODE == kRoundTteHw) {
#pragma unroll
            for (int i = 0; i < B; i += 8) {
                float u[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) u[j] = __fmul_rn(v[i + j], rcp);
                uint32_t w = e2m1_pack8_hw(u);
#pragma unroll
                for (int j = 0; j < 8; ++j) nib[i + j] = (w >> (4 * j)) & 0xFu;
            }
        } else {
#pragma unroll
            for (int i = 0; i < B; ++i) {
                uint32_t r14 = kSr ? r14_from_byte(s.rbits[g * B + i][c]) : 0u;
                nib[i] = e2m1_nibble<kSr>(__fmul_rn(v[i], rcp), r14);
            }
        }
        // transposed packed codes: rows become the contiguous axis
#pragma unroll
        for (int w = 0; w < B / 8; ++w) {
            uint32_t word = 0u;
#pragma unroll
            for (int j = 0; j < 8; ++j) word |= nib[w * 8 + j] << (4 * j);
            *reinterpret_cast<uint32_t*>(&s.stage_t[c][g * (B / 2) + w * 4]) = word;
        }
        if (TWO_D) {
            // natural packed codes: pair with the neighbouring column (lane ^ 1)
#pragma unroll
            for (int i = 0; i < B; ++i) {
                uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, nib[i], 1);
                if ((c & 1) == 0) s.stage_n[g * B + i][c / 2] = (uint8_t)(nib[i] | (other << 4));
            }
            if ((c % B) == 0) {
                int64_t sr = r0 / B + g, sc = (c0 + c) / B;
                if (sr < nbr && sc < nbc) {
                    if (a.scales) a.scales[sr * nbc + sc] = (uint8_t)code;
                    if (a.scales_t) a.scales_t[sc * nbr + sr] = (uint8_t)code;
                }
            }
        } else {
            s.scale_t[c][g] = (uint8_t)code;
        }
        if (want_fake) {
#pragma unroll
            for (int i = 0; i < B; ++i)
                s.tile[g * B + i][c] = fake_value(nib[i], scale, sd, ts.dec, a.fake_domain);
        }
    }
    __syncthreads();

    // ---- phase 3: shared -> global
    const bool full = r0 + kTileRows <= a.rows && c0 + kTileCols <= a.cols;
    const int64_t ld_t = (a.rows + 1) / 2;  // bytes per row of codes_t
    const int64_t ld_n = (a.cols + 1) / 2;  // bytes per row of codes
    if (a.codes_t) {
        if (full && (ld_t % 16) == 0) {
            int c = tid / 4, part = tid % 4;
            const uint32_t* src = reinterpret_cast<const uint32_t*>(&s.stage_t[c][part * 16]);
            uint4 w = make_uint4(src[0], src[1], src[2], src[3]);
            *reinterpret_cast<uint4*>(a.codes_t + (c0 + c) * ld_t + r0 / 2 + part * 16) = w;
        } else {
            for (int i = tid; i < kTileCols * (kTileRows / 2); i += 256) {
                int c = i / (kTileRows / 2), b = i % (kTileRows / 2);
                if (c0 + c < a.cols && r0 + 2 * b < a.rows)
                    a.codes_t[(c0 + c) * ld_t + r0 / 2 + b] = s.stage_t[c][b];
            }
        }
    }
    if (TWO_D && a.codes) {
        if (full && (ld_n % 16) == 0) {
            for (int i = tid; i < kTileRows * 2; i += 256) {
                int r = i / 2, part = i % 2;
                uint4 w = *reinterpret_cast<const uint4*>(&s.stage_n[r][part * 16]);
                *reinterpret_cast<uint4*>(a.codes + (r0 + r) * ld_n + c0 / 2 + part * 16) = w;
            }
        } else {
            for (int i = tid; i < kTileRows * (kTileCols / 2); i += 256) {
                int r = i / (kTileCols / 2), b = i % (kTileCols / 2);
                if (r0 + r < a.rows && c0 + 2 * b < a.cols)
                    a.codes[(r0 + r) * ld_n + c0 / 2 + b] = s.stage_n[r][b];
            }
        }
    }
    if (!TWO_D && a.scales_t) {
        for (int i = tid; i < kTileCols * kGroups; i += 256) {
            int c = i / kGroups, g = i % kGroups;
            int64_t sr = r0 / B + g;
            if (c0 + c < a.cols && sr < nbr) a.scales_t[(c0 + c) * nbr + sr] = s.scale_t[c][g];
        }
    }
    if (a.sf_t) {
        // 64 operand rows (tile columns) x two K atoms (tile rows 0..63, 64..127): one word each
        window_record_units(a.window_record, bad_units);
        const int64_t k_atoms = a.rows / 64;
        if (tid < 2 * kTileCols) {
            const int c = tid >> 1, half = tid & 1;
            const int64_t orow = c0 + c;
            const int64_t ka = r0 / 64 + half;
            if (ka < k_atoms) {
                uint32_t word = *reinterpret_cast<const uint32_t*>(&s.sf_t[c][4 * half]);
                uint32_t raw_word = *reinterpret_cast<const uint32_t*>(&s.sf_raw_t[c][4 * half]);
                if (orow >= a.cols) { word = 0x38383838u; raw_word = 0u; }
                const int64_t at = ((orow >> 7) * k_atoms + ka) * 128 + (orow & 31) * 4 + ((orow >> 5) & 3);
                a.sf_t[at] = word;
                if (a.sf_raw_t) a.sf_raw_t[at] = raw_word;
                // the last column tile also pads the rest of its 128-row atom
                if (c0 + kTileCols >= a.cols && ((c0 + kTileCols) & 127) != 0) {
                    const int64_t prow = orow + kTileCols;
                    const int64_t pat = ((prow >> 7) * k_atoms + ka) * 128 + (prow & 31) * 4 + ((prow >> 5) & 3);
                    a.sf_t[pat] = 0x38383838u;
                    if (a.sf_raw_t) a.sf_raw_t[pat] = 0u;
                }
            }
        }
    }
    if (a.fake) {
        for (int i = tid; i < kTileRows * (kTileCols / 8); i += 256) {
            int r = i / (kTileCols / 8), cc = (i % (kTileCols / 8)) * 8;
            int64_t gr = r0 + r, gc = c0 + cc;
            if (gr >= a.rows) continue;
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = s.tile[r][cc + j];
            if (a.vec_ok && gc + 8 <= a.cols) {
                store_fake8(a.fake, a.fake_dtype, gr * a.cols + gc, f);
            } else {
                for (int j = 0; j < 8 && gc + j < a.cols; ++j) {
                    if (a.fake_dtype == UE5M3_DTYPE_BF16)
                        static_cast<__nv_bfloat16*>(a.fake)[gr * a.cols + gc + j] = __float2bfloat16_rn(f[j]);
                    else
                        static_cast<float*>(a.fake)[gr * a.cols + gc + j] = f[j];
                }
            }
        }
    }
    if (a.fake_t) {
        const bool vec_t = full && (a.rows % 8) == 0;
        for (int i = tid; i < kTileCols * (kTileRows / 8); i += 256) {
            int c = i / (kTileRows / 8), rr = (i % (kTileRows / 8)) * 8;
            int64_t gc = c0 + c, gr = r0 + rr;
            if (gc >= a.cols) continue;
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = s.tile[rr + j][c];
            if (vec_t) {
                store_fake8(a.fake_t, a.fake_dtype, gc * a.rows + gr, f);
            } else {
                for (int j = 0; j < 8 && gr + j < a.rows; ++j) {
                    if (a.fake_dtype == UE5M3_DTYPE_BF16)
                        static_cast<__nv_bfloat16*>(a.fake_t)[gc * a.rows + gr + j] = __float2bfloat16_rn(f[j]);
                    else
                        static_cast<float*>(a.fake_t)[gc * a.rows + gr + j] = f[j];
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// packed -> values
// ---------------------------------------------------------------------------
__global__ void dequantize_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                  int64_t rows, int64_t cols, int B, int two_d,
                                  const float* __restrict__ amax_dev, float six_t,
                                  void* __restrict__ out, int out_dtype) {
    const TensorScale ts = tensor_scale(__ldg(amax_dev), six_t);
    const int64_t ld = (cols + 1) / 2;
    const int64_t nbc = (cols + B - 1) / B;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * ld;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / ld, c = (i % ld) * 2;
        uint32_t byte = codes[i];
        int64_t sr = two_d ? r / B : r;
        float sd = __fmul_rn(ue5m3_decode(scales[sr * nbc + c / B]), ts.dec);
        for (int h = 0; h < 2 && c + h < cols; ++h) {
            float f = __fmul_rn(e2m1_value((byte >> (4 * h)) & 0xFu), sd);
            if (out_dtype == UE5M3_DTYPE_BF16)
                static_cast<__nv_bfloat16*>(out)[r * cols + c + h] = __float2bfloat16_rn(f);
            else
                static_cast<float*>(out)[r * cols + c + h] = f;
        }
    }
}

__global__ void philox_bytes_kernel(const void* __restrict__ key, int64_t count, uint8_t* __restrict__ out) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (int64_t)gridDim.x * blockDim.x)
        out[e] = (uint8_t)philox_byte(key, e);
}

__global__ void alpha_kernel(const float* amax_a, const float* amax_b, float inv_denominator,
                             float* out) {
    out[0] = __fmul_rn(__fmul_rn(amax_a[0], amax_b[0]), inv_denominator);
}

__global__ void e2m1_cvt_test_kernel(uint32_t first, uint64_t count,
                                     unsigned long long* mismatches, uint32_t* first_bad) {
    for (uint64_t i = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < count;
         i += (uint64_t)gridDim.x * blockDim.x * 8) {
        float u[8];
        uint32_t bitsv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            bitsv[j] = first + (uint32_t)(i + j);
            u[j] = __uint_as_float(bitsv[j]);
        }
        uint32_t hw = e2m1_pack8_hw(u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (i + j >= count) break;
            if ((bitsv[j] & 0x7FFFFFFFu) > 0x7F800000u) continue;  // NaN
            uint32_t sw = e2m1_nibble<false>(u[j], 0u);
            if (sw != ((hw >> (4 * j)) & 0xFu)) {
                atomicAdd(mismatches, 1ull);
                atomicMin(first_bad, bitsv[j]);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// host dispatch
// ---------------------------------------------------------------------------
static int g_use_hw_cvt = -1;

bool use_hw_cvt() {
    if (g_use_hw_cvt < 0) {
        const char* e = getenv("UE5M3_E2M1_HW_CVT");
        g_use_hw_cvt = (e && e[0] == '0') ? 0 : 1;
    }
    return g_use_hw_cvt != 0;
}

template <typename T, int B, int RMODE, int BITS>
static void launch_row(const void* x, int64_t nunits, const float* amax_dev, float six_t,
                       const void* bits, uint8_t* codes, uint8_t* scales, void* fake,
                       int fake_dtype, int fake_domain, cudaStream_t stream) {
    int64_t want = (nunits + 511) / 512;
    int grid = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
    quantize_row_kernel<T, B, RMODE, BITS><<<grid, 256, 0, stream>>>(
        static_cast<const T*>(x), nunits, amax_dev, six_t, bits,
        reinterpret_cast<uint2*>(codes), scales, fake, fake_dtype, fake_domain);
}

template <typename T, int B>
static void dispatch_row(int rmode, int bits_dtype, const void* x, int64_t nchunks,
                         const float* amax_dev, float six_t, const void* bits, uint8_t* codes,
                         uint8_t* scales, void* fake, int fake_dtype, int fake_domain,
                         cudaStream_t stream) {
#define UE5M3_ROW(R, BT) \
    launch_row<T, B, R, BT>(x, nchunks, amax_dev, six_t, bits, codes, scales, fake, fake_dtype, fake_domain, stream)
    if (rmode == kRoundSr) {
        if (bits_dtype == UE5M3_BITS_U8) UE5M3_ROW(kRoundSr, UE5M3_BITS_U8);
        else if (bits_dtype == UE5M3_BITS_PHILOX) UE5M3_ROW(kRoundSr, UE5M3_BITS_PHILOX);
        else UE5M3_ROW(kRoundSr, UE5M3_BITS_I32);
    } else if (rmode == kRoundTteHw) {
        UE5M3_ROW(kRoundTteHw, UE5M3_BITS_U8);
    } else {
        UE5M3_ROW(kRoundTteSw, UE5M3_BITS_U8);
    }
#undef UE5M3_ROW
}

template <typename T, int B, bool TWO_D>
static int dispatch_tile(int rmode, int bits_dtype, const TileArgs& args, cudaStream_t stream) {
    dim3 grid((unsigned)((args.cols + kTileCols - 1) / kTileCols),
              (unsigned)((args.rows + kTileRows - 1) / kTileRows));
    if (grid.y > 65535u) return UE5M3_ERR_TOO_LARGE;
    size_t smem = sizeof(TileSmem);
#define UE5M3_TILE(R, BT)                                                                         \
    do {                                                                                          \
        auto kernel = quantize_tile_kernel<T, B, TWO_D, R, BT>;                                   \
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
        kernel<<<grid, 256, smem, stream>>>(args);                                                \
    } while (0)
    if (rmode == kRoundSr) {
        if (bits_dtype == UE5M3_BITS_U8) UE5M3_TILE(kRoundSr, UE5M3_BITS_U8);
        else if (bits_dtype == UE5M3_BITS_PHILOX) UE5M3_TILE(kRoundSr, UE5M3_BITS_PHILOX);
        else UE5M3_TILE(kRoundSr, UE5M3_BITS_I32);
    } else if (rmode == kRoundTteHw) {
        UE5M3_TILE(kRoundTteHw, UE5M3_BITS_U8);
    } else {
        UE5M3_TILE(kRoundTteSw, UE5M3_BITS_U8);
    }
#undef UE5M3_TILE
    return UE5M3_OK;
}

}  // namespace ue5m3

using namespace ue5m3;

namespace ue5m3 {
int quantize_operand_t_fast(const void* x, int dtype, int64_t rows, int64_t cols, int block, int blocking,
                            const float* amax_dev, float target, int rounding, const void* bits, int bits_dtype,
                            int shift, uint8_t* codes_t, uint8_t* sf_t, uint8_t* sf_raw_t, int* window_record,
                            bool rht, cudaStream_t stream);
}

static int quantize_dispatch(const void* x, int dtype, int64_t rows, int64_t cols, int block,
                             int blocking, const float* amax_dev, float target, int rounding,
                             const void* bits, int bits_dtype, uint8_t* codes, uint8_t* scales,
                             uint8_t* codes_t, uint8_t* scales_t, void* fake, void* fake_t,
                             int fake_dtype, int fake_domain, uint32_t* sf_t, uint32_t* sf_raw_t, int shift,
                             int* window_record, void* stream_v) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (!x || !amax_dev || rows <= 0 || cols <= 0) return UE5M3_ERR_INVALID_ARGUMENT;
    if (dtype != UE5M3_DTYPE_BF16 && dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (block != 16 && block != 32) return UE5M3_ERR_BLOCK_SIZE;
    if (!(target > 0.0f) || !(target < 3.0e38f)) return UE5M3_ERR_INVALID_ARGUMENT;
    if (blocking < UE5M3_BLOCK_ROW || blocking > UE5M3_BLOCK_2D) return UE5M3_ERR_INVALID_ARGUMENT;
    const bool sr = rounding == UE5M3_ROUND_STOCHASTIC_FAST;
    if (!sr && rounding != UE5M3_ROUND_TIES_TO_EVEN) return UE5M3_ERR_INVALID_ARGUMENT;
    if (sr && (!bits || (bits_dtype != UE5M3_BITS_U8 && bits_dtype != UE5M3_BITS_I32 &&
                         bits_dtype != UE5M3_BITS_PHILOX)))
        return UE5M3_ERR_INVALID_ARGUMENT;
    if (sr && bits_dtype == UE5M3_BITS_PHILOX && ((uintptr_t)bits % 8)) return UE5M3_ERR_ALIGNMENT;
    if (!sr && bits) return UE5M3_ERR_INVALID_ARGUMENT;
    if ((fake || fake_t) && (fake_domain < UE5M3_FAKE_ENCODED || fake_domain > UE5M3_FAKE_DEQUANT ||
                             (fake_dtype != UE5M3_DTYPE_BF16 && fake_dtype != UE5M3_DTYPE_FP32)))
        return UE5M3_ERR_INVALID_ARGUMENT;
    if (blocking == UE5M3_BLOCK_ROW && (codes_t || scales_t || fake_t)) return UE5M3_ERR_UNSUPPORTED;
    if (blocking == UE5M3_BLOCK_COL && (codes || scales)) return UE5M3_ERR_UNSUPPORTED;

    const float six_t = (float)((double)target * 6.0);
    const int rmode = sr ? kRoundSr : (use_hw_cvt() ? kRoundTteHw : kRoundTteSw);
    const size_t esize = dtype == UE5M3_DTYPE_BF16 ? 2 : 4;
    const bool x_vec = ((uintptr_t)x % 16) == 0 && (cols * esize) % 16 == 0;
    const bool bits_vec = !sr || (bits_dtype == UE5M3_BITS_PHILOX ? cols % 8 == 0 : bits_dtype == UE5M3_BITS_U8 ? ((uintptr_t)bits % 8) == 0 && cols % 8 == 0
                                                              : ((uintptr_t)bits % 16) == 0 && cols % 4 == 0);
    const size_t fsize = fake_dtype == UE5M3_DTYPE_BF16 ? 2 : 4;

    if (blocking == UE5M3_BLOCK_ROW) {
        const bool fake_vec = !fake || (((uintptr_t)fake % 16) == 0 && (cols * fsize) % 16 == 0);
        const bool bits32 = !sr || bits_dtype == UE5M3_BITS_PHILOX || (bits_dtype == UE5M3_BITS_U8 ? ((uintptr_t)bits % 16) == 0
                                                                : ((uintptr_t)bits % 32) == 0);
        const bool fast = cols % block == 0 && x_vec && bits_vec && fake_vec && bits32 &&
                          ((uintptr_t)x % 32) == 0 && (!codes || ((uintptr_t)codes % 8) == 0);
        if (fast) {
            int64_t nchunks = rows * cols / 16;
#define UE5M3_DR(T, B) \
    dispatch_row<T, B>(rmode, bits_dtype, x, nchunks, amax_dev, six_t, bits, codes, scales, fake, fake_dtype, fake_domain, stream)
            if (dtype == UE5M3_DTYPE_BF16) { if (block == 16) UE5M3_DR(__nv_bfloat16, 16); else UE5M3_DR(__nv_bfloat16, 32); }
            else { if (block == 16) UE5M3_DR(float, 16); else UE5M3_DR(float, 32); }
#undef UE5M3_DR
        } else {
            int64_t nblocks = rows * ((cols + block - 1) / block);
            int64_t want = (nblocks + 127) / 128;
            int grid = (int)(want < (int64_t)sm_count() * 16 ? want : (int64_t)sm_count() * 16);
            if (dtype == UE5M3_DTYPE_BF16)
                quantize_row_generic_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
                    static_cast<const __nv_bfloat16*>(x), rows, cols, block, amax_dev, six_t, sr, bits,
                    bits_dtype, codes, scales, fake, fake_dtype, fake_domain);
            else
                quantize_row_generic_kernel<float><<<grid, 128, 0, stream>>>(
                    static_cast<const float*>(x), rows, cols, block, amax_dev, six_t, sr, bits,
                    bits_dtype, codes, scales, fake, fake_dtype, fake_domain);
        }
        return check_launch();
    }

    TileArgs args;
    args.x = x; args.rows = rows; args.cols = cols; args.amax_dev = amax_dev; args.six_t = six_t;
    args.bits = bits; args.codes = codes; args.scales = scales; args.codes_t = codes_t;
    args.scales_t = scales_t; args.fake = fake; args.fake_t = fake_t; args.fake_dtype = fake_dtype;
    args.fake_domain = fake_domain;
    args.sf_t = sf_t; args.sf_raw_t = sf_raw_t; args.shift = shift; args.window_record = window_record;
    const bool fake_vec = !fake || (((uintptr_t)fake % 16) == 0 && (cols * fsize) % 16 == 0);
    const bool fake_t_ok = !fake_t || ((uintptr_t)fake_t % 16) == 0;
    if (!fake_t_ok) return UE5M3_ERR_ALIGNMENT;
    if (codes_t && ((uintptr_t)codes_t % 16) != 0) return UE5M3_ERR_ALIGNMENT;
    if (codes && ((uintptr_t)codes % 16) != 0) return UE5M3_ERR_ALIGNMENT;
    args.vec_ok = x_vec && bits_vec && fake_vec;
    int status;
    const bool two_d = blocking == UE5M3_BLOCK_2D;
#define UE5M3_DT(T, B) \
    (two_d ? dispatch_tile<T, B, true>(rmode, bits_dtype, args, stream) : dispatch_tile<T, B, false>(rmode, bits_dtype, args, stream))
    if (dtype == UE5M3_DTYPE_BF16) status = block == 16 ? UE5M3_DT(__nv_bfloat16, 16) : UE5M3_DT(__nv_bfloat16, 32);
    else status = block == 16 ? UE5M3_DT(float, 16) : UE5M3_DT(float, 32);
#undef UE5M3_DT
    if (status != UE5M3_OK) return status;
    return check_launch();
}

extern "C" int ue5m3_quantize(const void* x, int dtype, int64_t rows, int64_t cols, int block,
                              int blocking, const float* amax_dev, float target, int rounding,
                              const void* bits, int bits_dtype, uint8_t* codes, uint8_t* scales,
                              uint8_t* codes_t, uint8_t* scales_t, void* fake, void* fake_t,
                              int fake_dtype, int fake_domain, void* stream_v) {
    return quantize_dispatch(x, dtype, rows, cols, block, blocking, amax_dev, target, rounding, bits,
                             bits_dtype, codes, scales, codes_t, scales_t, fake, fake_t, fake_dtype,
                             fake_domain, nullptr, nullptr, 0, nullptr, stream_v);
}

extern "C" int ue5m3_quantize_fp4_operand_t(const void* x, int dtype, int64_t rows, int64_t cols,
                                            int block, int blocking, const float* amax_dev,
                                            float target, int rounding, const void* bits,
                                            int bits_dtype, int shift, uint8_t* codes_t, uint8_t* sf_t,
                                            uint8_t* sf_raw_t, int* window_record, void* stream_v) {
    if (!codes_t || !sf_t || !window_record || shift < -8 || shift > 16) return UE5M3_ERR_INVALID_ARGUMENT;
    if (blocking != UE5M3_BLOCK_COL && blocking != UE5M3_BLOCK_2D) return UE5M3_ERR_UNSUPPORTED;
    if (rows % 64) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if (((uintptr_t)sf_t % 16) || ((uintptr_t)sf_raw_t % 16)) return UE5M3_ERR_ALIGNMENT;
    if (!x || !amax_dev || rows <= 0 || cols <= 0) return UE5M3_ERR_INVALID_ARGUMENT;
    if (dtype != UE5M3_DTYPE_BF16 && dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (block != 16 && block != 32) return UE5M3_ERR_BLOCK_SIZE;
    if (!(target > 0.0f) || !(target < 3.0e38f)) return UE5M3_ERR_INVALID_ARGUMENT;
    const bool sr = rounding == UE5M3_ROUND_STOCHASTIC_FAST;
    if (!sr && rounding != UE5M3_ROUND_TIES_TO_EVEN) return UE5M3_ERR_INVALID_ARGUMENT;
    if (sr && (!bits || (bits_dtype != UE5M3_BITS_U8 && bits_dtype != UE5M3_BITS_I32 &&
                         bits_dtype != UE5M3_BITS_PHILOX)))
        return UE5M3_ERR_INVALID_ARGUMENT;
    if (!sr && bits) return UE5M3_ERR_INVALID_ARGUMENT;
    const char* general = getenv("UE5M3_TRANSPOSE_KERNEL");
    if (!(general && general[0] == '0')) {
        int fast = quantize_operand_t_fast(x, dtype, rows, cols, block, blocking, amax_dev, target, rounding, bits,
                                           bits_dtype, shift, codes_t, sf_t, sf_raw_t, window_record, false,
                                           static_cast<cudaStream_t>(stream_v));
        if (fast != UE5M3_ERR_UNSUPPORTED) return fast;
    }
    return quantize_dispatch(x, dtype, rows, cols, block, blocking, amax_dev, target, rounding, bits,
                             bits_dtype, nullptr, nullptr, codes_t, nullptr, nullptr, nullptr,
                             UE5M3_DTYPE_BF16, UE5M3_FAKE_NONE, reinterpret_cast<uint32_t*>(sf_t),
                             reinterpret_cast<uint32_t*>(sf_raw_t), shift, window_record, stream_v);
}

extern "C" int ue5m3_dequantize(const uint8_t* codes, const uint8_t* scales, int64_t rows,
                                int64_t cols, int block, int two_d, const float* amax_dev,
                                float target, void* out, int out_dtype, void* stream_v) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (!codes || !scales || !amax_dev || !out || rows <= 0 || cols <= 0) return UE5M3_ERR_INVALID_ARGUMENT;
    if (block != 16 && block != 32) return UE5M3_ERR_BLOCK_SIZE;
    if (out_dtype != UE5M3_DTYPE_BF16 && out_dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    const float six_t = (float)((double)target * 6.0);
    int64_t n = rows * ((cols + 1) / 2);
    int64_t want = (n + 255) / 256;
    int grid = (int)(want < (int64_t)sm_count() * 16 ? want : (int64_t)sm_count() * 16);
    dequantize_kernel<<<grid, 256, 0, stream>>>(codes, scales, rows, cols, block, two_d ? 1 : 0,
                                                amax_dev, six_t, out, out_dtype);
    return check_launch();
}

extern "C" int ue5m3_philox_bytes(const void* seed_stream_dev, int64_t count, uint8_t* out, void* stream_v) {
    if (!seed_stream_dev || !out || count <= 0 || ((uintptr_t)seed_stream_dev % 8)) return UE5M3_ERR_INVALID_ARGUMENT;
    int64_t want = (count + 255) / 256;
    int grid = (int)(want < (int64_t)sm_count() * 16 ? want : (int64_t)sm_count() * 16);
    philox_bytes_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_v)>>>(seed_stream_dev, count, out);
    return check_launch();
}

extern "C" int ue5m3_alpha(const float* amax_a, const float* amax_b, float inv_denominator,
                           float* alpha_out, void* stream_v) {
    if (!amax_a || !amax_b || !alpha_out) return UE5M3_ERR_INVALID_ARGUMENT;
    alpha_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream_v)>>>(amax_a, amax_b, inv_denominator, alpha_out);
    return check_launch();
}

extern "C" int ue5m3_test_e2m1_cvt(uint32_t first_bits, uint64_t count,
                                   unsigned long long* mismatch_count_dev,
                                   uint32_t* first_mismatch_dev, void* stream_v) {
    if (!mismatch_count_dev || !first_mismatch_dev) return UE5M3_ERR_INVALID_ARGUMENT;
    e2m1_cvt_test_kernel<<<sm_count() * 8, 256, 0, static_cast<cudaStream_t>(stream_v)>>>(
        first_bits, count, mismatch_count_dev, first_mismatch_dev);
    return check_launch();
}
