// Quantizer that writes a GEMM operand of the FP4 tensor-core path in one pass: packed E2M1
// codes (K-major) and the block scales already re-biased to UE4M3 and laid out in the 512-byte
// atoms the block-scaled MMA reads (see gemm_fp4_sm100.cu).  Blocks are 1 x B along K or
// B x B tiles; K is the contiguous axis of the input (no transpose).
//
// Work decomposition: one warp per (32 rows x 64 K-elements) piece, lane = row.  A lane owns
// 128 contiguous input bytes (bf16), 32 bytes of codes and one 32-bit word of an atom, so no
// shared memory and no block-level synchronisation is needed; a B x B block's amax is a
// butterfly over the B lanes that hold its rows.  The eight warps of a CTA take neighbouring
// K pieces of the same rows, which keeps DRAM pages open.
//
// Numerics: ue5m3_device.cuh (formats.py:350-457 of the reference).  The UE4M3 re-bias has no
// counterpart in the reference; it is exact inside the window and flagged outside.
#include "quantize_common.cuh"
#include "window_record.cuh"

namespace ue5m3 {

struct OperandArgs {
    const void* x;
    int64_t rows, cols;
    const float* amax_dev;
    float six_t;
    const void* bits;
    uint8_t* codes;     // [rows, cols / 2]
    uint32_t* sf;       // [ceil(rows / 128)][cols / 64][128] words, may be null
    uint32_t* sf_raw;   // same layout, unmodified UE5M3 bytes, may be null
    uint8_t* scales;    // raw UE5M3 bytes ([rows, cols/B] or [ceil(rows/B), cols/B]), may be null
    int shift;
    int* window_record; // see include/ue5m3_fp4.h
};

// U = 16-element units per lane and task: 4 (one whole atom row, 128 input bytes per lane) or
// 2 (half of it: fewer live registers, more resident warps).
template <typename T, int B, bool TWO_D, int RMODE, int BITS, int U>
__global__ void __launch_bounds__(256, RMODE == kRoundTteHw ? 4 : ((RMODE == kRoundSr && sizeof(T) == 2) ? 3 : 2))
quantize_operand_kernel(const OperandArgs a) {
    static_assert(U == 2 || U == 4, "units per task");
    constexpr bool kSr = RMODE == kRoundSr;
    const T* __restrict__ x = static_cast<const T*>(a.x);
    const TensorScale ts = tensor_scale(__ldg(a.amax_dev), a.six_t);
    const int lane = threadIdx.x & 31;
    const int64_t k_atoms = a.cols / 64;
    const int64_t k_tasks = a.cols / (16 * U);
    const int64_t row_groups = ((a.rows + 127) / 128) * 4;  // 32-row groups, padded to whole atoms
    const int64_t ntasks = row_groups * k_tasks;
    const int64_t nbc = a.cols / B;
    const int rebias = (8 + a.shift) << 3;
    int bad_units = 0;

    for (int64_t task = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); task < ntasks;
         task += (int64_t)gridDim.x * 8) {
        const int64_t rg = task / k_tasks, kt = task % k_tasks;
        const int64_t row = rg * 32 + lane;
        const bool valid = row < a.rows;
        const int64_t col0 = kt * (16 * U);
        const int64_t unit0 = (row * a.cols + col0) / 16;  // first 16-element unit of this lane

        RawUnit<T> raw[U];
        uint32_t rb[U][4];
        if (valid) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                load_raw_unit<T>(x, unit0 + u, raw[u]);
                if (kSr) load_unit_bits<BITS>(a.bits, unit0 + u, rb[u]);
            }
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                zero_raw_unit<T>(raw[u]);
#pragma unroll
                for (int i = 0; i < 4; ++i) rb[u][i] = 0u;
            }
        }

        float m[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float v[16];
            unit_values(raw[u], v);
            m[u] = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) m[u] = fmaxf(m[u], fabsf(v[i]));
        }
        if (B == 32) {
#pragma unroll
            for (int u = 0; u < U; u += 2) m[u] = m[u + 1] = fmaxf(m[u], m[u + 1]);
        }
        if (TWO_D) {
#pragma unroll
            for (int o = 1; o < B; o <<= 1) {
#pragma unroll
                for (int u = 0; u < U; u += B / 16)
                    m[u] = fmaxf(m[u], __shfl_xor_sync(0xFFFFFFFFu, m[u], o));
            }
            if (B == 32) {
#pragma unroll
                for (int u = 0; u < U; u += 2) m[u + 1] = m[u];
            }
        }

        uint32_t code[U];
        uint32_t sf_bytes = 0u, raw_bytes = 0u;
        uint32_t packed[U][2];
        float scale = 1.0f;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (B == 32 && (u & 1)) {
                code[u] = code[u - 1];  // same 32-wide block as the previous unit: same scale
            } else {
                block_scale_converged(m[u], ts, code[u], scale);
            }
            bool outside;
            sf_bytes |= ue4m3_window_byte(code[u], rebias, outside) << (8 * u);
            raw_bytes |= (m[u] == 0.0f ? 0u : code[u]) << (8 * u);   // 0 marks an all-zero block
            if (outside && valid && a.sf) {
                ++bad_units;
                window_record_row_cold(a.window_record, row);
            }
            const float rcp = payload_multiplier(scale, ts);
            float v[16];
            unit_values(raw[u], v);
#pragma unroll
            for (int i = 0; i < 16; i += 2) mul2_rn(v[i], v[i + 1], rcp);
            if (RMODE == kRoundTteHw) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float w[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) w[i] = v[h * 8 + i];
                    packed[u][h] = e2m1_pack8_hw(w);
                }
            } else if (kSr) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float w[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) w[i] = v[h * 8 + i];
                    if (sizeof(T) == 2) {
                        // sign bits straight from the stored bf16 words
                        uint32_t se, so;
                        bf16_sign_bytes(raw[u].w[4 * h], raw[u].w[4 * h + 1], raw[u].w[4 * h + 2],
                                        raw[u].w[4 * h + 3], se, so);
                        packed[u][h] = e2m1_pack8_sr_signed(w, rb[u][2 * h], rb[u][2 * h + 1], se, so);
                    } else {
                        packed[u][h] = e2m1_pack8_sr(w, rb[u][2 * h], rb[u][2 * h + 1]);
                    }
                }
            } else {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    packed[u][h] = 0u;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        packed[u][h] += e2m1_nibble<false>(v[h * 8 + i], 0u) * (1u << (4 * i));
                }
            }
        }

        if (valid) {
            uint4* dst = reinterpret_cast<uint4*>(a.codes + row * (a.cols / 2) + col0 / 2);
#pragma unroll
            for (int u = 0; u < U; u += 2)
                dst[u / 2] = make_uint4(packed[u][0], packed[u][1], packed[u + 1][0], packed[u + 1][1]);
            if (a.scales && (!TWO_D || (row % B) == 0)) {
                uint8_t* sp = a.scales + (TWO_D ? row / B : row) * nbc + col0 / B;
                if (B == 16) {
                    if (U == 4)
                        *reinterpret_cast<uint32_t*>(sp) = code[0] | (code[1] << 8) | (code[2] << 16) | (code[U - 1] << 24);
                    else
                        *reinterpret_cast<uint16_t*>(sp) = (uint16_t)(code[0] | (code[1] << 8));
                } else {
                    if (U == 4)
                        *reinterpret_cast<uint16_t*>(sp) = (uint16_t)(code[0] | (code[2] << 8));
                    else
                        *sp = (uint8_t)code[0];
                }
            }
        }
        if (a.sf) {
            const int64_t tile = rg >> 2;
            const int r1 = (int)(rg & 3);
            const int64_t ka = col0 / 64;
            uint32_t* word = a.sf + (tile * k_atoms + ka) * 128 + lane * 4 + r1;
            uint32_t* raw_word = a.sf_raw ? a.sf_raw + (word - a.sf) : nullptr;
            if (U == 4) {
                *word = valid ? sf_bytes : 0x38383838u;
                if (raw_word) *raw_word = valid ? raw_bytes : 0u;
            } else {
                const int half_index = (int)((col0 % 64) / 32);
                reinterpret_cast<uint16_t*>(word)[half_index] = valid ? (uint16_t)sf_bytes : (uint16_t)0x3838u;
                if (raw_word)
                    reinterpret_cast<uint16_t*>(raw_word)[half_index] = valid ? (uint16_t)raw_bytes : (uint16_t)0u;
            }
        }
    }
    if (a.sf) window_record_units(a.window_record, bad_units);
}

template <typename T, int B, bool TWO_D>
static void dispatch_operand(int rmode, int bits_dtype, const OperandArgs& args, cudaStream_t stream) {
    // ties-to-even fits 64 registers with two units per task (four resident CTAs per SM) and is
    // then faster; stochastic rounding is fastest with four units and three resident CTAs
    // (80 registers; measured against two units at 64 registers and four at 122)
    const int units = rmode == kRoundSr ? 4 : 2;
    const int64_t ntasks = ((args.rows + 127) / 128) * 4 * (args.cols / (16 * units));
    const int64_t want = (ntasks + 7) / 8;
    const int64_t cap = (int64_t)sm_count() * 8;
    const int grid = (int)(want < cap ? want : cap);
#define UE5M3_OP(R, BT)                                                                            \
    do {                                                                                           \
        if (units == 2) quantize_operand_kernel<T, B, TWO_D, R, BT, 2><<<grid, 256, 0, stream>>>(args); \
        else quantize_operand_kernel<T, B, TWO_D, R, BT, 4><<<grid, 256, 0, stream>>>(args);       \
    } while (0)
    if (rmode == kRoundSr) {
        if (bits_dtype == UE5M3_BITS_U8) UE5M3_OP(kRoundSr, UE5M3_BITS_U8);
        else if (bits_dtype == UE5M3_BITS_PHILOX) UE5M3_OP(kRoundSr, UE5M3_BITS_PHILOX);
        else UE5M3_OP(kRoundSr, UE5M3_BITS_I32);
    } else if (rmode == kRoundTteHw) {
        UE5M3_OP(kRoundTteHw, UE5M3_BITS_U8);
    } else {
        UE5M3_OP(kRoundTteSw, UE5M3_BITS_U8);
    }
#undef UE5M3_OP
}


// ---------------------------------------------------------------------------------------
// The operand x^T (reduction over the ROWS of x, blocks B x 1 or B x B): a 128 x 128 tile of x
// goes through shared memory in its storage type (bf16 pairs stay packed), then every lane
// owns two neighbouring columns and walks down 32 rows, so the per-element work is that of the
// streaming kernel: no per-element shared-memory staging of results, the codes of a column
// (32 rows = 16 bytes) and its two scale bytes leave in one store each.
// Warp w: columns (w & 1) * 64 + 2 * lane + {0, 1}, rows (w >> 1) * 32 .. + 31.
// ---------------------------------------------------------------------------------------
constexpr int kTT = 128;                        // tile extent in rows and in columns
constexpr int kTBitsPitch = kTT + 16;           // bytes per row of the random-byte tile

template <typename T>
struct TransposeTile {
    static constexpr int kWordsPerRow = kTT * (int)sizeof(T) / 4;
    static constexpr int kPitch = kWordsPerRow + 4;  // words; rows stay 16-byte aligned
};

struct OperandTArgs {
    const void* x;
    int64_t rows, cols;   // of x; the operand is [cols, rows]
    const float* amax_dev;
    float six_t;
    const void* bits;
    uint8_t* codes_t;     // [cols, rows / 2]
    uint8_t* sf_t;        // atoms of the [cols, rows] operand
    uint8_t* sf_raw_t;    // same layout, unmodified UE5M3 bytes, may be null
    int shift;
    int* window_record;   // see include/ue5m3_fp4.h
    unsigned int* transformed_amax;  // amax-only mode: max |transformed value| as fp32 bits
    // BOTH mode (2-D blocks, ties-to-even): the operand x itself as well, from the same tile
    uint8_t* codes;       // [rows, cols / 2]
    uint8_t* sf;          // atoms of the [rows, cols] operand
    uint8_t* sf_raw;
    int* window_record_rows;
};

// The fixed-sign, normalized B=16 Hadamard transform of the TE-settings comparator
// (nn/linear.py:23-40,80-114 of the reference) on the 16 consecutive reduction-axis values of
// one column: y_k = bf16( sum_i bf16(v_i * sign_i) * H[i][k] / 4 ).  The reference runs it as a
// BF16 matmul (exact products, FP32 accumulation, one rounding to BF16); here the sum is a
// fast Walsh-Hadamard butterfly in FP32, which is exact unless the 16 values span more than
// about 12 binades.
__device__ __forceinline__ void rht16(float (&v)[16]) {
    constexpr int kNegative = 0xD7E8;  // bit i set: sign_i = -1  (signs 1,1,1,-1,1,-1,-1,-1,-1,-1,-1,1,-1,1,-1,-1)
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float x = __bfloat162float(__float2bfloat16_rn(v[i]));
        v[i] = ((kNegative >> i) & 1) ? -x : x;
    }
#pragma unroll
    for (int len = 1; len < 16; len <<= 1) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if ((i & len) == 0) {
                const float a = v[i], b = v[i + len];
                v[i] = __fadd_rn(a, b);
                v[i + len] = __fadd_rn(a, -b);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(v[i], 0.25f)));
}

// two columns x 16 rows from the tile -> values (bf16: one word holds both columns)
__device__ __forceinline__ void tile_pair_values(const uint32_t* tile, int pitch, int row0, int word, __nv_bfloat16,
                                                 float (&c0)[16], float (&c1)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t w = tile[(row0 + i) * pitch + word];
        c0[i] = __uint_as_float(w << 16);
        c1[i] = __uint_as_float(w & 0xFFFF0000u);
    }
}

__device__ __forceinline__ void tile_pair_values(const uint32_t* tile, int pitch, int row0, int word, float,
                                                 float (&c0)[16], float (&c1)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint2 w = *reinterpret_cast<const uint2*>(&tile[(row0 + i) * pitch + 2 * word]);
        c0[i] = __uint_as_float(w.x);
        c1[i] = __uint_as_float(w.y);
    }
}

template <typename T, int B, bool TWO_D, int RMODE, int BITS, bool RHT, bool AMAX_ONLY, bool BOTH = false>
__global__ void __launch_bounds__(
    256, (RMODE == kRoundTteHw && !BOTH) ? 4
                                         : (((RMODE == kRoundSr && sizeof(T) == 2 && B == 16 && !TWO_D && !RHT) || (BOTH && sizeof(T) == 2)) ? 3 : 2))
quantize_operand_t_kernel(const OperandTArgs a) {
    static_assert(!RHT || (B == 16 && !TWO_D), "the transform is defined on 16 x 1 blocks");
    static_assert(!BOTH || (TWO_D && !RHT && !AMAX_ONLY && RMODE != kRoundSr),
                  "both orientations share scales only for B x B blocks; weights round ties-to-even");
    // BOTH: scale code (and 0 for an all-zero block) of every B x B block of the tile, for phase 3
    __shared__ uint8_t block_code[kTT / 16][kTT / 16], block_raw[kTT / 16][kTT / 16];
    constexpr bool kSr = RMODE == kRoundSr;
    constexpr int kPitch = TransposeTile<T>::kPitch;
    constexpr int kChunksPerRow = TransposeTile<T>::kWordsPerRow / 4;  // 16-byte chunks
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t* tile = reinterpret_cast<uint32_t*>(smem_raw);
    uint8_t* rbits = smem_raw + (size_t)kTT * kPitch * 4;

    const T* __restrict__ x = static_cast<const T*>(a.x);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t r0 = (int64_t)blockIdx.y * kTT, c0 = (int64_t)blockIdx.x * kTT;
    const TensorScale ts = tensor_scale(AMAX_ONLY ? 1.0f : __ldg(a.amax_dev), a.six_t);
    constexpr int kElemsPerChunk = 16 / (int)sizeof(T);

    // ---- phase 1: global -> shared, rows coalesced, zero padding outside the tensor
#pragma unroll 4
    for (int idx = tid; idx < kTT * kChunksPerRow; idx += 256) {
        const int row = idx / kChunksPerRow, chunk = idx % kChunksPerRow;
        const int64_t gr = r0 + row, gc = c0 + (int64_t)chunk * kElemsPerChunk;
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        if (gr < a.rows && gc < a.cols) w = __ldg(reinterpret_cast<const uint4*>(x + gr * a.cols + gc));
        *reinterpret_cast<uint4*>(&tile[row * kPitch + chunk * 4]) = w;
    }
    if (kSr) {
        for (int idx = tid; idx < kTT * (kTT / 16); idx += 256) {
            const int row = idx / (kTT / 16), unit = idx % (kTT / 16);
            const int64_t gr = r0 + row, gc = c0 + unit * 16;
            uint4 w = make_uint4(0u, 0u, 0u, 0u);
            if (gr < a.rows && gc < a.cols) {
                const int64_t elem = gr * a.cols + gc;  // a multiple of 16
                if (BITS == UE5M3_BITS_PHILOX) {
                    uint2 seed, stream;
                    philox_load_key(a.bits, seed, stream);
                    uint32_t r[4];
                    philox_unit(seed, stream, (uint64_t)(elem >> 4), r);
                    w = make_uint4(r[0], r[1], r[2], r[3]);
                } else {
                    w = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(a.bits) + elem));
                }
            }
            *reinterpret_cast<uint4*>(&rbits[row * kTBitsPitch + unit * 16]) = w;
        }
    }
    __syncthreads();

    // ---- phase 2: lane = two columns, 32 rows
    const int ch = warp & 1, rq = warp >> 1;
    const int word = ch * 32 + lane;             // column pair index inside the tile
    const int row_base = rq * 32;
    const int64_t col = c0 + 2 * word;           // first of the two columns
    const int64_t krow = r0 + row_base;          // first reduction index of this warp
    const bool rows_valid = krow < a.rows;       // rows % 64 == 0: a 32-row quarter is in or out

    // 16 x 1 blocks need nothing from outside their own 16 rows: their amax is taken in the main
    // loop below, from the values that are loaded there anyway
    constexpr bool kAmaxInLoop = B == 16 && !TWO_D && !AMAX_ONLY;
    float m[2][2];
    if (!kAmaxInLoop) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float u0[16], u1[16];
            tile_pair_values(tile, kPitch, row_base + 16 * h, word, T(), u0, u1);
            if (RHT) { rht16(u0); rht16(u1); }
            m[h][0] = m[h][1] = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                m[h][0] = fmaxf(m[h][0], fabsf(u0[i]));
                m[h][1] = fmaxf(m[h][1], fabsf(u1[i]));
            }
        }
    }
    if (AMAX_ONLY) {
        float v = fmaxf(fmaxf(m[0][0], m[0][1]), fmaxf(m[1][0], m[1][1]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
        if (lane == 0) atomicMax(a.transformed_amax, __float_as_uint(v));  // v >= 0: bit order = value order
        return;
    }
    if (B == 32) {
#pragma unroll
        for (int j = 0; j < 2; ++j) m[0][j] = m[1][j] = fmaxf(m[0][j], m[1][j]);
    }
    if (TWO_D) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float v = fmaxf(m[h][0], m[h][1]);
#pragma unroll
            for (int o = 1; o < B / 2; o <<= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
            m[h][0] = m[h][1] = v;
        }
    }

    const int rebias = (8 + a.shift) << 3;
    int bad_units = 0;
    uint32_t packed[2][4];   // [column][32 rows = 4 words]
    uint32_t sf_pair[2] = {0u, 0u}, raw_pair[2] = {0u, 0u};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float u[2][16];
        tile_pair_values(tile, kPitch, row_base + 16 * h, word, T(), u[0], u[1]);
        if (RHT) { rht16(u[0]); rht16(u[1]); }
        if (kAmaxInLoop) {
            m[h][0] = m[h][1] = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                m[h][0] = fmaxf(m[h][0], fabsf(u[0][i]));
                m[h][1] = fmaxf(m[h][1], fabsf(u[1][i]));
            }
        }
        uint32_t rw[2][4];   // random bytes of the 16 rows, per column
        uint32_t sign_even[2][2], sign_odd[2][2];  // [column][half]: sign bytes of rows 0,2,4,6 / 1,3,5,7
        constexpr bool kRawSigns = kSr && sizeof(T) == 2 && !RHT;
        if (kRawSigns) {
            // both columns' sign bits sit in the stored words (bits 15 and 31)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t wr[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) wr[i] = tile[(row_base + 16 * h + 8 * half + i) * kPitch + word];
                const uint32_t e02 = prmt(wr[0], wr[2], 0xFBD9u), e46 = prmt(wr[4], wr[6], 0xFBD9u);
                const uint32_t o13 = prmt(wr[1], wr[3], 0xFBD9u), o57 = prmt(wr[5], wr[7], 0xFBD9u);
                sign_even[0][half] = __byte_perm(e02, e46, 0x5410u);
                sign_even[1][half] = __byte_perm(e02, e46, 0x7632u);
                sign_odd[0][half] = __byte_perm(o13, o57, 0x5410u);
                sign_odd[1][half] = __byte_perm(o13, o57, 0x7632u);
            }
        }
        if (kSr) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t hw[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    hw[i] = *reinterpret_cast<const uint16_t*>(&rbits[(row_base + 16 * h + 4 * q + i) * kTBitsPitch + 2 * word]);
                const uint32_t p01 = hw[0] | (hw[1] << 16), p23 = hw[2] | (hw[3] << 16);
                rw[0][q] = __byte_perm(p01, p23, 0x6420u);
                rw[1][q] = __byte_perm(p01, p23, 0x7531u);
            }
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            uint32_t code;
            float scale;
            block_scale_converged(m[h][j], ts, code, scale);
            if (BOTH && j == 0 && (lane % (B / 2)) == 0 && (B == 16 || h == 0)) {
                const int rb = (row_base + 16 * h) / B, cb = (ch * 64 + 2 * lane) / B;
                block_code[rb][cb] = (uint8_t)code;
                block_raw[rb][cb] = m[h][j] == 0.0f ? (uint8_t)0 : (uint8_t)code;
            }
            bool outside;
            sf_pair[j] |= ue4m3_window_byte(code, rebias, outside) << (8 * h);
            raw_pair[j] |= (m[h][j] == 0.0f ? 0u : code) << (8 * h);   // 0 marks an all-zero block
            if (outside && rows_valid && col + j < a.cols) {
                ++bad_units;
                window_record_row_cold(a.window_record, col + j);
            }
            const float rcp = payload_multiplier(scale, ts);
#pragma unroll
            for (int i = 0; i < 16; i += 2) mul2_rn(u[j][i], u[j][i + 1], rcp);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) w[i] = u[j][half * 8 + i];
                uint32_t out;
                if (RMODE == kRoundTteHw) {
                    out = e2m1_pack8_hw(w);
                } else if (kRawSigns) {
                    out = e2m1_pack8_sr_signed(w, rw[j][2 * half], rw[j][2 * half + 1], sign_even[j][half],
                                               sign_odd[j][half]);
                } else if (kSr) {
                    out = e2m1_pack8_sr(w, rw[j][2 * half], rw[j][2 * half + 1]);
                } else {
                    out = 0u;
#pragma unroll
                    for (int i = 0; i < 8; ++i) out += e2m1_nibble<false>(w[i], 0u) * (1u << (4 * i));
                }
                packed[j][2 * h + half] = out;
            }
        }
    }

    if (rows_valid) {
        const int64_t k_atoms = a.rows / 64;
        const int64_t ka = krow / 64;
        const int kb0 = (int)((krow % 64) / 16);  // 0 or 2
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int64_t orow = col + j;  // operand row
            if (orow < a.cols)
                *reinterpret_cast<uint4*>(a.codes_t + orow * (a.rows / 2) + krow / 2) =
                    make_uint4(packed[j][0], packed[j][1], packed[j][2], packed[j][3]);
            // the tile spans one whole 128-row group of the operand: rows beyond `cols` get 1.0
            const int64_t byte_offset = (((orow >> 7) * k_atoms + ka) * 128 + (orow & 31) * 4 + ((orow >> 5) & 3)) * 4 + kb0;
            *reinterpret_cast<uint16_t*>(a.sf_t + byte_offset) = orow < a.cols ? (uint16_t)sf_pair[j] : (uint16_t)0x3838u;
            if (a.sf_raw_t)
                *reinterpret_cast<uint16_t*>(a.sf_raw_t + byte_offset) = orow < a.cols ? (uint16_t)raw_pair[j] : (uint16_t)0u;
        }
    }
    window_record_units(a.window_record, bad_units);

    // ---- phase 3 (BOTH): the operand x itself from the same tile.  Thread = one row x 64
    // columns (one atom word): the block scales are those of phase 2 (B x B blocks are the same
    // in both orientations), the payload arithmetic is quantize_operand_kernel's.
    if (BOTH) {
        __syncthreads();
        const int prow = tid >> 1, half = tid & 1;
        const int64_t grow = r0 + prow, gcol0 = c0 + half * 64;
        int bad_rows = 0;
        if (gcol0 < a.cols) {   // cols % 64 == 0: a 64-column half is in or out
            const bool valid = grow < a.rows;
            uint32_t sf_bytes = 0u, raw_bytes = 0u;
            uint32_t packed[4][2];
#pragma unroll
            for (int blk = 0; blk < 4; ++blk) {
                const uint32_t code = block_code[prow / B][(half * 64 + blk * 16) / B];
                bool outside;
                sf_bytes |= ue4m3_window_byte(code, rebias, outside) << (8 * blk);
                raw_bytes |= (uint32_t)block_raw[prow / B][(half * 64 + blk * 16) / B] << (8 * blk);
                if (outside && valid) {
                    ++bad_rows;
                    window_record_row_cold(a.window_record_rows, grow);
                }
                const float rcp = payload_multiplier(ue5m3_decode(code), ts);
                float v[16];
                if (sizeof(T) == 2) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t w = tile[prow * kPitch + (half * 64 + blk * 16) / 2 + i];
                        v[2 * i] = __uint_as_float(w << 16);
                        v[2 * i + 1] = __uint_as_float(w & 0xFFFF0000u);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(tile[prow * kPitch + half * 64 + blk * 16 + i]);
                }
#pragma unroll
                for (int i = 0; i < 16; i += 2) mul2_rn(v[i], v[i + 1], rcp);
#pragma unroll
                for (int h8 = 0; h8 < 2; ++h8) {
                    float w8[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) w8[i] = v[h8 * 8 + i];
                    if (RMODE == kRoundTteHw) {
                        packed[blk][h8] = e2m1_pack8_hw(w8);
                    } else {
                        packed[blk][h8] = 0u;
#pragma unroll
                        for (int i = 0; i < 8; ++i) packed[blk][h8] += e2m1_nibble<false>(w8[i], 0u) * (1u << (4 * i));
                    }
                }
            }
            if (valid) {
                uint4* dst = reinterpret_cast<uint4*>(a.codes + grow * (a.cols / 2) + gcol0 / 2);
                dst[0] = make_uint4(packed[0][0], packed[0][1], packed[1][0], packed[1][1]);
                dst[1] = make_uint4(packed[2][0], packed[2][1], packed[3][0], packed[3][1]);
            }
            // the tile spans one whole 128-row group of this operand too: rows beyond `rows` get 1.0
            const int64_t word = (((grow >> 7) * (a.cols / 64) + gcol0 / 64) * 128 + (grow & 31) * 4 + ((grow >> 5) & 3)) * 4;
            *reinterpret_cast<uint32_t*>(a.sf + word) = valid ? sf_bytes : 0x38383838u;
            if (a.sf_raw) *reinterpret_cast<uint32_t*>(a.sf_raw + word) = valid ? raw_bytes : 0u;
        }
        window_record_units(a.window_record_rows, bad_rows);
    }
}

template <typename T, int B, bool TWO_D, bool RHT>
static int dispatch_operand_t(int rmode, int bits_dtype, const OperandTArgs& args, cudaStream_t stream) {
    dim3 grid((unsigned)((args.cols + kTT - 1) / kTT), (unsigned)((args.rows + kTT - 1) / kTT));
    if (grid.y > 65535u) return UE5M3_ERR_TOO_LARGE;
    const size_t smem = (size_t)kTT * TransposeTile<T>::kPitch * 4 + (rmode == kRoundSr ? (size_t)kTT * kTBitsPitch : 0);
#define UE5M3_OPT(R, BT)                                                                         \
    do {                                                                                         \
        auto kernel = quantize_operand_t_kernel<T, B, TWO_D, R, BT, RHT, false>;                 \
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        kernel<<<grid, 256, smem, stream>>>(args);                                               \
    } while (0)
    if (rmode == kRoundSr) {
        if (bits_dtype == UE5M3_BITS_PHILOX) UE5M3_OPT(kRoundSr, UE5M3_BITS_PHILOX);
        else UE5M3_OPT(kRoundSr, UE5M3_BITS_U8);
    } else if (rmode == kRoundTteHw) {
        UE5M3_OPT(kRoundTteHw, UE5M3_BITS_U8);
    } else {
        UE5M3_OPT(kRoundTteSw, UE5M3_BITS_U8);
    }
#undef UE5M3_OPT
    return UE5M3_OK;
}

// The transposing kernel takes tensors whose rows are 16-byte multiples; everything else (and
// int32 bit tensors) stays on the general tile kernel.  Returns UE5M3_ERR_UNSUPPORTED when the
// caller should use that one.
int quantize_operand_t_fast(const void* x, int dtype, int64_t rows, int64_t cols, int block, int blocking,
                            const float* amax_dev, float target, int rounding, const void* bits, int bits_dtype,
                            int shift, uint8_t* codes_t, uint8_t* sf_t, uint8_t* sf_raw_t, int* window_record,
                            bool rht, cudaStream_t stream) {
    const bool sr = rounding == UE5M3_ROUND_STOCHASTIC_FAST;
    const size_t esize = dtype == UE5M3_DTYPE_BF16 ? 2 : 4;
    if (((uintptr_t)x % 16) || (cols * esize) % 16 || ((uintptr_t)codes_t % 16) || (rows % 64)) return UE5M3_ERR_UNSUPPORTED;
    if (sr) {
        if (bits_dtype == UE5M3_BITS_I32 || cols % 16) return UE5M3_ERR_UNSUPPORTED;
        if (bits_dtype == UE5M3_BITS_U8 && ((uintptr_t)bits % 16)) return UE5M3_ERR_UNSUPPORTED;
    }
    OperandTArgs args;
    args.x = x; args.rows = rows; args.cols = cols; args.amax_dev = amax_dev;
    args.six_t = (float)((double)target * 6.0);
    args.bits = bits; args.codes_t = codes_t; args.sf_t = sf_t; args.sf_raw_t = sf_raw_t; args.shift = shift;
    args.window_record = window_record;
    args.transformed_amax = nullptr;
    args.codes = nullptr; args.sf = nullptr; args.sf_raw = nullptr; args.window_record_rows = nullptr;
    const int rmode = sr ? kRoundSr : (use_hw_cvt() ? kRoundTteHw : kRoundTteSw);
    const bool two_d = blocking == UE5M3_BLOCK_2D;
    int status;
    if (rht) {
        if (block != 16 || two_d) return UE5M3_ERR_INVALID_ARGUMENT;
        status = dtype == UE5M3_DTYPE_BF16 ? dispatch_operand_t<__nv_bfloat16, 16, false, true>(rmode, bits_dtype, args, stream)
                                           : dispatch_operand_t<float, 16, false, true>(rmode, bits_dtype, args, stream);
        if (status != UE5M3_OK) return status;
        return check_launch();
    }
#define UE5M3_DOT(T, B) \
    (two_d ? dispatch_operand_t<T, B, true, false>(rmode, bits_dtype, args, stream) : dispatch_operand_t<T, B, false, false>(rmode, bits_dtype, args, stream))
    if (dtype == UE5M3_DTYPE_BF16) status = block == 16 ? UE5M3_DOT(__nv_bfloat16, 16) : UE5M3_DOT(__nv_bfloat16, 32);
    else status = block == 16 ? UE5M3_DOT(float, 16) : UE5M3_DOT(float, 32);
#undef UE5M3_DOT
    if (status != UE5M3_OK) return status;
    return check_launch();
}

// 2-D blocks, ties-to-even: x [rows, cols] -> both GEMM operands (x and x^T) in one launch.
template <typename T, int B>
static void launch_operand_both(const OperandTArgs& args, int rmode, cudaStream_t stream) {
    dim3 grid((unsigned)((args.cols + kTT - 1) / kTT), (unsigned)((args.rows + kTT - 1) / kTT));
    const size_t smem = (size_t)kTT * TransposeTile<T>::kPitch * 4;
    if (rmode == kRoundTteHw) {
        auto kernel = quantize_operand_t_kernel<T, B, true, kRoundTteHw, UE5M3_BITS_U8, false, false, true>;
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kernel<<<grid, 256, smem, stream>>>(args);
    } else {
        auto kernel = quantize_operand_t_kernel<T, B, true, kRoundTteSw, UE5M3_BITS_U8, false, false, true>;
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kernel<<<grid, 256, smem, stream>>>(args);
    }
}

}  // namespace ue5m3

using namespace ue5m3;

extern "C" int ue5m3_quantize_fp4_operand_both(const void* x, int dtype, int64_t rows, int64_t cols, int block,
                                               const float* amax_dev, float target, int shift, uint8_t* codes,
                                               uint8_t* sf, uint8_t* sf_raw, int* window_record, uint8_t* codes_t,
                                               uint8_t* sf_t, uint8_t* sf_raw_t, int* window_record_t,
                                               void* stream_v) {
    if (!x || !amax_dev || !codes || !sf || !window_record || !codes_t || !sf_t || !window_record_t || rows <= 0 || cols <= 0)
        return UE5M3_ERR_INVALID_ARGUMENT;
    if (dtype != UE5M3_DTYPE_BF16 && dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (block != 16 && block != 32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (!(target > 0.0f) || shift < -8 || shift > 16) return UE5M3_ERR_INVALID_ARGUMENT;
    if ((rows % 64) || (cols % 64)) return UE5M3_ERR_K_NOT_DIVISIBLE;   // both orientations are GEMM operands
    if (rows > 0x7FFFFFFF || cols > 0x7FFFFFFF || (rows + kTT - 1) / kTT > 65535) return UE5M3_ERR_TOO_LARGE;
    if (((uintptr_t)x % 16) || ((uintptr_t)codes % 16) || ((uintptr_t)codes_t % 16) || ((uintptr_t)sf % 4) ||
        ((uintptr_t)sf_t % 4) || ((uintptr_t)sf_raw % 4) || ((uintptr_t)sf_raw_t % 4))
        return UE5M3_ERR_ALIGNMENT;
    OperandTArgs args;
    args.x = x; args.rows = rows; args.cols = cols; args.amax_dev = amax_dev;
    args.six_t = (float)((double)target * 6.0);
    args.bits = nullptr; args.codes_t = codes_t; args.sf_t = sf_t; args.sf_raw_t = sf_raw_t; args.shift = shift;
    args.window_record = window_record_t; args.transformed_amax = nullptr;
    args.codes = codes; args.sf = sf; args.sf_raw = sf_raw; args.window_record_rows = window_record;
    const int rmode = use_hw_cvt() ? kRoundTteHw : kRoundTteSw;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (dtype == UE5M3_DTYPE_BF16) {
        if (block == 16) launch_operand_both<__nv_bfloat16, 16>(args, rmode, stream);
        else launch_operand_both<__nv_bfloat16, 32>(args, rmode, stream);
    } else {
        if (block == 16) launch_operand_both<float, 16>(args, rmode, stream);
        else launch_operand_both<float, 32>(args, rmode, stream);
    }
    return check_launch();
}

extern "C" int ue5m3_quantize_fp4_operand(const void* x, int dtype, int64_t rows, int64_t cols,
                                          int block, int blocking, const float* amax_dev,
                                          float target, int rounding, const void* bits,
                                          int bits_dtype, int shift, uint8_t* codes, uint8_t* sf,
                                          uint8_t* sf_raw, uint8_t* scales, int* window_record,
                                          void* stream_v) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (!x || !amax_dev || !codes || rows <= 0 || cols <= 0) return UE5M3_ERR_INVALID_ARGUMENT;
    if (dtype != UE5M3_DTYPE_BF16 && dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (block != 16 && block != 32) return UE5M3_ERR_BLOCK_SIZE;
    if (!(target > 0.0f) || !(target < 3.0e38f)) return UE5M3_ERR_INVALID_ARGUMENT;
    if (blocking != UE5M3_BLOCK_ROW && blocking != UE5M3_BLOCK_2D) return UE5M3_ERR_UNSUPPORTED;
    const bool sr = rounding == UE5M3_ROUND_STOCHASTIC_FAST;
    if (!sr && rounding != UE5M3_ROUND_TIES_TO_EVEN) return UE5M3_ERR_INVALID_ARGUMENT;
    if (sr && (!bits || (bits_dtype != UE5M3_BITS_U8 && bits_dtype != UE5M3_BITS_I32 &&
                         bits_dtype != UE5M3_BITS_PHILOX)))
        return UE5M3_ERR_INVALID_ARGUMENT;
    if (!sr && bits) return UE5M3_ERR_INVALID_ARGUMENT;
    if (sf && (!window_record || shift < -8 || shift > 16)) return UE5M3_ERR_INVALID_ARGUMENT;
    if (sf_raw && !sf) return UE5M3_ERR_INVALID_ARGUMENT;
    if (cols % 64) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if (((uintptr_t)x % 32) || ((uintptr_t)codes % 16) || ((uintptr_t)sf % 16) || ((uintptr_t)sf_raw % 16) ||
        ((uintptr_t)scales % 4))
        return UE5M3_ERR_ALIGNMENT;
    if (sr && ((uintptr_t)bits % (bits_dtype == UE5M3_BITS_PHILOX ? 8 : bits_dtype == UE5M3_BITS_U8 ? 16 : 32)))
        return UE5M3_ERR_ALIGNMENT;

    OperandArgs args;
    args.x = x; args.rows = rows; args.cols = cols; args.amax_dev = amax_dev;
    args.six_t = (float)((double)target * 6.0);
    args.bits = bits; args.codes = codes; args.sf = reinterpret_cast<uint32_t*>(sf);
    args.sf_raw = reinterpret_cast<uint32_t*>(sf_raw);
    args.scales = scales; args.shift = shift; args.window_record = window_record;
    const int rmode = sr ? kRoundSr : (use_hw_cvt() ? kRoundTteHw : kRoundTteSw);
    const bool two_d = blocking == UE5M3_BLOCK_2D;
#define UE5M3_DO(T, B) \
    (two_d ? dispatch_operand<T, B, true>(rmode, bits_dtype, args, stream) : dispatch_operand<T, B, false>(rmode, bits_dtype, args, stream))
    if (dtype == UE5M3_DTYPE_BF16) { if (block == 16) UE5M3_DO(__nv_bfloat16, 16); else UE5M3_DO(__nv_bfloat16, 32); }
    else { if (block == 16) UE5M3_DO(float, 16); else UE5M3_DO(float, 32); }
#undef UE5M3_DO
    return check_launch();
}

// max |y| over the transformed operand x^T (transform along the rows of x in blocks of 16)
extern "C" int ue5m3_rht_amax_t(const void* x, int dtype, int64_t rows, int64_t cols, float* amax_out_dev,
                                void* stream_v) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (!x || !amax_out_dev || rows <= 0 || cols <= 0) return UE5M3_ERR_INVALID_ARGUMENT;
    if (dtype != UE5M3_DTYPE_BF16 && dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    const size_t esize = dtype == UE5M3_DTYPE_BF16 ? 2 : 4;
    if (rows % 16) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if (((uintptr_t)x % 16) || (cols * esize) % 16) return UE5M3_ERR_ALIGNMENT;
    dim3 grid((unsigned)((cols + kTT - 1) / kTT), (unsigned)((rows + kTT - 1) / kTT));
    if (grid.y > 65535u) return UE5M3_ERR_TOO_LARGE;
    cudaError_t e = cudaMemsetAsync(amax_out_dev, 0, sizeof(float), stream);
    if (e != cudaSuccess) return record_cuda_error(e);
    OperandTArgs args = {};
    args.x = x; args.rows = rows; args.cols = cols; args.six_t = 1.0f;
    args.transformed_amax = reinterpret_cast<unsigned int*>(amax_out_dev);
    if (dtype == UE5M3_DTYPE_BF16) {
        auto kernel = quantize_operand_t_kernel<__nv_bfloat16, 16, false, kRoundTteHw, UE5M3_BITS_U8, true, true>;
        const size_t smem = (size_t)kTT * TransposeTile<__nv_bfloat16>::kPitch * 4;
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kernel<<<grid, 256, smem, stream>>>(args);
    } else {
        auto kernel = quantize_operand_t_kernel<float, 16, false, kRoundTteHw, UE5M3_BITS_U8, true, true>;
        const size_t smem = (size_t)kTT * TransposeTile<float>::kPitch * 4;
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kernel<<<grid, 256, smem, stream>>>(args);
    }
    return check_launch();
}

extern "C" int ue5m3_quantize_fp4_operand_t_rht(const void* x, int dtype, int64_t rows, int64_t cols,
                                                const float* amax_dev, float target, int rounding,
                                                const void* bits, int bits_dtype, int shift, uint8_t* codes_t,
                                                uint8_t* sf_t, uint8_t* sf_raw_t, int* window_record,
                                                void* stream_v) {
    if (!x || !amax_dev || !codes_t || !sf_t || !window_record || rows <= 0 || cols <= 0 || shift < -8 || shift > 16)
        return UE5M3_ERR_INVALID_ARGUMENT;
    if (dtype != UE5M3_DTYPE_BF16 && dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (!(target > 0.0f) || !(target < 3.0e38f)) return UE5M3_ERR_INVALID_ARGUMENT;
    const bool sr = rounding == UE5M3_ROUND_STOCHASTIC_FAST;
    if (!sr && rounding != UE5M3_ROUND_TIES_TO_EVEN) return UE5M3_ERR_INVALID_ARGUMENT;
    if (sr && (!bits || (bits_dtype != UE5M3_BITS_U8 && bits_dtype != UE5M3_BITS_PHILOX))) return UE5M3_ERR_INVALID_ARGUMENT;
    if (!sr && bits) return UE5M3_ERR_INVALID_ARGUMENT;
    if (rows % 64) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if (((uintptr_t)sf_t % 16) || ((uintptr_t)sf_raw_t % 16)) return UE5M3_ERR_ALIGNMENT;
    int status = quantize_operand_t_fast(x, dtype, rows, cols, 16, UE5M3_BLOCK_COL, amax_dev, target, rounding, bits,
                                         bits_dtype, shift, codes_t, sf_t, sf_raw_t, window_record, true,
                                         static_cast<cudaStream_t>(stream_v));
    return status == UE5M3_ERR_UNSUPPORTED ? UE5M3_ERR_ALIGNMENT : status;
}
