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

namespace ue5m3 {

struct OperandArgs {
    const void* x;
    int64_t rows, cols;
    const float* amax_dev;
    float six_t;
    const void* bits;
    uint8_t* codes;     // [rows, cols / 2]
    uint32_t* sf;       // [ceil(rows / 128)][cols / 64][128] words, may be null
    uint8_t* scales;    // raw UE5M3 bytes ([rows, cols/B] or [ceil(rows/B), cols/B]), may be null
    int shift;
    int* window_flag;
};

template <typename T, int B, bool TWO_D, int RMODE, int BITS>
__global__ void __launch_bounds__(256) quantize_operand_kernel(const OperandArgs a) {
    constexpr bool kSr = RMODE == kRoundSr;
    const T* __restrict__ x = static_cast<const T*>(a.x);
    const TensorScale ts = tensor_scale(__ldg(a.amax_dev), a.six_t);
    const int lane = threadIdx.x & 31;
    const int64_t k_atoms = a.cols / 64;
    const int64_t row_groups = ((a.rows + 127) / 128) * 4;  // 32-row groups, padded to whole atoms
    const int64_t ntasks = row_groups * k_atoms;
    const int64_t nbc = a.cols / B;
    const int rebias = (8 + a.shift) << 3;
    bool bad = false;

    for (int64_t task = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); task < ntasks;
         task += (int64_t)gridDim.x * 8) {
        const int64_t rg = task / k_atoms, ka = task % k_atoms;
        const int64_t row = rg * 32 + lane;
        const bool valid = row < a.rows;
        const int64_t unit0 = (row * a.cols + ka * 64) / 16;  // first 16-element unit of this lane

        RawUnit<T> raw[4];
        uint32_t rb[4][4];
        if (valid) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                load_raw_unit<T>(x, unit0 + u, raw[u]);
                if (kSr) load_unit_bits<BITS>(a.bits, unit0 + u, rb[u]);
            }
        } else {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                zero_raw_unit<T>(raw[u]);
#pragma unroll
                for (int i = 0; i < 4; ++i) rb[u][i] = 0u;
            }
        }

        float m[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float v[16];
            unit_values(raw[u], v);
            m[u] = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) m[u] = fmaxf(m[u], fabsf(v[i]));
        }
        if (B == 32) {
            m[0] = m[1] = fmaxf(m[0], m[1]);
            m[2] = m[3] = fmaxf(m[2], m[3]);
        }
        if (TWO_D) {
#pragma unroll
            for (int o = 1; o < B; o <<= 1) {
#pragma unroll
                for (int u = 0; u < 4; u += B / 16)
                    m[u] = fmaxf(m[u], __shfl_xor_sync(0xFFFFFFFFu, m[u], o));
            }
            if (B == 32) { m[1] = m[0]; m[3] = m[2]; }
        }

        uint32_t code[4];
        uint32_t sf_word = 0u;
        uint32_t packed[4][2];
        float scale = 1.0f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (B == 32 && (u & 1)) {
                code[u] = code[u - 1];  // same 32-wide block as the previous unit: same scale
            } else {
                block_scale_converged(m[u], ts, code[u], scale);
            }
            int code4 = (int)code[u] - rebias;
            if (code4 < 8 || code4 > 0x7E) {
                bad = bad || valid;
                code4 = code4 < 8 ? 8 : 0x7E;
            }
            sf_word |= (uint32_t)code4 << (8 * u);
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
                    packed[u][h] = e2m1_pack8_sr(w, rb[u][2 * h], rb[u][2 * h + 1]);
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
            uint4* dst = reinterpret_cast<uint4*>(a.codes + row * (a.cols / 2) + ka * 32);
            dst[0] = make_uint4(packed[0][0], packed[0][1], packed[1][0], packed[1][1]);
            dst[1] = make_uint4(packed[2][0], packed[2][1], packed[3][0], packed[3][1]);
            if (a.scales && (!TWO_D || (row % B) == 0)) {
                uint8_t* sp = a.scales + (TWO_D ? row / B : row) * nbc + ka * (64 / B);
                if (B == 16)
                    *reinterpret_cast<uint32_t*>(sp) = code[0] | (code[1] << 8) | (code[2] << 16) | (code[3] << 24);
                else
                    *reinterpret_cast<uint16_t*>(sp) = (uint16_t)(code[0] | (code[2] << 8));
            }
        }
        if (a.sf) {
            const int64_t tile = rg >> 2;
            const int r1 = (int)(rg & 3);
            a.sf[(tile * k_atoms + ka) * 128 + lane * 4 + r1] = valid ? sf_word : 0x38383838u;
        }
    }
    if (bad && a.window_flag) atomicExch(a.window_flag, 1);
}

template <typename T, int B, bool TWO_D>
static void dispatch_operand(int rmode, int bits_dtype, const OperandArgs& args, cudaStream_t stream) {
    const int64_t ntasks = ((args.rows + 127) / 128) * 4 * (args.cols / 64);
    const int64_t want = (ntasks + 7) / 8;
    const int64_t cap = (int64_t)sm_count() * 8;
    const int grid = (int)(want < cap ? want : cap);
#define UE5M3_OP(R, BT) quantize_operand_kernel<T, B, TWO_D, R, BT><<<grid, 256, 0, stream>>>(args)
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

}  // namespace ue5m3

using namespace ue5m3;

extern "C" int ue5m3_quantize_fp4_operand(const void* x, int dtype, int64_t rows, int64_t cols,
                                          int block, int blocking, const float* amax_dev,
                                          float target, int rounding, const void* bits,
                                          int bits_dtype, int shift, uint8_t* codes, uint8_t* sf,
                                          uint8_t* scales, int* window_flag, void* stream_v) {
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
    if (sf && (!window_flag || shift < -8 || shift > 16)) return UE5M3_ERR_INVALID_ARGUMENT;
    if (cols % 64) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if (((uintptr_t)x % 32) || ((uintptr_t)codes % 16) || ((uintptr_t)sf % 16) || ((uintptr_t)scales % 4))
        return UE5M3_ERR_ALIGNMENT;
    if (sr && ((uintptr_t)bits % (bits_dtype == UE5M3_BITS_PHILOX ? 8 : bits_dtype == UE5M3_BITS_U8 ? 16 : 32)))
        return UE5M3_ERR_ALIGNMENT;

    OperandArgs args;
    args.x = x; args.rows = rows; args.cols = cols; args.amax_dev = amax_dev;
    args.six_t = (float)((double)target * 6.0);
    args.bits = bits; args.codes = codes; args.sf = reinterpret_cast<uint32_t*>(sf);
    args.scales = scales; args.shift = shift; args.window_flag = window_flag;
    const int rmode = sr ? kRoundSr : (use_hw_cvt() ? kRoundTteHw : kRoundTteSw);
    const bool two_d = blocking == UE5M3_BLOCK_2D;
#define UE5M3_DO(T, B) \
    (two_d ? dispatch_operand<T, B, true>(rmode, bits_dtype, args, stream) : dispatch_operand<T, B, false>(rmode, bits_dtype, args, stream))
    if (dtype == UE5M3_DTYPE_BF16) { if (block == 16) UE5M3_DO(__nv_bfloat16, 16); else UE5M3_DO(__nv_bfloat16, 32); }
    else { if (block == 16) UE5M3_DO(float, 16); else UE5M3_DO(float, 32); }
#undef UE5M3_DO
    return check_launch();
}
