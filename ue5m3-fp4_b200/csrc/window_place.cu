// Row-wise placement of the UE4M3 scale window.
//
// The operand quantizers re-bias every UE5M3 block scale of a tensor by ONE power of two so
// that the tensor's largest possible scale sits at the top of UE4M3's 15 binades; a block whose
// scale falls below them gets its row flagged.  Most such rows are simply small as a whole
// (a token with a small gradient, a feature that hardly fires): their own largest scale is far
// below the tensor's, and their blocks fit 15 binades once the window is placed at the ROW's
// largest scale.  Scaling one operand row by a power of two scales every product of the output
// row (A operand) or column (B operand) it feeds by the same power of two, which the
// round-toward-zero accumulation commutes with exactly, so the GEMM epilogue undoes it with
// one exact multiply.
//
// This kernel visits the flagged rows of both operands of a product, reads their raw UE5M3
// scale bytes, and for each row either rewrites its UE4M3 bytes with the row's own shift
// (stored as the difference to the tensor's shift in the record) or, when the row's scales
// span more than the window, lists it for the recomputation pass.  With no flagged row every
// CTA returns after reading two integers.  No reference counterpart (the reference has no
// hardware scale type).
#include <cuda_runtime.h>
#include <stdint.h>

#include "abi_common.cuh"
#include "window_record.cuh"

namespace ue5m3 {

struct PlaceOperand {
    uint8_t* sf;          // UE4M3 atoms, rewritten for placed rows
    const uint8_t* raw;   // raw UE5M3 atoms (0 = all-zero block)
    int* rec;
    int rows;
    int shift;            // the tensor's shift
};

struct PlaceArgs {
    PlaceOperand op[2];
    int k_atoms;          // K / 64
};

// A UE5M3 byte as a position on the scale of NORMAL codes (8 per binade, 0x78 = 1.0): bytes
// 8..0xF7 are that already; the subnormal bytes 1..7 stand for m * 2^-17, each of which is a
// normal number with three fraction bits a few binades lower (1 -> 2^-17, 3 -> 1.5 * 2^-16, ...),
// so they continue the scale below zero.  UE4M3 = this position minus (8 + shift) * 8.
__device__ __forceinline__ int normal_position(uint32_t byte) {
    constexpr int kSubnormal[8] = {0, -16, -8, -4, 0, 2, 4, 6};
    return byte >= 8u ? (int)byte : kSubnormal[byte];
}

__device__ __forceinline__ void place_rows(const PlaceOperand& o, int k_atoms, int warp_global, int warps_total,
                                           int lane) {
    if (!o.rec || __ldg(o.rec + kRecFlagged) == 0) return;
    const int* flags = rec_flags(o.rec);
    int* row_shift = rec_row_shift(o.rec, o.rows);
    for (int row = warp_global; row < o.rows; row += warps_total) {
        if (flags[row] == 0) continue;
        const int64_t base = ((int64_t)(row >> 7) * k_atoms) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4;
        // largest and smallest scale of the row's non-zero blocks
        int top = -1000, bottom = 1000;
        for (int ka = lane; ka < k_atoms; ka += 32) {
            const uint32_t word = *reinterpret_cast<const uint32_t*>(o.raw + base + (int64_t)ka * 512);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t byte = (word >> (8 * b)) & 0xFFu;
                if (byte != 0u) {
                    top = max(top, normal_position(byte));
                    bottom = min(bottom, normal_position(byte));
                }
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            top = max(top, __shfl_xor_sync(0xFFFFFFFFu, top, d));
            bottom = min(bottom, __shfl_xor_sync(0xFFFFFFFFu, bottom, d));
        }
        if (top == -1000) continue;  // nothing but zero blocks
        // smallest shift that brings the largest scale to 0x7E or below: top - ((8 + s) << 3) <= 0x7E
        int shift = (top - 0x7E + 7) >> 3;   // ceil((top - 0x7E) / 8), also for negative values
        shift -= 8;
        const int rebias = (8 + shift) << 3;
        if (bottom - rebias < 8) {
            // the row's own scales span more than the window: recompute it
            if (lane == 0) {
                const int slot = atomicAdd(o.rec + kRecListed, 1);
                if (slot < kRecMaxRows) rec_list(o.rec)[slot] = row;
            }
            continue;
        }
        for (int ka = lane; ka < k_atoms; ka += 32) {
            const uint32_t word = *reinterpret_cast<const uint32_t*>(o.raw + base + (int64_t)ka * 512);
            uint32_t out = 0u;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t byte = (word >> (8 * b)) & 0xFFu;
                out |= (byte == 0u ? 0x38u : (uint32_t)(normal_position(byte) - rebias)) << (8 * b);
            }
            *reinterpret_cast<uint32_t*>(o.sf + base + (int64_t)ka * 512) = out;
        }
        if (lane == 0) {
            row_shift[row] = shift - o.shift;
            atomicAdd(o.rec + kRecPlaced, 1);
        }
    }
}

__global__ void __launch_bounds__(256) place_row_windows_kernel(const PlaceArgs args) {
    const int lane = threadIdx.x & 31;
    const int warp_global = (int)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int warps_total = (int)gridDim.x * 8;
    place_rows(args.op[0], args.k_atoms, warp_global, warps_total, lane);
    place_rows(args.op[1], args.k_atoms, warp_global, warps_total, lane);
}

// ---------------------------------------------------------------------------------------
// Histogram of an operand's UE5M3 block-scale bytes, read from its raw scale atoms (1/16 byte
// per element: the tensor itself is not touched again).  Bin b counts the blocks whose scale
// byte is b; bin 0 counts blocks whose elements are all zero.  One shared-memory histogram per
// CTA, flushed with one atomic per non-empty bin.  The device-side counterpart of the
// block-scale diagnostics of reproduce/scale_target/capture_scale_target_histograms.py:257-366
// of the reference (block count, zero blocks, saturated blocks, the code distribution).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) scale_byte_histogram_kernel(const uint32_t* __restrict__ raw, int64_t rows,
                                                                   int64_t k_atoms, int block, int row_group,
                                                                   unsigned long long* __restrict__ histogram) {
    __shared__ unsigned int bins[256];
    bins[threadIdx.x] = 0u;
    __syncthreads();
    const int64_t total = ((rows + 127) / 128) * k_atoms * 128;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int word = (int)(i % 128);                 // r0 * 4 + r1
        const int64_t tile = (i / 128) / k_atoms;
        const int64_t row = tile * 128 + (word & 3) * 32 + (word >> 2);
        if (row >= rows || (row % row_group) != 0) continue;   // B x B tiles: one count per tile, not per row
        const uint32_t bytes = __ldg(raw + i);
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            if (block == 32 && (kb & 1)) continue;       // a 32-wide block fills two 16-wide slots
            atomicAdd(&bins[(bytes >> (8 * kb)) & 0xFFu], 1u);
        }
    }
    __syncthreads();
    if (bins[threadIdx.x]) atomicAdd(histogram + threadIdx.x, (unsigned long long)bins[threadIdx.x]);
}

}  // namespace ue5m3

using namespace ue5m3;

extern "C" int ue5m3_scale_byte_histogram(const uint8_t* sf_raw, int64_t rows, int64_t K, int block, int two_d,
                                          unsigned long long* histogram_dev, void* stream_v) {
    if (!sf_raw || !histogram_dev || rows <= 0 || K <= 0) return UE5M3_ERR_INVALID_ARGUMENT;
    if (block != 16 && block != 32) return UE5M3_ERR_BLOCK_SIZE;
    if (K % 64) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if (((uintptr_t)sf_raw % 4) || ((uintptr_t)histogram_dev % 8)) return UE5M3_ERR_ALIGNMENT;
    const int64_t total = ((rows + 127) / 128) * (K / 64) * 128;
    const int64_t want = (total + 255) / 256;
    const int grid = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
    scale_byte_histogram_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_v)>>>(
        reinterpret_cast<const uint32_t*>(sf_raw), rows, K / 64, block, two_d ? block : 1, histogram_dev);
    return check_launch();
}

extern "C" int ue5m3_place_row_windows(uint8_t* a_sf, const uint8_t* a_sf_raw, int* a_record, int64_t a_rows,
                                       int a_shift, uint8_t* b_sf, const uint8_t* b_sf_raw, int* b_record,
                                       int64_t b_rows, int b_shift, int64_t K, void* stream_v) {
    if (K <= 0 || K % 64) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if ((a_record && (!a_sf || !a_sf_raw || a_rows <= 0)) || (b_record && (!b_sf || !b_sf_raw || b_rows <= 0)))
        return UE5M3_ERR_INVALID_ARGUMENT;
    if (!a_record && !b_record) return UE5M3_ERR_INVALID_ARGUMENT;
    if (a_rows > 0x7FFFFFFF || b_rows > 0x7FFFFFFF || K / 64 > 0x7FFFFFFF) return UE5M3_ERR_TOO_LARGE;
    if (((uintptr_t)a_sf % 4) || ((uintptr_t)a_sf_raw % 4) || ((uintptr_t)b_sf % 4) || ((uintptr_t)b_sf_raw % 4))
        return UE5M3_ERR_ALIGNMENT;
    PlaceArgs args;
    args.op[0] = PlaceOperand{a_sf, a_sf_raw, a_record, (int)a_rows, a_shift};
    args.op[1] = PlaceOperand{b_sf, b_sf_raw, b_record, (int)b_rows, b_shift};
    args.k_atoms = (int)(K / 64);
    place_row_windows_kernel<<<sm_count(), 256, 0, static_cast<cudaStream_t>(stream_v)>>>(args);
    return check_launch();
}
