// Device side of an operand's window record (layout: include/ue5m3_fp4.h).  The quantizers
// call these on the rare block whose UE5M3 scale does not fit the tensor core's UE4M3 range
// at the tensor's shift; ue5m3_place_row_windows then tries a shift of its own for every such
// row and lists the rows that still do not fit.
#pragma once

#include <stdint.h>

#include "abi_common.cuh"

namespace ue5m3 {

constexpr int kRecHeader = UE5M3_WINDOW_RECORD_HEADER;
constexpr int kRecMaxRows = UE5M3_FALLBACK_MAX_ROWS;
// header words
constexpr int kRecFlagged = 0;   // distinct rows flagged by the quantizer
constexpr int kRecUnits = 1;     // 16-element units outside the window at the tensor's shift
constexpr int kRecListed = 2;    // rows listed for recomputation (after row placement)
constexpr int kRecPlaced = 3;    // rows that got a shift of their own

__device__ __forceinline__ const int* rec_list(const int* rec) { return rec + kRecHeader; }
__device__ __forceinline__ int* rec_list(int* rec) { return rec + kRecHeader; }
__device__ __forceinline__ int* rec_flags(int* rec) { return rec + kRecHeader + kRecMaxRows; }
__device__ __forceinline__ const int* rec_row_shift(const int* rec, int64_t rows) { return rec + kRecHeader + kRecMaxRows + rows; }
__device__ __forceinline__ int* rec_row_shift(int* rec, int64_t rows) { return rec + kRecHeader + kRecMaxRows + rows; }

// Flags `row` once.  The plain read keeps rows with many such blocks off the atomic path.
__device__ __forceinline__ void window_record_row(int* rec, int64_t row) {
    int* flag = rec_flags(rec) + row;
    if (*((volatile int*)flag) == 0 && atomicExch(flag, 1) == 0) atomicAdd(rec + kRecFlagged, 1);
}

// The same as a call: for the quantizers' inner loops, where the flagging is rare and its inlined
// atomics would cost every thread registers.
static __device__ __noinline__ void window_record_row_cold(int* rec, int64_t row) { window_record_row(rec, row); }

// Adds a thread's count of out-of-window 16-element units, one atomic per warp at most.
__device__ __forceinline__ void window_record_units(int* rec, int units) {
    if (!__any_sync(0xFFFFFFFFu, units != 0)) return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) units += __shfl_xor_sync(0xFFFFFFFFu, units, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(rec + kRecUnits, units);
}

// UE5M3 byte -> UE4M3 byte at `rebias` = (8 + shift) << 3; `outside` reports a clamp.
__device__ __forceinline__ uint32_t ue4m3_window_byte(uint32_t code5, int rebias, bool& outside) {
    int code4 = (int)code5 - rebias;
    outside = code4 < 8 || code4 > 0x7E;
    if (outside) code4 = code4 < 8 ? 8 : 0x7E;
    return (uint32_t)code4;
}

// 2^e as fp32, |e| <= 126
__device__ __forceinline__ float exp2_int(int e) { return __int_as_float((127 + e) << 23); }

}  // namespace ue5m3
