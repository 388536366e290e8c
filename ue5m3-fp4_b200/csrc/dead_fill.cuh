// What a GEMM launch does instead of its work when its status word already holds a failure.
#pragma once

namespace ue5m3 {

// A launch that finds a failure recorded in its status word does none of its work; it marks
// the output it would have written instead, so that nobody mistakes stale memory for a result.
// All threads of the CTA store NaN into the rows x cols tile at (row0, col0) of a row-major
// bf16 (`is_bf16`) or fp32 output with `ldo` elements per row, clipped to M x N.
static __device__ __noinline__ void fill_tile_nan(void* out, bool is_bf16, long long ldo, int row0, int col0, int rows,
                                              int cols, int M, int N) {
    for (int idx = threadIdx.x; idx < rows * cols; idx += blockDim.x) {
        const int r = row0 + idx / cols, c = col0 + idx % cols;
        if (r >= M || c >= N) continue;
        if (is_bf16) static_cast<unsigned short*>(out)[r * ldo + c] = 0x7FC0u;
        else static_cast<unsigned int*>(out)[r * ldo + c] = 0x7FC00000u;
    }
}

}  // namespace ue5m3
