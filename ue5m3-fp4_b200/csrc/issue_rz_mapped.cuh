// The issue-RZ BF16 GEMM of gemm_sm100.cu launched over operands that the recomputation pass
// of the FP4 product has decoded into a workspace: which rows are listed, and how many, is
// known on the device only, and the output rows / columns are scattered through the lists.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "alpha_spec.cuh"

namespace ue5m3 {

struct MappedOperands {
    const void* a_listed;   // [cap, K] bf16: the listed rows of A in list order
    const void* b_listed;   // [cap, K]: the listed rows of B
    const void* a_full;     // [M, K]: all of A (filled only when B lists something, or after an overflow)
    const void* b_full;     // [N, K]
    int cap;
    const int* a_count;     // device: number of listed rows of A; above cap = the list overflowed
    const int* b_count;
    const int* a_list;      // device: output row of a_listed's row i
    const int* b_list;      // device: output column of b_listed's row i
};

// One persistent launch for listed A x full B, full A x listed B and - after an overflow - the
// whole product.  All buffers K-major and 16-byte aligned.  Returns a status code; the caller
// checks the launch.
int launch_issue_rz_mapped(const MappedOperands& ops, int64_t M, int64_t N, int64_t K, int snap, const AlphaSpec& alpha,
                           const void* bias, int bias_dtype, void* out, int out_dtype, int64_t ldo, int* status_dev,
                           cudaStream_t stream);

}  // namespace ue5m3
