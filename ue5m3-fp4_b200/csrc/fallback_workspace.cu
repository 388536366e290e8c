// The recomputation pass of the FP4 product with a caller-provided workspace.
//
// gemm_fallback.cu decodes packed operands inside the GEMM, per tile: every tile of the listed
// pass decodes its rows of BOTH operands again, which is fine for a handful of listed rows and
// 26-fold redundant when thousands of weight-gradient columns are listed.  Here every needed
// operand row is decoded ONCE (packed E2M1 codes x raw UE5M3 scales -> the exact encoded bf16
// value) into the workspace, and the TMA-fed issue-RZ kernel of gemm_sm100.cu runs on it:
//
//   listed rows of A (gathered)  x  all of B      -> scattered to the listed output rows
//   all of A                     x  listed rows of B (gathered) -> scattered to the listed columns
//   all of A                     x  all of B      -> after a list overflowed its capacity
//
// Two launches, still driven by the window records on the device: the decode kernel and the
// GEMM (persistent CTAs over the tiles of all three products) read the list lengths themselves
// and return at once when there is nothing to do; an operand is decoded in full only when the
// other one lists something.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "abi_common.cuh"
#include "alpha_spec.cuh"
#include "decode_bf16.cuh"
#include "issue_rz_mapped.cuh"
#include "window_record.cuh"

namespace ue5m3 {

namespace fb {

struct DecodeArgs {
    const uint8_t* codes[2];   // A, B: [rows, K / 2]
    const uint8_t* raw[2];     // raw UE5M3 scale atoms
    const int* rec[2];
    int rows[2];               // M, N
    int K;
    __nv_bfloat16* listed[2];  // [kRecMaxRows, K]: the listed rows of A / of B, in list order
    __nv_bfloat16* full[2];    // [rows, K]: all of A / of B
};

// An item is 32 consecutive elements of one operand row: 16 bytes of codes and two scale bytes
// in, 64 bytes out.  Four sections, walked with one grid-stride loop: A's listed rows, all of B
// (if A lists any), B's listed rows, all of A (if B lists any).
__global__ void __launch_bounds__(512) decode_operands_kernel(const DecodeArgs d) {
    int listed[2];
#pragma unroll
    for (int o = 0; o < 2; ++o) listed[o] = __ldg(d.rec[o] + kRecListed);
    if (listed[0] == 0 && listed[1] == 0) return;
    const bool overflow = listed[0] > kRecMaxRows || listed[1] > kRecMaxRows;   // whole product: both in full
    if (overflow) listed[0] = listed[1] = 0;
    const int64_t per_row = d.K / 32;
    const int64_t k_atoms = d.K / 64;
    // section s: operand (s == 1 || s == 2), gathered (s == 0 || s == 2), number of rows
    const int section_rows[4] = {listed[0], (listed[0] || overflow) ? d.rows[1] : 0, listed[1],
                                 (listed[1] || overflow) ? d.rows[0] : 0};
    int64_t first[5];
    first[0] = 0;
#pragma unroll
    for (int s = 0; s < 4; ++s) first[s + 1] = first[s] + (int64_t)section_rows[s] * per_row;
    for (int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; item < first[4];
         item += (int64_t)gridDim.x * blockDim.x) {
        const int s = item < first[1] ? 0 : (item < first[2] ? 1 : (item < first[3] ? 2 : 3));
        const int operand = (s == 1 || s == 2) ? 1 : 0;
        const bool gathered = (s & 1) == 0;
        const int64_t local = item - first[s];
        const int64_t index = local / per_row, chunk = local % per_row;
        const int64_t row = gathered ? (int64_t)__ldg(d.rec[operand] + kRecHeader + index) : index;
        const uint4 codes = __ldg(reinterpret_cast<const uint4*>(d.codes[operand] + row * (d.K / 2)) + chunk);
        const uint32_t scales = __ldg(reinterpret_cast<const uint16_t*>(
            d.raw[operand] + ((row >> 7) * k_atoms + (chunk >> 1)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 +
            (chunk & 1) * 2));
        const uint32_t scale2[2] = {scale_pair(scales & 0xFFu), scale_pair((scales >> 8) & 0xFFu)};
        const uint32_t words[4] = {codes.x, codes.y, codes.z, codes.w};
        uint4* dst = reinterpret_cast<uint4*>((gathered ? d.listed[operand] : d.full[operand]) + index * d.K + chunk * 32);
#pragma unroll
        for (int w = 0; w < 4; ++w) dst[w] = decode_word(words[w], scale2[w >> 1]);
    }
}

}  // namespace fb
}  // namespace ue5m3

using namespace ue5m3;

extern "C" size_t ue5m3_fallback_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return (size_t)(2 * (int64_t)kRecMaxRows + M + N) * (size_t)K * 2;
}

extern "C" int ue5m3_gemm_fp4_fallback_ws(const uint8_t* a_codes, const uint8_t* a_sf_raw, const int* a_record,
                                          const uint8_t* b_codes, const uint8_t* b_sf_raw, const int* b_record,
                                          int64_t M, int64_t N, int64_t K, int snap, const float* alpha_dev,
                                          const float* amax_a_dev, const float* amax_b_dev, float inv_denominator,
                                          const void* bias, int bias_dtype, void* out, int out_dtype, int64_t ldo,
                                          void* workspace, size_t workspace_bytes, int* status_dev, void* stream_v) {
    if (!a_codes || !a_sf_raw || !a_record || !b_codes || !b_sf_raw || !b_record || !out || !workspace || M <= 0 ||
        N <= 0 || K <= 0)
        return UE5M3_ERR_INVALID_ARGUMENT;
    if (K % 64) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if (out_dtype != UE5M3_DTYPE_BF16 && out_dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (bias && bias_dtype != UE5M3_DTYPE_BF16 && bias_dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (ldo < N) return UE5M3_ERR_INVALID_ARGUMENT;
    if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) return UE5M3_ERR_TOO_LARGE;
    if (workspace_bytes < ue5m3_fallback_workspace_bytes(M, N, K)) return UE5M3_ERR_INVALID_ARGUMENT;
    if (((uintptr_t)a_codes % 16) || ((uintptr_t)b_codes % 16) || ((uintptr_t)a_sf_raw % 4) || ((uintptr_t)b_sf_raw % 4) ||
        ((uintptr_t)workspace % 16))
        return UE5M3_ERR_ALIGNMENT;
    const AlphaSpec alpha{alpha_dev, amax_a_dev, amax_b_dev, inv_denominator};
    if (!alpha_spec_valid(alpha)) return UE5M3_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    __nv_bfloat16* base = static_cast<__nv_bfloat16*>(workspace);
    fb::DecodeArgs d;
    d.codes[0] = a_codes; d.codes[1] = b_codes; d.raw[0] = a_sf_raw; d.raw[1] = b_sf_raw;
    d.rec[0] = a_record; d.rec[1] = b_record; d.rows[0] = (int)M; d.rows[1] = (int)N; d.K = (int)K;
    d.listed[0] = base;
    d.listed[1] = d.listed[0] + (size_t)kRecMaxRows * K;
    d.full[0] = d.listed[1] + (size_t)kRecMaxRows * K;
    d.full[1] = d.full[0] + (size_t)M * K;
    // few, large CTAs: with nothing listed (the usual case) the launch costs what its CTAs cost to start
    fb::decode_operands_kernel<<<sm_count() * 2, 512, 0, stream>>>(d);

    MappedOperands ops{d.listed[0], d.listed[1], d.full[0], d.full[1], kRecMaxRows, a_record + kRecListed,
                       b_record + kRecListed, a_record + kRecHeader, b_record + kRecHeader};
    const int status = launch_issue_rz_mapped(ops, M, N, K, snap, alpha, bias, bias_dtype, out, out_dtype, ldo, status_dev,
                                              stream);
    if (status != UE5M3_OK) return status;
    return check_launch();
}
