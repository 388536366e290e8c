/*
 * C ABI of the B200 (sm_100a) UE5M3/E2M1 quantize + probe-matched GEMM library.
 *
 * Every entry point takes borrowed DEVICE pointers (unless a parameter says
 * "host"), plain sizes and an explicit CUDA stream (a cudaStream_t passed as
 * void*), launches asynchronously on that stream and returns a status code
 * (UE5M3_OK == 0).  The current device must be the stream's device on every call.
 * Nothing here allocates or frees device memory; the caller owns every buffer.
 * Global state of the library: per-process caches of driver entry points (TMA
 * descriptor encoder) and of per-device attributes (SM count, resident clusters), and,
 * as the one exception to "the caller owns every buffer", the fixed reduction scratch
 * of ue5m3_amax_static (a __device__ array per GPU plus a host-side cache of its
 * address per device ordinal).
 *
 * Each declaration cites the reference interface it replaces, by the file's path
 * inside the reference project, or says that it has no counterpart there.
 */
#ifndef UE5M3_FP4_H_
#define UE5M3_FP4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define UE5M3_ABI_VERSION 2

/* status codes */
#define UE5M3_OK 0
#define UE5M3_ERR_INVALID_ARGUMENT 1 /* null pointer, non-positive size, bad enum */
#define UE5M3_ERR_BLOCK_SIZE 2       /* block size is not 16 or 32 */
#define UE5M3_ERR_K_NOT_DIVISIBLE 3  /* reduction axis not divisible by block / by 64 */
#define UE5M3_ERR_ALIGNMENT 4        /* pointer or leading dimension breaks a 16-byte rule */
#define UE5M3_ERR_UNSUPPORTED 5      /* combination of options not implemented */
#define UE5M3_ERR_CUDA 6             /* a CUDA runtime / driver call failed */
#define UE5M3_ERR_SCRATCH 7          /* scratch buffer too small */
#define UE5M3_ERR_TOO_LARGE 8        /* size exceeds a stated maximum */

/* element types */
#define UE5M3_DTYPE_BF16 0
#define UE5M3_DTYPE_FP32 1

/* payload rounding; ids follow the reference, backends/triton/_rounding.py:18-19 */
#define UE5M3_ROUND_TIES_TO_EVEN 0
#define UE5M3_ROUND_STOCHASTIC_FAST 7

/* dtype of the explicit random-bit tensor (values 0..255, one per element) */
#define UE5M3_BITS_NONE 0
#define UE5M3_BITS_U8 1
#define UE5M3_BITS_I32 2 /* the reference's dtype, backends/triton/quantization.py:276 */
/*
 * No bit tensor: `bits` points to two uint64 on the device, {seed, stream}, and the byte of
 * element e (row-major index in x) is byte e % 16 of Philox4x32-10 with key = seed and
 * counter = {e / 16, stream} (words c0..c3 little-endian).  The reference draws its bits
 * from a torch generator (nn/linear.py:371-384), a stream that no kernel can reproduce;
 * ue5m3_philox_bytes writes the very bytes this mode uses, so that a run can be replayed
 * with an explicit UE5M3_BITS_U8 tensor.
 */
#define UE5M3_BITS_PHILOX 3

/* block geometry */
#define UE5M3_BLOCK_ROW 0 /* 1 x B, along the last axis (activations, dY)          */
#define UE5M3_BLOCK_COL 1 /* B x 1, along the first axis (wgrad operands)          */
#define UE5M3_BLOCK_2D 2  /* B x B tiles (weights; formats.py:294-328)             */

/* value domain of the optional fake-quantized tensor output */
#define UE5M3_FAKE_NONE 0
#define UE5M3_FAKE_ENCODED 1 /* p*s            backends/triton/quantization.py:135      */
#define UE5M3_FAKE_DECODED 2 /* (p*s)*dec      backends/triton/quantization.py:136-137  */
#define UE5M3_FAKE_DEQUANT 3 /* p*(s*dec)      formats.py:439,450                       */

int ue5m3_abi_version(void);
const char *ue5m3_status_string(int status);

/* Last CUDA error text recorded by this thread's most recent failing call (host string). */
const char *ue5m3_last_cuda_error(void);

/*
 * Tensor amax: amax_out[0] = max |x[i]| as fp32, in ONE pass, result left on the
 * device.  Non-finite inputs make the result +inf or NaN (bit pattern >=
 * 0x7f800000), which callers test instead of a separate isfinite pass.
 * Replaces: scaling/training.py:39 (`tensor.to(float32).abs().amax()`),
 * backends/triton/quantization.py:226.
 * scratch: ue5m3_amax_scratch_bytes() bytes of device memory, zero-filled once
 * by the caller before the first use; the kernel leaves it zeroed again.
 */
size_t ue5m3_amax_scratch_bytes(void);
int ue5m3_amax(const void *x, int dtype, int64_t n, float *amax_out, void *scratch,
               size_t scratch_bytes, void *stream);

/*
 * Tensor amax for callers that cannot allocate device memory.  It has no counterpart in
 * the reference.  Same result as ue5m3_amax, but the reduction scratch is a fixed array
 * inside the library (about 4 KiB per GPU that loads the library, held until exit), so
 * the caller passes only the input, the output and the stream.  Meant for hosts that
 * have no device allocator of their own to call - a plain C/C++ plugin whose device
 * memory all belongs to another runtime's pool - and for latency-critical threads where
 * cudaMalloc's device-wide synchronisation is not acceptable.  The call itself performs
 * no cudaMalloc/cudaFree and uses no allocating library routine.
 * Limits and rules:
 *  - n <= 2^32 elements, otherwise UE5M3_ERR_TOO_LARGE (use ue5m3_amax with own scratch);
 *  - the first call on each device looks up the array's device address (with that device
 *    current); make that first call outside any stream capture;
 *  - all calls on one device share the one array: calls that may overlap on the GPU
 *    (different streams, different threads) race and must be serialised by the caller.
 */
int ue5m3_amax_static(const void *x, int dtype, int64_t n, float *amax_out, void *stream);

/*
 * Fused single-pass block quantizer: E2M1 payload nibbles + UE5M3 scale bytes
 * (+ optional fake-quantized tensor) from a [rows, cols] row-major bf16/fp32
 * tensor and a held tensor amax (device scalar).
 * Replaces: backends/triton/quantization.py:34-200 (_fake_quantize_operands_kernel)
 * and formats.py:350-457 (_quantize_dequantize_blocks_impl).
 *
 * Packed layouts (byte = element 2j in the low nibble, 2j+1 in the high nibble;
 * nibble = sign<<3 | index into {0,.5,1,1.5,2,3,4,6}; scale byte = E<<3|M, bias 15):
 *   BLOCK_ROW: codes   [rows, ceil(cols/2)]   scales   [rows, ceil(cols/B)]
 *   BLOCK_COL: codes_t [cols, ceil(rows/2)]   scales_t [cols, ceil(rows/B)]
 *   BLOCK_2D : codes   [rows, ceil(cols/2)]   scales   [ceil(rows/B), ceil(cols/B)]
 *              codes_t [cols, ceil(rows/2)]   scales_t [ceil(cols/B), ceil(rows/B)]
 * fake   [rows, cols] and fake_t [cols, rows] hold the values of `fake_domain`
 * in `fake_dtype`.  Any output pointer may be NULL; outputs a geometry does not
 * define must be NULL.  Ragged edges are zero padded (formats.py:299-305).
 * bits: explicit random integers 0..255, same shape as x, required for
 * UE5M3_ROUND_STOCHASTIC_FAST (backends/triton/quantization.py:270-282).
 */
int ue5m3_quantize(const void *x, int dtype, int64_t rows, int64_t cols, int block,
                   int blocking, const float *amax_dev, float target, int rounding,
                   const void *bits, int bits_dtype, uint8_t *codes, uint8_t *scales,
                   uint8_t *codes_t, uint8_t *scales_t, void *fake, void *fake_t,
                   int fake_dtype, int fake_domain, void *stream);

/*
 * Packed -> values: out[r,c] = p * (s * dec), formats.py:439,450.
 * codes [rows, ceil(cols/2)]; scales [rows, ceil(cols/B)] (two_d == 0) or
 * [ceil(rows/B), ceil(cols/B)] (two_d != 0).
 */
int ue5m3_dequantize(const uint8_t *codes, const uint8_t *scales, int64_t rows,
                     int64_t cols, int block, int two_d, const float *amax_dev,
                     float target, void *out, int out_dtype, void *stream);

/*
 * alpha_out[0] = fl(fl(amax_a*amax_b) * inv_denominator): the tensor-scale decode
 * factor of backends/triton/quantization.py:412-420 with the host scalar
 * 1/((Ta*6)*(Tb*6)) passed in as fp32.
 */
int ue5m3_alpha(const float *amax_a, const float *amax_b, float inv_denominator,
                float *alpha_out, void *stream);

/*
 * Probe-matched GEMM on encoded bf16 operands, both K-major:
 *   out[M,N] = epilogue( A[M,K] * Bt[N,K]^T )
 * One tcgen05 issue per 64 reduction elements into a fresh TMEM accumulator;
 * issue partials are combined in ascending k with fp32 round-toward-zero adds;
 * then, fused: optional RNE snap to the 1/1024 grid, * alpha, + bias[n] (fp32 or bf16,
 * NULL = none), cast to out_dtype.  alpha is either alpha_dev[0] (device scalar), or, when
 * alpha_dev is NULL and amax_a_dev / amax_b_dev are given, fl(fl(amax_a[0] * amax_b[0]) *
 * inv_denominator) formed in the epilogue from the two held tensor amaxes (device scalars) and
 * the host-computed fp32 reciprocal of (Ta*6)*(Tb*6) - the expression of
 * backends/triton/quantization.py:412-420 as ATen evaluates it - or 1 when all three are NULL.
 * Replaces: backends/triton/gemm.py:26-88,110-160 (_issue_rz_kernel,
 * issue_rz_bf16_gemm), api.py:72-83 and nn/linear.py:334-336.
 * K % 64 == 0; a, bt 16-byte aligned; ldo = row stride of out in elements.
 * status_dev (nullable device int[4]): set non-zero if a bounded wait inside the
 * kernel expired; the kernel then returns without writing the affected tile.
 */
int ue5m3_gemm_issue_rz_bf16(const void *a, const void *bt, int64_t M, int64_t N, int64_t K,
                             int snap, const float *alpha_dev, const float *amax_a_dev,
                             const float *amax_b_dev, float inv_denominator, const void *bias,
                             int bias_dtype, void *out, int out_dtype, int64_t ldo,
                             int *status_dev, void *stream);

/*
 * Window record of one packed GEMM operand.  The FP4 tensor core takes UE4M3 block scales
 * (15 binades); UE5M3 spans 32 (formats.py:125-134).  The quantizers re-bias all scales of a
 * tensor by one power of two (`shift`); a block scale that then falls outside UE4M3's normal
 * range is clamped in the tensor-core scale atoms and its operand ROW is flagged here.
 * ue5m3_place_row_windows afterwards gives every flagged row whose own scales fit 15 binades a
 * shift of its own (exact: the GEMM epilogue multiplies the affected output rows / columns by
 * the matching power of two) and lists the rows that still do not fit, for
 * ue5m3_gemm_fp4_fallback to recompute.  Layout (int32, zero-filled by the caller before the
 * operand is quantized), R = operand rows:
 *   [0] distinct rows flagged by the quantizer
 *   [1] 16-element units whose scale was outside the window at the tensor's shift (diagnostic)
 *   [2] rows listed for recomputation (a value > UE5M3_FALLBACK_MAX_ROWS means the list
 *       overflowed and the whole product is recomputed)
 *   [3] rows that got a shift of their own
 *   [4 .. 4 + UE5M3_FALLBACK_MAX_ROWS)      the listed rows, in no particular order
 *   [.. + R)                                one flag per operand row
 *   [.. + R)                                per row: its shift minus the tensor's shift (0 if unplaced)
 * No reference counterpart (the reference has no packed operands and no scale window).
 */
#define UE5M3_FALLBACK_MAX_ROWS 4096
#define UE5M3_WINDOW_RECORD_HEADER 4
size_t ue5m3_window_record_ints(int64_t operand_rows);

/*
 * Row-wise placement of the scale window for the two operands of one product (either record
 * may be NULL): rewrites the UE4M3 atoms of flagged rows that fit a window of their own,
 * stores their extra exponents in the record and lists the others.  One launch; returns at
 * once on the device when nothing is flagged.  a_shift / b_shift: the tensors' shifts as
 * passed to the quantizers.  Call it between the quantizers and ue5m3_gemm_fp4.
 * No reference counterpart.
 */
int ue5m3_place_row_windows(uint8_t *a_sf, const uint8_t *a_sf_raw, int *a_record, int64_t a_rows,
                            int a_shift, uint8_t *b_sf, const uint8_t *b_sf_raw, int *b_record,
                            int64_t b_rows, int b_shift, int64_t K, void *stream);

/*
 * histogram_dev[b] += number of blocks of the operand whose UE5M3 scale byte is b (256
 * unsigned 64-bit counters, accumulated: clear them to start afresh); bin 0 = blocks whose
 * elements are all zero.  Reads the raw scale atoms (sf_raw) that the one-pass operand
 * quantizers write, i.e. 1/16 byte per element; two_d != 0 counts a block x block tile once.
 * Device-side counterpart of the block-scale diagnostics of
 * reproduce/scale_target/capture_scale_target_histograms.py:257-366 (block count, zero blocks,
 * saturated blocks = byte 0xF7, the scale-code distribution).
 */
int ue5m3_scale_byte_histogram(const uint8_t *sf_raw, int64_t rows, int64_t K, int block, int two_d,
                               unsigned long long *histogram_dev, void *stream);

/*
 * UE5M3 scale bytes -> the block-scaled tensor core's UE4M3 scale-factor layout.
 * scales: [rows, K/block] (two_d == 0) or [ceil(rows/block), K/block] (two_d != 0) as written
 * by ue5m3_quantize for a K-major operand.  sf_out: ue5m3_packed_scales_bytes(rows, K) bytes,
 * [ceil(rows/128)][K/64][512]; within a 512-byte atom the byte of row r0 + 32*r1 and 16-block
 * kb sits at r0*16 + r1*4 + kb.  Each byte is the UE5M3 byte minus ((8 + shift) << 3), i.e.
 * the same scale divided by 2^shift in UE4M3, clamped to UE4M3's normal range 0x08..0x7E when
 * it does not fit; such rows are flagged in window_record (see above).  sf_raw (nullable, same
 * size and layout) receives the unmodified UE5M3 bytes, which the row placement and the
 * recomputation pass read; the one-pass operand quantizers write 0 there for a block whose
 * elements are all zero (its scale is immaterial).
 * No reference counterpart.
 */
size_t ue5m3_packed_scales_bytes(int64_t rows, int64_t K);
int ue5m3_pack_scales_ue4m3(const uint8_t *scales, int64_t rows, int64_t K, int block, int two_d,
                            int shift, uint8_t *sf_out, uint8_t *sf_raw, int *window_record,
                            void *stream);

/* count bytes of the UE5M3_BITS_PHILOX stream {seed, stream} starting at element 0 */
int ue5m3_philox_bytes(const void *seed_stream_dev, int64_t count, uint8_t *out, void *stream);

/*
 * One-pass quantizer for an operand of ue5m3_gemm_fp4 whose reduction axis is the contiguous
 * axis of x (blocking UE5M3_BLOCK_ROW or UE5M3_BLOCK_2D; cols = K, K % 64 == 0): same
 * arithmetic as ue5m3_quantize (formats.py:350-457, backends/triton/quantization.py:34-200),
 * writing codes [rows, K/2] and, when sf != NULL, the scales directly in the layout and UE4M3
 * re-bias of ue5m3_pack_scales_ue4m3 (shift, sf_raw, window_record as there).  scales
 * (optional) receives the raw UE5M3 bytes as ue5m3_quantize would write them.  x 32-byte aligned, codes
 * and sf 16-byte aligned.  Operands whose reduction axis is strided (UE5M3_BLOCK_COL,
 * transposed outputs) go through ue5m3_quantize + ue5m3_pack_scales_ue4m3.
 */
int ue5m3_quantize_fp4_operand(const void *x, int dtype, int64_t rows, int64_t cols, int block,
                               int blocking, const float *amax_dev, float target, int rounding,
                               const void *bits, int bits_dtype, int shift, uint8_t *codes,
                               uint8_t *sf, uint8_t *sf_raw, uint8_t *scales, int *window_record,
                               void *stream);

/*
 * The same for an operand that is x transposed: the reduction axis is the ROW axis of x
 * (blocking UE5M3_BLOCK_COL: block x 1 blocks, or UE5M3_BLOCK_2D), rows = K, K % 64 == 0.
 * Writes codes_t [cols, K/2] and the scale atoms of the cols x K operand (dgrad W^T, wgrad dY^T
 * and X^T of nn/linear.py:359-363,385 without the transposed fp32 copies).
 */
int ue5m3_quantize_fp4_operand_t(const void *x, int dtype, int64_t rows, int64_t cols, int block,
                                 int blocking, const float *amax_dev, float target, int rounding,
                                 const void *bits, int bits_dtype, int shift, uint8_t *codes_t,
                                 uint8_t *sf_t, uint8_t *sf_raw_t, int *window_record,
                                 void *stream);

/*
 * A weight in both orientations from one read: x [rows, cols] with B x B blocks
 * (UE5M3_BLOCK_2D), ties-to-even -> the operand x (codes [rows, cols/2], its atoms, raw atoms
 * and window record) AND the operand x^T (codes_t [cols, rows/2], ...), i.e. what
 * ue5m3_quantize_fp4_operand and ue5m3_quantize_fp4_operand_t write, bit for bit: B x B blocks
 * have the same scale in both orientations (formats.py:294-328), so the forward GEMM's W and the
 * data-gradient GEMM's W^T of one training step (nn/linear.py:312-313,359-363 of the reference
 * re-quantize the weight for each) come out of one launch.  rows % 64 == 0 and cols % 64 == 0.
 */
int ue5m3_quantize_fp4_operand_both(const void *x, int dtype, int64_t rows, int64_t cols, int block,
                                    const float *amax_dev, float target, int shift,
                                    uint8_t *codes, uint8_t *sf, uint8_t *sf_raw,
                                    int *window_record, uint8_t *codes_t, uint8_t *sf_t,
                                    uint8_t *sf_raw_t, int *window_record_t, void *stream);

/*
 * The weight-gradient operands of the TE-settings comparator (nn/linear.py:23-40,80-114,
 * 389-400): the operand is x^T with the fixed-sign, normalized B=16 Hadamard transform applied
 * along its reduction axis (the rows of x) before 16 x 1 block quantization.
 * ue5m3_rht_amax_t writes max |transformed value| (the D=1 reference of the transformed
 * operand) to amax_out_dev; ue5m3_quantize_fp4_operand_t_rht quantizes with that reference.
 * rows % 16 == 0 (amax) / rows % 64 == 0 (operand), rows of x 16-byte multiples.
 */
int ue5m3_rht_amax_t(const void *x, int dtype, int64_t rows, int64_t cols, float *amax_out_dev,
                     void *stream);
int ue5m3_quantize_fp4_operand_t_rht(const void *x, int dtype, int64_t rows, int64_t cols,
                                     const float *amax_dev, float target, int rounding,
                                     const void *bits, int bits_dtype, int shift, uint8_t *codes_t,
                                     uint8_t *sf_t, uint8_t *sf_raw_t, int *window_record,
                                     void *stream);

/*
 * Probe-matched GEMM on PACKED operands with the FP4 block-scaled tensor cores:
 *   out[M,N] = epilogue( 2^shift_sum * sum over K=64 issues of (A codes x scales) . (B codes x scales) )
 * a_codes [M, K/2], b_codes [N, K/2] (E2M1 nibbles, reduction axis contiguous); a_sf, b_sf from
 * ue5m3_pack_scales_ue4m3; shift_sum = shift_a + shift_b.  One MMA instruction per K=64 issue,
 * accumulated by the tensor core in FP32; epilogue as ue5m3_gemm_issue_rz_bf16 (snap, alpha,
 * bias, cast).  a_record / b_record (nullable): the operands' window records after
 * ue5m3_place_row_windows; rows placed there are rescaled by their own power of two.
 * Replaces the same reference code as ue5m3_gemm_issue_rz_bf16
 * (backends/triton/gemm.py:26-160, api.py:72-83).  K % 64 == 0, (K/2) % 16 == 0.
 */
int ue5m3_gemm_fp4(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                   const uint8_t *b_sf, int64_t M, int64_t N, int64_t K, int shift_sum, int snap,
                   const float *alpha_dev, const float *amax_a_dev, const float *amax_b_dev,
                   float inv_denominator, const void *bias, int bias_dtype, void *out,
                   int out_dtype, int64_t ldo, const int *a_record, const int *b_record,
                   int *status_dev, void *stream);

/*
 * Second half of the FP4 product for operands whose window records are not empty: called
 * after ue5m3_gemm_fp4 on the same stream with the same epilogue arguments, it overwrites
 * the output rows listed in a_record and the output columns listed in b_record (the lists that
 * ue5m3_place_row_windows wrote; everything,
 * when a list overflowed) with the result of the issue-RZ kernel of ue5m3_gemm_issue_rz_bf16
 * on the exact encoded operands, which its producer warps decode from the codes and the raw
 * UE5M3 scale atoms (sf_raw of the quantizers) straight into shared memory.  The records are
 * read on the device: no host synchronisation, no workspace, and with empty records the two
 * launches (one per tile width: listed rows, listed columns) return at once.  This is what makes the FP4 path produce the reference model's
 * result for every tensor the reference accepts (its UE5M3 scales have no window,
 * formats.py:125-134, backends/triton/quantization.py:116-127).
 */
int ue5m3_gemm_fp4_fallback(const uint8_t *a_codes, const uint8_t *a_sf_raw, const int *a_record,
                            const uint8_t *b_codes, const uint8_t *b_sf_raw, const int *b_record,
                            int64_t M, int64_t N, int64_t K, int snap, const float *alpha_dev,
                            const float *amax_a_dev, const float *amax_b_dev,
                            float inv_denominator, const void *bias, int bias_dtype, void *out,
                            int out_dtype, int64_t ldo, int *status_dev, void *stream);

/*
 * ue5m3_gemm_fp4_fallback with a caller-provided device workspace of at least
 * ue5m3_fallback_workspace_bytes(M, N, K) bytes (16-byte aligned; contents need not be
 * preserved between calls): every needed operand row is decoded once into the workspace
 * (listed rows gathered; the other operand in full, and only when something is listed) and
 * the issue-RZ kernel of ue5m3_gemm_issue_rz_bf16 runs on it, instead of decoding per tile
 * inside the GEMM.  Same arguments, same results, still driven by the records on the device
 * (two launches that return at once when the records are empty); several times faster when
 * hundreds or thousands of rows are listed.  No reference counterpart beyond that of
 * ue5m3_gemm_fp4_fallback.
 */
size_t ue5m3_fallback_workspace_bytes(int64_t M, int64_t N, int64_t K);
int ue5m3_gemm_fp4_fallback_ws(const uint8_t *a_codes, const uint8_t *a_sf_raw, const int *a_record,
                               const uint8_t *b_codes, const uint8_t *b_sf_raw,
                               const int *b_record, int64_t M, int64_t N, int64_t K, int snap,
                               const float *alpha_dev, const float *amax_a_dev,
                               const float *amax_b_dev, float inv_denominator, const void *bias,
                               int bias_dtype, void *out, int out_dtype, int64_t ldo,
                               void *workspace, size_t workspace_bytes, int *status_dev,
                               void *stream);

/*
 * Test hook: compares the software E2M1 ties-to-even rounding with the sm_100a
 * cvt.rn.satfinite.e2m1x2.f32 instruction over `count` consecutive fp32 bit
 * patterns starting at `first_bits`; mismatch_count_dev[0] receives the number
 * of differing finite inputs, first_mismatch_dev[0] the smallest differing
 * pattern.  No reference counterpart.
 */
int ue5m3_test_e2m1_cvt(uint32_t first_bits, uint64_t count,
                        unsigned long long *mismatch_count_dev,
                        uint32_t *first_mismatch_dev, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* UE5M3_FP4_H_ */
