// Packed-FP4 GEMM on the sm_100a block-scaled tensor cores.
//
//   out[M,N] = epilogue( sum_k  A[m,k] * B[n,k] ),   A, B = E2M1 codes x per-16 block scales
//
// Operands are the packed outputs of the quantizer (two E2M1 nibbles per byte, reduction
// axis contiguous).  The block scales are UE5M3 bytes re-biased to the tensor core's UE4M3
// scale type by a per-tensor power of two (ue5m3_pack_scales_ue4m3 below): both formats
// carry three fraction bits, so inside a 15-binade window the re-biased scale is the same
// number divided by 2^shift, and the epilogue multiplies the result by 2^(shift_a+shift_b),
// which is exact.  A row whose scales do not fit the window at the tensor's shift is flagged in
// the operand's window record by the quantizer; ue5m3_place_row_windows (window_place.cu) gives
// such a row a shift of its own where its scales span at most 15 binades - the epilogue here then
// also multiplies by 2^(row shift + column shift) - and lists the rows that still do not fit,
// whose output rows / columns ue5m3_gemm_fp4_fallback (gemm_fallback.cu) overwrites afterwards.
//
// One tcgen05.mma.kind::mxf4nvf4.block_scale.scale_vec::4X instruction multiplies a
// 128 x 256 x 64 slab (256 x 256 x 64 for a CTA pair), i.e. exactly one K=64 issue of the
// reference model (four 16-blocks per operand row), and accumulates it into the FP32 tile in
// TMEM; the K loop is a plain chain of such instructions.
//
// Two kernels.  gemm_fp4_kernel (M <= 128): persistent CTAs (one per SM) walk 128 x 256 output
// tiles; a stage holds K = 256 (128 bytes per row, one 128-byte swizzle atom): A 16 KiB +
// B 32 KiB + scale atoms 2 + 4 KiB; four stages.  Warp 0 = TMA producer, warp 1 = MMA issue,
// warps 2..9 = epilogue (lane quadrant = warp % 4, column half = (warp - 2) / 4), warps 10..11 =
// scale copies shared -> TMEM.  gemm_fp4_pair_kernel (the default otherwise): the same roles in a
// cluster of two CTAs, described above its definition.  All waits are clock-bounded; a launch
// that finds a failure recorded in its status word fills its output with NaN instead of working.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "abi_common.cuh"
#include "alpha_spec.cuh"
#include "dead_fill.cuh"
#include "tcgen05_ptx.cuh"
#include "window_record.cuh"

namespace ue5m3 {

using namespace ptx;

constexpr int kFM = 128;            // tile rows
constexpr int kFN = 256;            // tile columns
constexpr int kFKStage = 256;       // reduction elements per stage (128 bytes per row)
constexpr int kFKMma = 64;          // reduction elements per MMA = one issue
constexpr int kFStages = 4;
constexpr int kFScaleWarps = 2;
constexpr int kFScaleWarp0 = 10;
constexpr int kFThreads = 32 * (kFScaleWarp0 + kFScaleWarps);  // producer, MMA, 8 epilogue, scale-copy warps
constexpr int kFEpilogueWarps = 8;
constexpr uint32_t kFTmemCols = 512;
constexpr uint32_t kSfAtomBytes = 512;  // 128 rows x 4 scale bytes
constexpr uint32_t kFBytesA = kFM * kFKStage / 2;
constexpr uint32_t kFBytesB = kFN * kFKStage / 2;
constexpr uint32_t kFBytesSfa = 4 * kSfAtomBytes;
constexpr uint32_t kFBytesSfb = 8 * kSfAtomBytes;
constexpr uint32_t kFStageBytes = kFBytesA + kFBytesB + kFBytesSfa + kFBytesSfb;
// TMEM columns: accumulator 0..255, scale slots of A from 256 (4 per MMA), of B from 320 (8 per MMA)
constexpr uint32_t kTmemSfa = 256;
constexpr uint32_t kTmemSfb = 320;

struct Fp4Params {
    int M, N, K;
    int snap;
    float rescale;  // 2^(shift_a + shift_b)
    AlphaSpec alpha;
    const void* bias;
    int bias_dtype;
    void* out;
    int out_dtype;
    long long ldo;
    int* status;
    const uint8_t* sfa;  // [ceil(M/128)][K/64][512]
    const uint8_t* sfb;  // [ceil(N/128)][K/64][512]
    int tiles_m, tiles_n;
    // window records of the operands (null: none).  Rows that got a scale window of their own
    // (window_place.cu) carry an extra exponent there; the epilogue multiplies by 2^(a[row] + b[col]).
    const int* rec_a;
    const int* rec_b;
};

// per-row exponent tables of the operands: null unless the record says that rows were placed
struct RowShifts {
    const int* a;
    const int* b;
};

__device__ __forceinline__ RowShifts resolve_row_shifts(const Fp4Params& p) {
    RowShifts shifts;
    shifts.a = (p.rec_a && __ldg(p.rec_a + kRecPlaced) > 0) ? rec_row_shift(p.rec_a, p.M) : nullptr;
    shifts.b = (p.rec_b && __ldg(p.rec_b + kRecPlaced) > 0) ? rec_row_shift(p.rec_b, p.N) : nullptr;
    return shifts;
}

struct __align__(8) Fp4Barriers {
    unsigned long long full[kFStages];
    unsigned long long empty[kFStages];
    unsigned long long sf_full[kFStages];
    unsigned long long tmem_full;
    unsigned long long tmem_empty;
    uint32_t tmem_base;
    int abort_flag;
    Fp4Params params;   // a copy that out-of-line code can point to
};

// D[tmem] (+)= A[smem] * B[smem] with per-16 block scales read from TMEM.
__device__ __forceinline__ void umma_fp4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                         uint32_t idesc, uint32_t accumulate, uint32_t tmem_sfa,
                                         uint32_t tmem_sfb) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

// 32 rows x 16 bytes from shared memory into 4 TMEM columns of every lane quadrant.
__device__ __forceinline__ void tmem_copy_sf(uint32_t taddr, uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc)
                 : "memory");
}

// Instruction descriptor of the block-scaled kind: A = B = E2M1 (code 1), both K-major,
// UE4M3 scales, K = 64.
__host__ __device__ constexpr uint32_t make_idesc_fp4(int m, int n) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Epilogue arithmetic and stores of one thread: 128 accumulator values of one output row
// (columns [tile_n * 256 + h * 128, + 128)): rescale by 2^shift, snap, alpha, bias, cast.
template <bool kShifts>
__device__ __forceinline__ void fp4_store_row(const Fp4Params& p, const RowShifts shifts, const uint32_t (&v)[4][32],
                                              long long row, int tile_n, int h, float alpha) {
    const float row_factor = (kShifts && shifts.a) ? __fmul_rn(p.rescale, exp2_int(__ldg(shifts.a + row))) : p.rescale;
#pragma unroll
    for (int chunk = 0; chunk < 4; ++chunk) {
        const int col0 = tile_n * kFN + h * (kFN / 2) + chunk * 32;
        if (col0 >= p.N) continue;
        float c[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float x = __fmul_rn(__uint_as_float(v[chunk][i]), row_factor);
            if (kShifts && shifts.b && col0 + i < p.N) x = __fmul_rn(x, exp2_int(__ldg(shifts.b + col0 + i)));
            if (p.snap) x = __fmul_rn(rint_rne(__fmul_rn(x, 1024.0f)), 0.0009765625f);
            x = __fmul_rn(x, alpha);   // alpha is 1 when the caller gave none: an exact no-op
            c[i] = x;
        }
        if (p.bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                int col = col0 + i;
                if (col < p.N) {
                    float bv = p.bias_dtype == UE5M3_DTYPE_BF16
                                   ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col])
                                   : static_cast<const float*>(p.bias)[col];
                    c[i] = __fadd_rn(c[i], bv);
                }
            }
        }
        if (p.out_dtype == UE5M3_DTYPE_BF16) {
            __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + row * p.ldo + col0;
            const bool vec = (p.ldo % 8) == 0 && ((uintptr_t)p.out % 16) == 0;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                if (vec && col0 + i + 8 <= p.N) {
                    uint4 w;
                    uint32_t hb[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        hb[e] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(c[i + e]));
                    w.x = hb[0] | (hb[1] << 16); w.y = hb[2] | (hb[3] << 16);
                    w.z = hb[4] | (hb[5] << 16); w.w = hb[6] | (hb[7] << 16);
                    *reinterpret_cast<uint4*>(out + i) = w;
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        if (col0 + i + e < p.N) out[i + e] = __float2bfloat16_rn(c[i + e]);
                }
            }
        } else {
            float* out = static_cast<float*>(p.out) + row * p.ldo + col0;
            const bool vec = (p.ldo % 4) == 0 && ((uintptr_t)p.out % 16) == 0;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                if (vec && col0 + i + 4 <= p.N) {
                    *reinterpret_cast<float4*>(out + i) = make_float4(c[i], c[i + 1], c[i + 2], c[i + 3]);
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (col0 + i + e < p.N) out[i + e] = c[i + e];
                }
            }
        }
    }
}

// The same epilogue arithmetic for one warp's 32 rows x 128 columns with BF16 output, stored
// through a per-warp 32 x 128-byte staging buffer so that every store instruction writes four
// full 128-byte lines (lane = 16 bytes of a row) instead of 16 bytes in each of 32 rows.
// 16-byte chunk c of row r sits at chunk position c ^ (r & 7): conflict-free both ways.
// Requires the whole 128-column half inside N, ldo % 8 == 0 and a 16-byte aligned base.
constexpr uint32_t kStageBytesPerWarp = 32 * 128;

template <bool kShifts>
__device__ __forceinline__ void fp4_store_rows_staged_bf16(const Fp4Params& p, const RowShifts shifts,
                                                           const uint32_t (&v)[4][32], long long row0, int tile_n,
                                                           int h, float alpha, unsigned char* stage, int lane) {
    float row_factor = p.rescale;
    if (kShifts && shifts.a && row0 + lane < p.M) row_factor = __fmul_rn(row_factor, exp2_int(__ldg(shifts.a + row0 + lane)));
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        const int col0 = tile_n * kFN + h * (kFN / 2) + pass * 64;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            uint32_t hb[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int idx = pass * 64 + c * 8 + e;
                float x = __fmul_rn(__uint_as_float(v[idx >> 5][idx & 31]), row_factor);
                if (kShifts && shifts.b) x = __fmul_rn(x, exp2_int(__ldg(shifts.b + col0 + c * 8 + e)));
                if (p.snap) x = __fmul_rn(rint_rne(__fmul_rn(x, 1024.0f)), 0.0009765625f);
                x = __fmul_rn(x, alpha);   // alpha is 1 when the caller gave none: an exact no-op
                if (p.bias) {
                    const int col = col0 + c * 8 + e;
                    const float bv = p.bias_dtype == UE5M3_DTYPE_BF16
                                         ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col])
                                         : static_cast<const float*>(p.bias)[col];
                    x = __fadd_rn(x, bv);
                }
                hb[e] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x));
            }
            uint4 w;
            w.x = hb[0] | (hb[1] << 16); w.y = hb[2] | (hb[3] << 16);
            w.z = hb[4] | (hb[5] << 16); w.w = hb[6] | (hb[7] << 16);
            *reinterpret_cast<uint4*>(stage + lane * 128 + ((c ^ (lane & 7)) << 4)) = w;
        }
        __syncwarp();
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
        for (int r4 = 0; r4 < 8; ++r4) {
            const int r = r4 * 4 + (lane >> 3);
            const int c = lane & 7;
            const uint4 w = *reinterpret_cast<const uint4*>(stage + r * 128 + ((c ^ (r & 7)) << 4));
            const long long row = row0 + r;
            if (row < p.M) *reinterpret_cast<uint4*>(out + row * p.ldo + col0 + c * 8) = w;
        }
        __syncwarp();
    }
}

// One epilogue warp's share of one tile: 32 accumulator rows x 128 columns out of TMEM (which is
// released as soon as the values are in registers: `release`), then arithmetic and stores.
// kShifts = true is the rare case that an operand has rows with a scale window of their own;
// it lives in a function of its own (below) so that the common case keeps its registers.
struct TileEpilogue {
    uint32_t taddr;               // TMEM address of this warp's lanes and columns
    long long row0;               // first output row of this warp
    int rows_per_thread_valid;    // unused padding to keep the struct trivially copyable
    int tile_n, h, lane;
    float alpha;
    unsigned char* stage;         // per-warp staging buffer, or null: direct stores
    unsigned long long* release_local;   // mbarrier to arrive on after the TMEM reads (this CTA's) ...
    uint32_t release_cluster;            // ... or its cluster address in the leader CTA (pair kernel); 0 = use local
};

template <bool kShifts>
__device__ __forceinline__ void fp4_tile_epilogue(const Fp4Params& p, const RowShifts shifts, const TileEpilogue& t) {
    uint32_t v[4][32];
#pragma unroll
    for (int chunk = 0; chunk < 4; ++chunk) tmem_load_32_async(t.taddr + chunk * 32, v[chunk]);
    tmem_wait_ld();
    tcgen05_fence_before();
    __syncwarp();
    if (t.lane == 0) {
        if (t.release_cluster) mbar_arrive_cluster(t.release_cluster);
        else mbar_arrive(t.release_local);
    }
    if (t.stage) {
        fp4_store_rows_staged_bf16<kShifts>(p, shifts, v, t.row0, t.tile_n, t.h, t.alpha, t.stage, t.lane);
        return;
    }
    const long long row = t.row0 + t.lane;
    if (row < p.M) fp4_store_row<kShifts>(p, shifts, v, row, t.tile_n, t.h, t.alpha);
}

// everything by value or through shared memory: a reference to the kernel's parameters or to a
// local struct would force a copy of them onto the caller's stack
__device__ __noinline__ void fp4_tile_epilogue_with_row_shifts(const Fp4Params* params_in_shared, const int* shift_a,
                                                               const int* shift_b, uint32_t taddr, long long row0,
                                                               int tile_n, int h, int lane, float alpha,
                                                               unsigned char* stage, unsigned long long* release_local,
                                                               uint32_t release_cluster) {
    TileEpilogue t;
    t.taddr = taddr; t.row0 = row0; t.rows_per_thread_valid = 0; t.tile_n = tile_n; t.h = h; t.lane = lane;
    t.alpha = alpha; t.stage = stage; t.release_local = release_local; t.release_cluster = release_cluster;
    fp4_tile_epilogue<true>(*params_in_shared, RowShifts{shift_a, shift_b}, t);
}

// tile index -> (tile_m, tile_n): groups of 8 tile rows sweep the tile columns together
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tile_m, int& tile_n) {
    constexpr int kGroupM = 8;
    const int tiles_per_group = kGroupM * tiles_n;
    const int group = tile / tiles_per_group;
    const int first_m = group * kGroupM;
    const int group_m = (tiles_m - first_m) < kGroupM ? (tiles_m - first_m) : kGroupM;
    tile_m = first_m + (tile % tiles_per_group) % group_m;
    tile_n = (tile % tiles_per_group) / group_m;
}

// Persistent: CTA c works on tiles c, c + gridDim.x, ...  The accumulator is drained into
// registers by eight epilogue warps right after a tile's last MMA and released at once, so
// the next tile's MMAs overlap the epilogue arithmetic and the global stores.
__global__ void __launch_bounds__(kFThreads, 1)
gemm_fp4_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const Fp4Params p) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    Fp4Barriers* bars = reinterpret_cast<Fp4Barriers*>(smem + kFStages * kFStageBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_issues = p.K / kFKMma;          // MMAs along K
    const int num_stages = (num_issues + 3) / 4;  // stages along K
    const int sf_k = num_issues;                  // scale atoms per row tile
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kFStages; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 1);
            mbar_init(&bars->sf_full[s], kFScaleWarps);
        }
        mbar_init(&bars->tmem_full, 1);
        mbar_init(&bars->tmem_empty, kFEpilogueWarps);
        bars->abort_flag = (p.status && *((volatile int*)p.status) != 0) ? 1 : 0;
        bars->params = p;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&bars->tmem_base, kFTmemCols);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *((volatile uint32_t*)&bars->tmem_base);
    const bool dead = *((volatile int*)&bars->abort_flag) != 0;

    if (dead) {
        // no work after a recorded failure: mark this CTA's tiles and fall through to the common exit
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            int tile_m, tile_n;
            tile_coords(tile, p.tiles_m, p.tiles_n, tile_m, tile_n);
            fill_tile_nan(p.out, p.out_dtype == UE5M3_DTYPE_BF16, p.ldo, tile_m * kFM, tile_n * kFN, kFM, kFN, p.M, p.N);
        }
    } else if (warp == 0) {
        // ---------------- producer: operands by TMA, scale atoms by bulk copy ----------------
        {
            uint32_t g = 0;  // stage counter across tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int tile_m, tile_n;
                tile_coords(tile, p.tiles_m, p.tiles_n, tile_m, tile_n);
                const int m0 = tile_m * kFM, n0 = tile_n * kFN;
                const bool second_b_tile = (2 * tile_n + 1) * 128 < p.N;  // columns 128..255 exist
                for (int j = 0; j < num_stages; ++j, ++g) {
                    const int s = g % kFStages;
                    const uint32_t use = g / kFStages;
                    if (use > 0) {
                        ok = mbar_wait(&bars->empty[s], (use - 1) & 1, &bars->abort_flag, p.status, 1, j);
                        ok = __all_sync(0xFFFFFFFFu, ok);
                        if (!ok) break;
                    }
                    unsigned char* sa = smem + s * kFStageBytes;
                    unsigned char* sb = sa + kFBytesA;
                    unsigned char* ssfa = sb + kFBytesB;
                    unsigned char* ssfb = ssfa + kFBytesSfa;
                    const int issues_here = (num_issues - 4 * j) < 4 ? (num_issues - 4 * j) : 4;
                    const uint32_t sf_bytes = (uint32_t)issues_here * kSfAtomBytes;
                    const uint32_t tx = kFBytesA + kFBytesB + sf_bytes * (second_b_tile ? 3u : 2u);
                    if (elect_one()) {
                        mbar_arrive_expect_tx(&bars->full[s], tx);
                        tma_load_2d(sa, &map_a, &bars->full[s], j * (kFKStage / 2), m0);
                        tma_load_2d(sb, &map_b, &bars->full[s], j * (kFKStage / 2), n0);
                        bulk_load(ssfa, p.sfa + ((size_t)tile_m * sf_k + 4 * j) * kSfAtomBytes, sf_bytes,
                                  &bars->full[s]);
                        bulk_load(ssfb, p.sfb + ((size_t)(2 * tile_n) * sf_k + 4 * j) * kSfAtomBytes, sf_bytes,
                                  &bars->full[s]);
                        if (second_b_tile)
                            bulk_load(ssfb + 4 * kSfAtomBytes,
                                      p.sfb + ((size_t)(2 * tile_n + 1) * sf_k + 4 * j) * kSfAtomBytes, sf_bytes,
                                      &bars->full[s]);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        {
            constexpr uint32_t idesc = make_idesc_fp4(kFM, kFN);
            uint32_t g = 0;
            bool ok = true;
            bool ready = false;  // the current stage's scale barrier was already seen complete
            int it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                if (it > 0) {  // the previous tile must have left the accumulator
                    ok = mbar_wait(&bars->tmem_empty, (it - 1) & 1, &bars->abort_flag, p.status, 2, it);
                    ok = __all_sync(0xFFFFFFFFu, ok);
                    if (!ok) break;
                    tcgen05_fence_after();
                }
                for (int j = 0; j < num_stages; ++j, ++g) {
                    const int s = g % kFStages;
                    // scales of this stage are in TMEM, which also means its operands have landed
                    if (!ready) {
                        ok = mbar_wait(&bars->sf_full[s], (g / kFStages) & 1, &bars->abort_flag, p.status, 3, j);
                        ok = __all_sync(0xFFFFFFFFu, ok);
                        if (!ok) break;
                    }
                    tcgen05_fence_after();
                    // probe the next stage's barrier before the issue (its latency overlaps the issue)
                    const uint32_t gn = g + 1;
                    const bool next_ready = mbar_test_wait(&bars->sf_full[gn % kFStages], (gn / kFStages) & 1);
                    const uint32_t sa = smem_u32(smem + s * kFStageBytes);
                    const uint32_t sb = sa + kFBytesA;
                    const uint64_t desc_a = smem_desc_sw128(sa);
                    const uint64_t desc_b = smem_desc_sw128(sb);
                    const uint32_t t_sfa = tmem_base + kTmemSfa + (uint32_t)s * 16u;
                    const uint32_t t_sfb = tmem_base + kTmemSfb + (uint32_t)s * 32u;
                    const int issues_here = (num_issues - 4 * j) < 4 ? (num_issues - 4 * j) : 4;
                    // 64 four-bit elements = 32 bytes inside the swizzle atom: +2 in 16-byte units
                    if (issues_here == 4) {
                        if (elect_one()) {
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                umma_fp4(tmem_base, desc_a + (uint64_t)(2 * k), desc_b + (uint64_t)(2 * k), idesc,
                                         (j > 0 || k > 0) ? 1u : 0u, t_sfa + k * 4, t_sfb + k * 8);
                            umma_commit(&bars->empty[s]);
                        }
                    } else {
                        if (elect_one()) {
                            for (int k = 0; k < issues_here; ++k)
                                umma_fp4(tmem_base, desc_a + (uint64_t)(2 * k), desc_b + (uint64_t)(2 * k), idesc,
                                         (j > 0 || k > 0) ? 1u : 0u, t_sfa + k * 4, t_sfb + k * 8);
                            umma_commit(&bars->empty[s]);
                        }
                    }
                    __syncwarp();
                    ready = __all_sync(0xFFFFFFFFu, next_ready);
                }
                if (ok && elect_one()) umma_commit(&bars->tmem_full);
                __syncwarp();
            }
        }
    } else if (warp >= kFScaleWarp0) {
        // ---------------- scale atoms: shared memory -> TMEM, one slot ring entry per stage ----------------
        // A landed stage (full) implies the MMAs that last read this stage's TMEM scale slots
        // have completed, because the producer refilled the stage only after their commit.
        {
            uint32_t g = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                for (int j = 0; j < num_stages; ++j, ++g) {
                    const int s = g % kFStages;
                    ok = mbar_wait(&bars->full[s], (g / kFStages) & 1, &bars->abort_flag, p.status, 5, j);
                    ok = __all_sync(0xFFFFFFFFu, ok);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t ssfa = smem_u32(smem + s * kFStageBytes) + kFBytesA + kFBytesB;
                    const uint32_t ssfb = ssfa + kFBytesSfa;
                    const int issues_here = (num_issues - 4 * j) < 4 ? (num_issues - 4 * j) : 4;
                    // the issuing thread is the bottleneck of these copies: split them over the warps
                    if (elect_one()) {
                        for (int k = warp - kFScaleWarp0; k < issues_here; k += kFScaleWarps) {
                            const uint32_t slot = (uint32_t)(s * 4 + k);
                            const uint32_t t_sfa = tmem_base + kTmemSfa + slot * 4;
                            const uint32_t t_sfb = tmem_base + kTmemSfb + slot * 8;
                            tmem_copy_sf(t_sfa, smem_desc_noswizzle_32x16(ssfa + k * kSfAtomBytes));
                            tmem_copy_sf(t_sfb, smem_desc_noswizzle_32x16(ssfb + k * kSfAtomBytes));
                            tmem_copy_sf(t_sfb + 4, smem_desc_noswizzle_32x16(ssfb + (4 + k) * kSfAtomBytes));
                        }
                        umma_commit(&bars->sf_full[s]);
                    }
                    __syncwarp();
                }
            }
        }
    } else {
        // ---------------- epilogue: TMEM -> registers (release) -> arithmetic -> global ----------------
        const int q = warp & 3;          // TMEM lane quadrant
        const int h = (warp - 2) >> 2;   // column half of the tile
        const float alpha = alpha_value(p.alpha);
        const RowShifts shifts = resolve_row_shifts(p);
        const bool has_shifts = shifts.a != nullptr || shifts.b != nullptr;
        int it = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
            int tile_m, tile_n;
            tile_coords(tile, p.tiles_m, p.tiles_n, tile_m, tile_n);
            bool ok = mbar_wait(&bars->tmem_full, it & 1, &bars->abort_flag, p.status, 4, it);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            TileEpilogue t;
            t.taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * (kFN / 2));
            t.row0 = (long long)tile_m * kFM + q * 32;
            t.rows_per_thread_valid = 0;
            t.tile_n = tile_n; t.h = h; t.lane = lane; t.alpha = alpha;
            t.stage = nullptr;
            t.release_local = &bars->tmem_empty;
            t.release_cluster = 0u;
            if (has_shifts)
                fp4_tile_epilogue_with_row_shifts(&bars->params, shifts.a, shifts.b, t.taddr, t.row0, t.tile_n, t.h, t.lane,
                                                  t.alpha, t.stage, t.release_local, t.release_cluster);
            else fp4_tile_epilogue<false>(p, shifts, t);
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kFTmemCols);
    }
}

// ---------------------------------------------------------------------------------------
// CTA-pair variant (cluster of two CTAs, tcgen05 cta_group::2): one 256 x 256 output tile per
// pair.  Each CTA loads its own 128 rows of A and its own half (128 rows) of the 256-column B
// tile, so a K=256 stage moves 38 KiB per CTA instead of 54 KiB and every MMA reads 8 KiB of
// shared memory per CTA instead of 12 KiB.  The leader CTA (rank 0) issues the scale copies,
// the MMAs and the commits for both; every load of both CTAs reports to the leader's `full`
// barrier (plain per-CTA TMA loads with cta_group::2, each CTA fetching only its own data).
// Each CTA drains its own 128 accumulator rows; BF16 output leaves through a 4 KiB per-warp
// staging buffer as full 128-byte lines.  The MMA warp's time per stage is what the tensor
// pipe can be fed at (measured: 128 cycles per MMA when nothing else delays the issue), so its
// loop is kept short: the four issues of a full stage are unrolled and the next stage's scale
// barrier is probed before the current issue.
// ---------------------------------------------------------------------------------------
constexpr int kPM = 256;
constexpr int kPStages = 5;
constexpr uint32_t kPBytesA = 128 * kFKStage / 2;
constexpr uint32_t kPBytesB = 128 * kFKStage / 2;
constexpr uint32_t kPStageBytes = kPBytesA + kPBytesB + kFBytesSfa + kFBytesSfb;
constexpr uint32_t kPTmemSfa = 256;                      // kPStages * 4 slots x 4 columns
constexpr uint32_t kPTmemSfb = kPTmemSfa + kPStages * 16;  // kPStages * 4 slots x 8 columns
static_assert(kPTmemSfb + kPStages * 32 <= 512, "TMEM columns");

struct __align__(8) Fp4PairBarriers {
    unsigned long long full[kPStages];     // leader's: bytes of both CTAs
    unsigned long long empty[kPStages];    // each CTA's own, signalled by the leader's commits
    unsigned long long sf_full[kPStages];  // leader's
    unsigned long long tmem_full;          // each CTA's own
    unsigned long long tmem_empty;         // leader's: epilogue warps of both CTAs
    uint32_t tmem_base;
    int abort_flag;
    Fp4Params params;                      // a copy that out-of-line code can point to
};

__device__ __forceinline__ void umma_fp4_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate, uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

// the copy runs in both CTAs, each from its own shared memory into its own TMEM
__device__ __forceinline__ void tmem_copy_sf_pair(uint32_t taddr, uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// pair tile index -> (tile_m, tile_n): groups of 16 tile rows (4096 rows of A) sweep the columns;
// the 74 tiles in flight then cover 16 x ~5 tiles (measured on the benchmark shape against groups
// of 2, 4, 8 and 32: 0.325, 0.324, 0.312 and 0.316 ms; 16: 0.307 ms)
__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tile_m, int& tile_n) {
    constexpr int kGroupM = 16;
    const int tiles_per_group = kGroupM * tiles_n;
    const int group = tile / tiles_per_group;
    const int first_m = group * kGroupM;
    const int group_m = (tiles_m - first_m) < kGroupM ? (tiles_m - first_m) : kGroupM;
    tile_m = first_m + (tile % tiles_per_group) % group_m;
    tile_n = (tile % tiles_per_group) / group_m;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kFThreads, 1)
gemm_fp4_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                     const Fp4Params p) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* stage_base = smem + kPStages * kPStageBytes;  // epilogue staging, 4 KiB per warp
    Fp4PairBarriers* bars = reinterpret_cast<Fp4PairBarriers*>(stage_base + kFEpilogueWarps * kStageBytesPerWarp);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    const int num_issues = p.K / kFKMma;
    const int num_stages = (num_issues + 3) / 4;
    const int sf_k = num_issues;
    const int num_tiles = p.tiles_m * p.tiles_n;  // 256 x 256 tiles
    const int where_base = 10 + 10 * (int)rank;   // wait sites reported as 11..15 (leader), 21..25 (peer)

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPStages; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 1);
            mbar_init(&bars->sf_full[s], kFScaleWarps);
        }
        mbar_init(&bars->tmem_full, 1);
        mbar_init(&bars->tmem_empty, 2 * kFEpilogueWarps);
        bars->abort_flag = (p.status && *((volatile int*)p.status) != 0) ? 1 : 0;
        bars->params = p;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc_pair(&bars->tmem_base, kFTmemCols);
    tcgen05_fence_before();
    cluster_sync_all();  // both CTAs' barriers exist before anything signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *((volatile uint32_t*)&bars->tmem_base);
    const bool dead = *((volatile int*)&bars->abort_flag) != 0;

    if (dead) {
        // no work after a recorded failure: mark this CTA's half of the pair's tiles, then the common exit
        for (int tile = pair; tile < num_tiles; tile += num_pairs) {
            int tile_m, tile_n;
            pair_tile_coords(tile, p.tiles_m, p.tiles_n, tile_m, tile_n);
            fill_tile_nan(p.out, p.out_dtype == UE5M3_DTYPE_BF16, p.ldo, tile_m * kPM + (int)rank * 128, tile_n * kFN, 128,
                          kFN, p.M, p.N);
        }
    } else if (warp == 0) {
        // ---------------- producer (both CTAs): own A rows, own B half, own scale atoms ----------------
        {
            uint32_t g = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                int tile_m, tile_n;
                pair_tile_coords(tile, p.tiles_m, p.tiles_n, tile_m, tile_n);
                const int m0 = tile_m * kPM + (int)rank * 128;
                const int n0 = tile_n * kFN + (int)rank * 128;
                const int sfa_row = (tile_m * 2 + (int)rank) * sf_k;
                const int sfb_row = (tile_n * 2) * sf_k;
                for (int j = 0; j < num_stages; ++j, ++g) {
                    const int s = g % kPStages;
                    const uint32_t use = g / kPStages;
                    if (use > 0) {
                        ok = mbar_wait_cluster(&bars->empty[s], (use - 1) & 1, &bars->abort_flag, p.status,
                                               where_base + 1, j);
                        ok = __all_sync(0xFFFFFFFFu, ok);
                        if (!ok) break;
                    }
                    unsigned char* sa = smem + s * kPStageBytes;
                    unsigned char* sb = sa + kPBytesA;
                    unsigned char* ssfa = sb + kPBytesB;
                    unsigned char* ssfb = ssfa + kFBytesSfa;
                    const uint32_t full_leader = map_to_cta(smem_u32(&bars->full[s]), 0);
                    if (elect_one()) {
                        // out-of-range rows / atoms are zero-filled and still counted, so the byte
                        // count of a stage is constant
                        if (leader) mbar_arrive_expect_tx(&bars->full[s], 2 * kPStageBytes);
                        tma_load_2d_pair(sa, &map_a, full_leader, j * (kFKStage / 2), m0);
                        tma_load_2d_pair(sb, &map_b, full_leader, j * (kFKStage / 2), n0);
                        tma_load_2d_pair(ssfa, &map_sfa, full_leader, 0, sfa_row + 4 * j);
                        tma_load_2d_pair(ssfb, &map_sfb, full_leader, 0, sfb_row + 4 * j);
                        tma_load_2d_pair(ssfb + 4 * kSfAtomBytes, &map_sfb, full_leader, 0, sfb_row + sf_k + 4 * j);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue (leader only) ----------------
        if (leader) {
            constexpr uint32_t idesc = make_idesc_fp4(kPM, kFN);
            const uint32_t empty_peer0 = map_to_cta(smem_u32(&bars->empty[0]), 1);
            const uint32_t tmem_full_peer = map_to_cta(smem_u32(&bars->tmem_full), 1);
            uint32_t g = 0;
            bool ok = true;
            bool ready = false;  // the current stage's scale barrier was already seen complete
            int it = 0;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
                if (it > 0) {  // both CTAs must have drained the previous tile
                    ok = mbar_wait_cluster(&bars->tmem_empty, (it - 1) & 1, &bars->abort_flag, p.status,
                                           where_base + 2, it);
                    ok = __all_sync(0xFFFFFFFFu, ok);
                    if (!ok) break;
                    tcgen05_fence_after();
                }
                for (int j = 0; j < num_stages; ++j, ++g) {
                    const int s = g % kPStages;
                    if (!ready) {
                        ok = mbar_wait(&bars->sf_full[s], (g / kPStages) & 1, &bars->abort_flag, p.status,
                                       where_base + 3, j);
                        ok = __all_sync(0xFFFFFFFFu, ok);
                        if (!ok) break;
                    }
                    tcgen05_fence_after();
                    // look at the next stage's barrier now: the probe's latency then overlaps the
                    // issue below instead of adding to this thread's time per stage
                    const uint32_t gn = g + 1;
                    const bool next_ready = mbar_test_wait(&bars->sf_full[gn % kPStages], (gn / kPStages) & 1);
                    const uint32_t sa = smem_u32(smem + s * kPStageBytes);
                    const uint32_t sb = sa + kPBytesA;
                    const uint64_t desc_a = smem_desc_sw128(sa);
                    const uint64_t desc_b = smem_desc_sw128(sb);
                    const uint32_t t_sfa = tmem_base + kPTmemSfa + (uint32_t)s * 16u;
                    const uint32_t t_sfb = tmem_base + kPTmemSfb + (uint32_t)s * 32u;
                    const int issues_here = (num_issues - 4 * j) < 4 ? (num_issues - 4 * j) : 4;
                    if (issues_here == 4) {
                        // fixed trip count: the four issues unroll with constant offsets
                        if (elect_one()) {
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                umma_fp4_pair(tmem_base, desc_a + (uint64_t)(2 * k), desc_b + (uint64_t)(2 * k), idesc,
                                              (j > 0 || k > 0) ? 1u : 0u, t_sfa + k * 4, t_sfb + k * 8);
                            // the stage is free in both CTAs once these MMAs have completed: one
                            // commit per CTA
                            umma_commit_pair(smem_u32(&bars->empty[s]));
                            umma_commit_pair(empty_peer0 + (uint32_t)s * 8u);
                        }
                    } else {
                        if (elect_one()) {
                            for (int k = 0; k < issues_here; ++k)
                                umma_fp4_pair(tmem_base, desc_a + (uint64_t)(2 * k), desc_b + (uint64_t)(2 * k), idesc,
                                              (j > 0 || k > 0) ? 1u : 0u, t_sfa + k * 4, t_sfb + k * 8);
                            umma_commit_pair(smem_u32(&bars->empty[s]));
                            umma_commit_pair(empty_peer0 + (uint32_t)s * 8u);
                        }
                    }
                    __syncwarp();
                    ready = __all_sync(0xFFFFFFFFu, next_ready);
                }
                if (ok && elect_one()) {
                    umma_commit_pair(smem_u32(&bars->tmem_full));
                    umma_commit_pair(tmem_full_peer);
                }
                __syncwarp();
            }
        }
    } else if (warp >= kFScaleWarp0) {
        // ---------------- scale atoms shared -> TMEM in both CTAs (issued by the leader) ----------------
        if (leader) {
            uint32_t g = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                for (int j = 0; j < num_stages; ++j, ++g) {
                    const int s = g % kPStages;
                    ok = mbar_wait_cluster(&bars->full[s], (g / kPStages) & 1, &bars->abort_flag, p.status,
                                           where_base + 5, j);
                    ok = __all_sync(0xFFFFFFFFu, ok);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t ssfa = smem_u32(smem + s * kPStageBytes) + kPBytesA + kPBytesB;
                    const uint32_t ssfb = ssfa + kFBytesSfa;
                    const int issues_here = (num_issues - 4 * j) < 4 ? (num_issues - 4 * j) : 4;
                    const int k0 = warp - kFScaleWarp0;
                    if (issues_here == 4) {
                        // fixed trip count (two issues per warp): unrolled, constant offsets
                        if (elect_one()) {
#pragma unroll
                            for (int i = 0; i < 4 / kFScaleWarps; ++i) {
                                const int k = k0 + i * kFScaleWarps;
                                const uint32_t slot = (uint32_t)(s * 4 + k);
                                const uint32_t t_sfa = tmem_base + kPTmemSfa + slot * 4;
                                const uint32_t t_sfb = tmem_base + kPTmemSfb + slot * 8;
                                tmem_copy_sf_pair(t_sfa, smem_desc_noswizzle_32x16(ssfa + k * kSfAtomBytes));
                                tmem_copy_sf_pair(t_sfb, smem_desc_noswizzle_32x16(ssfb + k * kSfAtomBytes));
                                tmem_copy_sf_pair(t_sfb + 4, smem_desc_noswizzle_32x16(ssfb + (4 + k) * kSfAtomBytes));
                            }
                            umma_commit_pair(smem_u32(&bars->sf_full[s]));
                        }
                    } else if (elect_one()) {
                        for (int k = k0; k < issues_here; k += kFScaleWarps) {
                            const uint32_t slot = (uint32_t)(s * 4 + k);
                            const uint32_t t_sfa = tmem_base + kPTmemSfa + slot * 4;
                            const uint32_t t_sfb = tmem_base + kPTmemSfb + slot * 8;
                            tmem_copy_sf_pair(t_sfa, smem_desc_noswizzle_32x16(ssfa + k * kSfAtomBytes));
                            tmem_copy_sf_pair(t_sfb, smem_desc_noswizzle_32x16(ssfb + k * kSfAtomBytes));
                            tmem_copy_sf_pair(t_sfb + 4, smem_desc_noswizzle_32x16(ssfb + (4 + k) * kSfAtomBytes));
                        }
                        umma_commit_pair(smem_u32(&bars->sf_full[s]));
                    }
                    __syncwarp();
                }
            }
        }
    } else {
        // ---------------- epilogue (both CTAs): own 128 accumulator rows ----------------
        const int q = warp & 3;
        const int h = (warp - 2) >> 2;
        const float alpha = alpha_value(p.alpha);
        const RowShifts shifts = resolve_row_shifts(p);
        const bool has_shifts = shifts.a != nullptr || shifts.b != nullptr;
        const uint32_t tmem_empty_leader = map_to_cta(smem_u32(&bars->tmem_empty), 0);
        int it = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
            int tile_m, tile_n;
            pair_tile_coords(tile, p.tiles_m, p.tiles_n, tile_m, tile_n);
            bool ok = mbar_wait_cluster(&bars->tmem_full, it & 1, &bars->abort_flag, p.status, where_base + 4, it);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            const bool staged = p.out_dtype == UE5M3_DTYPE_BF16 && (p.ldo % 8) == 0 &&
                                ((uintptr_t)p.out % 16) == 0 && tile_n * kFN + (h + 1) * (kFN / 2) <= p.N;
            TileEpilogue t;
            t.taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * (kFN / 2));
            t.row0 = (long long)tile_m * kPM + (long long)rank * 128 + q * 32;
            t.rows_per_thread_valid = 0;
            t.tile_n = tile_n; t.h = h; t.lane = lane; t.alpha = alpha;
            t.stage = staged ? stage_base + (warp - 2) * kStageBytesPerWarp : nullptr;
            t.release_local = nullptr;
            t.release_cluster = tmem_empty_leader;
            if (has_shifts)
                fp4_tile_epilogue_with_row_shifts(&bars->params, shifts.a, shifts.b, t.taddr, t.row0, t.tile_n, t.h, t.lane,
                                                  t.alpha, t.stage, t.release_local, t.release_cluster);
            else fp4_tile_epilogue<false>(p, shifts, t);
        }
    }

    // nobody leaves while the other CTA may still read its shared memory or signal its barriers
    tcgen05_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, kFTmemCols);
    }
}

// ---------------------------------------------------------------------------------------
// UE5M3 scale bytes -> UE4M3 scale bytes in the tensor core's scale-factor layout.
//
// Output: [ceil(rows/128)][K/64][512 bytes]; inside a 512-byte atom the byte of row
// r = r0 + 32*r1 (r0 < 32, r1 < 4) and 16-block kb (< 4) sits at r0*16 + r1*4 + kb.
// Source scales are [rows/row_group][K/block] bytes (row_group = 1 for 1-D blocks, = block
// for 2-D tiles); a 32-wide block feeds two consecutive 16-blocks.
// byte_out = byte_in - ((8 + shift) << 3): same fraction bits, exponent re-biased from 15 to
// 7 and divided by 2^shift.  Valid UE4M3 exponents are 1..15 (and not 0x7F); anything else is
// clamped and its row goes into the window record.  Rows beyond `rows` get 1.0 (0x38).
// ---------------------------------------------------------------------------------------
__global__ void pack_scales_kernel(const uint8_t* __restrict__ scales, int64_t rows, int64_t kblocks,
                                   int block, int row_group, int shift, uint32_t* __restrict__ out,
                                   uint32_t* __restrict__ out_raw, int64_t row_tiles, int64_t k_atoms,
                                   int* __restrict__ window_record) {
    const int64_t total = row_tiles * k_atoms * 128;
    const int per16 = block / 16;
    int bad_units = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int word = (int)(i % 128);           // r0 * 4 + r1
        const int64_t atom = i / 128;              // tile * k_atoms + ka
        const int64_t ka = atom % k_atoms, tile = atom / k_atoms;
        const int r0 = word >> 2, r1 = word & 3;
        const int64_t row = tile * 128 + r1 * 32 + r0;
        uint32_t packed = 0x38383838u, raw = 0u;   // rows beyond the operand: 1.0 for the tensor core, 0 = immaterial in the raw atoms
        if (row < rows) {
            packed = raw = 0u;
            const uint8_t* src = scales + (row / row_group) * kblocks;
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                const int64_t h = ka * 4 + kb;     // 16-wide block index along K
                const uint32_t code5 = src[h / per16];
                bool outside;
                packed |= ue4m3_window_byte(code5, (8 + shift) << 3, outside) << (8 * kb);
                raw |= code5 << (8 * kb);
                if (outside) {
                    ++bad_units;
                    window_record_row(window_record, row);
                }
            }
        }
        out[atom * 128 + word] = packed;
        if (out_raw) out_raw[atom * 128 + word] = raw;
    }
    window_record_units(window_record, bad_units);
}

static PFN_cuTensorMapEncodeTiled_v12000 fp4_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) != cudaSuccess ||
            query != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }
    return fn;
}

// [rows, K/2] bytes row-major -> 2-D map with a (128 byte x box_rows) box, 128B swizzle.
static int make_codes_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k_bytes,
                          uint32_t box_rows) {
    PFN_cuTensorMapEncodeTiled_v12000 encode = fp4_encode_fn();
    if (!encode) {
        record_error_text("cuTensorMapEncodeTiled is not available from the driver");
        return UE5M3_ERR_CUDA;
    }
    cuuint64_t dims[2] = {(cuuint64_t)k_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k_bytes};
    cuuint32_t box[2] = {128u, box_rows};
    cuuint32_t elem_strides[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                        elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        record_error_text("cuTensorMapEncodeTiled failed for packed codes");
        return UE5M3_ERR_CUDA;
    }
    return UE5M3_OK;
}

// scale atoms as a 2-D map: 128 words per atom, box = four consecutive atoms, no swizzle
static int make_sf_map(CUtensorMap* map, const void* base, int64_t atoms) {
    PFN_cuTensorMapEncodeTiled_v12000 encode = fp4_encode_fn();
    if (!encode) {
        record_error_text("cuTensorMapEncodeTiled is not available from the driver");
        return UE5M3_ERR_CUDA;
    }
    cuuint64_t dims[2] = {128u, (cuuint64_t)atoms};
    cuuint64_t strides[1] = {512u};
    cuuint32_t box[2] = {128u, 4u};
    cuuint32_t elem_strides[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box,
                        elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        record_error_text("cuTensorMapEncodeTiled failed for scale atoms");
        return UE5M3_ERR_CUDA;
    }
    return UE5M3_OK;
}

// The CTA-pair kernel is used when there is more than one 128-row tile; UE5M3_FP4_CTA_PAIR=0/1
// in the environment (read at every call) forces the single-CTA / the pair kernel.  The two are
// bit-equal; the pair kernel is the faster one wherever both apply (about 5 % on the
// 8192 x 21504 x 4096 product).
static bool use_cta_pair(int64_t M) {
    const char* e = getenv("UE5M3_FP4_CTA_PAIR");
    if (e && (e[0] == '0' || e[0] == '1')) return e[0] == '1';
    return M > 128;
}

}  // namespace ue5m3

using namespace ue5m3;

extern "C" size_t ue5m3_window_record_ints(int64_t operand_rows) {
    if (operand_rows <= 0) return 0;
    return (size_t)kRecHeader + (size_t)kRecMaxRows + 2 * (size_t)operand_rows;
}

extern "C" size_t ue5m3_packed_scales_bytes(int64_t rows, int64_t K) {
    if (rows <= 0 || K <= 0 || K % 64) return 0;
    return (size_t)((rows + 127) / 128) * (size_t)(K / 64) * kSfAtomBytes;
}

extern "C" int ue5m3_pack_scales_ue4m3(const uint8_t* scales, int64_t rows, int64_t K, int block,
                                       int two_d, int shift, uint8_t* sf_out, uint8_t* sf_raw,
                                       int* window_record, void* stream_v) {
    if (!scales || !sf_out || !window_record || rows <= 0 || K <= 0) return UE5M3_ERR_INVALID_ARGUMENT;
    if (block != 16 && block != 32) return UE5M3_ERR_BLOCK_SIZE;
    if (K % 64) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if (shift < -8 || shift > 8) return UE5M3_ERR_INVALID_ARGUMENT;
    if (((uintptr_t)sf_out % 16) != 0 || ((uintptr_t)sf_raw % 16) != 0) return UE5M3_ERR_ALIGNMENT;
    const int64_t row_tiles = (rows + 127) / 128, k_atoms = K / 64;
    const int64_t total = row_tiles * k_atoms * 128;
    int64_t want = (total + 255) / 256;
    int grid = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
    pack_scales_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_v)>>>(
        scales, rows, K / block, block, two_d ? block : 1, shift, reinterpret_cast<uint32_t*>(sf_out),
        reinterpret_cast<uint32_t*>(sf_raw), row_tiles, k_atoms, window_record);
    return check_launch();
}

extern "C" int ue5m3_gemm_fp4(const uint8_t* a_codes, const uint8_t* a_sf, const uint8_t* b_codes,
                              const uint8_t* b_sf, int64_t M, int64_t N, int64_t K, int shift_sum,
                              int snap, const float* alpha_dev, const float* amax_a_dev,
                              const float* amax_b_dev, float inv_denominator, const void* bias,
                              int bias_dtype, void* out, int out_dtype, int64_t ldo,
                              const int* a_record, const int* b_record, int* status_dev,
                              void* stream_v) {
    if (!a_codes || !a_sf || !b_codes || !b_sf || !out || M <= 0 || N <= 0 || K <= 0)
        return UE5M3_ERR_INVALID_ARGUMENT;
    if (K % kFKMma) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if (out_dtype != UE5M3_DTYPE_BF16 && out_dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (bias && bias_dtype != UE5M3_DTYPE_BF16 && bias_dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (ldo < N || shift_sum < -100 || shift_sum > 100) return UE5M3_ERR_INVALID_ARGUMENT;
    if (!alpha_spec_valid(AlphaSpec{alpha_dev, amax_a_dev, amax_b_dev, inv_denominator})) return UE5M3_ERR_INVALID_ARGUMENT;
    if (((uintptr_t)a_codes % 16) || ((uintptr_t)b_codes % 16) || ((uintptr_t)a_sf % 16) || ((uintptr_t)b_sf % 16))
        return UE5M3_ERR_ALIGNMENT;
    if (((K / 2) % 16) != 0) return UE5M3_ERR_ALIGNMENT;  // TMA row pitch
    if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) return UE5M3_ERR_TOO_LARGE;
    const bool pair = use_cta_pair(M);
    const int64_t tile_rows = pair ? kPM : kFM;
    const int64_t tiles_m = (M + tile_rows - 1) / tile_rows, tiles_n = (N + kFN - 1) / kFN;
    if (tiles_m * tiles_n > 0x7FFFFFFF) return UE5M3_ERR_TOO_LARGE;

    CUtensorMap map_a, map_b;
    int status = make_codes_map(&map_a, a_codes, M, K / 2, 128);
    if (status != UE5M3_OK) return status;
    status = make_codes_map(&map_b, b_codes, N, K / 2, pair ? 128 : kFN);
    if (status != UE5M3_OK) return status;

    Fp4Params p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.snap = snap ? 1 : 0;
    p.rescale = ldexpf(1.0f, shift_sum);
    p.alpha = AlphaSpec{alpha_dev, amax_a_dev, amax_b_dev, inv_denominator};
    p.bias = bias; p.bias_dtype = bias_dtype;
    p.out = out; p.out_dtype = out_dtype; p.ldo = ldo; p.status = status_dev;
    p.sfa = a_sf; p.sfb = b_sf;
    p.rec_a = a_record; p.rec_b = b_record;
    p.tiles_m = (int)tiles_m; p.tiles_n = (int)tiles_n;
    const int64_t tiles = tiles_m * tiles_n;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    if (pair) {
        CUtensorMap map_sfa, map_sfb;
        status = make_sf_map(&map_sfa, a_sf, ((M + 127) / 128) * (K / 64));
        if (status != UE5M3_OK) return status;
        status = make_sf_map(&map_sfb, b_sf, ((N + 127) / 128) * (K / 64));
        if (status != UE5M3_OK) return status;
        const size_t smem = (size_t)kPStages * kPStageBytes + kFEpilogueWarps * kStageBytesPerWarp +
                            sizeof(Fp4PairBarriers) + 1024;
        cudaError_t e = cudaFuncSetAttribute(gemm_fp4_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return record_cuda_error(e);
        static int max_pairs[64] = {0};
        int device = 0;
        cudaGetDevice(&device);
        if (device >= 0 && device < 64 && max_pairs[device] == 0) {
            cudaLaunchConfig_t config = {};
            config.gridDim = dim3(2 * (unsigned)(sm_count() / 2));
            config.blockDim = dim3(kFThreads);
            config.dynamicSmemBytes = smem;
            cudaLaunchAttribute attribute;
            attribute.id = cudaLaunchAttributeClusterDimension;
            attribute.val.clusterDim.x = 2; attribute.val.clusterDim.y = 1; attribute.val.clusterDim.z = 1;
            config.attrs = &attribute;
            config.numAttrs = 1;
            int clusters = 0;
            e = cudaOccupancyMaxActiveClusters(&clusters, gemm_fp4_pair_kernel, &config);
            if (e != cudaSuccess) return record_cuda_error(e);
            max_pairs[device] = clusters > 0 ? clusters : 1;
        }
        const int64_t resident = (device >= 0 && device < 64) ? max_pairs[device] : sm_count() / 2;
        const unsigned pairs = (unsigned)(tiles < resident ? tiles : resident);
        gemm_fp4_pair_kernel<<<2 * pairs, kFThreads, smem, stream>>>(map_a, map_b, map_sfa, map_sfb, p);
        return check_launch();
    }

    const size_t smem = (size_t)kFStages * kFStageBytes + sizeof(Fp4Barriers) + 1024;
    cudaError_t e = cudaFuncSetAttribute(gemm_fp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return record_cuda_error(e);
    const unsigned grid = (unsigned)(tiles < sm_count() ? tiles : sm_count());
    gemm_fp4_kernel<<<grid, kFThreads, smem, stream>>>(map_a, map_b, p);
    return check_launch();
}
