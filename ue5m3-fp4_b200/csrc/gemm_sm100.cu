// Probe-matched issue-RZ GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma
// (kind::f16, BF16 x BF16 -> FP32 in TMEM) -> CUDA-core epilogue.
//
// Numerical model (reference backends/triton/gemm.py:62-80,158-159 and
// api.py:72-83): the reduction axis is cut into issues of 64 elements; each
// issue is multiplied into a FRESH accumulator (four K=16 MMAs, the first one
// overwriting), the issue partial is read back from TMEM and folded into the
// running sum with an FP32 round-toward-zero add, in ascending k.  After the
// last issue the epilogue applies, in registers: RNE snap to the 1/1024 grid,
// the tensor-scale factor alpha, the bias, and the output cast.
//
// Tiling: one CTA per 128 x 256 output tile (all 128 TMEM lanes, 256 fp32
// columns).  TMEM holds two 256-column accumulators, so the MMA of issue j+1
// overlaps the epilogue of issue j.  Shared memory holds a 4-deep ring of
// (A 128x64, B 256x64) bf16 stages in the 128-byte-swizzled K-major layout
// written by TMA.  Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer and
// TMEM owner, warps 2..9 = epilogue (TMEM lane quadrant = warp % 4, column
// half = (warp - 2) / 4).
//
// Two instantiations.  Plain: one CTA per tile of a product of two bf16 operands
// (ue5m3_gemm_issue_rz_bf16).  Mapped: persistent CTAs walk the tiles of the up to three
// products of the FP4 path's recomputation pass - operands that fallback_workspace.cu has
// decoded into a workspace, extents and row / column lists read on the device - with the issue
// counter running on across tiles (issue_rz_mapped.cuh).
//
// Every wait is bounded by a clock budget; on expiry the kernel records where
// it gave up in the caller's status words, raises a CTA-wide abort flag and
// falls through to the common exit, where TMEM is released.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "abi_common.cuh"
#include "alpha_spec.cuh"
#include "issue_rz_mapped.cuh"
#include "dead_fill.cuh"

namespace ue5m3 {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kStages = 4;
constexpr int kUmmaK = 16;
constexpr int kNumThreads = 320;
constexpr int kEpilogueWarps = 8;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kStageBytesA = kBM * kBK * 2;  // 16 KiB
constexpr uint32_t kStageBytesB = kBN * kBK * 2;  // 32 KiB
constexpr uint32_t kStageBytes = kStageBytesA + kStageBytesB;
constexpr long long kWaitBudgetClocks = 4000000000LL;  // about two seconds

struct GemmParams {
    int M, N, K;
    int snap;
    AlphaSpec alpha;
    const void* bias;
    int bias_dtype;
    void* out;
    int out_dtype;
    long long ldo;
    int* status;
    int tiles_m, tiles_n;
    // Mapped launches only (the recomputation pass of the FP4 product, on operands decoded into a
    // workspace): the kernel gets four operand buffers - the listed rows of A and of B gathered
    // (map_a, map_b; capacity valid_cap rows) and A and B in full (map_a_full, map_b_full; M and N
    // rows) - and walks the tiles of up to three products: listed A x full B -> output rows
    // row_map[i]; full A x listed B -> output columns col_map[i]; full A x full B when a list
    // overflowed (a count above valid_cap).  The counts are read on the device.
    const int* valid_m;
    const int* valid_n;
    int valid_cap;
    const int* row_map;
    const int* col_map;
};

struct __align__(8) GemmBarriers {
    unsigned long long full[kStages];
    unsigned long long empty[kStages];
    unsigned long long tmem_full[2];
    unsigned long long tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// ---- PTX wrappers ---------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait.  Returns false when the budget expired or another role aborted.
// The clock and the abort flag are looked at once per 32 polls, so the common
// case is a tight try_wait loop.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity,
                                          GemmBarriers* bars, int* status, int where, int iter) {
#pragma unroll 1
    for (int spin = 0; spin < 32; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (true) {
#pragma unroll 1
        for (int spin = 0; spin < 32; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (*((volatile int*)&bars->abort_flag)) return false;
        if (clock64() - start > kWaitBudgetClocks) {
            *((volatile int*)&bars->abort_flag) = 1;
            if (status) {
                if (atomicCAS(&status[0], 0, 1) == 0) {
                    status[1] = where;
                    status[2] = iter;
                    status[3] = (int)blockIdx.x;
                }
            }
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map,
                                            unsigned long long* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(dst_smem)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], BF16 inputs, FP32 accumulate.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// mbarrier arrives once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
            smem_u32(bar))
        : "memory");
}

// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread.
__device__ __forceinline__ void tmem_load_32_async(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Two fp32 round-toward-zero adds in one instruction (sm_100 packed fp32 pipe).
__device__ __forceinline__ void fadd2_rz(float& c0, float& c1, uint32_t v0, uint32_t v1) {
    asm("{\n"
        ".reg .b64 a, b;\n"
        "mov.b64 a, {%0, %1};\n"
        "mov.b64 b, {%2, %3};\n"
        "add.rz.f32x2 a, a, b;\n"
        "mov.b64 {%0, %1}, a;\n"
        "}\n"
        : "+f"(c0), "+f"(c1)
        : "r"(v0), "r"(v1));
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups
// 1024 bytes apart, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address, bits [0,14)
    desc |= (uint64_t)1 << 16;                         // leading byte offset (unused with swizzle)
    desc |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset, bits [32,46)
    desc |= (uint64_t)1 << 46;                         // version
    desc |= (uint64_t)2 << 61;                         // SWIZZLE_128B
    return desc;
}

// Instruction descriptor for kind::f16: D = F32, A = B = BF16, both K-major.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// round-half-even to an integer (torch.round), full-rate float ops only
__device__ __forceinline__ float rint_rne(float v) {
    float a = fabsf(v);
    float r = a < 8388608.0f ? __fadd_rn(__fadd_rn(a, 8388608.0f), -8388608.0f) : a;
    return copysignf(r, v);
}

// Epilogue stores of a mapped launch: one thread's 128 finished values (after snap and alpha)
// of A row `row`, B rows col0 .. col0 + 127, to out[row_map[row]][col_map[col]] with the bias of
// the output column.
__device__ __forceinline__ void store_mapped_row(const GemmParams& p, float (&c)[kBN / 2], long long row, int col0,
                                                 int lim_n, const int* row_map, const int* col_map) {
    const long long out_row = row_map ? (long long)__ldg(row_map + row) : row;
#pragma unroll
    for (int i = 0; i < kBN / 2; ++i) {
        const int col = col0 + i;
        if (col >= lim_n) continue;
        const int out_col = col_map ? __ldg(col_map + col) : col;
        float v = c[i];
        if (p.bias)
            v = __fadd_rn(v, p.bias_dtype == UE5M3_DTYPE_BF16
                                 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[out_col])
                                 : static_cast<const float*>(p.bias)[out_col]);
        if (p.out_dtype == UE5M3_DTYPE_BF16)
            static_cast<__nv_bfloat16*>(p.out)[out_row * p.ldo + out_col] = __float2bfloat16_rn(v);
        else
            static_cast<float*>(p.out)[out_row * p.ldo + out_col] = v;
    }
}

// ---- kernel ----------------------------------------------------------------
template <bool kMapped>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_issue_rz_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_a_full, const __grid_constant__ CUtensorMap map_b_full,
                     const GemmParams p) {
    extern __shared__ unsigned char smem_dyn[];
    // 1024-byte alignment for the 128-byte swizzle atoms
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(smem + kStages * kStageBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_issues = p.K / kBK;

    // Plain launches: one tile per CTA, grouped raster (8 tile rows share each sweep over tile
    // columns).  Mapped launches: persistent CTAs walk the tiles of the rectangle of rows that
    // exist (known on the device only); the issue counter runs on across tiles, so the mbarrier
    // phases never need re-initialising.
    int first_tile = blockIdx.x, num_tiles = blockIdx.x + 1, tile_step = 1;
    int job_rows[3] = {0, 0, 0}, job_cols[3] = {0, 0, 0}, job_first[4] = {0, 0, 0, 0};   // mapped launches
    if (kMapped) {
        const int na = __ldg(p.valid_m), nb = __ldg(p.valid_n);
        const bool overflow = na > p.valid_cap || nb > p.valid_cap;
        job_rows[0] = overflow ? 0 : na; job_cols[0] = p.N;               // listed A x full B
        job_rows[1] = p.M;               job_cols[1] = overflow ? 0 : nb;  // full A x listed B
        job_rows[2] = overflow ? p.M : 0; job_cols[2] = p.N;              // full A x full B
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            const int tiles = job_rows[j] > 0 && job_cols[j] > 0
                                  ? ((job_rows[j] + kBM - 1) / kBM) * ((job_cols[j] + kBN - 1) / kBN) : 0;
            job_first[j + 1] = job_first[j] + tiles;
        }
        num_tiles = job_first[3];
        tile_step = gridDim.x;
        if ((int)blockIdx.x >= num_tiles) return;   // the whole CTA, before anything is set up
    }
    // tile -> origin in its product's own row / column numbering (and which product)
    auto tile_origin = [&](int tile, int& m0, int& n0) -> int {
        if (kMapped) {
            const int job = tile < job_first[1] ? 0 : (tile < job_first[2] ? 1 : 2);
            const int local = tile - job_first[job];
            const int tiles_n = (job_cols[job] + kBN - 1) / kBN;
            m0 = (local / tiles_n) * kBM;
            n0 = (local % tiles_n) * kBN;
            return job;
        }
        constexpr int kGroupM = 8;
        const int tiles_per_group = kGroupM * p.tiles_n;
        const int group = tile / tiles_per_group;
        const int first_m = group * kGroupM;
        const int group_m = (p.tiles_m - first_m) < kGroupM ? (p.tiles_m - first_m) : kGroupM;
        m0 = (first_m + (tile % tiles_per_group) % group_m) * kBM;
        n0 = ((tile % tiles_per_group) / group_m) * kBN;
        return 0;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bars->tmem_full[b], 1);
            mbar_init(&bars->tmem_empty[b], kEpilogueWarps);
        }
        // a launch that follows a recorded failure does no work at all
        bars->abort_flag = (p.status && *((volatile int*)p.status) != 0) ? 1 : 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&bars->tmem_base, kTmemCols);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *((volatile uint32_t*)&bars->tmem_base);
    const bool dead = *((volatile int*)&bars->abort_flag) != 0;

    if (dead) {
        // no work after a recorded failure: mark this CTA's tile and fall through to the common exit
        // (a mapped launch rewrites parts of an output that the preceding FP4 launch has marked)
        if (!kMapped) {
            int m0, n0;
            tile_origin(first_tile, m0, n0);
            fill_tile_nan(p.out, p.out_dtype == UE5M3_DTYPE_BF16, p.ldo, m0, n0, kBM, kBN, p.M, p.N);
        }
    } else if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int g = 0;   // issues since the kernel started
            bool ok = true;
            for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
                int m0, n0;
                const int job = tile_origin(tile, m0, n0);
                const CUtensorMap* tile_a = (kMapped && job != 0) ? &map_a_full : &map_a;
                const CUtensorMap* tile_b = (kMapped && job != 1) ? &map_b_full : &map_b;
                for (int j = 0; j < num_issues; ++j, ++g) {
                    const int s = g % kStages;
                    const uint32_t use = g / kStages;
                    if (use > 0 && !mbar_wait(&bars->empty[s], (use - 1) & 1, bars, p.status, 1, j)) {
                        ok = false;
                        break;
                    }
                    unsigned char* sa = smem + s * kStageBytes;
                    unsigned char* sb = sa + kStageBytesA;
                    mbar_arrive_expect_tx(&bars->full[s], kStageBytes);
                    tma_load_2d(sa, tile_a, &bars->full[s], j * kBK, m0);
                    tma_load_2d(sb, tile_b, &bars->full[s], j * kBK, n0);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(kBM, kBN);
            int g = 0;
            bool ok = true;
            for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
                for (int j = 0; j < num_issues; ++j, ++g) {
                    const int s = g % kStages;
                    const int b = g & 1;
                    const uint32_t use_b = g >> 1;
                    if (use_b > 0 && !mbar_wait(&bars->tmem_empty[b], (use_b - 1) & 1, bars, p.status, 2, j)) {
                        ok = false;
                        break;
                    }
                    if (!mbar_wait(&bars->full[s], (g / kStages) & 1, bars, p.status, 3, j)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t sa = smem_u32(smem + s * kStageBytes);
                    const uint32_t sb = sa + kStageBytesA;
                    const uint64_t desc_a = make_smem_desc(sa);
                    const uint64_t desc_b = make_smem_desc(sb);
                    const uint32_t tmem_d = tmem_base + (uint32_t)b * kBN;
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        // advance 16 bf16 = 32 bytes inside the swizzle atom: +2 in 16-byte units
                        umma_bf16(tmem_d, desc_a + (uint64_t)(2 * k), desc_b + (uint64_t)(2 * k), idesc,
                                  k > 0 ? 1u : 0u);
                    }
                    umma_commit(&bars->empty[s]);      // smem stage reusable once the MMAs have read it
                    umma_commit(&bars->tmem_full[b]);  // issue partial complete in TMEM
                }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int q = warp & 3;            // TMEM lane quadrant
        const int h = (warp - 2) >> 2;     // column half of the tile
        int g = 0;
        bool ok = true;
        for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
            int m0, n0;
            const int job = tile_origin(tile, m0, n0);
            const int lim_m = kMapped ? job_rows[job] : p.M;
            const int lim_n = kMapped ? job_cols[job] : p.N;
            float c[kBN / 2];
#pragma unroll
            for (int i = 0; i < kBN / 2; ++i) c[i] = 0.0f;
            for (int j = 0; j < num_issues; ++j, ++g) {
                const int b = g & 1;
                ok = mbar_wait(&bars->tmem_full[b], (g >> 1) & 1, bars, p.status, 4, j);
                ok = __all_sync(0xFFFFFFFFu, ok);  // keep the warp convergent for tcgen05.ld
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * kBN + h * (kBN / 2));
                // two 32-column loads in flight per wait; packed round-toward-zero adds
#pragma unroll
                for (int half = 0; half < kBN / 2 / 64; ++half) {
                    uint32_t v0[32], v1[32];
                    tmem_load_32_async(taddr + half * 64, v0);
                    tmem_load_32_async(taddr + half * 64 + 32, v1);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        fadd2_rz(c[half * 64 + i], c[half * 64 + i + 1], v0[i], v0[i + 1]);
                        fadd2_rz(c[half * 64 + 32 + i], c[half * 64 + 33 + i], v1[i], v1[i + 1]);
                    }
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->tmem_empty[b]);
            }
            if (ok) {
                const float alpha = alpha_value(p.alpha);
                const bool scale_by_alpha = alpha_enabled(p.alpha);
                const long long row = (long long)m0 + q * 32 + lane;
                const int col0 = n0 + h * (kBN / 2);
                if (row < lim_m) {
#pragma unroll
                    for (int i = 0; i < kBN / 2; ++i) {
                        float v = c[i];
                        if (p.snap) v = __fmul_rn(rint_rne(__fmul_rn(v, 1024.0f)), 0.0009765625f);
                        if (scale_by_alpha) v = __fmul_rn(v, alpha);
                        c[i] = v;
                    }
                }
                if (kMapped) {
                    if (row < lim_m)
                        store_mapped_row(p, c, row, col0, lim_n, job == 0 ? p.row_map : nullptr, job == 1 ? p.col_map : nullptr);
                } else if (row < p.M) {
                    if (p.bias) {
#pragma unroll
                        for (int i = 0; i < kBN / 2; ++i) {
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
                        for (int i = 0; i < kBN / 2; i += 8) {
                            if (vec && col0 + i + 8 <= p.N) {
                                uint4 w;
                                w.x = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(c[i + 0])) |
                                      ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(c[i + 1])) << 16);
                                w.y = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(c[i + 2])) |
                                      ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(c[i + 3])) << 16);
                                w.z = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(c[i + 4])) |
                                      ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(c[i + 5])) << 16);
                                w.w = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(c[i + 6])) |
                                      ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(c[i + 7])) << 16);
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
                        for (int i = 0; i < kBN / 2; i += 4) {
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
        }
    }

    // common exit: every role's loop is bounded, so all threads arrive here
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- host side ---------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 encode_tiled_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) !=
                cudaSuccess ||
            query != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }
    return fn;
}

// [rows, K] bf16 row-major -> 2-D tiled map with a (64 x box_rows) box, 128B swizzle.
static int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K,
                            uint32_t box_rows) {
    PFN_cuTensorMapEncodeTiled_v12000 encode = encode_tiled_fn();
    if (!encode) {
        record_error_text("cuTensorMapEncodeTiled is not available from the driver");
        return UE5M3_ERR_CUDA;
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
    cuuint32_t elem_strides[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                        strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        record_error_text("cuTensorMapEncodeTiled failed");
        return UE5M3_ERR_CUDA;
    }
    return UE5M3_OK;
}

// The mapped launch (issue_rz_mapped.cuh).
int launch_issue_rz_mapped(const MappedOperands& ops, int64_t M, int64_t N, int64_t K, int snap, const AlphaSpec& alpha,
                           const void* bias, int bias_dtype, void* out, int out_dtype, int64_t ldo, int* status_dev,
                           cudaStream_t stream) {
    const int64_t tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + kBN - 1) / kBN;
    if (tiles_m * tiles_n > 0x7FFFFFFF) return UE5M3_ERR_TOO_LARGE;
    CUtensorMap map_a, map_b, map_a_full, map_b_full;
    int status = make_operand_map(&map_a, ops.a_listed, ops.cap, K, kBM);
    if (status == UE5M3_OK) status = make_operand_map(&map_b, ops.b_listed, ops.cap, K, kBN);
    if (status == UE5M3_OK) status = make_operand_map(&map_a_full, ops.a_full, M, K, kBM);
    if (status == UE5M3_OK) status = make_operand_map(&map_b_full, ops.b_full, N, K, kBN);
    if (status != UE5M3_OK) return status;
    GemmParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.snap = snap ? 1 : 0;
    p.alpha = alpha;
    p.bias = bias; p.bias_dtype = bias_dtype;
    p.out = out; p.out_dtype = out_dtype; p.ldo = ldo; p.status = status_dev;
    p.tiles_m = (int)tiles_m; p.tiles_n = (int)tiles_n;
    p.valid_m = ops.a_count; p.valid_n = ops.b_count; p.valid_cap = ops.cap;
    p.row_map = ops.a_list; p.col_map = ops.b_list;
    const size_t smem = (size_t)kStages * kStageBytes + sizeof(GemmBarriers) + 1024;
    cudaError_t e = cudaFuncSetAttribute(gemm_issue_rz_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return record_cuda_error(e);
    // persistent CTAs (one per SM at most): with nothing listed every one of them returns at once
    gemm_issue_rz_kernel<true><<<sm_count(), kNumThreads, smem, stream>>>(map_a, map_b, map_a_full, map_b_full, p);
    return UE5M3_OK;
}

}  // namespace ue5m3

using namespace ue5m3;

extern "C" int ue5m3_gemm_issue_rz_bf16(const void* a, const void* bt, int64_t M, int64_t N,
                                        int64_t K, int snap, const float* alpha_dev,
                                        const float* amax_a_dev, const float* amax_b_dev,
                                        float inv_denominator, const void* bias, int bias_dtype,
                                        void* out, int out_dtype, int64_t ldo, int* status_dev,
                                        void* stream_v) {
    if (!a || !bt || !out || M <= 0 || N <= 0 || K <= 0) return UE5M3_ERR_INVALID_ARGUMENT;
    if (K % kBK) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if (out_dtype != UE5M3_DTYPE_BF16 && out_dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (bias && bias_dtype != UE5M3_DTYPE_BF16 && bias_dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (ldo < N) return UE5M3_ERR_INVALID_ARGUMENT;
    if (!alpha_spec_valid(AlphaSpec{alpha_dev, amax_a_dev, amax_b_dev, inv_denominator})) return UE5M3_ERR_INVALID_ARGUMENT;
    if (((uintptr_t)a % 16) || ((uintptr_t)bt % 16)) return UE5M3_ERR_ALIGNMENT;
    if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) return UE5M3_ERR_TOO_LARGE;
    const int64_t tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + kBN - 1) / kBN;
    if (tiles_m * tiles_n > 0x7FFFFFFF) return UE5M3_ERR_TOO_LARGE;

    CUtensorMap map_a, map_b;
    int status = make_operand_map(&map_a, a, M, K, kBM);
    if (status != UE5M3_OK) return status;
    status = make_operand_map(&map_b, bt, N, K, kBN);
    if (status != UE5M3_OK) return status;

    GemmParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.snap = snap ? 1 : 0;
    p.alpha = AlphaSpec{alpha_dev, amax_a_dev, amax_b_dev, inv_denominator};
    p.bias = bias; p.bias_dtype = bias_dtype;
    p.out = out; p.out_dtype = out_dtype; p.ldo = ldo; p.status = status_dev;
    p.tiles_m = (int)tiles_m; p.tiles_n = (int)tiles_n;

    const size_t smem = (size_t)kStages * kStageBytes + sizeof(GemmBarriers) + 1024;
    p.valid_m = nullptr; p.valid_n = nullptr; p.valid_cap = 0; p.row_map = nullptr; p.col_map = nullptr;
    cudaError_t e = cudaFuncSetAttribute(gemm_issue_rz_kernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return record_cuda_error(e);
    gemm_issue_rz_kernel<false><<<(unsigned)(tiles_m * tiles_n), kNumThreads, smem,
                                  static_cast<cudaStream_t>(stream_v)>>>(map_a, map_b, map_a, map_b, p);
    return check_launch();
}
