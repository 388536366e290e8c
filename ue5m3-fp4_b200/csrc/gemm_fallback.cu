// Second half of the FP4 tensor-core product: recomputes, with the issue-RZ BF16 instruction
// sequence of gemm_sm100.cu, the part of the output that the FP4 kernel could not get right
// because a UE5M3 block scale fell outside the tensor core's UE4M3 window.
//
// The quantizers list such operand rows in a window record (include/ue5m3_fp4.h).  The kernel
// is driven by those records ON THE DEVICE, so the host launches it after every FP4 GEMM
// without looking at the data; with empty records every CTA returns after reading two integers.
//
// Persistent CTAs walk the tiles of up to three products,
//   (listed A rows) x B            -> scattered to those output rows,
//   A x (listed B rows)            -> scattered to those output columns,
//   A x B over the whole output    -> when a list overflowed its capacity,
// and per tile do what gemm_sm100.cu does: four K=16 BF16 MMAs into a fresh TMEM accumulator
// per K=64 issue, round-toward-zero adds across issues in registers, then snap, alpha, bias,
// cast.  The operands are not read as bf16 from memory: producer warps decode the packed
// E2M1 codes and the RAW UE5M3 scale atoms (p * s is exact in bf16) straight into the
// 128-byte-swizzled K-major shared-memory tiles the MMA reads, gathering listed rows through
// the record (every thread looks its rows up once per tile and has the next issue's global loads
// in flight while it decodes the current one).  No workspace, no separate decode pass.  The
// issue counter runs on across tiles, so the mbarrier phases never need re-initialising.
//
// The kernel is instantiated for two tile widths and launched once for each (struct Pass):
// 128 x 32 tiles for the listed rows of A, 128 x 128 tiles for the listed rows of B and for the
// whole product.  Warps: producers first (10 / 7), then the MMA issuer and TMEM owner, then the
// epilogue warps (4 x 32 columns / 8 x 64 columns; TMEM lane quadrant = warp % 4).  Of the
// producers and of the epilogue warps only one warp each polls its mbarrier; the others sleep on
// a hardware barrier and take the outcome from shared memory (group_wait).  Every mbarrier wait
// is clock-bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "abi_common.cuh"
#include "alpha_spec.cuh"
#include "decode_bf16.cuh"
#include "tcgen05_ptx.cuh"
#include "ue5m3_device.cuh"
#include "window_record.cuh"

namespace ue5m3 {

using namespace ptx;

namespace fb {

constexpr int kBM = 128;
constexpr int kBK = 64;

struct Plan {
    int na, nb;        // listed rows of A / of B (0 when a list overflowed)
    bool full;         // a list overflowed: recompute everything
    int tiles[3];      // tiles of the row pass, the column pass, the full pass
};

struct Params {
    int M, N, K;
    int snap;
    AlphaSpec alpha;
    const void* bias;
    int bias_dtype;
    void* out;
    int out_dtype;
    long long ldo;
    int* status;
    const uint8_t* codes_a;   // [M, K / 2]
    const uint8_t* codes_b;   // [N, K / 2]
    const uint8_t* raw_a;     // raw UE5M3 scale atoms
    const uint8_t* raw_b;
    const int* rec_a;
    const int* rec_b;
    int jobs;                 // bit 0: listed rows of A, bit 1: listed rows of B, bit 2: whole product after an overflow
};

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

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

// writes made with ordinary shared-memory stores become visible to the tensor core's reads
__device__ __forceinline__ void fence_generic_to_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// which product, which tile of it, and where its results go
struct Tile {
    int job;            // 0 row pass, 1 column pass, 2 full pass
    int m0, n0;         // tile origin in the job's own row / column numbering
    int rows, cols;     // extent of the job's output
};

// Barrier `id` of the CTA over `threads` threads: waiting warps take no issue slots, unlike
// warps polling an mbarrier.  Every thread of the group must arrive.
__device__ __forceinline__ void group_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// One warp of a group waits on the mbarrier, the others sleep on a hardware barrier and learn
// the outcome from shared memory - so that they all leave their loop in the same iteration and
// nobody is left behind at the hardware barrier, which has no time limit of its own.  `word` is
// double-buffered by the caller (iteration parity).
__device__ __forceinline__ bool group_wait(bool poller, int id, int threads, volatile int* word, unsigned long long* bar,
                                           uint32_t parity, int* abort_flag, int* status, int where, int iter) {
    __syncwarp();   // the hardware barrier wants the whole warp at once
    if (poller) {
        bool ok = mbar_wait(bar, parity, abort_flag, status, where, iter);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if ((threadIdx.x & 31) == 0) *word = ok ? 1 : 0;
    }
    group_sync(id, threads);
    return *word != 0;
}


template <typename OutT>
__device__ __forceinline__ OutT to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// One pass of the kernel for one tile width.  The listed-row pass (BN = 32) has one or two row
// tiles, so narrow tiles spread it over the SMs and every CTA decodes few rows of the full
// operand per issue.  The listed-column pass and the full pass (BN = 128) have a row tile per
// 128 rows of A, which every column tile decodes again: wide tiles there.
template <int BN>
struct Pass {
    static constexpr int kBN = BN;
    static constexpr int kStages = BN == 32 ? 10 : 6;
    static constexpr int kProducerWarps = BN == 32 ? 10 : 7;   // 16 warps in all either way: register files are handed out per four warps
    static constexpr int kCols = BN == 32 ? 32 : 64;   // columns per epilogue warp
    static constexpr int kEpilogueWarps = 4 * (BN / kCols);
    static constexpr int kMmaWarp = kProducerWarps;
    static constexpr int kEpilogueWarp0 = kMmaWarp + 1;
    static constexpr int kThreads = 32 * (kEpilogueWarp0 + kEpilogueWarps);
    static constexpr uint32_t kTmemCols = 2 * kBN;   // two accumulators
    static constexpr uint32_t kStageBytesA = kBM * kBK * 2;
    static constexpr uint32_t kStageBytesB = kBN * kBK * 2;
    static constexpr uint32_t kStageBytes = kStageBytesA + kStageBytesB;

    static __device__ __forceinline__ Plan make_plan(const int* rec_a, const int* rec_b, int M, int N, int jobs) {
        Plan plan;
        const int na = __ldg(rec_a + kRecListed), nb = __ldg(rec_b + kRecListed);
        plan.full = na > kRecMaxRows || nb > kRecMaxRows;
        plan.na = plan.full ? 0 : na;
        plan.nb = plan.full ? 0 : nb;
        const int tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + kBN - 1) / kBN;
        plan.tiles[0] = (jobs & 1) ? ((plan.na + kBM - 1) / kBM) * tiles_n : 0;
        plan.tiles[1] = (jobs & 2) ? tiles_m * ((plan.nb + kBN - 1) / kBN) : 0;
        plan.tiles[2] = ((jobs & 4) && plan.full) ? tiles_m * tiles_n : 0;
        return plan;
    }


    struct __align__(8) Barriers {
        unsigned long long full[kStages];
        unsigned long long empty[kStages];
        unsigned long long tmem_full[2];
        unsigned long long tmem_empty[2];
        uint32_t tmem_base;
        int abort_flag;
        int producers_go[2];   // outcome of the producers' / the epilogue's current wait (group_wait)
        int epilogue_go[2];
    };

    static __device__ __forceinline__ Tile locate_tile(const Plan& plan, int t, int M, int N) {
        Tile tile;
        const int tiles_n = (N + kBN - 1) / kBN;
        if (t < plan.tiles[0]) {
            tile.job = 0; tile.m0 = (t / tiles_n) * kBM; tile.n0 = (t % tiles_n) * kBN;
            tile.rows = plan.na; tile.cols = N;
            return tile;
        }
        t -= plan.tiles[0];
        if (t < plan.tiles[1]) {
            const int col_tiles = (plan.nb + kBN - 1) / kBN;
            tile.job = 1; tile.m0 = (t / col_tiles) * kBM; tile.n0 = (t % col_tiles) * kBN;
            tile.rows = M; tile.cols = plan.nb;
            return tile;
        }
        t -= plan.tiles[1];
        tile.job = 2; tile.m0 = (t / tiles_n) * kBM; tile.n0 = (t % tiles_n) * kBN;
        tile.rows = M; tile.cols = N;
        return tile;
    }

    // One K=64 slab of the tile's A rows and B rows -> bf16 in the 128-byte-swizzled K-major
    // layout: row r of a tile occupies 128 bytes at r * 128, its 16-byte chunk c sits at chunk
    // position c ^ (r & 7).  An item is (row, half of the issue): 16 bytes of codes (32 elements,
    // two 16-element blocks) and their two scale bytes in, four 16-byte chunks out.  The 512 items
    // of a stage go one to a producer thread; the 32 left over are second items of warp 0, taken
    // from the operand that a row or column pass has few rows of (see item_row).  Every thread has
    // the next issue's global loads in flight while it decodes the current one.
    static constexpr int kStageItems = (kBM + kBN) * 2;
    static constexpr int kItems = (kStageItems + kProducerWarps * 32 - 1) / (kProducerWarps * 32);   // the last one may not exist
    static_assert(kItems * kProducerWarps * 32 >= kStageItems && kEpilogueWarps * 32 * kCols == kBM * kBN, "warp roles cover a stage and a tile");

    static constexpr int kPrefetch = 1;

    struct StageLoads {
        uint4 codes[kItems];
        uint32_t scales[kItems];   // two bytes
    };

    // where a thread's items of the current tile live: the codes of (row, half) at issue 0, the
    // row's two raw scale bytes of that half in atom 0, and the row's 128 bytes in a stage.  A null
    // pointer marks a row beyond the operand: zeros are stored for it.  stage_offset < 0: no item.
    struct ItemSources {
        const uint4* codes[kItems];
        const uint16_t* scale[kItems];
        int stage_offset[kItems];
    };

    // Row of the stage (0..kBM-1 operand A, kBM.. operand B) that an item belongs to.  In a row pass
    // operand B comes first, so that the leftover items are rows of A's tile, of which such a pass
    // has few; in the other passes operand A comes first.
    static __device__ __forceinline__ int item_row(int item, int job) {
        const int r = item >> 1;
        return job == 0 ? (r < kBN ? r + kBM : r - kBN) : r;
    }

    static __device__ __forceinline__ void load_stage(StageLoads& loads, const ItemSources& src, int issue) {
    #pragma unroll
        for (int i = 0; i < kItems; ++i) {
            if (src.codes[i]) {
                loads.codes[i] = __ldg(src.codes[i] + issue * 2);             // 32 bytes of codes per row and issue
                loads.scales[i] = __ldg(src.scale[i] + (int64_t)issue * 256);  // one 512-byte atom per 128 rows and issue
            }
        }
    }

    static __device__ __forceinline__ void store_stage(unsigned char* stage, const StageLoads& loads, const ItemSources& src) {
    #pragma unroll
        for (int i = 0; i < kItems; ++i) {
            if (src.stage_offset[i] < 0) break;
            unsigned char* row = stage + (src.stage_offset[i] & ~1);
            const int half = src.stage_offset[i] & 1;
            const int swizzle = (src.stage_offset[i] >> 7) & 7;   // both operands' regions start on 1024 bytes
            const uint32_t words[4] = {loads.codes[i].x, loads.codes[i].y, loads.codes[i].z, loads.codes[i].w};
            uint32_t scale2[2] = {0u, 0u};
            if (src.codes[i]) {
                scale2[0] = scale_pair(loads.scales[i] & 0xFFu);
                scale2[1] = scale_pair((loads.scales[i] >> 8) & 0xFFu);
            }
    #pragma unroll
            for (int w = 0; w < 4; ++w) {
                const int c = half * 4 + w;   // 8-element chunk of the issue; chunks 2k, 2k+1 share block k's scale
                // rows beyond the operand are zero (their results are never stored)
                const uint4 value = src.codes[i] ? decode_word(words[w], scale2[w >> 1]) : make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(row + ((c ^ swizzle) << 4)) = value;
            }
        }
    }

    // one thread's finished values of one output row
    template <typename OutT>
    static __device__ __forceinline__ void store_row(const Params& p, const Tile& tile, const float (&c)[kCols],
                                              long long out_row, int col0) {
        OutT* out = static_cast<OutT*>(p.out) + out_row * p.ldo;
        const int* col_map = tile.job == 1 ? p.rec_b + kRecHeader : nullptr;
        constexpr int kVec = 16 / (int)sizeof(OutT);
        const bool vec = !col_map && (p.ldo % kVec) == 0 && ((uintptr_t)p.out % 16) == 0;
    #pragma unroll
        for (int i = 0; i < kCols; i += kVec) {
            if (vec && col0 + i + kVec <= tile.cols) {
                OutT tmp[kVec];
    #pragma unroll
                for (int e = 0; e < kVec; ++e) tmp[e] = to_out<OutT>(c[i + e]);
                *reinterpret_cast<uint4*>(out + col0 + i) = *reinterpret_cast<const uint4*>(tmp);
            } else {
    #pragma unroll
                for (int e = 0; e < kVec; ++e) {
                    const int col = col0 + i + e;
                    if (col < tile.cols) out[col_map ? __ldg(col_map + col) : col] = to_out<OutT>(c[i + e]);
                }
            }
        }
    }

    static __device__ __forceinline__ void run(const Params& p) {
        const Plan plan = make_plan(p.rec_a, p.rec_b, p.M, p.N, p.jobs);
        const int total_tiles = plan.tiles[0] + plan.tiles[1] + plan.tiles[2];
        if ((int)blockIdx.x >= total_tiles) return;  // the whole CTA, before anything is set up

        extern __shared__ unsigned char smem_dyn[];
        unsigned char* smem = reinterpret_cast<unsigned char*>(
            (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
        Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * kStageBytes);

        const int warp = threadIdx.x >> 5;
        const int lane = threadIdx.x & 31;
        const int num_issues = p.K / kBK;

        if (threadIdx.x == 0) {
            for (int s = 0; s < kStages; ++s) {
                mbar_init(&bars->full[s], kProducerWarps);
                mbar_init(&bars->empty[s], 1);
            }
            for (int b = 0; b < 2; ++b) {
                mbar_init(&bars->tmem_full[b], 1);
                mbar_init(&bars->tmem_empty[b], kEpilogueWarps);
            }
            // a launch that follows a recorded failure does no work at all
            bars->abort_flag = (p.status && *((volatile int*)p.status) != 0) ? 1 : 0;
            mbar_fence_init();
        }
        if (warp == kMmaWarp) tmem_alloc(&bars->tmem_base, kTmemCols);
        tcgen05_fence_before();
        __syncthreads();
        tcgen05_fence_after();
        const uint32_t tmem_base = *((volatile uint32_t*)&bars->tmem_base);
        const bool dead = *((volatile int*)&bars->abort_flag) != 0;

        if (dead) {
            // fall through to the common exit
        } else if (warp < kProducerWarps) {
            // ---------------- producers: decode packed operands into the stage ----------------
            int g = 0;  // issues since the kernel started, over all tiles of this CTA
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const Tile tile = locate_tile(plan, t, p.M, p.N);
                // sources of this thread's items, looked up once per tile
                ItemSources src;
                const int64_t k_atoms = p.K / 64;
    #pragma unroll
                for (int i = 0; i < kItems; ++i) {
                    const int item = threadIdx.x + i * (kProducerWarps * 32);
                    const int r = item_row(item, tile.job), half = item & 1;
                    const bool is_a = r < kBM;
                    const int local = is_a ? r : r - kBM;
                    const int index = (is_a ? tile.m0 : tile.n0) + local;
                    const int count = is_a ? tile.rows : tile.cols;
                    src.codes[i] = nullptr;
                    src.scale[i] = nullptr;
                    src.stage_offset[i] = item < kStageItems ? ((is_a ? 0 : (int)kStageBytesA) + local * 128) | half : -1;
                    if (item < kStageItems && index < count) {
                        int64_t row;
                        if (is_a) row = tile.job == 0 ? __ldg(p.rec_a + kRecHeader + index) : index;
                        else row = tile.job == 1 ? __ldg(p.rec_b + kRecHeader + index) : index;
                        src.codes[i] = reinterpret_cast<const uint4*>((is_a ? p.codes_a : p.codes_b) + row * (p.K / 2)) + half;
                        src.scale[i] = reinterpret_cast<const uint16_t*>(
                            (is_a ? p.raw_a : p.raw_b) + (row >> 7) * k_atoms * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + half * 2);
                    }
                }
                StageLoads ring[kPrefetch + 1];
    #pragma unroll
                for (int u = 0; u < kPrefetch; ++u)
                    if (u < num_issues) load_stage(ring[u], src, u);
                for (int j0 = 0; j0 < num_issues && ok; j0 += kPrefetch + 1) {
    #pragma unroll
                    for (int u = 0; u < kPrefetch + 1; ++u) {
                        const int j = j0 + u;
                        if (j >= num_issues) break;
                        if (j + kPrefetch < num_issues) load_stage(ring[(u + kPrefetch) % (kPrefetch + 1)], src, j + kPrefetch);
                        const int s = g % kStages;
                        const uint32_t use = g / kStages;
                        if (use > 0) {
                            ok = group_wait(warp == 0, 1, kProducerWarps * 32, &bars->producers_go[g & 1], &bars->empty[s],
                                            (use - 1) & 1, &bars->abort_flag, p.status, 11, g);
                            if (!ok) break;
                        }
                        store_stage(smem + s * kStageBytes, ring[u], src);
                        fence_generic_to_async_smem();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bars->full[s]);
                        ++g;
                    }
                }
            }
        } else if (warp == kMmaWarp) {
            // ---------------- MMA issuer ----------------
            if (lane == 0) {
                constexpr uint32_t idesc = make_idesc(kBM, kBN);
                int g = 0;
                bool ok = true;
                for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                    for (int j = 0; j < num_issues; ++j, ++g) {
                        const int s = g % kStages;
                        const int b = g & 1;
                        const uint32_t use_b = g >> 1;
                        if (use_b > 0 && !mbar_wait(&bars->tmem_empty[b], (use_b - 1) & 1, &bars->abort_flag, p.status, 12, g)) {
                            ok = false;
                            break;
                        }
                        if (!mbar_wait(&bars->full[s], (g / kStages) & 1, &bars->abort_flag, p.status, 13, g)) {
                            ok = false;
                            break;
                        }
                        tcgen05_fence_after();
                        const uint32_t sa = smem_u32(smem + s * kStageBytes);
                        const uint64_t desc_a = smem_desc_sw128(sa);
                        const uint64_t desc_b = smem_desc_sw128(sa + kStageBytesA);
                        const uint32_t tmem_d = tmem_base + (uint32_t)b * kBN;
    #pragma unroll
                        for (int k = 0; k < kBK / 16; ++k)
                            umma_bf16(tmem_d, desc_a + (uint64_t)(2 * k), desc_b + (uint64_t)(2 * k), idesc, k > 0 ? 1u : 0u);
                        umma_commit(&bars->empty[s]);
                        umma_commit(&bars->tmem_full[b]);
                    }
                }
            }
        } else {
            // ---------------- epilogue ----------------
            const int q = warp & 3;
            const int h = (warp - kEpilogueWarp0) >> 2;
            const float alpha = alpha_value(p.alpha);
            int g = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const Tile tile = locate_tile(plan, t, p.M, p.N);
                float c[kCols];
    #pragma unroll
                for (int i = 0; i < kCols; ++i) c[i] = 0.0f;
                for (int j = 0; j < num_issues; ++j, ++g) {
                    const int b = g & 1;
                    ok = group_wait(warp == kEpilogueWarp0, 2, kEpilogueWarps * 32, &bars->epilogue_go[b], &bars->tmem_full[b],
                                    (g >> 1) & 1, &bars->abort_flag, p.status, 14, g);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * kBN + h * kCols);
    #pragma unroll
                    for (int chunk = 0; chunk < kCols / 32; ++chunk) {
                        uint32_t v[32];
                        tmem_load_32_async(taddr + chunk * 32, v);
                        tmem_wait_ld();
    #pragma unroll
                        for (int i = 0; i < 32; i += 2) fadd2_rz(c[chunk * 32 + i], c[chunk * 32 + i + 1], v[i], v[i + 1]);
                    }
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->tmem_empty[b]);
                }
                if (!ok) break;
                const int local_row = tile.m0 + q * 32 + lane;
                if (local_row >= tile.rows) continue;
                const long long out_row = tile.job == 0 ? (long long)__ldg(p.rec_a + kRecHeader + local_row) : local_row;
                const int col0 = tile.n0 + h * kCols;
                const int* col_map = tile.job == 1 ? p.rec_b + kRecHeader : nullptr;
    #pragma unroll
                for (int i = 0; i < kCols; ++i) {
                    float v = c[i];
                    if (p.snap) v = __fmul_rn(rint_rne(__fmul_rn(v, 1024.0f)), 0.0009765625f);
                    c[i] = __fmul_rn(v, alpha);   // alpha is 1 when the caller gave none: an exact no-op
                }
                if (p.bias) {
    #pragma unroll
                    for (int i = 0; i < kCols; ++i) {
                        const int col = col0 + i;
                        if (col < tile.cols) {
                            const int out_col = col_map ? __ldg(col_map + col) : col;
                            const float bv = p.bias_dtype == UE5M3_DTYPE_BF16
                                                 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[out_col])
                                                 : static_cast<const float*>(p.bias)[out_col];
                            c[i] = __fadd_rn(c[i], bv);
                        }
                    }
                }
                if (p.out_dtype == UE5M3_DTYPE_BF16) store_row<__nv_bfloat16>(p, tile, c, out_row, col0);
                else store_row<float>(p, tile, c, out_row, col0);
            }
        }

        // common exit: every role's loop is bounded, so all threads arrive here
        tcgen05_fence_before();
        __syncthreads();
        if (warp == kMmaWarp) {
            tcgen05_fence_after();
            tmem_dealloc(tmem_base, kTmemCols);
        }
    }

};

template <int BN>
__global__ void __launch_bounds__(Pass<BN>::kThreads, 1) gemm_fallback_kernel(const Params p) {
    Pass<BN>::run(p);
}

template <int BN>
static int launch_pass(const Params& p, cudaStream_t stream) {
    using P = Pass<BN>;
    const size_t smem = (size_t)P::kStages * P::kStageBytes + sizeof(typename P::Barriers) + 1024;
    static bool configured[64] = {false};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64 || !configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_fallback_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (device >= 0 && device < 64) configured[device] = true;
    }
    gemm_fallback_kernel<BN><<<sm_count(), P::kThreads, smem, stream>>>(p);
    return UE5M3_OK;
}

}  // namespace fb
}  // namespace ue5m3

using namespace ue5m3;

extern "C" int ue5m3_gemm_fp4_fallback(const uint8_t* a_codes, const uint8_t* a_sf_raw, const int* a_record,
                                       const uint8_t* b_codes, const uint8_t* b_sf_raw, const int* b_record,
                                       int64_t M, int64_t N, int64_t K, int snap, const float* alpha_dev,
                                       const float* amax_a_dev, const float* amax_b_dev, float inv_denominator,
                                       const void* bias, int bias_dtype, void* out, int out_dtype, int64_t ldo,
                                       int* status_dev, void* stream_v) {
    if (!a_codes || !a_sf_raw || !a_record || !b_codes || !b_sf_raw || !b_record || !out || M <= 0 || N <= 0 || K <= 0)
        return UE5M3_ERR_INVALID_ARGUMENT;
    if (K % fb::kBK) return UE5M3_ERR_K_NOT_DIVISIBLE;
    if (out_dtype != UE5M3_DTYPE_BF16 && out_dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (bias && bias_dtype != UE5M3_DTYPE_BF16 && bias_dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (ldo < N) return UE5M3_ERR_INVALID_ARGUMENT;
    if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) return UE5M3_ERR_TOO_LARGE;
    if (((M + fb::kBM - 1) / fb::kBM) * ((N + 31) / 32) > 0x3FFFFFFF) return UE5M3_ERR_TOO_LARGE;
    if (((uintptr_t)a_codes % 16) || ((uintptr_t)b_codes % 16) || ((uintptr_t)a_sf_raw % 4) || ((uintptr_t)b_sf_raw % 4))
        return UE5M3_ERR_ALIGNMENT;

    fb::Params p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.snap = snap ? 1 : 0;
    p.alpha = AlphaSpec{alpha_dev, amax_a_dev, amax_b_dev, inv_denominator};
    if (!alpha_spec_valid(p.alpha)) return UE5M3_ERR_INVALID_ARGUMENT;
    p.bias = bias; p.bias_dtype = bias_dtype;
    p.out = out; p.out_dtype = out_dtype; p.ldo = ldo; p.status = status_dev;
    p.codes_a = a_codes; p.codes_b = b_codes; p.raw_a = a_sf_raw; p.raw_b = b_sf_raw;
    p.rec_a = a_record; p.rec_b = b_record;
    // two launches, both driven by the records on the device: the listed rows of A (narrow tiles),
    // then the listed rows of B and, after a list overflow, the whole product (wide tiles)
    p.jobs = 1;
    const int status_rows = fb::launch_pass<32>(p, static_cast<cudaStream_t>(stream_v));
    if (status_rows != UE5M3_OK) return status_rows;
    p.jobs = 2 | 4;
    const int status_cols = fb::launch_pass<128>(p, static_cast<cudaStream_t>(stream_v));
    if (status_cols != UE5M3_OK) return status_cols;
    return check_launch();
}
