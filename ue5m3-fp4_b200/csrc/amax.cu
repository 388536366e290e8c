// Tensor amax as a single-pass device reduction (HBM bound: one read of x).
//
// |x| of a finite or non-finite float orders like its unsigned bit pattern
// (sign cleared), with +inf below every NaN.  The reduction therefore runs on
// unsigned integers: the result is exact for finite inputs, and any non-finite
// input surfaces as a result >= 0x7f800000 without a second pass.
//
// Blocks write one partial each into caller-provided scratch; the last block
// to finish (atomic ticket) folds the partials, stores the result and clears
// the ticket, so the scratch is ready for the next launch on the same stream.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "abi_common.cuh"

namespace ue5m3 {

constexpr int kAmaxMaxBlocks = 1024;
constexpr int kAmaxThreads = 256;

struct AmaxScratch {
    uint32_t partial[kAmaxMaxBlocks];
    uint32_t ticket;
    uint32_t pad[3];
};

__device__ __forceinline__ uint32_t umax(uint32_t a, uint32_t b) { return a > b ? a : b; }

// abs bits of two packed bf16 -> max as fp32 bit pattern
__device__ __forceinline__ uint32_t bf16x2_abs_max_bits(uint32_t w, uint32_t m) {
    m = umax(m, (w << 16) & 0x7FFF0000u);
    return umax(m, w & 0x7FFF0000u);
}

__device__ __forceinline__ uint32_t block_reduce_umax(uint32_t m) {
    __shared__ uint32_t warp_max[kAmaxThreads / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = umax(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = threadIdx.x < kAmaxThreads / 32 ? warp_max[threadIdx.x] : 0u;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) m = umax(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    }
    return m;  // valid in thread 0
}

// Folds this block's maximum into scratch and, in the last block, into out.
__device__ __forceinline__ void finish_amax(uint32_t m, AmaxScratch* scratch, float* out) {
    m = block_reduce_umax(m);
    __shared__ bool is_last;
    if (threadIdx.x == 0) {
        scratch->partial[blockIdx.x] = m;
        __threadfence();
        uint32_t ticket = atomicAdd(&scratch->ticket, 1u);
        is_last = ticket == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    uint32_t t = 0u;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += kAmaxThreads)
        t = umax(t, *((volatile uint32_t*)&scratch->partial[i]));
    __syncthreads();  // block_reduce_umax reuses its shared array
    t = block_reduce_umax(t);
    if (threadIdx.x == 0) {
        out[0] = __uint_as_float(t);
        scratch->ticket = 0u;
    }
}

__device__ __forceinline__ uint32_t thread_amax_bits(const void* x, int dtype, int64_t n) {
    uint32_t m = 0u;
    const int64_t tid = (int64_t)blockIdx.x * kAmaxThreads + threadIdx.x;
    const int64_t nthreads = (int64_t)gridDim.x * kAmaxThreads;
    if (dtype == UE5M3_DTYPE_BF16) {
        const uint16_t* p = static_cast<const uint16_t*>(x);
        // head up to a 16-byte boundary, vector body, tail
        int64_t head = ((16 - ((uintptr_t)p & 15)) & 15) / 2;
        if (head > n) head = n;
        int64_t nvec = (n - head) / 8;
        const uint4* v = reinterpret_cast<const uint4*>(p + head);
        for (int64_t i = tid; i < nvec; i += nthreads) {
            uint4 w = __ldg(v + i);
            m = bf16x2_abs_max_bits(w.x, m);
            m = bf16x2_abs_max_bits(w.y, m);
            m = bf16x2_abs_max_bits(w.z, m);
            m = bf16x2_abs_max_bits(w.w, m);
        }
        for (int64_t i = tid; i < head; i += nthreads) m = umax(m, ((uint32_t)p[i] << 16) & 0x7FFF0000u);
        for (int64_t i = head + nvec * 8 + tid; i < n; i += nthreads)
            m = umax(m, ((uint32_t)p[i] << 16) & 0x7FFF0000u);
    } else {
        const uint32_t* p = static_cast<const uint32_t*>(x);
        int64_t head = ((16 - ((uintptr_t)p & 15)) & 15) / 4;
        if (head > n) head = n;
        int64_t nvec = (n - head) / 4;
        const uint4* v = reinterpret_cast<const uint4*>(p + head);
        for (int64_t i = tid; i < nvec; i += nthreads) {
            uint4 w = __ldg(v + i);
            m = umax(m, w.x & 0x7FFFFFFFu);
            m = umax(m, w.y & 0x7FFFFFFFu);
            m = umax(m, w.z & 0x7FFFFFFFu);
            m = umax(m, w.w & 0x7FFFFFFFu);
        }
        for (int64_t i = tid; i < head; i += nthreads) m = umax(m, p[i] & 0x7FFFFFFFu);
        for (int64_t i = head + nvec * 4 + tid; i < n; i += nthreads) m = umax(m, p[i] & 0x7FFFFFFFu);
    }
    return m;
}

__global__ void __launch_bounds__(kAmaxThreads)
amax_kernel(const void* __restrict__ x, int dtype, int64_t n, float* __restrict__ out,
            AmaxScratch* __restrict__ scratch) {
    finish_amax(thread_amax_bits(x, dtype, n), scratch, out);
}

// Reduction scratch of ue5m3_amax_static: lives in the library image, one copy per GPU
// that loads the library, zero at load time.  Host code may not use this name as a
// pointer; its device address is looked up once per device (static_scratch_for_device).
static __device__ __align__(256) AmaxScratch g_static_amax_scratch;

constexpr int kMaxDevices = 64;
constexpr int64_t kStaticAmaxMaxElements = (int64_t)1 << 32;

static int amax_grid(int dtype, int64_t n) {
    int64_t per_thread = dtype == UE5M3_DTYPE_BF16 ? 8 : 4;
    int64_t want = (n + per_thread * kAmaxThreads * 4 - 1) / (per_thread * kAmaxThreads * 4);
    int64_t cap = (int64_t)sm_count() * 6;
    if (cap > kAmaxMaxBlocks) cap = kAmaxMaxBlocks;
    if (want > cap) want = cap;
    return (int)(want < 1 ? 1 : want);
}

}  // namespace ue5m3

using namespace ue5m3;

// Device address of the static scratch on the current device, resolved on first use.  The
// table is written without a lock: two threads that race on a device's first call both look
// the address up and both store the same value, so the worst case is one redundant lookup.
// It is keyed by the CURRENT device, which therefore has to be the stream's device on every
// call, not only on the first.
static int static_scratch_for_device(AmaxScratch** out) {
    static AmaxScratch* cache[kMaxDevices] = {nullptr};
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (device < 0 || device >= kMaxDevices) return UE5M3_ERR_UNSUPPORTED;
    if (cache[device] == nullptr) {
        void* address = nullptr;
        e = cudaGetSymbolAddress(&address, g_static_amax_scratch);
        if (e != cudaSuccess) return record_cuda_error(e);
        cache[device] = static_cast<AmaxScratch*>(address);
    }
    *out = cache[device];
    return UE5M3_OK;
}

extern "C" size_t ue5m3_amax_scratch_bytes(void) { return sizeof(AmaxScratch); }

extern "C" int ue5m3_amax_static(const void* x, int dtype, int64_t n, float* amax_out,
                                 void* stream_v) {
    if (!x || !amax_out || n <= 0) return UE5M3_ERR_INVALID_ARGUMENT;
    if (dtype != UE5M3_DTYPE_BF16 && dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (n > kStaticAmaxMaxElements) {
        record_error_text("ue5m3_amax_static: more than 2^32 elements; use ue5m3_amax with caller scratch");
        return UE5M3_ERR_TOO_LARGE;
    }
    AmaxScratch* scratch = nullptr;
    int status = static_scratch_for_device(&scratch);
    if (status != UE5M3_OK) return status;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    // The ticket must start at zero; the array keeps whatever the previous call left.
    cudaError_t e = cudaMemsetAsync(&scratch->ticket, 0, sizeof(uint32_t), stream);
    if (e != cudaSuccess) return record_cuda_error(e);
    amax_kernel<<<amax_grid(dtype, n), kAmaxThreads, 0, stream>>>(x, dtype, n, amax_out, scratch);
    return check_launch();
}

extern "C" int ue5m3_amax(const void* x, int dtype, int64_t n, float* amax_out, void* scratch,
                          size_t scratch_bytes, void* stream_v) {
    if (!x || !amax_out || !scratch || n <= 0) return UE5M3_ERR_INVALID_ARGUMENT;
    if (dtype != UE5M3_DTYPE_BF16 && dtype != UE5M3_DTYPE_FP32) return UE5M3_ERR_INVALID_ARGUMENT;
    if (scratch_bytes < sizeof(AmaxScratch)) return UE5M3_ERR_SCRATCH;
    if (((uintptr_t)scratch % 16) != 0) return UE5M3_ERR_ALIGNMENT;
    amax_kernel<<<amax_grid(dtype, n), kAmaxThreads, 0, static_cast<cudaStream_t>(stream_v)>>>(
        x, dtype, n, amax_out, static_cast<AmaxScratch*>(scratch));
    return check_launch();
}
