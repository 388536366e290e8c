// The tensor-scale decode factor of a GEMM epilogue: either a ready device scalar, or the two
// held amax scalars and the host-computed fp32 reciprocal of (Ta*6)*(Tb*6), from which every
// epilogue thread forms alpha = fl(fl(amax_a * amax_b) * inv_denominator) - the two roundings of
// backends/triton/quantization.py:412-420 as ATen evaluates them on CUDA tensors - so that no
// separate launch is needed for it.
#pragma once

#include <cuda_runtime.h>

namespace ue5m3 {

struct AlphaSpec {
    const float* alpha;    // device scalar, or null
    const float* amax_a;   // device scalars, or null
    const float* amax_b;
    float inv_denominator;
};

__device__ __forceinline__ bool alpha_enabled(const AlphaSpec& s) { return s.alpha != nullptr || s.amax_a != nullptr; }

__device__ __forceinline__ float alpha_value(const AlphaSpec& s) {
    if (s.alpha) return __ldg(s.alpha);
    if (s.amax_a) return __fmul_rn(__fmul_rn(__ldg(s.amax_a), __ldg(s.amax_b)), s.inv_denominator);
    return 1.0f;
}

inline bool alpha_spec_valid(const AlphaSpec& s) {
    if ((s.amax_a == nullptr) != (s.amax_b == nullptr)) return false;
    return !(s.alpha && s.amax_a);
}

}  // namespace ue5m3
