// Status strings, error text and device queries of the C ABI.
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include "abi_common.cuh"

namespace ue5m3 {

static thread_local char g_error_text[256] = "";

void record_error_text(const char* text) {
    strncpy(g_error_text, text, sizeof(g_error_text) - 1);
    g_error_text[sizeof(g_error_text) - 1] = '\0';
}

int record_cuda_error(cudaError_t error) {
    if (error == cudaSuccess) return UE5M3_OK;
    record_error_text(cudaGetErrorString(error));
    return UE5M3_ERR_CUDA;
}

int check_launch() { return record_cuda_error(cudaGetLastError()); }

int sm_count() {
    static int counts[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    if (counts[device] == 0) {
        int value = 0;
        if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
            value <= 0)
            value = 148;
        counts[device] = value;
    }
    return counts[device];
}

}  // namespace ue5m3

extern "C" int ue5m3_abi_version(void) { return UE5M3_ABI_VERSION; }

extern "C" const char* ue5m3_status_string(int status) {
    switch (status) {
        case UE5M3_OK: return "ok";
        case UE5M3_ERR_INVALID_ARGUMENT: return "invalid argument";
        case UE5M3_ERR_BLOCK_SIZE: return "block_size must be 16 or 32";
        case UE5M3_ERR_K_NOT_DIVISIBLE: return "reduction dimension is not divisible as required";
        case UE5M3_ERR_ALIGNMENT: return "pointer or leading dimension is not 16-byte aligned";
        case UE5M3_ERR_UNSUPPORTED: return "unsupported combination of options";
        case UE5M3_ERR_CUDA: return "CUDA error";
        case UE5M3_ERR_SCRATCH: return "scratch buffer too small";
        case UE5M3_ERR_TOO_LARGE: return "size exceeds the supported maximum";
        default: return "unknown status";
    }
}

extern "C" const char* ue5m3_last_cuda_error(void) { return ue5m3::g_error_text; }
