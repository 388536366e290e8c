// Host-side helpers shared by the translation units of the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <stdlib.h>

#include "../../include/ue5m3_fp4.h"

namespace ue5m3 {

// Number of SMs of the current device (cached per device ordinal).
int sm_count();

// cudaGetLastError() -> status code; records the error text for
// ue5m3_last_cuda_error().
int check_launch();
int record_cuda_error(cudaError_t error);
void record_error_text(const char* text);

}  // namespace ue5m3
