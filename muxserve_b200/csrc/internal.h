// Declarations shared by the translation units of libmuxb200 (not installed).
#pragma once
#include <cuda_runtime.h>

#include "../../include/muxb200.h"

namespace mux {

// Device address of the status word of the CURRENT device (one word per device,
// a file-scope __device__ variable; resolved once per device and cached).
// Returns nullptr and records the CUDA error when the lookup fails.
unsigned* device_status_ptr();

// Records the error of a failed CUDA call for mux_last_cuda_error and returns MUX_ERR_CUDA.
int record_cuda_error(cudaError_t e);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace mux
