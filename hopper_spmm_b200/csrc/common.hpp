// Status plumbing shared by the host-side translation units.  The reference turns every CUDA
// failure into exit(1) (src/utils/utils.h:9-21); here a failing call is recorded for the
// calling thread and surfaces as B200SPMM_ERR_CUDA.
#pragma once

#include <cuda_runtime.h>

#include "../../include/b200_spmm.h"

namespace b200spmm {

// Remembers `what: cudaGetErrorString(e)` for b200spmm_last_cuda_error().
void record_cuda_error(cudaError_t e, const char *what);
// Same, for a fixed message: keeps the pointer, allocates nothing.
void set_last_error_static(const char *message);

// How long a device-side wait may spin before the kernel gives up (nanoseconds).
constexpr unsigned long long kDeviceWaitLimitNs = 2000000000ull;

// Bits of the device status word a kernel may raise.
enum : unsigned { kDevStatusTimeout = 1u };

}  // namespace b200spmm

#define B200_CUDA_TRY(expr)                              \
    do {                                                 \
        cudaError_t e__ = (expr);                        \
        if (e__ != cudaSuccess) {                        \
            ::b200spmm::record_cuda_error(e__, #expr);   \
            return B200SPMM_ERR_CUDA;                    \
        }                                                \
    } while (0)
