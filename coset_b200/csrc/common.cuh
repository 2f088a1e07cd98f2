// Shared host-side helpers of the C-ABI translation units: error reporting and launch checks.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/coset_b200.h"

namespace coset {

// Stores a message for coset_last_error_string() (thread local) and returns `code`.
int fail(int code, const char* fmt, ...);
// cudaGetLastError() after a launch -> 0 or a positive cudaError_t (message stored).
int check_launch(const char* what);
int check_cuda(cudaError_t e, const char* what);

// Number of SMs of the current device (cached per device).
int sm_count();

// Device pointer to the q=4 single-level residual table of the current device:
// 65536 entries x 8 bytes = twice the residual G b - 4 Q(G b / 4) of level word `b`, plus 7.
// Built once per device by the library's own literal decoder; nullptr on failure (message stored).
const uint2* residual_table_q4(cudaStream_t stream);

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace coset
