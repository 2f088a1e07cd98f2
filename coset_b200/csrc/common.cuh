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
// The same residuals packed into 4 bytes per level word (layout at e8::biased_bytes_q4m2), 256 KB:
// mostly L1-resident, for the bandwidth-bound decoder whose gathers otherwise wait on L2.  Kernels
// bound by instruction issue keep the 8-byte entries, which unpack with 12 fewer instructions.
const uint32_t* residual_table_q4_packed(cudaStream_t stream);

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace coset
