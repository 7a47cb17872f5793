// Per-device kernel status word.  Kernels never trap: a kernel that has to give up (a bounded
// wait ran out) records a negative STK_ERR_* code here and returns; the host reads it on demand.
#pragma once
#include <cuda_runtime.h>

namespace stk {

__device__ int g_device_status = 0;

// Keeps the first reported problem.
__device__ __forceinline__ void report_status(int code) { atomicCAS(&g_device_status, 0, code); }

// Where the first bounded wait ran out: warp | cluster rank << 8 | barrier's shared-memory offset << 12 |
// parity << 31 (0: no wait has run out).  A diagnostic next to the status word, cleared with it.
__device__ unsigned int g_timeout_site = 0;

}  // namespace stk
