// Per-device kernel status word.  Kernels never trap: a kernel that has to give up (a bounded
// wait ran out) records a negative STK_ERR_* code here and returns; the host reads it on demand.
#pragma once
#include <cuda_runtime.h>

namespace stk {

__device__ int g_device_status = 0;

// Keeps the first reported problem.
__device__ __forceinline__ void report_status(int code) { atomicCAS(&g_device_status, 0, code); }

}  // namespace stk
