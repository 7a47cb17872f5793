// The one translation unit of libstk_b200.so: the C ABI declared in include/stk_b200.h.
// The kernels live in the headers included below; they share one device status word, which is
// why the library is built as a single unit.
#include <cuda_runtime.h>

#include "../../include/stk_b200.h"
#include "status.cuh"
#include "bsmm_api.cuh"
#include "meta_sm100.cuh"
#include "plan_sm100.cuh"
#include "dmoe_sm100.cuh"

extern "C" int stk_b200_version(void) { return STK_B200_VERSION; }

extern "C" const char* stk_b200_error_string(int code) {
  switch (code) {
    case STK_OK: return "ok";
    case STK_ERR_NULL_POINTER: return "a required pointer is NULL";
    case STK_ERR_BAD_DIMS: return "incompatible dimensions (M and N must be multiples of 128, K of 32; sizes non-negative)";
    case STK_ERR_BAD_DTYPE: return "unsupported element type";
    case STK_ERR_BAD_LAYOUT: return "pointer not 16-byte aligned or leading dimension not a multiple of 8 elements";
    case STK_ERR_TENSOR_MAP: return "cuTensorMapEncodeTiled failed";
    case STK_ERR_LAUNCH: return "CUDA launch or runtime error";
    case STK_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case STK_ERR_DRIVER: return "CUDA driver entry point unavailable";
    case STK_ERR_TOO_LARGE: return "size beyond what this entry point supports";
    case STK_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel ran out";
    default: return "unknown stk_b200 status";
  }
}

extern "C" int stk_b200_last_tensor_map_error(void) { return stk::g_last_encode_result; }

extern "C" int stk_b200_timeout_site(unsigned int* site_host) {
  if (site_host == nullptr) return STK_ERR_NULL_POINTER;
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, stk::g_timeout_site, sizeof(v)) != cudaSuccess) return STK_ERR_LAUNCH;
  if (v != 0) {
    const unsigned int zero = 0;
    if (cudaMemcpyToSymbol(stk::g_timeout_site, &zero, sizeof(zero)) != cudaSuccess) return STK_ERR_LAUNCH;
  }
  *site_host = v;
  return STK_OK;
}

extern "C" int stk_b200_device_status(int* status_host) {
  if (status_host == nullptr) return STK_ERR_NULL_POINTER;
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, stk::g_device_status, sizeof(int)) != cudaSuccess) return STK_ERR_LAUNCH;
  if (v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(stk::g_device_status, &zero, sizeof(int)) != cudaSuccess) return STK_ERR_LAUNCH;
  }
  *status_host = v;
  return STK_OK;
}

