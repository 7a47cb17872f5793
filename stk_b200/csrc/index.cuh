// Block row / column indices come as int16 (the reference's format, stk/matrix.py:96-99, good for up
// to 32767 blocks per side) or as int32 (beyond that; the reference leaves this as a TODO,
// stk/matrix.py:161-167).  Kernels read and write them through this view; the width is uniform over
// a launch, so the branch costs nothing next to the memory access it selects.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace stk {

struct IndexArray {
  const void* ptr;
  int wide;  // 0: int16, 1: int32
  __device__ __forceinline__ int operator[](long long i) const {
    return wide ? __ldg(static_cast<const int32_t*>(ptr) + i)
                : static_cast<int>(__ldg(static_cast<const int16_t*>(ptr) + i));
  }
  __device__ __forceinline__ void store(long long i, int v) const {
    if (wide) static_cast<int32_t*>(const_cast<void*>(ptr))[i] = v;
    else static_cast<int16_t*>(const_cast<void*>(ptr))[i] = static_cast<int16_t>(v);
  }
  __host__ __device__ bool null() const { return ptr == nullptr; }
};

// Largest number of block rows / columns an index width can name.
static inline long long index_limit(int wide) { return wide ? 0x7fffffffll : 32767ll; }

}  // namespace stk
