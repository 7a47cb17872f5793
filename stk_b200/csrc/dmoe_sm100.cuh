// Kernels around the block-sparse products in a dropless-MoE layer: moving token rows into and out
// of padded expert bins, and writing the block-diagonal topology (with its transposed metadata, in
// closed form) for a given number of block rows per expert.  HBM-bound row copies with 16-byte
// accesses, and tiny integer kernels.  The reference has no counterpart (it is a matmul library);
// these are the callers' side of stk.Matrix(...) / stk.ops.sdd / stk.ops.dsd.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/stk_b200.h"

namespace stk {

// dst[i] = index[i] >= 0 ? src[index[i]] : 0, rows of `vec_per_row` 16-byte vectors.  One warp per
// output row; every output row is written exactly once (padding rows as zeros).
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                   const int32_t* __restrict__ index, int64_t n_rows, int vec_per_row) {
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int32_t s = index[row];
  uint4* out = dst + row * vec_per_row;
  if (s < 0) {
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    for (int v = lane; v < vec_per_row; v += 32) out[v] = z;
  } else {
    const uint4* in = src + static_cast<int64_t>(s) * vec_per_row;
    for (int v = lane; v < vec_per_row; v += 32) out[v] = __ldg(in + v);
  }
}

// dst[index[i]] = src[i] for index[i] >= 0.
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                    const int32_t* __restrict__ index, int64_t n_rows, int vec_per_row) {
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int32_t d = index[row];
  if (d < 0) return;
  const uint4* in = src + row * vec_per_row;
  uint4* out = dst + static_cast<int64_t>(d) * vec_per_row;
  for (int v = lane; v < vec_per_row; v += 32) out[v] = __ldg(in + v);
}

// Gather index of the padded expert bins of one rank.  Rows arrive from `world` peers, each peer's
// rows ordered by local expert: counts[p * local + e] rows from peer p for expert e.  Bin e holds
// the rows for expert e ordered by peer, then zero padding up to a multiple of `block`.
// index[r] = source row of padded row r, or -1 for padding; with `compose`, the source row is looked
// up through it (compose[source]), e.g. the sort order that produced the received rows.
// bin_rows[e] = padded rows / block.
__global__ void __launch_bounds__(256)
bin_index_kernel(const int64_t* __restrict__ counts, int world, int local, int block,
                 const int32_t* __restrict__ compose, int32_t* __restrict__ index,
                 int64_t total_padded, int32_t* __restrict__ bin_rows) {
  extern __shared__ int64_t sm[];
  int64_t* bin_start = sm;              // [local + 1] padded
  int64_t* src_start = sm + local + 1;  // [world * local] position of segment (p, e) in the received rows
  if (threadIdx.x == 0) {
    int64_t run = 0;
    for (int p = 0; p < world; ++p)
      for (int e = 0; e < local; ++e) {
        src_start[p * local + e] = run;
        run += counts[p * local + e];
      }
    int64_t pad = 0;
    for (int e = 0; e < local; ++e) {
      int64_t n = 0;
      for (int p = 0; p < world; ++p) n += counts[p * local + e];
      bin_start[e] = pad;
      const int64_t rows = (n + block - 1) / block;
      if (blockIdx.x == 0 && bin_rows != nullptr) bin_rows[e] = static_cast<int32_t>(rows);
      pad += rows * block;
    }
    bin_start[local] = pad;
  }
  __syncthreads();
  const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= total_padded) return;
  int e = 0;
  while (e + 1 < local && bin_start[e + 1] <= r) ++e;
  int64_t q = r - bin_start[e];  // position inside bin e
  int32_t src = -1;
  for (int p = 0; p < world; ++p) {
    const int64_t n = counts[p * local + e];
    if (q < n) {
      src = static_cast<int32_t>(src_start[p * local + e] + q);
      break;
    }
    q -= n;
  }
  index[r] = (src >= 0 && compose != nullptr) ? compose[src] : src;
}

// Block-diagonal topology: expert e owns bin_rows[e] consecutive block rows and the block columns
// [e*cpb, (e+1)*cpb).  One thread per block writes both the row-major and the column-major
// metadata; nothing is sorted.
__global__ void __launch_bounds__(256)
dmoe_topology_kernel(const int32_t* __restrict__ bin_rows, int experts, int cpb, int64_t nnz,
                     int block_rows, int16_t* __restrict__ row_indices,
                     int16_t* __restrict__ column_indices, int32_t* __restrict__ offsets,
                     int16_t* __restrict__ column_indices_t, int32_t* __restrict__ offsets_t,
                     int32_t* __restrict__ block_offsets_t) {
  extern __shared__ int32_t row_start[];  // [experts + 1] first block row of every expert
  if (threadIdx.x == 0) {
    int32_t run = 0;
    for (int e = 0; e < experts; ++e) {
      row_start[e] = run;
      run += bin_rows[e];
    }
    row_start[experts] = run;
  }
  __syncthreads();
  const int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // column-major offsets: one entry per block column (plus the end), written by the first threads
  const int64_t block_cols = static_cast<int64_t>(experts) * cpb;
  if (p <= block_cols) {
    if (p == block_cols) {
      offsets_t[p] = static_cast<int32_t>(nnz);
    } else {
      const int e = static_cast<int>(p / cpb), j = static_cast<int>(p - static_cast<int64_t>(e) * cpb);
      offsets_t[p] = row_start[e] * cpb + j * bin_rows[e];
    }
  }
  if (p <= block_rows) offsets[p] = static_cast<int32_t>(p * cpb);
  if (p >= nnz) return;
  // row-major position p: block row r, j-th column block of its expert
  const int r = static_cast<int>(p / cpb), j = static_cast<int>(p - static_cast<int64_t>(r) * cpb);
  int lo = 0, hi = experts - 1;  // expert e with row_start[e] <= r < row_start[e+1]
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (row_start[mid] <= r) lo = mid; else hi = mid - 1;
  }
  const int e = lo;
  row_indices[p] = static_cast<int16_t>(r);
  column_indices[p] = static_cast<int16_t>(e * cpb + j);
  // the same block in column-major order: column e*cpb + j, k-th block row of the expert
  const int k = r - row_start[e];
  const int64_t q = static_cast<int64_t>(row_start[e]) * cpb + static_cast<int64_t>(j) * bin_rows[e] + k;
  column_indices_t[q] = static_cast<int16_t>(r);
  block_offsets_t[q] = static_cast<int32_t>(p);
}

}  // namespace stk

using namespace stk;

static int rows_args_ok(const void* src, const void* dst, const int32_t* index, int64_t n_rows,
                        int64_t row_bytes) {
  if (n_rows < 0 || row_bytes <= 0 || row_bytes % 16) return STK_ERR_BAD_DIMS;
  if (row_bytes / 16 > INT32_MAX) return STK_ERR_TOO_LARGE;
  if (n_rows == 0) return STK_OK;
  if (src == nullptr || dst == nullptr || index == nullptr) return STK_ERR_NULL_POINTER;
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) return STK_ERR_BAD_LAYOUT;
  return STK_OK;
}

extern "C" int stk_b200_gather_rows(const void* src, void* dst, const int32_t* index, int64_t n_rows,
                                    int64_t row_bytes, void* stream) {
  const int rc = rows_args_ok(src, dst, index, n_rows, row_bytes);
  if (rc != STK_OK || n_rows == 0) return rc;
  const int64_t ctas = (n_rows + 7) / 8;
  if (ctas > INT32_MAX) return STK_ERR_TOO_LARGE;
  gather_rows_kernel<<<static_cast<unsigned>(ctas), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), index, n_rows,
      static_cast<int>(row_bytes / 16));
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

extern "C" int stk_b200_scatter_rows(const void* src, void* dst, const int32_t* index,
                                     int64_t n_rows, int64_t row_bytes, void* stream) {
  const int rc = rows_args_ok(src, dst, index, n_rows, row_bytes);
  if (rc != STK_OK || n_rows == 0) return rc;
  const int64_t ctas = (n_rows + 7) / 8;
  if (ctas > INT32_MAX) return STK_ERR_TOO_LARGE;
  scatter_rows_kernel<<<static_cast<unsigned>(ctas), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), index, n_rows,
      static_cast<int>(row_bytes / 16));
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

extern "C" int stk_b200_bin_index(const int64_t* counts, int world, int local_experts, int block,
                                  const int32_t* compose, int32_t* index, int64_t total_padded,
                                  int32_t* bin_rows, void* stream) {
  if (world <= 0 || local_experts <= 0 || block <= 0 || total_padded < 0) return STK_ERR_BAD_DIMS;
  if (static_cast<int64_t>(world) * local_experts > 4096 || total_padded > INT32_MAX) return STK_ERR_TOO_LARGE;
  if (counts == nullptr || (total_padded > 0 && index == nullptr)) return STK_ERR_NULL_POINTER;
  const size_t smem = (static_cast<size_t>(local_experts) + 1 + static_cast<size_t>(world) * local_experts) * sizeof(int64_t);
  const int64_t ctas = total_padded > 0 ? (total_padded + 255) / 256 : 1;
  bin_index_kernel<<<static_cast<unsigned>(ctas), 256, smem, static_cast<cudaStream_t>(stream)>>>(
      counts, world, local_experts, block, compose, index, total_padded, bin_rows);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

extern "C" int stk_b200_dmoe_topology(const int32_t* bin_rows, int experts, int cols_per_expert,
                                      int64_t block_rows, int16_t* row_indices,
                                      int16_t* column_indices, int32_t* offsets,
                                      int16_t* column_indices_t, int32_t* offsets_t,
                                      int32_t* block_offsets_t, void* stream) {
  if (experts <= 0 || cols_per_expert <= 0 || block_rows < 0) return STK_ERR_BAD_DIMS;
  const int64_t block_cols = static_cast<int64_t>(experts) * cols_per_expert;
  if (experts > 8192 || block_rows > 32767 || block_cols > 32767) return STK_ERR_TOO_LARGE;
  if (bin_rows == nullptr || offsets == nullptr || offsets_t == nullptr) return STK_ERR_NULL_POINTER;
  const int64_t nnz = block_rows * cols_per_expert;
  if (nnz > INT32_MAX) return STK_ERR_TOO_LARGE;
  if (nnz > 0 && (row_indices == nullptr || column_indices == nullptr ||
                  column_indices_t == nullptr || block_offsets_t == nullptr))
    return STK_ERR_NULL_POINTER;
  int64_t threads = nnz;
  if (threads < block_cols + 1) threads = block_cols + 1;
  if (threads < block_rows + 1) threads = block_rows + 1;
  const int64_t ctas = (threads + 255) / 256;
  dmoe_topology_kernel<<<static_cast<unsigned>(ctas), 256, (experts + 1) * sizeof(int32_t),
                         static_cast<cudaStream_t>(stream)>>>(
      bin_rows, experts, cols_per_expert, nnz, static_cast<int>(block_rows), row_indices,
      column_indices, offsets, column_indices_t, offsets_t, block_offsets_t);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}
