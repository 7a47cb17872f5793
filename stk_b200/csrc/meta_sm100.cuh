// Integer metadata and dense<->sparse conversion kernels.  All HBM-bound byte/integer work:
// coalesced, 16-byte vectorised where the layout allows, every output written once.
//
//   row_indices      CSR offsets -> COO block-row index        (reference: triton_kernels.py:381-393)
//   transpose_meta   stable counting sort of blocks by column  (reference: matrix.py:105-123)
//   block_mask / mask_to_offsets / mask_to_indices / gather_blocks
//                    the phases of to_sparse                   (reference: matrix_ops.py:50-85)
//   to_dense         blocks -> dense, zero elsewhere           (reference: matrix_ops.py:15-47)
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/stk_b200.h"
#include "index.cuh"
#include "status.cuh"

namespace stk {

// ------------------------------------------------------------------------------------------
// row_indices: block p belongs to the block row r with offsets[r] <= p < offsets[r+1].
// One thread per block, binary search, fully coalesced stores.
__global__ void row_indices_kernel(const int32_t* __restrict__ offsets, IndexArray out, int block_rows,
                                   int nnz) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= nnz) return;
  int lo = 0, hi = block_rows - 1;  // smallest r with offsets[r+1] > p
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (offsets[mid + 1] > p) hi = mid; else lo = mid + 1;
  }
  out.store(p, lo);
}

// ------------------------------------------------------------------------------------------
// Exclusive scan of v[0..n) in place by one 1024-thread CTA; the total goes to v[n].
__global__ void __launch_bounds__(1024, 1) exclusive_scan_kernel(int32_t* v, int n) {
  __shared__ int32_t warp_sums[32];
  const int tid = threadIdx.x;
  const int ipt = (n + 1023) / 1024;
  const int begin = min(n, tid * ipt);
  const int end = min(n, begin + ipt);
  int32_t sum = 0;
  for (int i = begin; i < end; ++i) sum += v[i];
  // block-wide exclusive scan of `sum`
  const int lane = tid & 31, warp = tid >> 5;
  int32_t incl = sum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int32_t t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int32_t w = warp_sums[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t t = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += t;
    }
    warp_sums[lane] = w;  // inclusive over warps
  }
  __syncthreads();
  int32_t run = incl - sum + (warp > 0 ? warp_sums[warp - 1] : 0);
  for (int i = begin; i < end; ++i) {
    const int32_t t = v[i];
    v[i] = run;
    run += t;
  }
  if (tid == 1023) v[n] = run;  // the last thread's running sum is the total
}

// ------------------------------------------------------------------------------------------
// transpose_meta.
//
// The blocks arrive sorted by (row, column); the transposed order is the STABLE sort by column.
// The block list is cut into G contiguous groups, one warp each.  hist[g][c] first counts the
// blocks of group g in column c, then (prefix over g) becomes the rank of the group's first such
// block inside column c.  A warp then walks its group 32 blocks at a time; blocks of one column
// inside a window keep their lane order, so the result is deterministic and stable.

struct TransposePlan {
  int groups;       // G
  int chunk;        // blocks per group, a multiple of 32
  bool fused;       // single-CTA shared-memory path
};

constexpr int kFusedThreads = 1024;
constexpr int kFusedGroups = 32;
constexpr int64_t kFusedMaxCols = 1536;    // 32*Cb*4 + (Cb+1)*4 bytes of shared memory <= ~200 KiB
constexpr int64_t kFusedMaxNnz = 8192;     // beyond this one CTA is slower than the multi-kernel path
constexpr int64_t kHistEntriesCap = 1 << 20;  // 4 MiB of workspace at most

static inline TransposePlan plan_transpose(int64_t nnz, int64_t block_cols,
                                           int64_t hist_entries_cap = kHistEntriesCap) {
  TransposePlan pl;
  if (block_cols <= kFusedMaxCols && nnz <= kFusedMaxNnz) {
    pl.fused = true;
    pl.groups = kFusedGroups;
    int64_t chunk = (nnz + kFusedGroups - 1) / kFusedGroups;
    pl.chunk = static_cast<int>(((chunk + 31) / 32) * 32);
    if (pl.chunk == 0) pl.chunk = 32;
    return pl;
  }
  pl.fused = false;
  int64_t g = hist_entries_cap / block_cols;
  if (g > 1024) g = 1024;
  if (g < 1) g = 1;
  const int64_t windows = (nnz + 31) / 32;
  if (g > windows) g = windows;
  int64_t chunk = (nnz + g - 1) / g;
  chunk = ((chunk + 31) / 32) * 32;
  pl.chunk = static_cast<int>(chunk);
  pl.groups = static_cast<int>((nnz + chunk - 1) / chunk);
  return pl;
}

// Shared by both paths: one warp scatters blocks [begin, end) given per-column start positions
// `colstart` and its group's rank counters `hist_g` (shared or global memory).
// A block whose column index lies outside [0, block_cols) is left out (the reference's histc drops
// such values too) and reported through the status word; it never indexes the counters.
__device__ __forceinline__ void scatter_group(IndexArray rows, IndexArray cols, int begin, int end,
                                              int block_cols, const int32_t* colstart, int32_t* hist_g,
                                              IndexArray column_indices_t,
                                              int32_t* __restrict__ block_offsets_t) {
  const int lane = threadIdx.x & 31;
  const uint32_t lt_mask = (1u << lane) - 1u;
  for (int base = begin; base < end; base += 32) {
    const int i = base + lane;
    int c = i < end ? cols[i] : -1;
    const bool active = static_cast<unsigned>(c) < static_cast<unsigned>(block_cols);
    // Inactive lanes get distinct negative keys so that they never match a column.
    const int key = active ? c : -1 - lane;
    const uint32_t peers = __match_any_sync(0xffffffffu, key);
    const int rank = __popc(peers & lt_mask);
    const int leader = __ffs(peers) - 1;
    int32_t first = 0;
    if (active && rank == 0) first = atomicAdd(&hist_g[key], __popc(peers));
    first = __shfl_sync(0xffffffffu, first, leader);
    if (active) {
      const int dst = colstart[key] + first + rank;
      column_indices_t.store(dst, rows[i]);
      block_offsets_t[dst] = i;
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(kFusedThreads, 1)
transpose_fused_kernel(IndexArray rows, IndexArray cols, int nnz, int block_cols, int chunk,
                       IndexArray column_indices_t,
                       int32_t* __restrict__ offsets_t, int32_t* __restrict__ block_offsets_t) {
  extern __shared__ int32_t tsm[];
  int32_t* hist = tsm;                                  // [32][block_cols]
  int32_t* colstart = tsm + kFusedGroups * block_cols;  // [block_cols + 1]
  __shared__ int32_t warp_sums[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < kFusedGroups * block_cols; i += kFusedThreads) hist[i] = 0;
  __syncthreads();
  const int begin = min(nnz, warp * chunk), end = min(nnz, begin + chunk);
  for (int i = begin + lane; i < end; i += 32) {
    const int c = cols[i];
    if (static_cast<unsigned>(c) < static_cast<unsigned>(block_cols)) atomicAdd(&hist[warp * block_cols + c], 1);
    else report_status(STK_ERR_BAD_DIMS);
  }
  __syncthreads();
  // prefix over groups; colstart[c] = blocks in column c
  for (int c = tid; c < block_cols; c += kFusedThreads) {
    int32_t run = 0;
#pragma unroll 8
    for (int g = 0; g < kFusedGroups; ++g) {
      const int32_t t = hist[g * block_cols + c];
      hist[g * block_cols + c] = run;
      run += t;
    }
    colstart[c] = run;
  }
  __syncthreads();
  // exclusive scan of colstart over the columns
  {
    const int ipt = (block_cols + kFusedThreads - 1) / kFusedThreads;
    const int b0 = min(block_cols, tid * ipt), b1 = min(block_cols, b0 + ipt);
    int32_t sum = 0;
    for (int i = b0; i < b1; ++i) sum += colstart[i];
    int32_t incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t t = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += t;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int32_t w = warp_sums[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int32_t t = __shfl_up_sync(0xffffffffu, w, d);
        if (lane >= d) w += t;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    int32_t run = incl - sum + (warp > 0 ? warp_sums[warp - 1] : 0);
    for (int i = b0; i < b1; ++i) {
      const int32_t t = colstart[i];
      colstart[i] = run;
      offsets_t[i] = run;
      run += t;
    }
    if (tid == kFusedThreads - 1) {
      colstart[block_cols] = run;
      offsets_t[block_cols] = run;
    }
  }
  __syncthreads();
  scatter_group(rows, cols, begin, end, block_cols, colstart, hist + warp * block_cols, column_indices_t,
                block_offsets_t);
}

// General path, kernel 1: hist[g][c] = number of blocks of group g in column c (hist pre-zeroed).
__global__ void transpose_count_kernel(IndexArray cols, int nnz, int block_cols,
                                       int chunk, int groups, int32_t* __restrict__ hist) {
  const int g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (g >= groups) return;
  const int begin = min(nnz, g * chunk), end = min(nnz, begin + chunk);
  int32_t* hist_g = hist + static_cast<int64_t>(g) * block_cols;
  for (int i = begin + lane; i < end; i += 32) {
    const int c = cols[i];
    if (static_cast<unsigned>(c) < static_cast<unsigned>(block_cols)) atomicAdd(&hist_g[c], 1);
    else report_status(STK_ERR_BAD_DIMS);
  }
}

// General path, kernel 2: per column, exclusive prefix over the groups; column totals to counts[c].
// A warp per column, 32 groups per step with a warp scan (a thread per column walking the groups one
// by one took 165 us for the 64 columns x 1024 groups of a top-2 slot sort: a chain of L2 round trips).
__global__ void __launch_bounds__(256)
transpose_group_prefix_kernel(int32_t* __restrict__ hist, int block_cols, int groups,
                              int32_t* __restrict__ counts) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (c >= block_cols) return;
  int32_t run = 0;
  for (int g0 = 0; g0 < groups; g0 += 32) {
    const int g = g0 + lane;
    const int64_t idx = static_cast<int64_t>(g) * block_cols + c;
    const int32_t t = g < groups ? hist[idx] : 0;
    int32_t incl = t;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    if (g < groups) hist[idx] = run + incl - t;
    run += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) counts[c] = run;
}

// General path, kernel 4 (kernel 3 is exclusive_scan_kernel on offsets_t).
__global__ void transpose_scatter_kernel(IndexArray rows, IndexArray cols, int nnz, int block_cols,
                                         int chunk, int groups, int32_t* __restrict__ hist,
                                         const int32_t* __restrict__ offsets_t,
                                         IndexArray column_indices_t,
                                         int32_t* __restrict__ block_offsets_t) {
  const int g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (g >= groups) return;
  const int begin = min(nnz, g * chunk), end = min(nnz, begin + chunk);
  scatter_group(rows, cols, begin, end, block_cols, offsets_t, hist + static_cast<int64_t>(g) * block_cols,
                column_indices_t, block_offsets_t);
}

// ------------------------------------------------------------------------------------------
// block_mask.

// Vector path: 16-bit elements, blocking % 8 == 0, rows 16-byte aligned.  A CTA covers one block
// row, 2048 columns and 1/gridDim.z of the block's rows; a thread ORs one 16-byte column strip.
__global__ void __launch_bounds__(256)
block_mask_vec_kernel(const uint16_t* __restrict__ x, int64_t ld, int cols, int blocking,
                      int block_cols, int br0, uint8_t* __restrict__ mask) {
  const int col0 = (blockIdx.x * 256 + threadIdx.x) * 8;
  const int br = br0 + blockIdx.y;  // the grid's y extent is limited: tall matrices take several launches
  const int rows_per_split = (blocking + gridDim.z - 1) / gridDim.z;
  const int r0 = blockIdx.z * rows_per_split;
  const int r1 = min(blocking, r0 + rows_per_split);
  bool nz = false;
  if (col0 < cols) {
    const uint16_t* src = x + (static_cast<int64_t>(br) * blocking + r0) * ld + col0;
    uint32_t acc = 0;
#pragma unroll 4
    for (int r = r0; r < r1; ++r, src += ld) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
      // drop the sign bits: +0 and -0 are both zero
      acc |= (v.x | v.y | v.z | v.w) & 0x7fff7fffu;
    }
    nz = acc != 0;
  }
  // Neighbouring lanes of one block report once.
  const int bc = col0 / blocking;
  const int prev_bc = __shfl_up_sync(0xffffffffu, bc, 1);
  const int prev_nz = __shfl_up_sync(0xffffffffu, nz ? 1 : 0, 1);
  const bool dup = (threadIdx.x & 31) != 0 && prev_bc == bc && prev_nz;
  if (nz && !dup) mask[static_cast<int64_t>(br) * block_cols + bc] = 1;
}

// Generic path: one thread per block.
template <typename T, T kAbsMask>
__global__ void block_mask_generic_kernel(const T* __restrict__ x, int64_t ld, int blocking,
                                          int block_rows, int block_cols,
                                          uint8_t* __restrict__ mask) {
  const int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (b >= static_cast<int64_t>(block_rows) * block_cols) return;
  const int br = static_cast<int>(b / block_cols), bc = static_cast<int>(b % block_cols);
  const T* src = x + static_cast<int64_t>(br) * blocking * ld + static_cast<int64_t>(bc) * blocking;
  T acc = 0;
  for (int r = 0; r < blocking; ++r)
    for (int c = 0; c < blocking; ++c) acc |= src[r * ld + c] & kAbsMask;
  mask[b] = acc != 0 ? 1 : 0;
}

// counts[r] = set bytes in mask row r.  One warp per row.
__global__ void mask_row_count_kernel(const uint8_t* __restrict__ mask, int block_rows,
                                      int block_cols, int32_t* __restrict__ counts) {
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= block_rows) return;
  const uint8_t* m = mask + static_cast<int64_t>(r) * block_cols;
  int32_t n = 0;
  for (int c = lane; c < block_cols; c += 32) n += m[c] != 0;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) n += __shfl_xor_sync(0xffffffffu, n, d);
  if (lane == 0) counts[r] = n;
}

// Ordered compaction of one mask row per warp.
__global__ void mask_to_indices_kernel(const uint8_t* __restrict__ mask, int block_rows,
                                       int block_cols, const int32_t* __restrict__ offsets,
                                       IndexArray row_indices, IndexArray column_indices) {
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= block_rows) return;
  const uint8_t* m = mask + static_cast<int64_t>(r) * block_cols;
  int32_t pos = offsets[r];
  for (int c0 = 0; c0 < block_cols; c0 += 32) {
    const int c = c0 + lane;
    const bool set = c < block_cols && m[c] != 0;
    const uint32_t bal = __ballot_sync(0xffffffffu, set);
    if (set) {
      const int dst = pos + __popc(bal & ((1u << lane) - 1u));
      row_indices.store(dst, r);
      column_indices.store(dst, c);
    }
    pos += __popc(bal);
  }
}

// ------------------------------------------------------------------------------------------
// gather_blocks: data[p] = x[r_p*b : +b, c_p*b : +b].

// Vector path: one CTA per block, 16-byte copies, rows of the block are contiguous in `data`.
__global__ void __launch_bounds__(256)
gather_blocks_vec_kernel(const uint16_t* __restrict__ x, int64_t ld, int blocking, int block_rows,
                         int block_cols, IndexArray row_indices, IndexArray column_indices,
                         uint16_t* __restrict__ data) {
  const int64_t p = blockIdx.x;
  const int vec_per_row = blocking / 8;
  const int nvec = blocking * vec_per_row;
  const int br = row_indices[p], bc = column_indices[p];
  uint4* dst = reinterpret_cast<uint4*>(data + p * blocking * blocking);
  if (br < 0 || br >= block_rows || bc < 0 || bc >= block_cols) {
    // a block outside the matrix is never read: its values become zeros and the call is reported
    if (threadIdx.x == 0) report_status(STK_ERR_BAD_DIMS);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const uint16_t* src = x + static_cast<int64_t>(br) * blocking * ld + static_cast<int64_t>(bc) * blocking;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const int r = v / vec_per_row, c = v - r * vec_per_row;
    dst[v] = __ldg(reinterpret_cast<const uint4*>(src + r * ld) + c);
  }
}

template <typename T>
__global__ void gather_blocks_generic_kernel(const T* __restrict__ x, int64_t ld, int blocking, int block_rows,
                                             int block_cols, IndexArray row_indices,
                                             IndexArray column_indices, int64_t total, T* __restrict__ data) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int64_t bb = static_cast<int64_t>(blocking) * blocking;
  const int64_t p = i / bb;
  const int rem = static_cast<int>(i - p * bb);
  const int r = rem / blocking, c = rem - r * blocking;
  const int br = row_indices[p], bc = column_indices[p];
  if (br < 0 || br >= block_rows || bc < 0 || bc >= block_cols) {
    if (rem == 0) report_status(STK_ERR_BAD_DIMS);
    data[i] = 0;
    return;
  }
  data[i] = x[(static_cast<int64_t>(br) * blocking + r) * ld + static_cast<int64_t>(bc) * blocking + c];
}

// ------------------------------------------------------------------------------------------
// to_dense: every output tile is either a copy of its block or zeros; found by binary search in
// the block row's (sorted) column list.
__device__ __forceinline__ int find_block(const int32_t* __restrict__ offsets,
                                          IndexArray column_indices, int br,
                                          int bc) {
  int lo = offsets[br], hi = offsets[br + 1];
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    const int c = column_indices[mid];
    if (c == bc) return mid;
    if (c < bc) lo = mid + 1; else hi = mid;
  }
  return -1;
}

__global__ void __launch_bounds__(256)
to_dense_vec_kernel(const uint16_t* __restrict__ data, const int32_t* __restrict__ offsets,
                    IndexArray column_indices, int blocking, int br0,
                    uint16_t* __restrict__ out, int64_t ld_out) {
  const int bc = blockIdx.x, br = br0 + blockIdx.y;
  const int p = find_block(offsets, column_indices, br, bc);
  const int vec_per_row = blocking / 8;
  const int nvec = blocking * vec_per_row;
  uint16_t* dst = out + static_cast<int64_t>(br) * blocking * ld_out +
                  static_cast<int64_t>(bc) * blocking;
  const uint4* src =
      p >= 0 ? reinterpret_cast<const uint4*>(data + static_cast<int64_t>(p) * blocking * blocking)
             : nullptr;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const int r = v / vec_per_row, c = v - r * vec_per_row;
    const uint4 val = src ? __ldg(src + v) : make_uint4(0u, 0u, 0u, 0u);
    reinterpret_cast<uint4*>(dst + r * ld_out)[c] = val;
  }
}

// Small blocks (blocking < 64): a CTA per block would move 128 B - 2 KiB.  Instead a CTA covers one
// block row and 2048 columns; a thread owns one 16-byte column strip (8 elements, inside one block
// because blocking % 8 == 0), finds its block once (binary search in the row's column list) and walks
// down the block's rows: output rows are written as contiguous 4 KiB runs by the CTA.
__global__ void __launch_bounds__(256)
to_dense_strip_kernel(const uint16_t* __restrict__ data, const int32_t* __restrict__ offsets,
                      IndexArray column_indices, int blocking, int cols, int br0,
                      uint16_t* __restrict__ out, int64_t ld_out) {
  const int col0 = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (col0 >= cols) return;
  const int br = br0 + blockIdx.y, bc = col0 / blocking;
  const int p = find_block(offsets, column_indices, br, bc);
  uint16_t* dst = out + static_cast<int64_t>(br) * blocking * ld_out + col0;
  if (p < 0) {
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 4
    for (int r = 0; r < blocking; ++r, dst += ld_out) *reinterpret_cast<uint4*>(dst) = z;
    return;
  }
  const uint16_t* src = data + static_cast<int64_t>(p) * blocking * blocking + (col0 - bc * blocking);
#pragma unroll 4
  for (int r = 0; r < blocking; ++r, dst += ld_out, src += blocking)
    *reinterpret_cast<uint4*>(dst) = __ldg(reinterpret_cast<const uint4*>(src));
}

// The same geometry for gather_blocks: threads whose block is absent have nothing to do.
__global__ void __launch_bounds__(256)
gather_blocks_strip_kernel(const uint16_t* __restrict__ x, int64_t ld, int blocking, int cols,
                           const int32_t* __restrict__ offsets,
                           IndexArray column_indices, int br0, uint16_t* __restrict__ data) {
  const int col0 = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (col0 >= cols) return;
  const int br = br0 + blockIdx.y, bc = col0 / blocking;
  const int p = find_block(offsets, column_indices, br, bc);
  if (p < 0) return;
  const uint16_t* src = x + static_cast<int64_t>(br) * blocking * ld + col0;
  uint16_t* dst = data + static_cast<int64_t>(p) * blocking * blocking + (col0 - bc * blocking);
#pragma unroll 4
  for (int r = 0; r < blocking; ++r, src += ld, dst += blocking)
    *reinterpret_cast<uint4*>(dst) = __ldg(reinterpret_cast<const uint4*>(src));
}

template <typename T>
__global__ void to_dense_generic_kernel(const T* __restrict__ data,
                                        const int32_t* __restrict__ offsets,
                                        IndexArray column_indices, int blocking,
                                        int64_t rows, int64_t cols, T* __restrict__ out,
                                        int64_t ld_out) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * cols) return;
  const int64_t row = i / cols, col = i - row * cols;
  const int br = static_cast<int>(row / blocking), bc = static_cast<int>(col / blocking);
  const int p = find_block(offsets, column_indices, br, bc);
  T v = 0;
  if (p >= 0)
    v = data[static_cast<int64_t>(p) * blocking * blocking + (row - static_cast<int64_t>(br) * blocking) * blocking +
             (col - static_cast<int64_t>(bc) * blocking)];
  out[row * ld_out + col] = v;
}

static inline bool ptr_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline int launch_status() { return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH; }

}  // namespace stk

using namespace stk;

// ====================================================================== host side
// Every routine that takes or produces block indices exists twice in the C ABI: with int16 indices
// (the reference's format) and, suffixed _i32, with int32 indices.  Both are thin wrappers of the
// *_impl functions below, which see the indices through IndexArray.
namespace stk {

constexpr int kMaxGridY = 65535;

static int row_indices_impl(const int32_t* offsets, IndexArray out, int64_t block_rows, int64_t nnz,
                            void* stream) {
  if (block_rows < 0 || nnz < 0) return STK_ERR_BAD_DIMS;
  if (block_rows > index_limit(out.wide) || nnz > INT32_MAX) return STK_ERR_TOO_LARGE;
  if (nnz == 0) return STK_OK;
  if (offsets == nullptr || out.null()) return STK_ERR_NULL_POINTER;
  if (block_rows == 0) return STK_ERR_BAD_DIMS;
  const int threads = 256;
  const int blocks = static_cast<int>((nnz + threads - 1) / threads);
  row_indices_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      offsets, out, static_cast<int>(block_rows), static_cast<int>(nnz));
  return launch_status();
}

// Shared by the caller-workspace entry point and the variant with built-in scratch.
static int transpose_meta_launch(IndexArray row_indices, IndexArray column_indices, int64_t nnz,
                                 int64_t block_cols, IndexArray column_indices_t, int32_t* offsets_t,
                                 int32_t* block_offsets_t, void* workspace, cudaStream_t s,
                                 int64_t hist_entries_cap = kHistEntriesCap) {
  const TransposePlan pl = plan_transpose(nnz, block_cols, hist_entries_cap);
  const int n = static_cast<int>(nnz), cb = static_cast<int>(block_cols);
  if (pl.fused) {
    static bool opted_in[64] = {};
    const size_t smem = (static_cast<size_t>(kFusedGroups) * cb + cb + 1) * sizeof(int32_t);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return STK_ERR_LAUNCH;
    if (!opted_in[dev]) {
      if (cudaFuncSetAttribute(transpose_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>((kFusedGroups * kFusedMaxCols + kFusedMaxCols + 1) *
                                                sizeof(int32_t))) != cudaSuccess) {
        cudaGetLastError();
        return STK_ERR_LAUNCH;
      }
      opted_in[dev] = true;
    }
    transpose_fused_kernel<<<1, kFusedThreads, smem, s>>>(row_indices, column_indices, n, cb,
                                                          pl.chunk, column_indices_t, offsets_t,
                                                          block_offsets_t);
    return launch_status();
  }
  int32_t* hist = static_cast<int32_t*>(workspace);
  const size_t hist_bytes = static_cast<size_t>(pl.groups) * cb * sizeof(int32_t);
  if (cudaMemsetAsync(hist, 0, hist_bytes, s) != cudaSuccess) return STK_ERR_LAUNCH;
  const int warps_per_cta = 8;
  const int group_ctas = (pl.groups + warps_per_cta - 1) / warps_per_cta;
  transpose_count_kernel<<<group_ctas, warps_per_cta * 32, 0, s>>>(column_indices, n, cb, pl.chunk,
                                                                   pl.groups, hist);
  transpose_group_prefix_kernel<<<(cb + 7) / 8, 256, 0, s>>>(hist, cb, pl.groups, offsets_t);
  exclusive_scan_kernel<<<1, 1024, 0, s>>>(offsets_t, cb);
  transpose_scatter_kernel<<<group_ctas, warps_per_cta * 32, 0, s>>>(
      row_indices, column_indices, n, cb, pl.chunk, pl.groups, hist, offsets_t, column_indices_t,
      block_offsets_t);
  return launch_status();
}

static size_t transpose_workspace_bytes(int64_t nnz, int64_t block_cols) {
  if (nnz <= 0 || block_cols <= 0) return 0;
  const TransposePlan pl = plan_transpose(nnz, block_cols);
  if (pl.fused) return 0;
  return static_cast<size_t>(pl.groups) * static_cast<size_t>(block_cols) * sizeof(int32_t);
}

static int transpose_meta_impl(IndexArray row_indices, IndexArray column_indices, int64_t nnz,
                               int64_t block_cols, IndexArray column_indices_t, int32_t* offsets_t,
                               int32_t* block_offsets_t, void* workspace, size_t workspace_bytes,
                               void* stream) {
  if (nnz < 0 || block_cols <= 0) return STK_ERR_BAD_DIMS;
  // the per-group counters are indexed [group][column]: keep their number within int range
  if (block_cols > index_limit(column_indices.wide) || block_cols > (1 << 24) || nnz > INT32_MAX)
    return STK_ERR_TOO_LARGE;
  if (offsets_t == nullptr) return STK_ERR_NULL_POINTER;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (nnz == 0) {
    return cudaMemsetAsync(offsets_t, 0, (block_cols + 1) * sizeof(int32_t), s) == cudaSuccess
               ? STK_OK
               : STK_ERR_LAUNCH;
  }
  if (row_indices.null() || column_indices.null() || column_indices_t.null() ||
      block_offsets_t == nullptr)
    return STK_ERR_NULL_POINTER;
  const size_t need = transpose_workspace_bytes(nnz, block_cols);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need || !ptr_aligned16(workspace)))
    return STK_ERR_WORKSPACE;
  return transpose_meta_launch(row_indices, column_indices, nnz, block_cols, column_indices_t,
                               offsets_t, block_offsets_t, workspace, s);
}

static int mask_to_indices_impl(const uint8_t* mask, int64_t block_rows, int64_t block_cols,
                                const int32_t* offsets, IndexArray row_indices,
                                IndexArray column_indices, void* stream) {
  if (block_rows < 0 || block_cols < 0) return STK_ERR_BAD_DIMS;
  const long long limit = index_limit(row_indices.wide);
  if (block_rows > limit || block_cols > limit || block_rows > (1 << 28)) return STK_ERR_TOO_LARGE;
  if (block_rows == 0 || block_cols == 0) return STK_OK;
  if (mask == nullptr || offsets == nullptr || row_indices.null() || column_indices.null())
    return STK_ERR_NULL_POINTER;
  const int R = static_cast<int>(block_rows), Cb = static_cast<int>(block_cols);
  mask_to_indices_kernel<<<(R + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      mask, R, Cb, offsets, row_indices, column_indices);
  return launch_status();
}

static int gather_blocks_impl(const void* x, int64_t rows, int64_t cols, int64_t ld, int blocking,
                              int elem_bytes, const int32_t* offsets, IndexArray row_indices,
                              IndexArray column_indices, int64_t nnz, void* data, void* stream) {
  if (blocking <= 0 || rows < 0 || cols < 0 || nnz < 0 || rows % blocking || cols % blocking ||
      ld < cols)
    return STK_ERR_BAD_DIMS;
  if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4) return STK_ERR_BAD_DTYPE;
  if (nnz == 0) return STK_OK;
  if (nnz > INT32_MAX || cols > INT32_MAX) return STK_ERR_TOO_LARGE;
  if (x == nullptr || data == nullptr || row_indices.null() || column_indices.null())
    return STK_ERR_NULL_POINTER;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec = elem_bytes == 2 && blocking % 8 == 0 && ld % 8 == 0 && ptr_aligned16(x) &&
                   ptr_aligned16(data);
  if (rows / blocking > INT32_MAX || cols / blocking > INT32_MAX) return STK_ERR_TOO_LARGE;
  const int block_rows = static_cast<int>(rows / blocking), block_cols = static_cast<int>(cols / blocking);
  if (vec && blocking < 64 && offsets != nullptr) {
    const int64_t R = rows / blocking;
    for (int64_t br0 = 0; br0 < R; br0 += kMaxGridY) {
      const dim3 grid(static_cast<unsigned>((cols / 8 + 255) / 256),
                      static_cast<unsigned>(R - br0 < kMaxGridY ? R - br0 : kMaxGridY));
      gather_blocks_strip_kernel<<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(x), ld, blocking,
                                                      static_cast<int>(cols), offsets, column_indices,
                                                      static_cast<int>(br0), static_cast<uint16_t*>(data));
    }
  } else if (vec) {
    gather_blocks_vec_kernel<<<static_cast<unsigned>(nnz), 256, 0, s>>>(
        static_cast<const uint16_t*>(x), ld, blocking, block_rows, block_cols, row_indices, column_indices,
        static_cast<uint16_t*>(data));
  } else {
    const int64_t total = nnz * blocking * blocking;
    const int64_t blocks = (total + 255) / 256;
    if (blocks > INT32_MAX) return STK_ERR_TOO_LARGE;
    if (elem_bytes == 1)
      gather_blocks_generic_kernel<uint8_t><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
          static_cast<const uint8_t*>(x), ld, blocking, block_rows, block_cols, row_indices, column_indices,
          total, static_cast<uint8_t*>(data));
    else if (elem_bytes == 2)
      gather_blocks_generic_kernel<uint16_t><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
          static_cast<const uint16_t*>(x), ld, blocking, block_rows, block_cols, row_indices, column_indices,
          total, static_cast<uint16_t*>(data));
    else
      gather_blocks_generic_kernel<uint32_t><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
          static_cast<const uint32_t*>(x), ld, blocking, block_rows, block_cols, row_indices, column_indices,
          total, static_cast<uint32_t*>(data));
  }
  return launch_status();
}

static int to_dense_impl(const void* data, const int32_t* offsets, IndexArray column_indices,
                         int64_t block_rows, int64_t block_cols, int blocking, int elem_bytes,
                         void* out, int64_t ld_out, void* stream) {
  if (blocking <= 0 || block_rows < 0 || block_cols < 0 || ld_out < block_cols * blocking)
    return STK_ERR_BAD_DIMS;
  if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4) return STK_ERR_BAD_DTYPE;
  const long long limit = index_limit(column_indices.wide);
  if (block_rows > limit || block_cols > limit || block_cols * blocking > INT32_MAX ||
      block_rows > (1 << 28))
    return STK_ERR_TOO_LARGE;
  if (block_rows == 0 || block_cols == 0) return STK_OK;
  // `data` and `column_indices` may be NULL when there is no block at all.
  if (offsets == nullptr || out == nullptr) return STK_ERR_NULL_POINTER;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec = elem_bytes == 2 && blocking % 8 == 0 && ld_out % 8 == 0 && ptr_aligned16(out) &&
                   ptr_aligned16(data);
  if (vec) {
    const int64_t cols = block_cols * blocking;
    for (int64_t br0 = 0; br0 < block_rows; br0 += kMaxGridY) {
      const unsigned gy = static_cast<unsigned>(block_rows - br0 < kMaxGridY ? block_rows - br0 : kMaxGridY);
      if (blocking < 64) {
        const dim3 grid(static_cast<unsigned>((cols / 8 + 255) / 256), gy);
        to_dense_strip_kernel<<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(data), offsets,
                                                   column_indices, blocking, static_cast<int>(cols),
                                                   static_cast<int>(br0), static_cast<uint16_t*>(out), ld_out);
      } else {
        const dim3 grid(static_cast<unsigned>(block_cols), gy);
        to_dense_vec_kernel<<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(data), offsets,
                                                 column_indices, blocking, static_cast<int>(br0),
                                                 static_cast<uint16_t*>(out), ld_out);
      }
    }
  } else {
    const int64_t rows = block_rows * blocking, cols = block_cols * blocking;
    const int64_t blocks = (rows * cols + 255) / 256;
    if (blocks > INT32_MAX) return STK_ERR_TOO_LARGE;
    if (elem_bytes == 1)
      to_dense_generic_kernel<uint8_t><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
          static_cast<const uint8_t*>(data), offsets, column_indices, blocking, rows, cols,
          static_cast<uint8_t*>(out), ld_out);
    else if (elem_bytes == 2)
      to_dense_generic_kernel<uint16_t><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
          static_cast<const uint16_t*>(data), offsets, column_indices, blocking, rows, cols,
          static_cast<uint16_t*>(out), ld_out);
    else
      to_dense_generic_kernel<uint32_t><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
          static_cast<const uint32_t*>(data), offsets, column_indices, blocking, rows, cols,
          static_cast<uint32_t*>(out), ld_out);
  }
  return launch_status();
}

// transpose_meta with built-in scratch, for callers that cannot allocate device memory.
constexpr int64_t kStaticScratchEntries = 1 << 18;        // 1 MiB of int32 counters
constexpr int64_t kStaticMaxBlockCols = 8192;             // leaves >= 32 groups of counters
constexpr int64_t kStaticMaxNnz = 1 << 20;
// The group-by-column counters of the multi-kernel transpose path.  In host code this name is only
// a handle for cudaGetSymbolAddress; the device address is looked up once per device below.
static __device__ __align__(256) int32_t g_transpose_scratch[kStaticScratchEntries];

}  // namespace stk

using namespace stk;

extern "C" int stk_b200_row_indices(const int32_t* offsets, int16_t* out, int64_t block_rows,
                                    int64_t nnz, void* stream) {
  return row_indices_impl(offsets, IndexArray{out, 0}, block_rows, nnz, stream);
}
extern "C" int stk_b200_row_indices_i32(const int32_t* offsets, int32_t* out, int64_t block_rows,
                                        int64_t nnz, void* stream) {
  return row_indices_impl(offsets, IndexArray{out, 1}, block_rows, nnz, stream);
}

extern "C" size_t stk_b200_transpose_meta_workspace_bytes(int64_t nnz, int64_t block_cols) {
  return transpose_workspace_bytes(nnz, block_cols);
}
extern "C" int stk_b200_transpose_meta(const int16_t* row_indices, const int16_t* column_indices,
                                       int64_t nnz, int64_t block_cols, int16_t* column_indices_t,
                                       int32_t* offsets_t, int32_t* block_offsets_t, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  return transpose_meta_impl(IndexArray{row_indices, 0}, IndexArray{column_indices, 0}, nnz, block_cols,
                             IndexArray{column_indices_t, 0}, offsets_t, block_offsets_t, workspace,
                             workspace_bytes, stream);
}
extern "C" int stk_b200_transpose_meta_i32(const int32_t* row_indices, const int32_t* column_indices,
                                           int64_t nnz, int64_t block_cols, int32_t* column_indices_t,
                                           int32_t* offsets_t, int32_t* block_offsets_t,
                                           void* workspace, size_t workspace_bytes, void* stream) {
  return transpose_meta_impl(IndexArray{row_indices, 1}, IndexArray{column_indices, 1}, nnz, block_cols,
                             IndexArray{column_indices_t, 1}, offsets_t, block_offsets_t, workspace,
                             workspace_bytes, stream);
}

extern "C" int stk_b200_block_mask(const void* x, int64_t rows, int64_t cols, int64_t ld,
                                   int blocking, int elem_bytes, uint8_t* mask, void* stream) {
  if (blocking <= 0 || rows < 0 || cols < 0 || rows % blocking || cols % blocking || ld < cols)
    return STK_ERR_BAD_DIMS;
  if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4) return STK_ERR_BAD_DTYPE;
  if (rows == 0 || cols == 0) return STK_OK;
  if (x == nullptr || mask == nullptr) return STK_ERR_NULL_POINTER;
  const int64_t R = rows / blocking, Cb = cols / blocking;
  if (R > (1 << 28) || Cb > (1 << 28) || cols > INT32_MAX) return STK_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec = elem_bytes == 2 && blocking % 8 == 0 && ld % 8 == 0 && ptr_aligned16(x);
  if (vec) {
    if (cudaMemsetAsync(mask, 0, R * Cb, s) != cudaSuccess) return STK_ERR_LAUNCH;
    const int splits = blocking >= 128 ? 4 : (blocking >= 32 ? 2 : 1);
    for (int64_t br0 = 0; br0 < R; br0 += kMaxGridY) {
      const dim3 grid(static_cast<unsigned>((cols / 8 + 255) / 256),
                      static_cast<unsigned>(R - br0 < kMaxGridY ? R - br0 : kMaxGridY), splits);
      block_mask_vec_kernel<<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(x), ld,
                                                 static_cast<int>(cols), blocking,
                                                 static_cast<int>(Cb), static_cast<int>(br0), mask);
    }
  } else {
    const int64_t nb = R * Cb;
    if ((nb + 255) / 256 > INT32_MAX) return STK_ERR_TOO_LARGE;
    const unsigned blocks = static_cast<unsigned>((nb + 255) / 256);
    if (elem_bytes == 1)  // 8-bit floats: the element-wise kernels only
      block_mask_generic_kernel<uint8_t, 0x7f><<<blocks, 256, 0, s>>>(
          static_cast<const uint8_t*>(x), ld, blocking, static_cast<int>(R), static_cast<int>(Cb), mask);
    else if (elem_bytes == 2)
      block_mask_generic_kernel<uint16_t, 0x7fff><<<blocks, 256, 0, s>>>(
          static_cast<const uint16_t*>(x), ld, blocking, static_cast<int>(R), static_cast<int>(Cb), mask);
    else
      block_mask_generic_kernel<uint32_t, 0x7fffffffu><<<blocks, 256, 0, s>>>(
          static_cast<const uint32_t*>(x), ld, blocking, static_cast<int>(R), static_cast<int>(Cb), mask);
  }
  return launch_status();
}

extern "C" int stk_b200_mask_to_offsets(const uint8_t* mask, int64_t block_rows, int64_t block_cols,
                                        int32_t* offsets, void* stream) {
  if (block_rows < 0 || block_cols < 0) return STK_ERR_BAD_DIMS;
  if (block_rows > (1 << 28) || block_cols > (1 << 28)) return STK_ERR_TOO_LARGE;
  if (offsets == nullptr) return STK_ERR_NULL_POINTER;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (block_rows == 0 || block_cols == 0) {
    return cudaMemsetAsync(offsets, 0, (block_rows + 1) * sizeof(int32_t), s) == cudaSuccess
               ? STK_OK
               : STK_ERR_LAUNCH;
  }
  if (mask == nullptr) return STK_ERR_NULL_POINTER;
  const int R = static_cast<int>(block_rows), Cb = static_cast<int>(block_cols);
  mask_row_count_kernel<<<(R + 7) / 8, 256, 0, s>>>(mask, R, Cb, offsets);
  exclusive_scan_kernel<<<1, 1024, 0, s>>>(offsets, R);
  return launch_status();
}

extern "C" int stk_b200_mask_to_indices(const uint8_t* mask, int64_t block_rows, int64_t block_cols,
                                        const int32_t* offsets, int16_t* row_indices,
                                        int16_t* column_indices, void* stream) {
  return mask_to_indices_impl(mask, block_rows, block_cols, offsets, IndexArray{row_indices, 0},
                              IndexArray{column_indices, 0}, stream);
}
extern "C" int stk_b200_mask_to_indices_i32(const uint8_t* mask, int64_t block_rows,
                                            int64_t block_cols, const int32_t* offsets,
                                            int32_t* row_indices, int32_t* column_indices,
                                            void* stream) {
  return mask_to_indices_impl(mask, block_rows, block_cols, offsets, IndexArray{row_indices, 1},
                              IndexArray{column_indices, 1}, stream);
}

extern "C" int stk_b200_gather_blocks(const void* x, int64_t rows, int64_t cols, int64_t ld,
                                      int blocking, int elem_bytes, const int32_t* offsets,
                                      const int16_t* row_indices, const int16_t* column_indices,
                                      int64_t nnz, void* data, void* stream) {
  return gather_blocks_impl(x, rows, cols, ld, blocking, elem_bytes, offsets, IndexArray{row_indices, 0},
                            IndexArray{column_indices, 0}, nnz, data, stream);
}
extern "C" int stk_b200_gather_blocks_i32(const void* x, int64_t rows, int64_t cols, int64_t ld,
                                          int blocking, int elem_bytes, const int32_t* offsets,
                                          const int32_t* row_indices, const int32_t* column_indices,
                                          int64_t nnz, void* data, void* stream) {
  return gather_blocks_impl(x, rows, cols, ld, blocking, elem_bytes, offsets, IndexArray{row_indices, 1},
                            IndexArray{column_indices, 1}, nnz, data, stream);
}

// ------------------------------------------------------------------------------------------
// regroup_blocks: b x b blocks (b = 16, 32 or 64) <-> their places inside 128 x 128 blocks, which is how the
// matmul kernels (built for 128 x 128 blocks) run products of matrices with smaller blocks: slot[p] =
// coarse block * q*q + (block row % q) * q + block column % q with q = 128 / b.  16-byte copies, a thread
// per vector, consecutive threads along a block's rows.
__global__ void __launch_bounds__(256)
regroup_blocks_kernel(uint4* __restrict__ fine, uint4* __restrict__ coarse, const int32_t* __restrict__ slot,
                      int64_t total_vecs, int64_t coarse_slots, int blocking, int vec_per_row, int to_coarse) {
  const int q = 128 / blocking;
  const int vecs_per_block = blocking * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total_vecs;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t p = i / vecs_per_block;
    const int v = static_cast<int>(i - p * vecs_per_block);
    const int row = v / vec_per_row, cv = v - row * vec_per_row;
    const int64_t s = slot[p];
    if (s < 0 || s >= coarse_slots) {
      // a slot outside the coarse matrix is never touched: gathered values become zeros, the call is reported
      if (v == 0) report_status(STK_ERR_BAD_DIMS);
      if (!to_coarse) fine[i] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const int64_t cb = s / (q * q);
    const int within = static_cast<int>(s - cb * (q * q));
    const int rq = within / q, cq = within - rq * q;
    const int64_t ci = (cb * 128 + rq * blocking + row) * (static_cast<int64_t>(vec_per_row) * q) + cq * vec_per_row + cv;
    if (to_coarse) coarse[ci] = fine[i];
    else fine[i] = coarse[ci];
  }
}

extern "C" int stk_b200_regroup_blocks(void* fine, void* coarse, const int32_t* slot, int64_t nnz,
                                       int64_t coarse_blocks, int blocking, int elem_bytes, int to_coarse,
                                       void* stream) {
  if ((blocking != 16 && blocking != 32 && blocking != 64) || nnz < 0 || coarse_blocks < 0) return STK_ERR_BAD_DIMS;
  if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4) return STK_ERR_BAD_DTYPE;
  if (nnz == 0) return STK_OK;
  if (fine == nullptr || coarse == nullptr || slot == nullptr) return STK_ERR_NULL_POINTER;
  if (!ptr_aligned16(fine) || !ptr_aligned16(coarse)) return STK_ERR_BAD_LAYOUT;
  const int q = 128 / blocking;
  if (coarse_blocks > INT32_MAX / (q * q)) return STK_ERR_TOO_LARGE;
  const int vec_per_row = blocking * elem_bytes / 16;
  const int64_t total = nnz * blocking * vec_per_row;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = 148 * 16;
  if (blocks > cap) blocks = cap;
  regroup_blocks_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(fine), static_cast<uint4*>(coarse), slot, total, coarse_blocks * q * q, blocking,
      vec_per_row, to_coarse);
  return launch_status();
}

extern "C" int stk_b200_to_dense(const void* data, const int32_t* offsets,
                                 const int16_t* column_indices, int64_t block_rows,
                                 int64_t block_cols, int blocking, int elem_bytes, void* out,
                                 int64_t ld_out, void* stream) {
  return to_dense_impl(data, offsets, IndexArray{column_indices, 0}, block_rows, block_cols, blocking,
                       elem_bytes, out, ld_out, stream);
}
extern "C" int stk_b200_to_dense_i32(const void* data, const int32_t* offsets,
                                     const int32_t* column_indices, int64_t block_rows,
                                     int64_t block_cols, int blocking, int elem_bytes, void* out,
                                     int64_t ld_out, void* stream) {
  return to_dense_impl(data, offsets, IndexArray{column_indices, 1}, block_rows, block_cols, blocking,
                       elem_bytes, out, ld_out, stream);
}

extern "C" int stk_b200_transpose_meta_static(const int16_t* row_indices,
                                              const int16_t* column_indices, int64_t nnz,
                                              int64_t block_cols, int16_t* column_indices_t,
                                              int32_t* offsets_t, int32_t* block_offsets_t,
                                              void* stream) {
  if (nnz < 0 || block_cols <= 0) return STK_ERR_BAD_DIMS;
  if (block_cols > kStaticMaxBlockCols || nnz > kStaticMaxNnz) return STK_ERR_TOO_LARGE;
  if (offsets_t == nullptr) return STK_ERR_NULL_POINTER;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (nnz == 0) {
    return cudaMemsetAsync(offsets_t, 0, (block_cols + 1) * sizeof(int32_t), s) == cudaSuccess
               ? STK_OK
               : STK_ERR_LAUNCH;
  }
  if (row_indices == nullptr || column_indices == nullptr || column_indices_t == nullptr ||
      block_offsets_t == nullptr)
    return STK_ERR_NULL_POINTER;
  // Device address of the scratch array: resolved on the first call on each device, with that
  // device current (the first call on a device should therefore come before any stream capture).
  static void* scratch_addr[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return STK_ERR_LAUNCH;
  if (scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_transpose_scratch) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return STK_ERR_LAUNCH;
    }
    scratch_addr[dev] = ptr;
  }
  // The counters are cleared inside (cudaMemsetAsync on the part this call uses); the array
  // keeps whatever the previous call left elsewhere.
  return transpose_meta_launch(IndexArray{row_indices, 0}, IndexArray{column_indices, 0}, nnz, block_cols,
                               IndexArray{column_indices_t, 0}, offsets_t, block_offsets_t,
                               scratch_addr[dev], s, kStaticScratchEntries);
}
