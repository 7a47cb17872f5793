// Per-topology preparation for the CTA-pair kernel (bsmm_pair_sm100.cuh), computed once per
// topology instead of in every launch:
//
//   pair_stats  how well neighbouring block rows / block columns pair up, and whether the metadata
//               is ordered the way the pair kernel's merge walks need it.  The host reads the five
//               numbers (they may be written straight into pinned host memory) and picks a kernel.
//   pair_plan   the work-item table of the pair kernel: the block rows (or block columns) cut into
//               runs where two neighbours' lists cannot overlap, paired inside each run, the groups
//               listed longest list first.  The pair kernel reads one table entry per work item.
//
// Small integer kernels, one CTA each; latency-bound.  The reference has no counterpart (its Triton
// kernels take one 128x128 tile per program, stk/backend/triton_kernels.py:21-220).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/stk_b200.h"
#include "index.cuh"

namespace stk {

constexpr int kPlanThreads = 1024;
constexpr int kPlanSortMaxGroups = 4096;  // beyond this the groups stay in row order

// Position of column `c` in block row `r` (lists ascending), or -1.
__device__ __forceinline__ int plan_find(const int32_t* __restrict__ offsets,
                                         IndexArray cols, int r, int c) {
  int lo = offsets[r], hi = offsets[r + 1];
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    const int v = cols[mid];
    if (v == c) return mid;
    if (v < c) lo = mid + 1; else hi = mid;
  }
  return -1;
}

// stats[0] = distinct (row pair, column) positions      -> useful share of row pairs  = nnz / (2 stats[0])
// stats[1] = distinct (row, column pair) positions      -> useful share of column pairs
// stats[2] = distinct (row pair, column pair) positions -> useful share of 2x2 tiles  = nnz / (4 stats[2])
// stats[3] = 1 if the blocks are listed in strictly ascending (row, column) order, consistently
//            with `offsets`, and every index is in range; else 0 (then stats[0..2] mean nothing)
// stats[4] = 1 if every block column's segment of column_indices_t ascends and is in range, 0 if
//            not, -1 if the transposed metadata was not given
// stats[5] = 1, written last (a completion mark for a host that polls the memory)
__global__ void __launch_bounds__(kPlanThreads, 1)
pair_stats_kernel(const int32_t* __restrict__ offsets, IndexArray rows, IndexArray cols,
                  const int32_t* __restrict__ offsets_t, IndexArray cols_t, int block_rows, int block_cols, int nnz,
                  volatile int32_t* stats) {
  __shared__ int acc[5];
  if (threadIdx.x < 5) acc[threadIdx.x] = threadIdx.x >= 3 ? 1 : 0;
  __syncthreads();
  // pass 1: order and ranges (everything else relies on them)
  int ordered = 1;
  for (int r = threadIdx.x; r < block_rows; r += kPlanThreads) {
    const int a = offsets[r], b = offsets[r + 1];
    if (a > b || a < 0 || b > nnz || (r == 0 && a != 0) || (r == block_rows - 1 && b != nnz)) ordered = 0;
  }
  for (int p = threadIdx.x; p < nnz; p += kPlanThreads) {
    const int r = rows[p], c = cols[p];
    if (r < 0 || r >= block_rows || c < 0 || c >= block_cols) { ordered = 0; continue; }
    const int a = offsets[r], b = offsets[r + 1];
    if (p < a || p >= b) ordered = 0;
    if (p > 0) {
      const int pr = rows[p - 1], pc = cols[p - 1];
      if (pr > r || (pr == r && pc >= c)) ordered = 0;
    }
  }
  if (!ordered) atomicAnd(&acc[3], 0);
  __syncthreads();
  if (acc[3]) {
    int n_rp = 0, n_cp = 0, n_t = 0;
    for (int p = threadIdx.x; p < nnz; p += kPlanThreads) {
      const int r = rows[p], c = cols[p];
      // a position is counted by the first of the blocks that share it
      const bool left = (c & 1) && p > offsets[r] && cols[p - 1] == c - 1;  // (r, c-1) exists
      bool up = false, up_tile = false;
      if (r & 1) {
        up = plan_find(offsets, cols, r - 1, c) >= 0;
        up_tile = up || plan_find(offsets, cols, r - 1, c ^ 1) >= 0;
      }
      n_rp += up ? 0 : 1;
      n_cp += left ? 0 : 1;
      n_t += (left || up_tile) ? 0 : 1;
    }
    atomicAdd(&acc[0], n_rp);
    atomicAdd(&acc[1], n_cp);
    atomicAdd(&acc[2], n_t);
  }
  if (offsets_t != nullptr && !cols_t.null()) {
    int ok = 1;
    for (int c = threadIdx.x; c < block_cols; c += kPlanThreads) {
      const int a = offsets_t[c], b = offsets_t[c + 1];
      if (a > b || a < 0 || b > nnz) { ok = 0; continue; }
      for (int q = a; q < b; ++q) {
        const int r = cols_t[q];
        if (r < 0 || r >= block_rows || (q > a && cols_t[q - 1] >= r)) ok = 0;
      }
    }
    if (!ok) atomicAnd(&acc[4], 0);
  }
  __syncthreads();
  if (threadIdx.x < 5) {
    int v = acc[threadIdx.x];
    if (threadIdx.x == 4 && (offsets_t == nullptr || cols_t.null())) v = -1;
    stats[threadIdx.x] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) stats[5] = 1;
}

// Exclusive block scans over one value per thread (sum / max), 1024 threads.
__device__ __forceinline__ int plan_block_scan_sum(int v, int* warp_tmp, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += t;
  }
  __syncthreads();
  if (lane == 31) warp_tmp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_tmp[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += t;
    }
    warp_tmp[lane] = w;
  }
  __syncthreads();
  if (total != nullptr) *total = warp_tmp[31];
  return incl - v + (warp > 0 ? warp_tmp[warp - 1] : 0);
}
__device__ __forceinline__ int plan_block_scan_max(int v, int* warp_tmp) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl = max(incl, t);
  }
  __syncthreads();
  if (lane == 31) warp_tmp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_tmp[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w = max(w, t);
    }
    warp_tmp[lane] = w;
  }
  __syncthreads();
  // exclusive: the maximum over the threads before this one
  int before = __shfl_up_sync(0xffffffffu, incl, 1);
  if (lane == 0) before = -1;
  if (warp > 0) before = max(before, warp_tmp[warp - 1]);
  return before;
}

// Lists r and r + 1 cannot share a K position: both non-empty and their column ranges disjoint.
__device__ __forceinline__ bool plan_is_cut(const int32_t* __restrict__ offsets, IndexArray cols, int r) {
  const int a0 = offsets[r], a1 = offsets[r + 1], b1 = offsets[r + 2];
  if (a0 >= a1 || a1 >= b1) return false;
  const int a_first = cols[a0], a_last = cols[a1 - 1], b_first = cols[a1], b_last = cols[b1 - 1];
  return a_last < b_first || b_last < a_first;
}

// plan[0] = number of groups G; plan[1 + g] = first list of group g | (single << 30): a group is
// lists (r, r + 1), or list r alone where a run of lists has odd length.  Groups are listed by
// descending length of their first list (stable), so that a round-robin deal hands every CTA pair its
// expensive items first; beyond kPlanSortMaxGroups they stay in list order.  plan[1 + num_lists ..]
// is scratch of the same size.
__global__ void __launch_bounds__(kPlanThreads, 1)
pair_plan_kernel(const int32_t* __restrict__ offsets, IndexArray cols, int num_lists,
                 int32_t* __restrict__ plan) {
  __shared__ int warp_tmp[32];
  __shared__ int total_groups;
  int32_t* group_row = plan + 1 + num_lists;  // groups in list order (scratch)
  const int ipt = (num_lists + kPlanThreads - 1) / kPlanThreads;
  const int b0 = min(num_lists, static_cast<int>(threadIdx.x) * ipt), b1 = min(num_lists, b0 + ipt);
  // start of the run that contains each list: the last cut before it, plus one
  int last_start = -1;
  for (int r = b0; r < b1; ++r)
    if (r > 0 && plan_is_cut(offsets, cols, r - 1)) last_start = r;
  int run_start = max(0, plan_block_scan_max(last_start, warp_tmp));  // for list b0, before its own cuts
  int firsts = 0;
  for (int r = b0, s = run_start; r < b1; ++r) {
    if (r > 0 && plan_is_cut(offsets, cols, r - 1)) s = r;
    firsts += ((r - s) & 1) ? 0 : 1;
  }
  int g = plan_block_scan_sum(firsts, warp_tmp, &total_groups);
  for (int r = b0, s = run_start; r < b1; ++r) {
    if (r > 0 && plan_is_cut(offsets, cols, r - 1)) s = r;
    if ((r - s) & 1) continue;
    const bool single = r + 1 >= num_lists || plan_is_cut(offsets, cols, r);
    group_row[g++] = r | (single ? (1 << 30) : 0);
  }
  __syncthreads();
  const int G = total_groups;
  if (threadIdx.x == 0) plan[0] = G;
  if (G > kPlanSortMaxGroups) {
    for (int i = threadIdx.x; i < G; i += kPlanThreads) plan[1 + i] = group_row[i];
    return;
  }
  // stable sort by descending list length, by rank counting (G^2 / 1024 comparisons per thread)
  for (int i = threadIdx.x; i < G; i += kPlanThreads) {
    const int e = group_row[i], r = e & 0x3fffffff;
    const int cost = offsets[r + 1] - offsets[r];
    int rank = 0;
    for (int j = 0; j < G; ++j) {
      const int rj = group_row[j] & 0x3fffffff;
      const int cj = offsets[rj + 1] - offsets[rj];
      rank += (cj > cost || (cj == cost && j < i)) ? 1 : 0;
    }
    plan[1 + rank] = e;
  }
}

}  // namespace stk

namespace stk {
static int pair_stats_impl(const int32_t* offsets, IndexArray row_indices, IndexArray column_indices,
                           const int32_t* offsets_t, IndexArray column_indices_t, int64_t block_rows,
                           int64_t block_cols, int64_t nnz, int32_t* stats, void* stream) {
  if (block_rows <= 0 || block_cols <= 0 || nnz < 0) return STK_ERR_BAD_DIMS;
  const long long limit = index_limit(column_indices.wide);
  if (block_rows > limit || block_cols > limit || nnz > INT32_MAX) return STK_ERR_TOO_LARGE;
  if (stats == nullptr || offsets == nullptr) return STK_ERR_NULL_POINTER;
  if (nnz > 0 && (row_indices.null() || column_indices.null())) return STK_ERR_NULL_POINTER;
  pair_stats_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      offsets, row_indices, column_indices, offsets_t, column_indices_t, static_cast<int>(block_rows),
      static_cast<int>(block_cols), static_cast<int>(nnz), stats);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}
static int pair_plan_impl(const int32_t* offsets, IndexArray column_indices, int64_t num_lists,
                          int32_t* plan, size_t plan_bytes, void* stream) {
  if (num_lists <= 0) return STK_ERR_BAD_DIMS;
  if (num_lists > (1 << 29)) return STK_ERR_TOO_LARGE;
  if (offsets == nullptr || plan == nullptr) return STK_ERR_NULL_POINTER;
  if (plan_bytes < stk_b200_pair_plan_bytes(num_lists)) return STK_ERR_WORKSPACE;
  pair_plan_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      offsets, column_indices, static_cast<int>(num_lists), plan);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}
}  // namespace stk

extern "C" size_t stk_b200_pair_plan_bytes(int64_t num_lists) {
  return num_lists < 0 ? 0 : static_cast<size_t>(2 * num_lists + 4) * sizeof(int32_t);
}
extern "C" int stk_b200_pair_stats(const int32_t* offsets, const int16_t* row_indices,
                                   const int16_t* column_indices, const int32_t* offsets_t,
                                   const int16_t* column_indices_t, int64_t block_rows,
                                   int64_t block_cols, int64_t nnz, int32_t* stats, void* stream) {
  return stk::pair_stats_impl(offsets, stk::IndexArray{row_indices, 0}, stk::IndexArray{column_indices, 0},
                              offsets_t, stk::IndexArray{column_indices_t, 0}, block_rows, block_cols, nnz, stats,
                              stream);
}
extern "C" int stk_b200_pair_stats_i32(const int32_t* offsets, const int32_t* row_indices,
                                       const int32_t* column_indices, const int32_t* offsets_t,
                                       const int32_t* column_indices_t, int64_t block_rows,
                                       int64_t block_cols, int64_t nnz, int32_t* stats, void* stream) {
  return stk::pair_stats_impl(offsets, stk::IndexArray{row_indices, 1}, stk::IndexArray{column_indices, 1},
                              offsets_t, stk::IndexArray{column_indices_t, 1}, block_rows, block_cols, nnz, stats,
                              stream);
}
extern "C" int stk_b200_pair_plan(const int32_t* offsets, const int16_t* column_indices,
                                  int64_t num_lists, int32_t* plan, size_t plan_bytes, void* stream) {
  return stk::pair_plan_impl(offsets, stk::IndexArray{column_indices, 0}, num_lists, plan, plan_bytes, stream);
}
extern "C" int stk_b200_pair_plan_i32(const int32_t* offsets, const int32_t* column_indices,
                                      int64_t num_lists, int32_t* plan, size_t plan_bytes, void* stream) {
  return stk::pair_plan_impl(offsets, stk::IndexArray{column_indices, 1}, num_lists, plan, plan_bytes, stream);
}
