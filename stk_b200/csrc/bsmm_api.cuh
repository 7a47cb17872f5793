// C entry points of the three block-sparse products: argument checks, tensor-map encoding and
// the dispatch to the 128x128 kernel, the CTA-pair 256x256 kernel or the 128x256 row kernel.
#pragma once
#include "bsmm_pair_sm100.cuh"
#include "bsmm_wide_sm100.cuh"
#include "bsmm_row_sm100.cuh"
#include "bsmm_sm100.cuh"

namespace stk {

static int check_dtype_dims(int dtype, int64_t M, int64_t N, int64_t K, int64_t nnz, int64_t k_mult,
                            int pair_mode) {
  if (dtype != STK_F16 && dtype != STK_BF16 && dtype != STK_F8E4M3) return STK_ERR_BAD_DTYPE;
  if (dtype == STK_F8E4M3 && pair_mode == 3) return STK_ERR_BAD_DTYPE;  // the 128x256 kernels are 16-bit only
  if (M <= 0 || N <= 0 || K <= 0 || nnz < 0 || M % kBlk || N % kBlk || K % k_mult) return STK_ERR_BAD_DIMS;
  if (pair_mode < 0 || pair_mode > 3) return STK_ERR_BAD_DIMS;
  if (nnz * kBlk > INT32_MAX - 2 * kBlk || M > INT32_MAX / 2 || N > INT32_MAX / 2 || K > INT32_MAX / 2 ||
      (M / kBlk) * (N / kBlk) > INT32_MAX)
    return STK_ERR_TOO_LARGE;
  return STK_OK;
}

// Lists (block rows / columns) per tile-order group of the row kernel: as many as keep the group's
// sparse blocks (32 KiB each) within a share of the L2 that leaves room for the dense panels in use.
static int row_raster_group(int64_t nnz, int64_t num_lists) {
  const int64_t budget_blocks = (48ll << 20) / (kBlk * kBlk * 2);
  const int64_t per_list = (nnz + num_lists - 1) / num_lists;
  int64_t g = budget_blocks / (per_list > 0 ? per_list : 1);
  if (g < 1) g = 1;
  if (g > num_lists) g = num_lists;
  return static_cast<int>(g);
}

// 8-bit float operands: one byte per element, so a 16-byte-aligned row needs a multiple of 16 elements.
static int check_dense8(const void* ptr, int64_t ld, int64_t min_ld) {
  if (ptr == nullptr) return STK_ERR_NULL_POINTER;
  if (!aligned16(ptr) || ld < min_ld || (ld % 16) != 0) return STK_ERR_BAD_LAYOUT;
  return STK_OK;
}

}  // namespace stk

using namespace stk;

static int sdd_impl(const void* lhs, const void* rhs, void* out, const int32_t* offsets,
                    IndexArray row_indices, IndexArray column_indices, int64_t M, int64_t N, int64_t K,
                    int64_t nnz, int lhs_colmajor, int64_t ld_lhs, int rhs_colmajor, int64_t ld_rhs,
                    int dtype, int pair_mode, int epilogue, void* aux, const int32_t* pair_plan,
                    void* stream) {
  int rc = check_dtype_dims(dtype, M, N, K, nnz, 32, pair_mode);
  if (rc != STK_OK) return rc;
  if (epilogue < kEpilogueNone || epilogue > kEpilogueGeluGrad) return STK_ERR_BAD_DIMS;
  const bool has_aux = epilogue == kEpilogueGeluKeep || epilogue == kEpilogueGeluGrad;
  if (has_aux && nnz != 0 && aux == nullptr) return STK_ERR_NULL_POINTER;
  if (has_aux && !aligned16(aux)) return STK_ERR_BAD_LAYOUT;
  if (nnz == 0) return STK_OK;
  if (out == nullptr || row_indices.null() || column_indices.null()) return STK_ERR_NULL_POINTER;
  if (pair_mode && pair_mode != 3 && offsets == nullptr) return STK_ERR_NULL_POINTER;
  if (!aligned16(out)) return STK_ERR_BAD_LAYOUT;
  const int in8 = dtype == STK_F8E4M3 ? 1 : 0;
  const int out_fmt = in8 ? STK_BF16 : dtype;
  if (in8) {
    if (has_aux) return STK_ERR_BAD_DIMS;  // plain or GeLU epilogue only
    if ((rc = check_dense8(lhs, ld_lhs, lhs_colmajor ? M : K)) != STK_OK) return rc;
    if ((rc = check_dense8(rhs, ld_rhs, rhs_colmajor ? K : N)) != STK_OK) return rc;
  } else {
    if ((rc = check_dense(lhs, ld_lhs, lhs_colmajor ? M : K)) != STK_OK) return rc;
    if ((rc = check_dense(rhs, ld_rhs, rhs_colmajor ? K : N)) != STK_OK) return rc;
  }

  CUtensorMap tmA, tmB;
  // lhs [M,K]: row-major means K contiguous.
  if ((rc = encode_dense(&tmA, lhs, dtype, M, K, ld_lhs, !lhs_colmajor)) != STK_OK) return rc;
  // rhs [K,N]: row-major means N contiguous; column-major means K contiguous.
  if ((rc = encode_dense(&tmB, rhs, dtype, N, K, ld_rhs, rhs_colmajor)) != STK_OK) return rc;
  const int stage_k = in8 ? 2 * kBK : kBK;
  const int k_steps = static_cast<int>((K + stage_k - 1) / stage_k);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUtensorMap tmC;  // the output blocks as one [nnz*128, 128] matrix, stored 128 x 64 at a time
  if ((rc = encode_map(&tmC, out, out_fmt, kBlk, nnz * kBlk, kBlk, kBlk)) != STK_OK) return rc;
  CUtensorMap tmX = tmC;  // the auxiliary tensor has the layout of out
  if (has_aux && (rc = encode_map(&tmX, aux, out_fmt, kBlk, nnz * kBlk, kBlk, kBlk)) != STK_OK) return rc;

  if (pair_mode == 3) {  // two blocks of a block row per tile
    BsmmParams p{};
    p.mode = kModeSDD;
    p.a_mn = lhs_colmajor ? 1 : 0;
    p.b_mn = rhs_colmajor ? 0 : 1;
    p.fmt = dtype;
    p.epilogue = epilogue;
    p.num_tiles = static_cast<int>((nnz + 1) / 2);
    p.tiles_inner = 1;
    p.k_steps = k_steps;
    p.row_idx = row_indices;
    p.col_idx = column_indices;
    p.out = out;
    p.ldc = kBlk;
    p.nnz = static_cast<int>(nnz);
    p.aux = aux;
    return launch_row(tmA, tmB, tmC, tmX, p, s);
  }
  if (pair_mode) {
    PairDeviceInfo* d = nullptr;
    if ((rc = pair_device_info(&d)) != STK_OK) return rc;
    const int block_rows = static_cast<int>(M / kBlk), block_cols = static_cast<int>(N / kBlk);
    const int row_pairs = (block_rows + 1) / 2;
    // Every row pair's column range is split into `segments` items.  The items are dealt round-robin,
    // so a launch lasts (rounds of items) x (tiles per item): the split is chosen to minimise that
    // product for a topology whose row pairs have about nnz / block_rows / 2 tiles each (dMoE: all
    // alike), among the splits that cut a row pair's tiles into equal parts, preferring fewer,
    // longer items on a tie (every item starts with a short chain of dependent metadata loads).
    int tiles_per_group = static_cast<int>(((nnz + block_rows - 1) / block_rows + 1) / 2);
    if (tiles_per_group > (block_cols + 1) / 2) tiles_per_group = (block_cols + 1) / 2;
    if (tiles_per_group < 1) tiles_per_group = 1;
    int segments = 1;
    long long best = -1;
    for (int cand = 1; cand <= tiles_per_group; ++cand) {
      if (tiles_per_group % cand != 0) continue;
      const long long items = static_cast<long long>(row_pairs) * cand;
      const long long rounds = (items + d->max_pairs - 1) / d->max_pairs;
      const long long cost = rounds * (tiles_per_group / cand) * 64 + rounds;  // + a little per item start
      if (best < 0 || cost < best) {
        best = cost;
        segments = cand;
      }
    }
    PairParams p{};
    p.mode = kModeSDD;
    p.a_mn = lhs_colmajor ? 1 : 0;
    p.b_mn = rhs_colmajor ? 0 : 1;
    p.fmt = out_fmt;
    p.in8 = in8;
    p.epilogue = epilogue;
    p.inner = segments;
    p.num_items = row_pairs * segments;
    p.k_steps = k_steps;
    p.num_lists = block_rows;
    p.col_idx = column_indices;
    p.offsets = offsets;
    p.out = out;
    p.ldc = kBlk;
    p.aux = aux;
    p.plan = pair_plan;
    return launch_pair(tmA, tmB, tmC, tmX, p, s);
  }

  BsmmParams p{};
  p.mode = kModeSDD;
  p.a_mn = lhs_colmajor ? 1 : 0;
  p.b_mn = rhs_colmajor ? 0 : 1;
  p.fmt = out_fmt;
  p.in8 = in8;
  p.epilogue = epilogue;
  p.num_tiles = static_cast<int>(nnz);
  p.tiles_inner = 1;
  p.k_steps = k_steps;
  p.row_idx = row_indices;
  p.col_idx = column_indices;
  p.out = out;
  p.ldc = kBlk;
  p.aux = aux;
  return launch(tmA, tmB, tmC, tmX, p, s);
}

static int dsd_impl(const void* data, const int32_t* offsets, IndexArray column_indices,
                    const int32_t* block_offsets, const void* rhs, void* out, int64_t M, int64_t N,
                    int64_t K, int64_t nnz, int trans_sparse, int rhs_colmajor, int64_t ld_rhs,
                    int64_t ld_out, int dtype, int pair_mode, const int32_t* pair_plan, void* stream) {
  int rc = check_dtype_dims(dtype, M, N, K, nnz, kBlk, pair_mode);
  if (rc != STK_OK) return rc;
  if ((rc = check_dense(out, ld_out, N)) != STK_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (nnz == 0) {
    // No blocks at all: the product is zero.
    return cudaMemset2DAsync(out, ld_out * 2, 0, N * 2, M, s) == cudaSuccess ? STK_OK
                                                                             : STK_ERR_LAUNCH;
  }
  if (data == nullptr || offsets == nullptr || column_indices.null()) return STK_ERR_NULL_POINTER;
  if (trans_sparse && block_offsets == nullptr) return STK_ERR_NULL_POINTER;
  if (!aligned16(data)) return STK_ERR_BAD_LAYOUT;
  const int in8 = dtype == STK_F8E4M3 ? 1 : 0;
  const int out_fmt = in8 ? STK_BF16 : dtype;
  if (in8) {
    if ((rc = check_dense8(rhs, ld_rhs, rhs_colmajor ? K : N)) != STK_OK) return rc;
  } else if ((rc = check_dense(rhs, ld_rhs, rhs_colmajor ? K : N)) != STK_OK) {
    return rc;
  }

  CUtensorMap tmA, tmB;
  // A = data[blk] as stored (its columns are K) or transposed (its columns are M).
  if ((rc = encode_sparse(&tmA, data, dtype, nnz, !trans_sparse)) != STK_OK) return rc;
  if ((rc = encode_dense(&tmB, rhs, dtype, N, K, ld_rhs, rhs_colmajor)) != STK_OK) return rc;

  CUtensorMap tmC;
  if ((rc = encode_map(&tmC, out, out_fmt, N, M, ld_out, kBlk)) != STK_OK) return rc;

  if (pair_mode == 3) {  // one block row x 256 dense columns per CTA
    BsmmParams p{};
    p.mode = kModeDSD;
    p.a_mn = trans_sparse ? 1 : 0;
    p.b_mn = rhs_colmajor ? 0 : 1;
    p.fmt = dtype;
    p.tiles_inner = static_cast<int>((N + 2 * kBlk - 1) / (2 * kBlk));
    p.num_tiles = static_cast<int>((M / kBlk) * p.tiles_inner);
    p.col_idx = column_indices;
    p.offsets = offsets;
    p.blk_idx = block_offsets;
    p.out = out;
    p.ldc = ld_out;
    p.out_cols = static_cast<int>(N);
    p.raster_group = row_raster_group(nnz, M / kBlk);
    return launch_row(tmA, tmB, tmC, tmC, p, s);
  }
  if (pair_mode) {
    PairParams p{};
    p.mode = kModeDSD;
    p.a_mn = trans_sparse ? 1 : 0;
    p.b_mn = rhs_colmajor ? 0 : 1;
    p.fmt = out_fmt;
    p.in8 = in8;
    p.num_lists = static_cast<int>(M / kBlk);
    // dense columns per work item: 256, or 512 (two accumulators fed by one sparse tile)
    const int64_t panel = pair_mode == 2 ? 4 * kBlk : 2 * kBlk;
    p.inner = static_cast<int>((N + panel - 1) / panel);
    p.num_items = ((p.num_lists + 1) / 2) * p.inner;
    p.zero_coord = static_cast<int>(nnz * kBlk);
    p.out_rows = static_cast<int>(M);
    p.out_cols = static_cast<int>(N);
    p.col_idx = column_indices;
    p.offsets = offsets;
    p.blk_idx = block_offsets;
    p.out = out;
    p.ldc = ld_out;
    p.plan = pair_plan;
    return pair_mode == 2 ? launch_wide(tmA, tmB, p, s) : launch_pair(tmA, tmB, tmC, tmC, p, s);
  }

  BsmmParams p{};
  p.mode = kModeDSD;
  p.a_mn = trans_sparse ? 1 : 0;
  p.b_mn = rhs_colmajor ? 0 : 1;
  p.fmt = out_fmt;
  p.in8 = in8;
  p.tiles_inner = static_cast<int>(N / kBlk);
  p.num_tiles = static_cast<int>((M / kBlk) * (N / kBlk));
  p.col_idx = column_indices;
  p.offsets = offsets;
  p.blk_idx = block_offsets;
  p.out = out;
  p.ldc = ld_out;
  return launch(tmA, tmB, tmC, tmC, p, s);
}

static int dds_impl(const void* lhs, const void* data, const int32_t* offsets, IndexArray column_indices,
                    const int32_t* block_offsets, void* out, int64_t M, int64_t N, int64_t K, int64_t nnz,
                    int lhs_colmajor, int64_t ld_lhs, int trans_sparse, int64_t ld_out, int dtype,
                    int pair_mode, const int32_t* pair_plan, void* stream) {
  int rc = check_dtype_dims(dtype, M, N, K, nnz, kBlk, pair_mode);
  if (rc != STK_OK) return rc;
  if ((rc = check_dense(out, ld_out, N)) != STK_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (nnz == 0) {
    return cudaMemset2DAsync(out, ld_out * 2, 0, N * 2, M, s) == cudaSuccess ? STK_OK
                                                                             : STK_ERR_LAUNCH;
  }
  if (data == nullptr || offsets == nullptr || column_indices.null()) return STK_ERR_NULL_POINTER;
  if (!trans_sparse && block_offsets == nullptr) return STK_ERR_NULL_POINTER;
  if (!aligned16(data)) return STK_ERR_BAD_LAYOUT;
  const int in8 = dtype == STK_F8E4M3 ? 1 : 0;
  const int out_fmt = in8 ? STK_BF16 : dtype;
  if (in8) {
    if ((rc = check_dense8(lhs, ld_lhs, lhs_colmajor ? M : K)) != STK_OK) return rc;
  } else if ((rc = check_dense(lhs, ld_lhs, lhs_colmajor ? M : K)) != STK_OK) {
    return rc;
  }

  CUtensorMap tmA, tmB;
  if ((rc = encode_dense(&tmA, lhs, dtype, M, K, ld_lhs, !lhs_colmajor)) != STK_OK) return rc;
  // B = data[blk] as stored (its columns are N) or transposed (its columns are K).
  if ((rc = encode_sparse(&tmB, data, dtype, nnz, trans_sparse)) != STK_OK) return rc;

  CUtensorMap tmC;
  if ((rc = encode_map(&tmC, out, out_fmt, N, M, ld_out, kBlk)) != STK_OK) return rc;

  if (pair_mode == 3) {  // 256 dense rows x one block column per CTA
    BsmmParams p{};
    p.mode = kModeDDS;
    p.a_mn = lhs_colmajor ? 1 : 0;
    p.b_mn = trans_sparse ? 0 : 1;
    p.fmt = dtype;
    p.tiles_inner = static_cast<int>((M + 2 * kBlk - 1) / (2 * kBlk));
    p.num_tiles = static_cast<int>((N / kBlk) * p.tiles_inner);
    p.col_idx = column_indices;
    p.offsets = offsets;
    p.blk_idx = block_offsets;
    p.out = out;
    p.ldc = ld_out;
    p.out_rows = static_cast<int>(M);
    p.raster_group = row_raster_group(nnz, N / kBlk);
    return launch_row(tmA, tmB, tmC, tmC, p, s);
  }
  if (pair_mode) {
    PairParams p{};
    p.mode = kModeDDS;
    p.a_mn = lhs_colmajor ? 1 : 0;
    p.b_mn = trans_sparse ? 0 : 1;
    p.fmt = out_fmt;
    p.in8 = in8;
    p.num_lists = static_cast<int>(N / kBlk);
    // dense rows per work item: 256, or 512 (two accumulators fed by one sparse tile)
    const int64_t panel = pair_mode == 2 ? 4 * kBlk : 2 * kBlk;
    p.inner = static_cast<int>((M + panel - 1) / panel);
    p.num_items = ((p.num_lists + 1) / 2) * p.inner;
    p.zero_coord = static_cast<int>(nnz * kBlk);
    p.out_rows = static_cast<int>(M);
    p.out_cols = static_cast<int>(N);
    p.col_idx = column_indices;
    p.offsets = offsets;
    p.blk_idx = block_offsets;
    p.out = out;
    p.ldc = ld_out;
    p.plan = pair_plan;
    return pair_mode == 2 ? launch_wide(tmA, tmB, p, s) : launch_pair(tmA, tmB, tmC, tmC, p, s);
  }

  BsmmParams p{};
  p.mode = kModeDDS;
  p.a_mn = lhs_colmajor ? 1 : 0;
  p.b_mn = trans_sparse ? 0 : 1;
  p.fmt = out_fmt;
  p.in8 = in8;
  p.tiles_inner = static_cast<int>(M / kBlk);
  p.num_tiles = static_cast<int>((M / kBlk) * (N / kBlk));
  p.col_idx = column_indices;
  p.offsets = offsets;
  p.blk_idx = block_offsets;
  p.out = out;
  p.ldc = ld_out;
  return launch(tmA, tmB, tmC, tmC, p, s);
}

// The exported entry points: block indices as int16 (the reference's format) or, with the _i32
// suffix, as int32.
extern "C" int stk_b200_sdd(const void* lhs, const void* rhs, void* out, const int32_t* offsets,
                            const int16_t* row_indices, const int16_t* column_indices, int64_t M,
                            int64_t N, int64_t K, int64_t nnz, int lhs_colmajor, int64_t ld_lhs,
                            int rhs_colmajor, int64_t ld_rhs, int dtype, int pair_mode,
                            int epilogue, void* aux, const int32_t* pair_plan, void* stream) {
  return sdd_impl(lhs, rhs, out, offsets, IndexArray{row_indices, 0}, IndexArray{column_indices, 0}, M, N, K,
                  nnz, lhs_colmajor, ld_lhs, rhs_colmajor, ld_rhs, dtype, pair_mode, epilogue, aux, pair_plan,
                  stream);
}
extern "C" int stk_b200_sdd_i32(const void* lhs, const void* rhs, void* out, const int32_t* offsets,
                                const int32_t* row_indices, const int32_t* column_indices, int64_t M,
                                int64_t N, int64_t K, int64_t nnz, int lhs_colmajor, int64_t ld_lhs,
                                int rhs_colmajor, int64_t ld_rhs, int dtype, int pair_mode,
                                int epilogue, void* aux, const int32_t* pair_plan, void* stream) {
  return sdd_impl(lhs, rhs, out, offsets, IndexArray{row_indices, 1}, IndexArray{column_indices, 1}, M, N, K,
                  nnz, lhs_colmajor, ld_lhs, rhs_colmajor, ld_rhs, dtype, pair_mode, epilogue, aux, pair_plan,
                  stream);
}

extern "C" int stk_b200_dsd(const void* data, const int32_t* offsets, const int16_t* column_indices,
                            const int32_t* block_offsets, const void* rhs, void* out, int64_t M,
                            int64_t N, int64_t K, int64_t nnz, int trans_sparse, int rhs_colmajor,
                            int64_t ld_rhs, int64_t ld_out, int dtype, int pair_mode,
                            const int32_t* pair_plan, void* stream) {
  return dsd_impl(data, offsets, IndexArray{column_indices, 0}, block_offsets, rhs, out, M, N, K, nnz,
                  trans_sparse, rhs_colmajor, ld_rhs, ld_out, dtype, pair_mode, pair_plan, stream);
}
extern "C" int stk_b200_dsd_i32(const void* data, const int32_t* offsets, const int32_t* column_indices,
                                const int32_t* block_offsets, const void* rhs, void* out, int64_t M,
                                int64_t N, int64_t K, int64_t nnz, int trans_sparse, int rhs_colmajor,
                                int64_t ld_rhs, int64_t ld_out, int dtype, int pair_mode,
                                const int32_t* pair_plan, void* stream) {
  return dsd_impl(data, offsets, IndexArray{column_indices, 1}, block_offsets, rhs, out, M, N, K, nnz,
                  trans_sparse, rhs_colmajor, ld_rhs, ld_out, dtype, pair_mode, pair_plan, stream);
}
extern "C" int stk_b200_dds(const void* lhs, const void* data, const int32_t* offsets,
                            const int16_t* column_indices, const int32_t* block_offsets, void* out,
                            int64_t M, int64_t N, int64_t K, int64_t nnz, int lhs_colmajor,
                            int64_t ld_lhs, int trans_sparse, int64_t ld_out, int dtype,
                            int pair_mode, const int32_t* pair_plan, void* stream) {
  return dds_impl(lhs, data, offsets, IndexArray{column_indices, 0}, block_offsets, out, M, N, K, nnz,
                  lhs_colmajor, ld_lhs, trans_sparse, ld_out, dtype, pair_mode, pair_plan, stream);
}
extern "C" int stk_b200_dds_i32(const void* lhs, const void* data, const int32_t* offsets,
                                const int32_t* column_indices, const int32_t* block_offsets, void* out,
                                int64_t M, int64_t N, int64_t K, int64_t nnz, int lhs_colmajor,
                                int64_t ld_lhs, int trans_sparse, int64_t ld_out, int dtype,
                                int pair_mode, const int32_t* pair_plan, void* stream) {
  return dds_impl(lhs, data, offsets, IndexArray{column_indices, 1}, block_offsets, out, M, N, K, nnz,
                  lhs_colmajor, ld_lhs, trans_sparse, ld_out, dtype, pair_mode, pair_plan, stream);
}
