/*
 * stk_b200 — C ABI of the B200 (sm_100a) block-sparse matmul backend.
 *
 * This header is the whole drop-in boundary: plain pointers, sizes and flags, no
 * torch types.  Every pointer is a DEVICE pointer owned by the caller unless the
 * comment says "host".  Every call is asynchronous on `stream` (a cudaStream_t
 * passed as void*), never synchronises the device, and allocates nothing.
 * Return value: 0 on success, a negative STK_ERR_* code otherwise (see
 * stk_b200_error_string).  Nothing aborts and no kernel traps.
 *
 * Each entry point names the interface of the reference project
 * (stanford-futuredata/stk, paths relative to its root) that it replaces.
 *
 * Sparse operand format (blocked CSR-COO, blocking = 128 for the matmuls):
 *   data            [nnz,128,128]  fp16/bf16, blocks ordered by (block-row, block-col)
 *   row_indices     [nnz]          int16
 *   column_indices  [nnz]          int16
 *   offsets         [R+1]          int32   (R = block rows)
 *   column_indices_t[nnz]          int16   (block-row of the k-th block in column-major order)
 *   offsets_t       [Cb+1]         int32   (Cb = block columns)
 *   block_offsets_t [nnz]          int32   (index into data of the k-th block in column-major order)
 */
#ifndef STK_B200_H_
#define STK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STK_B200_VERSION 100

/* element types of the matmul operands */
#define STK_F16 0
#define STK_BF16 1
#define STK_F8E4M3 2   /* sdd / dsd / dds: 8-bit float operands (1 byte each), bf16 output; see below */

/* epilogue of stk_b200_sdd */
#define STK_EPILOGUE_NONE 0
#define STK_EPILOGUE_GELU 1
#define STK_EPILOGUE_GELU_KEEP 2
#define STK_EPILOGUE_GELU_GRAD 3

/* status codes */
#define STK_OK 0
#define STK_ERR_NULL_POINTER (-1)   /* a required pointer is NULL */
#define STK_ERR_BAD_DIMS (-2)       /* M,N not multiples of 128, K not a multiple of 32, negative size ... */
#define STK_ERR_BAD_DTYPE (-3)      /* dtype / element size not supported */
#define STK_ERR_BAD_LAYOUT (-4)     /* pointer not 16-byte aligned or leading dimension not a multiple of 8 elements */
#define STK_ERR_TENSOR_MAP (-5)     /* cuTensorMapEncodeTiled failed */
#define STK_ERR_LAUNCH (-6)         /* kernel launch / CUDA runtime error */
#define STK_ERR_WORKSPACE (-7)      /* workspace missing or too small */
#define STK_ERR_DRIVER (-8)         /* driver entry point unavailable */
#define STK_ERR_TOO_LARGE (-9)      /* size beyond what the entry point supports */
#define STK_ERR_DEVICE_TIMEOUT (-10)/* a bounded wait inside a kernel ran out (reported by stk_b200_device_status) */

int stk_b200_version(void);
const char* stk_b200_error_string(int code);

/*
 * Reads and clears this device's kernel status word (0 = no kernel has reported a
 * problem since the last call).  Synchronises the device: debugging / tests only.
 * No counterpart in the reference (its kernels cannot report anything).
 */
int stk_b200_device_status(int* status_host);
/* Diagnostic for STK_ERR_DEVICE_TIMEOUT: which wait ran out first (0: none), read and cleared like the
 * status word: warp of the waiting thread | its CTA's rank in the cluster << 8 | shared-memory address
 * of the barrier << 12 | awaited parity << 31.  Synchronises the device. */
int stk_b200_timeout_site(unsigned int* site_host);
/* Diagnostic for STK_ERR_TENSOR_MAP: the CUresult of the calling thread's last cuTensorMapEncodeTiled
 * (0 = success; 1 = CUDA_ERROR_INVALID_VALUE: an address, stride or extent the hardware cannot describe). */
int stk_b200_last_tensor_map_error(void);

/*
 * pair_mode (sdd / dsd / dds): 0 runs one 128x128 output tile per CTA.  1 runs 256x256 supertiles on
 * CTA pairs (tcgen05 cta_group::2): two neighbouring block rows / columns of the sparse operand are
 * processed together over the merge of their block lists, which halves the operand traffic per
 * FLOP when the neighbours' lists mostly coincide (dMoE topologies) and wastes MMA work when they
 * do not.  3 runs 128x256 tiles on one CTA with one N = 256 MMA per K step: one block row of op(S) x
 * 256 dense columns (dsd), 256 dense rows x one block column (dds, computed transposed), or two
 * blocks of one block row (sdd: blocks 2i and 2i+1 of the list; row_indices / column_indices in
 * row-major order).  Three quarters of mode 0's operand traffic for any topology, no pairing
 * needed - the choice for topologies that do not pair up.  2 (dsd / dds; sdd treats it as 1) is mode 1
 * with work items of 256x512 (dsd) / 512x256 (dds): every sparse tile is fetched once for two dense
 * tiles and feeds both accumulators of tensor memory - a quarter less operand traffic per FLOP than
 * mode 1, but the epilogue of an item no longer overlaps the next item's MMAs, so it pays when the
 * block lists are long.  Any other value is STK_ERR_BAD_DIMS.
 * All modes give the same results; modes 1 and 2 need every block row's column_indices (and every
 * block column's column_indices_t) in ascending order, and take the same pair_plan.
 *
 * dtype (sdd / dsd / dds): STK_F16 or STK_BF16 - operands and output in that format - or STK_F8E4M3:
 * every operand (lhs, rhs, the sparse values read by dsd / dds) is an 8-bit float, e4m3, one byte per
 * element, and the output (the blocks written by sdd, the dense result of dsd / dds) is bf16; fp32
 * accumulation as always, no scaling (a caller that quantised with scales applies their product to
 * the result).  Not in the reference.  The 8-bit kernels (tcgen05.mma kind::f8f6f4, 128 of K per
 * pipeline stage) take the same layouts as the 16-bit ones (row- or column-major dense operands,
 * blocks as stored or transposed).  Leading dimensions of 8-bit operands are multiples of 16
 * elements.  pair_mode 0, 1 and 2; 3 is STK_ERR_BAD_DTYPE, and the epilogues with an auxiliary
 * tensor are STK_ERR_BAD_DIMS.
 */

/*
 * SDD: out[p] = lhs[r_p*128:+128, :] @ rhs[:, c_p*128:+128] for every nonzero block p,
 * fp32 accumulation, output rounded to `dtype`.
 * Replaces stk/backend/triton_kernels.py:332-379 (sdd) and :21-68 (_sdd_kernel).
 *   lhs: logical [M,K]; row-major (lhs_colmajor=0, element (m,k) at m*ld_lhs+k) or
 *        column-major (lhs_colmajor=1, element (m,k) at k*ld_lhs+m - an exact .t() view).
 *   rhs: logical [K,N]; same convention with ld_rhs.
 *   out: [nnz,128,128] contiguous.
 *   offsets: CSR offsets [M/128+1]; only read when pair_mode = 1 (may be NULL otherwise).
 *   epilogue: 0 stores the product; 1 (STK_EPILOGUE_GELU) stores GeLU(product), the exact erf form
 *             applied to the fp32 accumulator before rounding - the step between SDD and DSD in a
 *             dMoE layer, fused so that the hidden activations are written once.  The reference
 *             has no fused form (it runs a separate elementwise kernel on Matrix.data).
 *             2 (STK_EPILOGUE_GELU_KEEP) stores the product in `out` AND GeLU(product) in `aux`
 *             (a training step keeps the pre-activations for the backward pass).
 *             3 (STK_EPILOGUE_GELU_GRAD) stores product * GeLU'(aux), `aux` holding pre-activations:
 *             the backward of GeLU fused into the product dy @ w2^T that yields the gradient of
 *             the activations.
 *   aux: [nnz,128,128] contiguous like out, written (2) or read (3); NULL for epilogue 0 / 1.
 *   pair_plan: work-item table from stk_b200_pair_plan(offsets, column_indices, M/128, ...) for
 *        pair_mode = 1, or NULL (block rows are then paired blindly; see stk_b200_pair_plan).
 * nnz == 0 is a no-op.
 */
int stk_b200_sdd(const void* lhs, const void* rhs, void* out, const int32_t* offsets,
                 const int16_t* row_indices, const int16_t* column_indices,
                 int64_t M, int64_t N, int64_t K, int64_t nnz,
                 int lhs_colmajor, int64_t ld_lhs, int rhs_colmajor, int64_t ld_rhs,
                 int dtype, int pair_mode, int epilogue, void* aux, const int32_t* pair_plan,
                 void* stream);

/*
 * DSD: out[M,N] = op(S)[M,K] @ rhs[K,N].
 * Replaces stk/backend/triton_kernels.py:222-276 (dsd) and :70-145 (_dsd_kernel).
 *   trans_sparse = 0: pass offsets, column_indices and block_offsets = NULL
 *                     (block j of block-row i is data[j]).
 *   trans_sparse = 1: pass offsets_t, column_indices_t and block_offsets_t
 *                     (block j of block-row i of S^T is data[block_offsets_t[j]]^T).
 *   M,K: logical (already transposed) shape of op(S).  Block rows without blocks give zeros.
 *   rhs: row-major or column-major as for stk_b200_sdd.  out: row-major, leading dimension ld_out.
 *   pair_plan: table from stk_b200_pair_plan over the SAME offsets / column_indices arrays that are
 *        passed here (M/128 lists), for pair_mode = 1; or NULL.
 */
int stk_b200_dsd(const void* data, const int32_t* offsets, const int16_t* column_indices,
                 const int32_t* block_offsets, const void* rhs, void* out,
                 int64_t M, int64_t N, int64_t K, int64_t nnz,
                 int trans_sparse, int rhs_colmajor, int64_t ld_rhs, int64_t ld_out,
                 int dtype, int pair_mode, const int32_t* pair_plan, void* stream);

/*
 * DDS: out[M,N] = lhs[M,K] @ op(S)[K,N].
 * Replaces stk/backend/triton_kernels.py:278-330 (dds) and :147-220 (_dds_kernel).
 *   trans_sparse = 0: pass offsets_t, column_indices_t and block_offsets_t (the block
 *                     columns of S are walked through the transposed metadata).
 *   trans_sparse = 1: pass offsets, column_indices and block_offsets = NULL
 *                     (block column n of S^T is block row n of S, blocks used transposed).
 *   K,N: logical shape of op(S).
 *   pair_plan: table from stk_b200_pair_plan over the offsets / column_indices arrays passed here
 *        (N/128 lists), for pair_mode = 1; or NULL.
 */
int stk_b200_dds(const void* lhs, const void* data, const int32_t* offsets,
                 const int16_t* column_indices, const int32_t* block_offsets, void* out,
                 int64_t M, int64_t N, int64_t K, int64_t nnz,
                 int lhs_colmajor, int64_t ld_lhs, int trans_sparse, int64_t ld_out,
                 int dtype, int pair_mode, const int32_t* pair_plan, void* stream);

/*
 * Preparation for pair_mode = 1, once per topology.  No counterpart in the reference (its kernels
 * take one 128x128 tile per program, stk/backend/triton_kernels.py:21-220).
 *
 * pair_stats: how well the topology suits the CTA-pair kernel.  Writes six int32 to `stats`, which
 *   may be device memory or pinned host memory mapped into the device (the kernel stores to it):
 *   [0] distinct (row pair, column) positions, [1] distinct (row, column pair) positions,
 *   [2] distinct (row pair, column pair) positions - the useful share of the pair kernel's MMA work
 *   is nnz / (2 [0]) when block rows are paired (dsd with S as stored, dds with S transposed),
 *   nnz / (2 [1]) when block columns are paired, nnz / (4 [2]) for sdd;
 *   [3] 1 iff the blocks are listed in strictly ascending (row, column) order consistent with
 *   offsets and all indices are in range (otherwise [0..2] are meaningless and pair_mode 1 must not
 *   be used); [4] 1 iff every block column's segment of column_indices_t ascends (needed when block
 *   columns are paired), 0 if not, -1 if offsets_t / column_indices_t were NULL; [5] = 1, stored last.
 * pair_plan: the pair kernel's work-item table for one list family - (offsets, column_indices) with
 *   num_lists = block rows, or (offsets_t, column_indices_t) with num_lists = block columns.  Lists
 *   are cut into runs where two neighbours cannot share a position (expert boundaries of a dMoE
 *   topology), paired inside each run, and ordered longest first.  `plan` needs
 *   stk_b200_pair_plan_bytes(num_lists) bytes of device memory and is passed to sdd / dsd / dds.
 */
int stk_b200_pair_stats(const int32_t* offsets, const int16_t* row_indices,
                        const int16_t* column_indices, const int32_t* offsets_t,
                        const int16_t* column_indices_t, int64_t block_rows, int64_t block_cols,
                        int64_t nnz, int32_t* stats, void* stream);
size_t stk_b200_pair_plan_bytes(int64_t num_lists);
int stk_b200_pair_plan(const int32_t* offsets, const int16_t* column_indices, int64_t num_lists,
                       int32_t* plan, size_t plan_bytes, void* stream);

/*
 * CSR offsets -> COO row index of every block (int16).
 * Replaces stk/backend/triton_kernels.py:381-393 (_row_indices_kernel, row_indices).
 */
int stk_b200_row_indices(const int32_t* offsets, int16_t* out, int64_t block_rows, int64_t nnz,
                         void* stream);

/*
 * Transpose metadata: stable counting sort of the blocks by column.
 * Replaces stk/matrix.py:105-123 (_transpose: argsort + gather + histc + cumsum).
 * Ties (blocks of one column) come out in ascending storage order, i.e. ascending block row.
 * The caller supplies `workspace` of at least stk_b200_transpose_meta_workspace_bytes()
 * bytes, 16-byte aligned; its contents on entry do not matter.
 */
size_t stk_b200_transpose_meta_workspace_bytes(int64_t nnz, int64_t block_cols);
int stk_b200_transpose_meta(const int16_t* row_indices, const int16_t* column_indices,
                            int64_t nnz, int64_t block_cols,
                            int16_t* column_indices_t, int32_t* offsets_t, int32_t* block_offsets_t,
                            void* workspace, size_t workspace_bytes, void* stream);

/*
 * Transpose metadata without any allocation, by the caller or by the library.  No counterpart in
 * the reference.  It is stk_b200_transpose_meta with the group-by-column counters kept in a
 * 1 MiB array that is part of the library image on every GPU that loads it, for callers that
 * cannot obtain device memory at the point of the call: code running under a framework whose
 * allocator may not be re-entered (inside an allocator callback, while a memory pool is frozen),
 * or a host language binding that only hands over the buffers it was given.
 *   Limits: block_cols <= 8192 and nnz <= 1048576; larger sizes return STK_ERR_TOO_LARGE.
 *   The first call on each device looks up the array's device address (cudaGetSymbolAddress);
 *   make that first call outside any stream capture.
 *   All calls on one device share the array: the part a call uses is cleared by that call, and
 *   two calls whose kernels overlap on the GPU (different streams) race with each other.
 * Results are identical to stk_b200_transpose_meta.
 */
int stk_b200_transpose_meta_static(const int16_t* row_indices, const int16_t* column_indices,
                                   int64_t nnz, int64_t block_cols,
                                   int16_t* column_indices_t, int32_t* offsets_t,
                                   int32_t* block_offsets_t, void* stream);

/*
 * to_sparse, in phases, because the number of nonzero blocks sizes the output.
 * Together they replace stk/ops/matrix_ops.py:50-85 (_mask, to_sparse).
 *
 * 1. block_mask: mask[br*Cb+bc] = 1 iff block (br,bc) of x holds an element that is not +-0
 *    (NaN and Inf count as nonzero, as sum(|x|) != 0 does in the reference).
 *    x: [rows, cols] row-major with leading dimension ld (elements), elem_bytes in {2,4}, or 1 for
 *    8-bit floats (sign bit 0x80; element-wise kernels only, as in gather_blocks and to_dense).
 * 2. mask_to_offsets: offsets[0]=0, offsets[r+1] = number of set bytes in mask rows 0..r.
 *    The caller reads offsets[R] back to size data / row_indices / column_indices.
 * 3. mask_to_indices: row-major list of the set positions as int16 row / column indices.
 * 4. gather_blocks: data[p] = x[r_p*b:+b, c_p*b:+b], copied bit-exactly.  `offsets` (the CSR offsets of
 *    step 2; may be NULL) lets blocks smaller than 64 be copied by block-row strips instead of one
 *    CTA per block.  A listed block outside the matrix is not read: it becomes zeros and
 *    STK_ERR_BAD_DIMS is recorded in the device status word.
 */
int stk_b200_block_mask(const void* x, int64_t rows, int64_t cols, int64_t ld,
                        int blocking, int elem_bytes, uint8_t* mask, void* stream);
int stk_b200_mask_to_offsets(const uint8_t* mask, int64_t block_rows, int64_t block_cols,
                             int32_t* offsets, void* stream);
int stk_b200_mask_to_indices(const uint8_t* mask, int64_t block_rows, int64_t block_cols,
                             const int32_t* offsets, int16_t* row_indices, int16_t* column_indices,
                             void* stream);
int stk_b200_gather_blocks(const void* x, int64_t rows, int64_t cols, int64_t ld,
                           int blocking, int elem_bytes, const int32_t* offsets,
                           const int16_t* row_indices, const int16_t* column_indices, int64_t nnz,
                           void* data, void* stream);

/*
 * to_dense: out[rows, cols] (row-major, leading dimension ld_out) = zeros with every block
 * written at (row*b, col*b); every output element is written exactly once.
 * Replaces stk/ops/matrix_ops.py:36-47 (to_dense) and :15-31 (_expand_for_blocking).
 */
int stk_b200_to_dense(const void* data, const int32_t* offsets, const int16_t* column_indices,
                      int64_t block_rows, int64_t block_cols, int blocking, int elem_bytes,
                      void* out, int64_t ld_out, void* stream);

/*
 * regroup_blocks: products of matrices with 16, 32 or 64 blocks.  The reference's kernels exist for
 * 128 x 128 blocks only (stk/backend/triton_kernels.py:8-11 TritonConfig, BLOCK_SIZE = 128 in every launch);
 * here a matrix with smaller blocks runs as the matrix of the 128 x 128 blocks that contain its blocks,
 * zero where it has none, which is exact.  This call moves the values: fine = [nnz, b, b],
 * coarse = [coarse_blocks, 128, 128] (zero-filled by the caller when to_coarse = 1),
 * slot[p] = coarse block * q*q + (block row % q) * q + block column % q with q = 128 / b.
 * to_coarse = 1: coarse[slot] = fine;  to_coarse = 0: fine = coarse[slot].  Bit-exact copies; both
 * buffers 16-byte aligned; a slot outside [0, coarse_blocks * q*q) is skipped (zeros when gathering)
 * and reported as STK_ERR_BAD_DIMS through stk_b200_device_status.
 */
int stk_b200_regroup_blocks(void* fine, void* coarse, const int32_t* slot, int64_t nnz,
                            int64_t coarse_blocks, int blocking, int elem_bytes, int to_coarse,
                            void* stream);

/*
 * dMoE plumbing around the products (the callers' side of stk.Matrix / sdd / dsd in a dropless-MoE
 * layer; the reference is a matmul library and has no counterpart for these).
 *
 * gather_rows : dst[i] = index[i] >= 0 ? src[index[i] / index_div] : zeros   (i < n_rows output rows)
 *   index_div = 1 for plain row indices; index_div = k when index holds top-k slots
 *   (slot = token * k + choice) and src holds one row per token.
 * scatter_rows: dst[index[i]] = src[i] for index[i] >= 0            (i < n_rows input rows)
 *   Rows are row_bytes long (a multiple of 16), src / dst 16-byte aligned.
 * weighted_sum_rows: dst[t] = sum_{j<k} weights[t*k+j] * src[pos ? pos[t*k+j] : t*k+j] for t < tokens,
 *   fp32 accumulation, one rounding to `dtype` (STK_F16 / STK_BF16): the weighted top-k combine.
 *   pos == NULL: src is slot-ordered; weights == NULL: all ones; a negative pos contributes nothing.
 * bin_index   : gather index that puts the token rows received from `world` peers (each peer's rows
 *   ordered by local expert; counts[p*local_experts+e] rows from peer p for expert e, int64) into
 *   per-expert bins padded to a multiple of `block` rows: rows of expert e ordered by peer, then
 *   padding (index -1).  total_padded = sum of the padded bin sizes (the caller knows the counts).
 *   If `compose` is not NULL the source row s is replaced by compose[s] (e.g. a sort order).
 *   bin_rows[e] (optional) receives padded rows of expert e / block.  inverse (optional, as long as
 *   the largest index + 1): inverse[index[r]] = r for every row r that is not padding.
 * dmoe_topology: blocked CSR-COO metadata, row- and column-major, of the block-diagonal matrix in
 *   which expert e owns bin_rows[e] block rows and block columns [e*cpb, (e+1)*cpb).  bin_rows lives on
 *   the device, so its sum is checked there: bins that are negative or do not add up to block_rows
 *   (the number the arrays were sized for) leave the arrays unwritten and record STK_ERR_BAD_DIMS in
 *   the device status word.
 */
int stk_b200_gather_rows(const void* src, void* dst, const int32_t* index, int64_t n_rows,
                         int64_t row_bytes, int index_div, void* stream);
int stk_b200_scatter_rows(const void* src, void* dst, const int32_t* index, int64_t n_rows,
                          int64_t row_bytes, void* stream);
int stk_b200_weighted_sum_rows(const void* src, const int32_t* pos, const float* weights, void* dst,
                               int64_t tokens, int top_k, int64_t row_bytes, int dtype, void* stream);
int stk_b200_bin_index(const int64_t* counts, int world, int local_experts, int block,
                       const int32_t* compose, int32_t* index, int64_t total_padded,
                       int32_t* bin_rows, int32_t* inverse, void* stream);
int stk_b200_dmoe_topology(const int32_t* bin_rows, int experts, int cols_per_expert,
                           int64_t block_rows, int16_t* row_indices, int16_t* column_indices,
                           int32_t* offsets, int16_t* column_indices_t, int32_t* offsets_t,
                           int32_t* block_offsets_t, void* stream);

/*
 * Copies up to 1 MiB with a kernel (one CTA) instead of the copy engine.  `dst` may be pinned host
 * memory: a small read-back (expert counts, padded row count) then does not wait behind a large
 * device-to-host copy queued on the copy engine.  No counterpart in the reference.
 */
int stk_b200_copy_bytes(const void* src, void* dst, int64_t nbytes, void* stream);

/*
 * Expert-parallel token exchange over peer memory (NVLink), top-k routing.  No counterpart in the
 * reference, which is single-GPU; these move the rows that stk.ops.sdd / dsd work on between the
 * ranks of an expert-parallel dMoE layer without a host-side collective.  A rank holds `tokens`
 * tokens with top_k expert choices each (slot = token * top_k + choice).  It pushes the token row of
 * every slot into the padded bin of the slot's expert on the rank that owns the expert, with a tag
 * naming the slot's home; after the experts' MLP the owner pushes every result row into the home
 * rank's slot-ordered buffer, and stk_b200_weighted_sum_rows combines the top_k rows of a token.
 * Only stores go to a peer.  `peer_*[r]` is rank r's buffer as mapped in THIS process (symmetric
 * memory); the caller puts a barrier between ranks after the count exchange, after dispatch and
 * after return.  A row that would fall outside a buffer is skipped and STK_ERR_WORKSPACE is
 * recorded in the status word (stk_b200_device_status).
 * The local experts of every rank can be handled in `chunks` groups of consecutive experts (chunk c =
 * local experts [c*L/chunks, (c+1)*L/chunks), L = experts / world), so that the exchange of one group
 * overlaps the products of another; chunks <= STK_EP_MAX_CHUNKS.
 *   ep_barrier: all ranks meet on the stream.  peer_flags[r] = rank r's flag array (int64 [world],
 *               zero before the first use); every rank stores `epoch` into slot `rank` of every
 *               array and waits until its own array holds `epoch` everywhere.  `epoch` starts at 1 and
 *               grows by one per barrier on the same arrays, identically on all ranks.  The wait gives
 *               up after timeout_ms and records STK_ERR_DEVICE_TIMEOUT in the status word (nothing
 *               traps).  One rank per GPU: ranks sharing a GPU must not use it.
 *   ep_share_counts: row `rank` of every rank's count matrix (peer_counts[r], int32
 *               [world*experts]) <- offsets[e+1] - offsets[e], this rank's slots per expert.
 *   ep_plan:    counts_all[s*experts+e] = slots of rank s for global expert e (int32, the same
 *               matrix on every rank).  Writes dest_base[e] (row in the owner's buffer where this
 *               rank's rows of expert e start), bin_rows[le] (blocks of this rank's local bins),
 *               totals[0] = padded rows of this rank, totals[1] = rows it receives, totals[2] = the
 *               largest padded row count of any rank (identical on all ranks: compare it with the
 *               capacity and every rank takes the same decision), totals[3+c] = padded rows of this
 *               rank's chunk c.  totals: int64 [3 + chunks].
 *   ep_zero_padding: zero rows that close each local bin in `recv`; their tags become -1.
 *   ep_dispatch: for every sorted position q in expert segment e whose expert lies in chunk `chunk`
 *               of its owner: x[order[q] / top_k] -> owner's buffer row dest_base[e] + (q - offsets[e]),
 *               tag rank << 40 | order[q] -> owner's tags (order / offsets as produced by a stable
 *               sort of the slots by expert).
 *   ep_return:  rows [row0, row0 + n_rows) of `result` -> row (tag & (2^40 - 1)) of the slot-ordered
 *               buffer of rank tag >> 40 (peer_slots); rows with a negative tag are padding.
 */
#define STK_EP_MAX_CHUNKS 8
int stk_b200_ep_barrier(const uint64_t* peer_flags, int world, int rank, int64_t epoch, int64_t timeout_ms,
                        void* stream);
int stk_b200_ep_share_counts(const int32_t* offsets, const uint64_t* peer_counts, int world, int experts,
                             int rank, void* stream);
int stk_b200_ep_plan(const int32_t* counts_all, int world, int experts, int rank, int block, int chunks,
                     int64_t* dest_base, int32_t* bin_rows, int64_t* totals, void* stream);
int stk_b200_ep_zero_padding(const int32_t* counts_all, int world, int experts, int rank, int block,
                             void* recv, int64_t* tags, int64_t row_bytes, int64_t cap_rows, void* stream);
int stk_b200_ep_dispatch(const void* x, const int32_t* order, const int32_t* offsets,
                         const int64_t* dest_base, const uint64_t* peer_bufs, const uint64_t* peer_tags,
                         int64_t slots, int top_k, int world, int experts, int rank, int chunk, int chunks,
                         int64_t row_bytes, int64_t cap_rows, void* stream);
int stk_b200_ep_return(const void* result, const int64_t* tags, const uint64_t* peer_slots, int64_t row0,
                       int64_t n_rows, int world, int64_t row_bytes, int64_t slot_cap, void* stream);

/*
 * 32-bit block indices.  The reference stores block row / column indices as int16 and rejects matrices
 * with more than 32767 blocks per side (stk/matrix.py:161-167, dtype handling left as a TODO at
 * :178-181).  Every entry point above that takes or produces int16 index arrays (row_indices,
 * column_indices, column_indices_t) has a twin with the suffix _i32 that takes int32 arrays instead;
 * all other arguments, the results and the error codes are the same.  offsets, offsets_t and
 * block_offsets_t are int32 in both.
 */
int stk_b200_sdd_i32(const void* lhs, const void* rhs, void* out, const int32_t* offsets,
                     const int32_t* row_indices, const int32_t* column_indices,
                     int64_t M, int64_t N, int64_t K, int64_t nnz,
                     int lhs_colmajor, int64_t ld_lhs, int rhs_colmajor, int64_t ld_rhs,
                     int dtype, int pair_mode, int epilogue, void* aux, const int32_t* pair_plan,
                     void* stream);
int stk_b200_dsd_i32(const void* data, const int32_t* offsets, const int32_t* column_indices,
                     const int32_t* block_offsets, const void* rhs, void* out,
                     int64_t M, int64_t N, int64_t K, int64_t nnz,
                     int trans_sparse, int rhs_colmajor, int64_t ld_rhs, int64_t ld_out,
                     int dtype, int pair_mode, const int32_t* pair_plan, void* stream);
int stk_b200_dds_i32(const void* lhs, const void* data, const int32_t* offsets,
                     const int32_t* column_indices, const int32_t* block_offsets, void* out,
                     int64_t M, int64_t N, int64_t K, int64_t nnz,
                     int lhs_colmajor, int64_t ld_lhs, int trans_sparse, int64_t ld_out,
                     int dtype, int pair_mode, const int32_t* pair_plan, void* stream);
int stk_b200_pair_stats_i32(const int32_t* offsets, const int32_t* row_indices,
                            const int32_t* column_indices, const int32_t* offsets_t,
                            const int32_t* column_indices_t, int64_t block_rows, int64_t block_cols,
                            int64_t nnz, int32_t* stats, void* stream);
int stk_b200_pair_plan_i32(const int32_t* offsets, const int32_t* column_indices, int64_t num_lists,
                           int32_t* plan, size_t plan_bytes, void* stream);
int stk_b200_row_indices_i32(const int32_t* offsets, int32_t* out, int64_t block_rows, int64_t nnz,
                             void* stream);
int stk_b200_transpose_meta_i32(const int32_t* row_indices, const int32_t* column_indices,
                                int64_t nnz, int64_t block_cols,
                                int32_t* column_indices_t, int32_t* offsets_t, int32_t* block_offsets_t,
                                void* workspace, size_t workspace_bytes, void* stream);
int stk_b200_mask_to_indices_i32(const uint8_t* mask, int64_t block_rows, int64_t block_cols,
                                 const int32_t* offsets, int32_t* row_indices, int32_t* column_indices,
                                 void* stream);
int stk_b200_gather_blocks_i32(const void* x, int64_t rows, int64_t cols, int64_t ld,
                               int blocking, int elem_bytes, const int32_t* offsets,
                               const int32_t* row_indices, const int32_t* column_indices, int64_t nnz,
                               void* data, void* stream);
int stk_b200_to_dense_i32(const void* data, const int32_t* offsets, const int32_t* column_indices,
                          int64_t block_rows, int64_t block_cols, int blocking, int elem_bytes,
                          void* out, int64_t ld_out, void* stream);
int stk_b200_dmoe_topology_i32(const int32_t* bin_rows, int experts, int cols_per_expert,
                               int64_t block_rows, int32_t* row_indices, int32_t* column_indices,
                               int32_t* offsets, int32_t* column_indices_t, int32_t* offsets_t,
                               int32_t* block_offsets_t, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* STK_B200_H_ */
