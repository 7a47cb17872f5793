// Kernels around the block-sparse products in a dropless-MoE layer: moving token rows into and out
// of padded expert bins, and writing the block-diagonal topology (with its transposed metadata, in
// closed form) for a given number of block rows per expert.  HBM-bound row copies with 16-byte
// accesses, and tiny integer kernels.  The reference has no counterpart (it is a matmul library);
// these are the callers' side of stk.Matrix(...) / stk.ops.sdd / stk.ops.dsd.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/stk_b200.h"
#include "index.cuh"
#include "status.cuh"

namespace stk {

// dst[i] = index[i] >= 0 ? src[index[i] / index_div] : 0, rows of `vec_per_row` 16-byte vectors.  One
// warp per output row; every output row is written exactly once (padding rows as zeros).  index_div > 1:
// the index names a (token, choice) slot of top-k routing, slot = token * k + choice, and the row
// fetched is the token's.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                   const int32_t* __restrict__ index, int64_t n_rows, int vec_per_row, int index_div) {
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  int32_t s = index[row];
  if (s >= 0 && index_div > 1) s /= index_div;
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
// bin_rows[e] = padded rows / block.  inverse (optional): inverse[index[r]] = r for every real row.
__global__ void __launch_bounds__(256)
bin_index_kernel(const int64_t* __restrict__ counts, int world, int local, int block,
                 const int32_t* __restrict__ compose, int32_t* __restrict__ index,
                 int64_t total_padded, int32_t* __restrict__ bin_rows, int32_t* __restrict__ inverse) {
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
  if (src >= 0 && compose != nullptr) src = compose[src];
  index[r] = src;
  if (src >= 0 && inverse != nullptr) inverse[src] = static_cast<int32_t>(r);  // where source row src went
}

// Block-diagonal topology: expert e owns bin_rows[e] consecutive block rows and the block columns
// [e*cpb, (e+1)*cpb).  One thread per block writes both the row-major and the column-major
// metadata; nothing is sorted.
__global__ void __launch_bounds__(256)
dmoe_topology_kernel(const int32_t* __restrict__ bin_rows, int experts, int cpb, int64_t nnz,
                     int block_rows, IndexArray row_indices, IndexArray column_indices,
                     int32_t* __restrict__ offsets, IndexArray column_indices_t,
                     int32_t* __restrict__ offsets_t,
                     int32_t* __restrict__ block_offsets_t) {
  extern __shared__ int32_t row_start[];  // [experts + 1] first block row of every expert
  if (threadIdx.x == 0) {
    int64_t run = 0;
    bool bad = false;
    for (int e = 0; e < experts; ++e) {
      row_start[e] = static_cast<int32_t>(run);
      bad |= bin_rows[e] < 0;
      run += max(bin_rows[e], 0);
      if (run > block_rows) {  // keeps the prefix inside int32 whatever the bins hold
        bad = true;
        run = block_rows;
      }
    }
    // Every position written below is in range only if the bins add up to the block rows the
    // arrays were sized for: anything else writes nothing and is reported.
    row_start[experts] = (bad || run != block_rows) ? -1 : static_cast<int32_t>(run);
  }
  __syncthreads();
  if (row_start[experts] < 0) {
    if (blockIdx.x == 0 && threadIdx.x == 0) report_status(STK_ERR_BAD_DIMS);
    return;
  }
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
  row_indices.store(p, r);
  column_indices.store(p, e * cpb + j);
  // the same block in column-major order: column e*cpb + j, k-th block row of the expert
  const int k = r - row_start[e];
  const int64_t q = static_cast<int64_t>(row_start[e]) * cpb + static_cast<int64_t>(j) * bin_rows[e] + k;
  column_indices_t.store(q, r);
  block_offsets_t[q] = static_cast<int32_t>(p);
}

// dst[t] = sum over j < k of weights[t*k + j] * src[pos ? pos[t*k + j] : t*k + j], accumulated in fp32
// and rounded once: the top-k weighted combine of a dMoE layer (k = 1 with weight 1 is the plain
// un-permute).  A slot whose position is negative (a row that was dropped) contributes nothing.
// One warp per token, 16-byte accesses; kBf16 selects the 16-bit format.
template <bool kBf16>
__global__ void __launch_bounds__(256)
weighted_sum_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ pos,
                         const float* __restrict__ weights, uint4* __restrict__ dst, int64_t tokens, int k,
                         int vec_per_row) {
  const int64_t t = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  for (int v = lane; v < vec_per_row; v += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int64_t slot = t * k + j;
      const int64_t row = pos != nullptr ? static_cast<int64_t>(pos[slot]) : slot;
      if (row < 0) continue;
      const float w = weights != nullptr ? weights[slot] : 1.0f;
      const uint4 x = __ldg(src + row * vec_per_row + v);
      const uint32_t words[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f;
        if (kBf16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[i]));
        else f = __half22float2(*reinterpret_cast<const __half2*>(&words[i]));
        acc[2 * i] = fmaf(w, f.x, acc[2 * i]);
        acc[2 * i + 1] = fmaf(w, f.y, acc[2 * i + 1]);
      }
    }
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (kBf16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        out[i] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __half2 h = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
        out[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    dst[t * vec_per_row + v] = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

// A few bytes copied by a kernel instead of the copy engine: the destination may be pinned host
// memory (mapped into the device's address space), so that a small read-back - expert counts, the
// number of padded rows - does not queue behind a large device-to-host copy on the copy engine.
__global__ void __launch_bounds__(256)
copy_bytes_kernel(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst, int64_t nbytes,
                  int words) {
  if (words) {
    const uint32_t* s4 = reinterpret_cast<const uint32_t*>(src);
    uint32_t* d4 = reinterpret_cast<uint32_t*>(dst);
    for (int64_t i = threadIdx.x; i < nbytes / 4; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int64_t i = threadIdx.x; i < nbytes; i += blockDim.x) dst[i] = src[i];
  }
}

// ------------------------------------------------------------------ expert-parallel exchange
// Token exchange over peer memory (NVLink) for top-k routing.  Every rank holds `tokens` tokens with
// k expert choices each: slot = token * k + choice.  A rank PUSHES the token row of every slot
// straight into the padded bin of the slot's expert on the rank that owns the expert, together with
// a tag (home rank, slot); after the experts' MLP the owner PUSHES every result row back into the
// home rank's slot-ordered buffer, where the k rows of a token are combined with their weights.  The
// peers' buffers are ordinary device pointers (symmetric memory); only plain stores go to a peer, no
// load of any kind reads one.  A barrier between ranks (not part of these kernels) separates the
// phases.  Every address sent to a peer is checked against the buffer's capacity first; a row that
// would not fit is skipped and reported through the status word.
//
// Layout on rank d: bin of local expert le = rows [bin_start[le], bin_start[le] + padded[le]), the
// rows from rank 0 first, then rank 1, ..., each rank's rows in its own (stable) slot order, then
// zero rows up to a multiple of `block`.  The local experts are cut into `chunks` groups of
// consecutive experts so that a caller can overlap the exchange of one group with the products of
// another: chunk c of every rank holds local experts [c * local / chunks, (c + 1) * local / chunks).

constexpr int64_t kTagRowMask = (1ll << 40) - 1;

// Barrier between the ranks of the exchange, on the stream: every rank stores `epoch` into slot
// `rank` of every rank's flag array (peer stores, released at system scope so that everything this
// rank wrote before - its own rows in the peers' buffers - is visible to whoever reads the flag), then
// waits until all `world` slots of its own array have reached `epoch`.  Epochs only grow (one counter
// per flag array on the host, the same on every rank).  The wait is bounded: after `timeout_ns` the
// kernel records STK_ERR_DEVICE_TIMEOUT in the status word and returns, it never traps or spins on.
// One thread per rank.  The ranks must run on different GPUs (a waiting kernel and the kernel it
// waits for are not guaranteed to run at the same time on one GPU).
__global__ void __launch_bounds__(64)
ep_barrier_kernel(const uint64_t* __restrict__ peer_flags, int world, int rank, long long epoch,
                  unsigned long long timeout_ns) {
  const int r = threadIdx.x;
  if (r >= world) return;
  long long* remote = reinterpret_cast<long long*>(peer_flags[r]) + rank;
  asm volatile("st.release.sys.global.s64 [%0], %1;" ::"l"(remote), "l"(epoch) : "memory");
  const long long* mine = reinterpret_cast<const long long*>(peer_flags[rank]) + r;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  while (true) {
    long long v;
    asm volatile("ld.acquire.sys.global.s64 %0, [%1];" : "=l"(v) : "l"(mine) : "memory");
    if (v >= epoch) break;
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - t0 > timeout_ns) {
      report_status(STK_ERR_DEVICE_TIMEOUT);
      break;
    }
    __nanosleep(200);
  }
}

// Row `rank` of every rank's count matrix <- this rank's slots per expert (offsets[e+1] - offsets[e]).
__global__ void __launch_bounds__(128)
ep_share_counts_kernel(const int32_t* __restrict__ offsets, const uint64_t* __restrict__ peer_counts,
                       int world, int experts, int rank) {
  for (int i = threadIdx.x; i < experts * world; i += blockDim.x) {
    const int peer = i / experts, e = i - peer * experts;
    reinterpret_cast<int32_t*>(peer_counts[peer])[rank * experts + e] = offsets[e + 1] - offsets[e];
  }
}

__device__ __forceinline__ int ep_chunk_of(int le, int local, int chunks) {
  return static_cast<int>((static_cast<long long>(le) * chunks) / local);
}

// counts_all[s * E + e] = slots of rank s routed to global expert e (the same matrix on every rank).
// One CTA, E * world small.
//   dest_base[e]  = row in the owner's buffer where THIS rank's rows for expert e start
//   bin_rows[le]  = padded rows / block of this rank's local expert le
//   totals[0] = padded rows of this rank, totals[1] = rows it receives (unpadded),
//   totals[2] = the largest padded row count over ALL ranks (every rank computes the same value, so a
//               buffer overflow anywhere is seen everywhere), totals[3 + c] = padded rows of this
//               rank's chunk c
__global__ void __launch_bounds__(128)
ep_plan_kernel(const int32_t* __restrict__ counts_all, int world, int experts, int local, int rank,
               int block, int chunks, int64_t* __restrict__ dest_base, int32_t* __restrict__ bin_rows,
               int64_t* __restrict__ totals) {
  // column sums first (one round of loads), so that the serial parts below run out of shared memory
  extern __shared__ int32_t ep_sm[];
  int32_t* col_sum = ep_sm;              // [experts] slots of all ranks per expert
  int32_t* before_me = ep_sm + experts;  // [experts] slots of the ranks before this one
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int32_t n = 0, b = 0;
    for (int s = 0; s < world; ++s) {
      const int32_t c = counts_all[s * experts + e];
      n += c;
      if (s < rank) b += c;
    }
    col_sum[e] = n;
    before_me[e] = b;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int owner = e / local, le = e - owner * local;
    int64_t start = 0;
    for (int k = 0; k < le; ++k)
      start += (static_cast<int64_t>(col_sum[owner * local + k]) + block - 1) / block * block;
    dest_base[e] = start + before_me[e];
  }
  if (threadIdx.x == 0) {
    int64_t padded_total = 0, received = 0, worst = 0;
    for (int c = 0; c < chunks; ++c) totals[3 + c] = 0;
    for (int g = 0; g < world; ++g) {
      int64_t sum = 0;
      for (int le = 0; le < local; ++le) {
        const int64_t n = col_sum[g * local + le];
        const int64_t padded = (n + block - 1) / block * block;
        sum += padded;
        if (g == rank) {
          bin_rows[le] = static_cast<int32_t>(padded / block);
          received += n;
          totals[3 + ep_chunk_of(le, local, chunks)] += padded;
        }
      }
      if (g == rank) padded_total = sum;
      if (sum > worst) worst = sum;
    }
    totals[0] = padded_total;
    totals[1] = received;
    totals[2] = worst;
  }
}

// Zero rows that close each local bin (nobody writes them), and mark them in `tags` as belonging to
// nobody.  One warp per padding row.
__global__ void __launch_bounds__(256)
ep_zero_padding_kernel(const int32_t* __restrict__ counts_all, int world, int experts, int local,
                       int rank, int block, uint4* __restrict__ recv, int64_t* __restrict__ tags,
                       int vec_per_row, int64_t cap_rows) {
  const int le = blockIdx.y;
  int64_t start = 0, n = 0;
  for (int k = 0; k <= le; ++k) {
    n = 0;
    for (int s = 0; s < world; ++s) n += counts_all[s * experts + rank * local + k];
    if (k < le) start += (n + block - 1) / block * block;
  }
  const int64_t pad = (n + block - 1) / block * block - n;
  const int64_t w = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= pad) return;
  const int64_t row = start + n + w;
  if (row >= cap_rows) return;
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  for (int v = lane; v < vec_per_row; v += 32) recv[row * vec_per_row + v] = z;
  if (lane == 0 && tags != nullptr) tags[row] = -1;
}

// The push kernels run beside the product kernels of another stream, one CTA per SM: a 256x256 pair
// kernel CTA leaves 1.8 KiB of an SM's shared memory, and every resident CTA costs 1 KiB of it whether
// it asks for shared memory or not, so exactly one more CTA fits; 512 threads x 32 registers fit
// beside the product CTA's 352 x 120.
constexpr int kPushThreads = 512;

// Sorted position q (slots ordered by expert: slot order[q], expert segments offsets[e..e+1]) goes to
// row dest_base[e] + (q - offsets[e]) of the buffer of rank e / local: the row of token order[q] / k,
// and the tag (this rank << 40 | slot) into the owner's tag array.  Only the experts of chunk `chunk`
// of every owner are handled (chunks = 1: all).  A warp per row, the warps of the one-CTA-per-SM grid
// striding over one expert's rows after the other (a CTA per eight rows, 32768 queued CTAs, kept the
// first products waiting until the NEXT chunk's push had been dealt out).
__global__ void __launch_bounds__(kPushThreads, 4)  // 32 registers
ep_dispatch_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ order,
                   const int32_t* __restrict__ offsets, const int64_t* __restrict__ dest_base,
                   const uint64_t* __restrict__ peer_bufs, const uint64_t* __restrict__ peer_tags,
                   int k, int world, int local, int rank, int chunk, int chunks,
                   int vec_per_row, int64_t cap_rows) {
  const int warp0 = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  // local experts le with ep_chunk_of(le) == chunk
  const int le0 = static_cast<int>((static_cast<long long>(chunk) * local + chunks - 1) / chunks);
  const int le1 = static_cast<int>((static_cast<long long>(chunk + 1) * local + chunks - 1) / chunks);
  for (int owner = 0; owner < world; ++owner) {
    int64_t* tags = reinterpret_cast<int64_t*>(peer_tags[owner]);
    uint4* buf = reinterpret_cast<uint4*>(peer_bufs[owner]);
    for (int le = le0; le < le1; ++le) {
      const int e = owner * local + le;
      const int begin = offsets[e], n = offsets[e + 1] - begin;
      const int64_t base = dest_base[e];
      for (int i = warp0; i < n; i += nwarps) {
        const int64_t row = base + i;
        if (row < 0 || row >= cap_rows) {
          if (lane == 0) report_status(STK_ERR_WORKSPACE);
          continue;
        }
        const int32_t slot = order[begin + i];
        if (lane == 0) tags[row] = (static_cast<int64_t>(rank) << 40) | slot;
        const uint4* in = x + static_cast<int64_t>(slot / k) * vec_per_row;
        uint4* out = buf + row * vec_per_row;
        for (int v = lane; v < vec_per_row; v += 32) out[v] = __ldg(in + v);
      }
    }
  }
}

// The way back: rows [row0, row0 + n_rows) of this rank's result go to the home rank's slot-ordered
// buffer, row tag & mask of rank tag >> 40; padding rows (tag < 0) go nowhere.  A warp per row, bounded
// grid as above.
__global__ void __launch_bounds__(kPushThreads, 4)
ep_return_kernel(const uint4* __restrict__ result, const int64_t* __restrict__ tags,
                 const uint64_t* __restrict__ peer_slots, int64_t row0, int64_t n_rows, int world,
                 int vec_per_row, int64_t slot_cap) {
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int64_t w = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; w < n_rows; w += nwarps) {
    const int64_t row = row0 + w;
    const int64_t tag = tags[row];
    if (tag < 0) continue;
    const int64_t home = tag >> 40, slot = tag & kTagRowMask;
    if (home >= world || slot >= slot_cap) {
      if (lane == 0) report_status(STK_ERR_WORKSPACE);
      continue;
    }
    const uint4* in = result + row * vec_per_row;
    uint4* out = reinterpret_cast<uint4*>(peer_slots[home]) + slot * vec_per_row;
    for (int v = lane; v < vec_per_row; v += 32) out[v] = __ldg(in + v);
  }
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
                                    int64_t row_bytes, int index_div, void* stream) {
  const int rc = rows_args_ok(src, dst, index, n_rows, row_bytes);
  if (rc != STK_OK || n_rows == 0) return rc;
  if (index_div < 1) return STK_ERR_BAD_DIMS;
  const int64_t ctas = (n_rows + 7) / 8;
  if (ctas > INT32_MAX) return STK_ERR_TOO_LARGE;
  gather_rows_kernel<<<static_cast<unsigned>(ctas), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), index, n_rows,
      static_cast<int>(row_bytes / 16), index_div);
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
                                  int32_t* bin_rows, int32_t* inverse, void* stream) {
  if (world <= 0 || local_experts <= 0 || block <= 0 || total_padded < 0) return STK_ERR_BAD_DIMS;
  if (static_cast<int64_t>(world) * local_experts > 4096 || total_padded > INT32_MAX) return STK_ERR_TOO_LARGE;
  if (counts == nullptr || (total_padded > 0 && index == nullptr)) return STK_ERR_NULL_POINTER;
  const size_t smem = (static_cast<size_t>(local_experts) + 1 + static_cast<size_t>(world) * local_experts) * sizeof(int64_t);
  const int64_t ctas = total_padded > 0 ? (total_padded + 255) / 256 : 1;
  bin_index_kernel<<<static_cast<unsigned>(ctas), 256, smem, static_cast<cudaStream_t>(stream)>>>(
      counts, world, local_experts, block, compose, index, total_padded, bin_rows, inverse);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

static int dmoe_topology_impl(const int32_t* bin_rows, int experts, int cols_per_expert,
                              int64_t block_rows, IndexArray row_indices, IndexArray column_indices,
                              int32_t* offsets, IndexArray column_indices_t, int32_t* offsets_t,
                              int32_t* block_offsets_t, void* stream) {
  if (experts <= 0 || cols_per_expert <= 0 || block_rows < 0) return STK_ERR_BAD_DIMS;
  const int64_t block_cols = static_cast<int64_t>(experts) * cols_per_expert;
  const long long limit = index_limit(row_indices.wide);
  if (experts > 8192 || block_rows > limit || block_cols > limit) return STK_ERR_TOO_LARGE;
  if (bin_rows == nullptr || offsets == nullptr || offsets_t == nullptr) return STK_ERR_NULL_POINTER;
  const int64_t nnz = block_rows * cols_per_expert;
  if (nnz > INT32_MAX) return STK_ERR_TOO_LARGE;
  if (nnz > 0 && (row_indices.null() || column_indices.null() || column_indices_t.null() ||
                  block_offsets_t == nullptr))
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

extern "C" int stk_b200_dmoe_topology(const int32_t* bin_rows, int experts, int cols_per_expert,
                                      int64_t block_rows, int16_t* row_indices,
                                      int16_t* column_indices, int32_t* offsets,
                                      int16_t* column_indices_t, int32_t* offsets_t,
                                      int32_t* block_offsets_t, void* stream) {
  return dmoe_topology_impl(bin_rows, experts, cols_per_expert, block_rows, IndexArray{row_indices, 0},
                            IndexArray{column_indices, 0}, offsets, IndexArray{column_indices_t, 0}, offsets_t,
                            block_offsets_t, stream);
}
extern "C" int stk_b200_dmoe_topology_i32(const int32_t* bin_rows, int experts, int cols_per_expert,
                                          int64_t block_rows, int32_t* row_indices,
                                          int32_t* column_indices, int32_t* offsets,
                                          int32_t* column_indices_t, int32_t* offsets_t,
                                          int32_t* block_offsets_t, void* stream) {
  return dmoe_topology_impl(bin_rows, experts, cols_per_expert, block_rows, IndexArray{row_indices, 1},
                            IndexArray{column_indices, 1}, offsets, IndexArray{column_indices_t, 1}, offsets_t,
                            block_offsets_t, stream);
}

namespace stk {
// CTAs of a push kernel (ep_dispatch, ep_return): one per SM (see kPushThreads).
// An SM splits one array between L1 and shared memory and changes the split only when it is empty:
// the kernels that run beside the product kernels (which take the largest shared-memory split) ask
// for the same split, or their CTAs would keep product CTAs off their SMs until they have finished.
static bool ep_prefer_product_carveout() {
  const int most = cudaSharedmemCarveoutMaxShared;
  const bool ok =
      cudaFuncSetAttribute(ep_dispatch_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, most) == cudaSuccess &&
      cudaFuncSetAttribute(ep_return_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, most) == cudaSuccess &&
      cudaFuncSetAttribute(ep_barrier_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, most) == cudaSuccess;
  if (!ok) cudaGetLastError();
  return ok;
}
static int64_t ep_push_grid() {
  static int sms[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return -1;
    if (!ep_prefer_product_carveout()) return -1;
    sms[dev] = n;
  }
  return sms[dev];
}
}  // namespace stk

extern "C" int stk_b200_ep_share_counts(const int32_t* offsets, const uint64_t* peer_counts, int world,
                                        int experts, int rank, void* stream) {
  if (!offsets || !peer_counts) return STK_ERR_NULL_POINTER;
  if (world < 1 || experts < 1 || rank < 0 || rank >= world) return STK_ERR_BAD_DIMS;
  stk::ep_share_counts_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(offsets, peer_counts,
                                                                                 world, experts, rank);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

extern "C" int stk_b200_ep_barrier(const uint64_t* peer_flags, int world, int rank, int64_t epoch,
                                   int64_t timeout_ms, void* stream) {
  if (!peer_flags) return STK_ERR_NULL_POINTER;
  if (world < 1 || world > 64 || rank < 0 || rank >= world || epoch < 1 || timeout_ms < 1) return STK_ERR_BAD_DIMS;
  if (stk::ep_push_grid() <= 0) return STK_ERR_LAUNCH;  // (sets the kernels' shared-memory split once per device)
  stk::ep_barrier_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
      peer_flags, world, rank, static_cast<long long>(epoch),
      static_cast<unsigned long long>(timeout_ms) * 1000000ull);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

extern "C" int stk_b200_ep_plan(const int32_t* counts_all, int world, int experts, int rank, int block,
                                int chunks, int64_t* dest_base, int32_t* bin_rows, int64_t* totals,
                                void* stream) {
  if (!counts_all || !dest_base || !bin_rows || !totals) return STK_ERR_NULL_POINTER;
  if (world < 1 || experts < 1 || experts % world != 0 || rank < 0 || rank >= world || block < 1 ||
      chunks < 1 || chunks > experts / world || chunks > STK_EP_MAX_CHUNKS)
    return STK_ERR_BAD_DIMS;
  if (experts > 4096) return STK_ERR_TOO_LARGE;
  stk::ep_plan_kernel<<<1, 128, 2 * experts * sizeof(int32_t), static_cast<cudaStream_t>(stream)>>>(
      counts_all, world, experts, experts / world, rank, block, chunks, dest_base, bin_rows, totals);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

extern "C" int stk_b200_ep_zero_padding(const int32_t* counts_all, int world, int experts, int rank,
                                        int block, void* recv, int64_t* tags, int64_t row_bytes,
                                        int64_t cap_rows, void* stream) {
  if (!counts_all || !recv) return STK_ERR_NULL_POINTER;
  if (world < 1 || experts < 1 || experts % world != 0 || rank < 0 || rank >= world || block < 1 ||
      row_bytes <= 0 || row_bytes % 16 != 0 || cap_rows < 0)
    return STK_ERR_BAD_DIMS;
  const int local = experts / world;
  const dim3 grid(static_cast<unsigned>((block * 32 + 255) / 256), static_cast<unsigned>(local));
  stk::ep_zero_padding_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      counts_all, world, experts, local, rank, block, static_cast<uint4*>(recv), tags,
      static_cast<int>(row_bytes / 16), cap_rows);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

extern "C" int stk_b200_ep_dispatch(const void* x, const int32_t* order, const int32_t* offsets,
                                    const int64_t* dest_base, const uint64_t* peer_bufs,
                                    const uint64_t* peer_tags, int64_t slots, int top_k, int world,
                                    int experts, int rank, int chunk, int chunks, int64_t row_bytes,
                                    int64_t cap_rows, void* stream) {
  if (slots == 0) return STK_OK;
  if (!x || !order || !offsets || !dest_base || !peer_bufs || !peer_tags) return STK_ERR_NULL_POINTER;
  if (slots < 0 || top_k < 1 || world < 1 || experts < 1 || experts % world != 0 || rank < 0 ||
      rank >= world || chunks < 1 || chunk < 0 || chunk >= chunks || row_bytes <= 0 ||
      row_bytes % 16 != 0 || cap_rows < 0)
    return STK_ERR_BAD_DIMS;
  if (slots > INT32_MAX) return STK_ERR_TOO_LARGE;
  int64_t blocks = (slots * 32 + stk::kPushThreads - 1) / stk::kPushThreads;  // a warp per row at most
  const int64_t bound = stk::ep_push_grid();
  if (bound <= 0) return STK_ERR_LAUNCH;
  if (blocks > bound) blocks = bound;
  stk::ep_dispatch_kernel<<<static_cast<unsigned>(blocks), stk::kPushThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), order, offsets, dest_base, peer_bufs, peer_tags, top_k, world,
      experts / world, rank, chunk, chunks, static_cast<int>(row_bytes / 16), cap_rows);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

extern "C" int stk_b200_ep_return(const void* result, const int64_t* tags, const uint64_t* peer_slots,
                                  int64_t row0, int64_t n_rows, int world, int64_t row_bytes,
                                  int64_t slot_cap, void* stream) {
  if (n_rows == 0) return STK_OK;
  if (!result || !tags || !peer_slots) return STK_ERR_NULL_POINTER;
  if (row0 < 0 || n_rows < 0 || world < 1 || row_bytes <= 0 || row_bytes % 16 != 0 || slot_cap < 0)
    return STK_ERR_BAD_DIMS;
  int64_t blocks = (n_rows * 32 + stk::kPushThreads - 1) / stk::kPushThreads;
  const int64_t bound = stk::ep_push_grid();
  if (bound <= 0) return STK_ERR_LAUNCH;
  if (blocks > bound) blocks = bound;
  stk::ep_return_kernel<<<static_cast<unsigned>(blocks), stk::kPushThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(result), tags, peer_slots, row0, n_rows, world,
      static_cast<int>(row_bytes / 16), slot_cap);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

extern "C" int stk_b200_weighted_sum_rows(const void* src, const int32_t* pos, const float* weights,
                                          void* dst, int64_t tokens, int top_k, int64_t row_bytes,
                                          int dtype, void* stream) {
  if (tokens == 0) return STK_OK;
  if (dtype != STK_F16 && dtype != STK_BF16) return STK_ERR_BAD_DTYPE;
  if (tokens < 0 || top_k < 1 || row_bytes <= 0 || row_bytes % 16 != 0) return STK_ERR_BAD_DIMS;
  if (!src || !dst) return STK_ERR_NULL_POINTER;
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) return STK_ERR_BAD_LAYOUT;
  const int64_t blocks = (tokens * 32 + 255) / 256;
  if (blocks > INT32_MAX || row_bytes / 16 > INT32_MAX) return STK_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == STK_BF16)
    stk::weighted_sum_rows_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        static_cast<const uint4*>(src), pos, weights, static_cast<uint4*>(dst), tokens, top_k,
        static_cast<int>(row_bytes / 16));
  else
    stk::weighted_sum_rows_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        static_cast<const uint4*>(src), pos, weights, static_cast<uint4*>(dst), tokens, top_k,
        static_cast<int>(row_bytes / 16));
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

extern "C" int stk_b200_copy_bytes(const void* src, void* dst, int64_t nbytes, void* stream) {
  if (nbytes == 0) return STK_OK;
  if (!src || !dst) return STK_ERR_NULL_POINTER;
  if (nbytes < 0) return STK_ERR_BAD_DIMS;
  if (nbytes > (1 << 20)) return STK_ERR_TOO_LARGE;
  const int words = (reinterpret_cast<uintptr_t>(src) % 4 == 0 && reinterpret_cast<uintptr_t>(dst) % 4 == 0 &&
                     nbytes % 4 == 0) ? 1 : 0;
  stk::copy_bytes_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned char*>(src), static_cast<unsigned char*>(dst), nbytes, words);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}
