// Block-sparse matmul on CTA PAIRS (tcgen05 cta_group::2): 256x256 output supertiles.
//
// Why: the kernel in bsmm_sm100.cuh computes one 128x128 tile per CTA and has to pull 32 KiB of
// operands through shared memory for every 128x128x64 of MMA work (64 FLOP/B); TMA writes into
// shared memory and the tensor pipe's reads out of it share its bandwidth, and measured on B200
// that kernel keeps the tensor pipe busy about a third of the time.  A pair of CTAs that shares
// one 256-row MMA needs the same 32 KiB per CTA for twice the work (128 FLOP/B): each CTA loads
// its own 128 rows of A and its own 128 columns of B, the hardware reads both halves.
//
// A supertile needs two A row-blocks that walk the SAME K sequence and two B column-blocks:
//
//   DSD  rows (r, r+1) of op(S)  x  256 columns of the dense operand.  The K sequence is the MERGE of
//        the two block rows' column lists; where a row has no block at a K position its A tile is
//        fetched from an out-of-range TMA coordinate, which yields zeros.
//   DDS  256 rows of the dense operand  x  block columns (2t, 2t+1) of op(S), K = merge of their lists.
//   SDD  block rows (r, r+1)  x  block columns (2u, 2u+1); the four blocks that exist are stored.
//   Which rows pair up is decided per launch (see decode_item): runs of rows cut at expert boundaries.
//
// Results are exact for ANY sorted topology; the layout only pays off when neighbouring block
// rows / columns share most of their lists (dMoE topologies do: all rows of one expert are alike).
// The host picks this kernel, the 128x256 row kernel or the 128x128 kernel per call.
//
// Roles per CTA (352 threads): warp 0 = TMA producer of the A tiles, warp 6 = TMA producer of the B
// tiles, warp 1 = TMEM owner (and, in the leader CTA, the MMA issuer), warps 2..5 and 7..10 = two
// epilogue groups that drain alternate 64-column sub-tiles of an accumulator.  The MMA issuer does not know the tiles: it consumes a
// stream of pipeline stages, each tagged FIRST / LAST (of a tile) or END by the leader's producer.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/stk_b200.h"
#include "bsmm_sm100.cuh"
#include "sm100_ptx.cuh"
#include "status.cuh"

namespace stk {

constexpr int kPThreads = 352;       // warps: 0 A-producer, 1 MMA / TMEM, 2..5 and 7..10 epilogue, 6 B-producer
constexpr int kPEpilogueWarps = 8;   // two groups of four; a group covers the four TMEM lane quarters
constexpr int kPProducerBWarp = 6;
constexpr int kPStages = 6;
constexpr int kPAccCols = 256;   // one accumulator: 128 lanes x 256 fp32 columns per CTA
constexpr int kPTmemCols = 512;  // two accumulators
constexpr int kPNumBars = 2 * kPStages + 4;
#ifndef STK_DEPENDENT_LAUNCH
#define STK_DEPENDENT_LAUNCH 1
#endif
constexpr bool kUseDependentLaunch = STK_DEPENDENT_LAUNCH != 0;
constexpr int kPSmemBytes =
    kPStages * kStageBytes + 2 * kOutStageBytes + kPNumBars * 8 + kPStages * 4 + 32 + 1024;
constexpr int kNoBlock = 0x7fffffff;

enum : uint32_t { kFlagFirst = 1u, kFlagLast = 2u, kFlagEnd = 4u };


struct PairParams {
  int mode;
  int a_mn, b_mn, fmt;
  int in8;          // 1: 8-bit float operands (e4m3), both K-major; fmt then only names the output format
  int epilogue;     // kEpilogueNone / kEpilogueGelu
  int num_items;    // static work items, dealt round-robin to the CTA pairs
  int inner;        // DSD: N supertiles per row pair; DDS: M supertiles per column pair; SDD: segments per row pair
  int k_steps;      // SDD: ceil(K / 64)
  int num_lists;    // DSD: block rows of op(S); DDS: block columns of op(S); SDD: block rows of the topology
  int zero_coord;   // an out-of-range row of the sparse tensor map (nnz * 128): reads as zeros
  int out_rows, out_cols;  // DSD/DDS: extent of the dense output in elements
  IndexArray col_idx;
  const int32_t* offsets;
  const int32_t* blk_idx;  // nullptr: block j is data[j]
  void* out;
  long long ldc;
  const void* aux;  // SDD with kEpilogueGeluKeep / kEpilogueGeluGrad: the auxiliary tensor
  const int32_t* plan;  // work-item table written by pair_plan_kernel (plan_sm100.cuh), or nullptr
  unsigned int* pace;   // counter of finished items that keeps the CTA pairs in step (see pace_gate), or nullptr
};

// Two-pointer merge of the K lists of a pair of block rows (DSD) / block columns (DDS).  The heads of
// both lists (column and data index) are held in registers and reloaded as soon as a list advances, so
// that the loads of one step are in flight while the step before it waits for its pipeline stage:
// with 8-bit operands a stage is a whole block and the walk runs once per stage.
struct MergeWalker {
  IndexArray col;
  const int32_t* blk;
  int ia, a1, ib, b1;
  int ca, cb;  // columns of the head blocks, kNoBlock for an exhausted list
  int ba, bb;  // their indices into data
  __device__ __forceinline__ void load_a() {
    ca = ia < a1 ? col[ia] : kNoBlock;
    ba = ia < a1 ? (blk ? __ldg(blk + ia) : ia) : kNoBlock;
  }
  __device__ __forceinline__ void load_b() {
    cb = ib < b1 ? col[ib] : kNoBlock;
    bb = ib < b1 ? (blk ? __ldg(blk + ib) : ib) : kNoBlock;
  }
  // Lists la and la + 1 (part 0), or list la alone (part 1).
  __device__ __forceinline__ void init(const PairParams& p, int la, int part = 0) {
    col = p.col_idx;
    blk = p.blk_idx;
    const int lb = la + 1;
    ia = p.offsets[la];
    a1 = p.offsets[la + 1];
    if (lb < p.num_lists && part != 1) {
      ib = a1;  // consecutive lists are adjacent in the metadata
      b1 = p.offsets[lb + 1];
    } else {
      ib = b1 = 0;
    }
    load_a();
    load_b();
  }
  __device__ __forceinline__ bool empty() const { return ia >= a1 && ib >= b1; }
  // Next K position; blk_a / blk_b = index into data of the block each list has there, or kNoBlock.
  __device__ __forceinline__ void next(int& kpos, int& blk_a, int& blk_b) {
    kpos = min(ca, cb);
    blk_a = blk_b = kNoBlock;
    const bool take_a = ca == kpos, take_b = cb == kpos;
    if (take_a) {
      blk_a = ba;
      ++ia;
      load_a();
    }
    if (take_b) {
      blk_b = bb;
      ++ib;
      load_b();
    }
  }
};

// Walks the 2x2 block tiles of one row pair of an SDD topology inside one column segment.
struct TileWalker {
  IndexArray col;
  int ia, a1, ib, b1, u_end;
  __device__ __forceinline__ int lower_bound(int lo, int hi, int c_min) const {
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (col[mid] < c_min) lo = mid + 1; else hi = mid;
    }
    return lo;
  }
  // First position in [lo, hi) whose column is >= c_min.  Rows of dMoE topologies are runs of
  // consecutive columns, so the position is first guessed by offset and checked with two loads;
  // only a wrong guess pays for the binary search (a chain of dependent loads).
  __device__ __forceinline__ int seek(int lo, int hi, int c_min) const {
    if (lo >= hi) return lo;
    const int first = col[lo];
    if (first >= c_min) return lo;
    const int guess = lo + (c_min - first);
    if (guess < hi && col[guess] >= c_min &&
        col[guess - 1] < c_min)
      return guess;
    return lower_bound(lo, hi, c_min);
  }
  // Rows ra and ra + 1 (part 0), or row ra alone (part 1).
  __device__ __forceinline__ void init(const PairParams& p, int ra, int seg, int part = 0) {
    col = p.col_idx;
    const int rb = ra + 1;
    int a0 = p.offsets[ra];
    a1 = p.offsets[ra + 1];
    int b0 = a1;
    b1 = rb < p.num_lists ? p.offsets[rb + 1] : a1;
    if (part == 1) b0 = b1;
    ia = a1;
    ib = b1;
    u_end = 0;
    if (a0 >= a1 && b0 >= b1) return;  // no block in either row
    int c_min = kNoBlock, c_max = -1;
    if (a0 < a1) {
      c_min = min(c_min, col[a0]);
      c_max = max(c_max, col[a1 - 1]);
    }
    if (b0 < b1) {
      c_min = min(c_min, col[b0]);
      c_max = max(c_max, col[b1 - 1]);
    }
    const int u_min = c_min >> 1, n_u = (c_max >> 1) - u_min + 1;
    const int u_lo = u_min + static_cast<int>((static_cast<long long>(seg) * n_u) / p.inner);
    u_end = u_min + static_cast<int>((static_cast<long long>(seg + 1) * n_u) / p.inner);
    ia = seek(a0, a1, 2 * u_lo);
    ib = seek(b0, b1, 2 * u_lo);
  }
  // Next tile: u = column pair; p[r][h] = block index of (row ra+r, column 2u+h) or kNoBlock.
  __device__ __forceinline__ bool next(int& u, int (&p)[2][2]) {
    const int ca = ia < a1 ? col[ia] : kNoBlock;
    const int cb = ib < b1 ? col[ib] : kNoBlock;
    const int c = min(ca, cb);
    if (c == kNoBlock || (c >> 1) >= u_end) return false;
    u = c >> 1;
    p[0][0] = p[0][1] = p[1][0] = p[1][1] = kNoBlock;
#pragma unroll
    for (int rep = 0; rep < 2; ++rep) {
      if (ia < a1) {
        const int cc = col[ia];
        if ((cc >> 1) == u) { p[0][cc & 1] = ia; ++ia; }
      }
      if (ib < b1) {
        const int cc = col[ib];
        if ((cc >> 1) == u) { p[1][cc & 1] = ib; ++ib; }
      }
    }
    return true;
  }
};

__device__ __forceinline__ void load_operand_pair(const CUtensorMap* tm, uint32_t smem_dst,
                                                  uint32_t leader_bar, int mn_major, int mn_elem,
                                                  int k_elem, bool bytes8 = false) {
  if (!mn_major) {
    tma_load_2d_pair(smem_dst, tm, leader_bar, k_elem, mn_elem);
  } else if (bytes8) {
    tma_load_2d_pair(smem_dst, tm, leader_bar, mn_elem, k_elem);  // see load_operand
  } else {
    tma_load_3d_pair(smem_dst, tm, leader_bar, 0, k_elem, mn_elem >> 6);
  }
}

// Work items.  The block rows (DSD, SDD) or block columns (DDS) are taken two at a time, each CTA
// of the pair computing one of them.  Blind pairs (0,1), (2,3), ... go wrong where two experts of a
// dMoE topology meet at an odd row: the two rows' block lists cannot overlap (the last column of one
// lies before the first column of the other), so the pair runs for the sum of both lists with half
// of every MMA wasted, and every pair behind it may be misaligned as well.  The lists are therefore
// cut into runs at those places and paired inside each run, a run of odd length ending in a single
// list; that table is computed once per topology (pair_plan_kernel) and read here, one entry per
// item.  Without a table the kernel pairs blindly, which is still exact.
struct PairItem {
  int r, part, inner;  // first list of the group, 0 = lists r and r + 1 / 1 = list r alone, dense supertile
};
// Item order: item = group * inner + inner position, the inner position (dense supertile of a
// DSD / DDS group, column segment of an SDD row group) running fastest, dealt round-robin to the CTA
// pairs.
__device__ __forceinline__ PairItem decode_item(const PairParams& p, int item) {
  PairItem it;
  const int g = item / p.inner;
  it.inner = item - g * p.inner;
  if (p.plan != nullptr) {
    const int e = __ldg(p.plan + 1 + g);
    it.r = e & 0x3fffffff;
    it.part = (e >> 30) & 1;
    // a table that does not belong to this topology must not send anyone out of bounds
    if (it.r + (it.part ? 0 : 1) >= p.num_lists) {
      report_status(STK_ERR_BAD_DIMS);
      it.r = p.num_lists - 1;
      it.part = 1;
    }
  } else {
    it.r = 2 * g;
    it.part = it.r + 1 >= p.num_lists ? 1 : 0;
  }
  return it;
}

// Keeping the CTA pairs in step.  The items are dealt round-robin, so in round k the 74 pairs work on 74
// consecutive items, which share operand tiles (the supertiles of one row group share its sparse
// blocks, the same supertile of neighbouring groups shares the dense panel).  A shared tile comes out
// of the L2 for every pair after the first only while the pairs stay within the L2's turnover time of
// each other (~20 us at the fill rate of these kernels); left alone they drift apart by a few per
// cent per round (SMs differ in their distance to the L2 slices) and most sharing is lost - measured:
// 4x the compulsory DRAM reads.  So the leader's A producer counts finished items in a global counter
// and starts its k-th item only when (almost) all pairs have finished k items - a barrier with slack
// and a short time limit, never a hard wait: a pair that would wait longer goes on (pairs that were
// scheduled late, behind the tail of the previous kernel, are caught up with a few microseconds per
// round).  The static schedule ends with its slowest pair anyway, so the waiting costs no time.  The
// pair that finishes the very last item resets the counter for the next launch.
#ifndef STK_PACE_PAIRS
#define STK_PACE_PAIRS 1
#endif
constexpr bool kPacePairs = STK_PACE_PAIRS != 0;
// (Measured on the full-size dMoE products: slack 0, 3, 8 and limits of 12 and 40 us are level; a limit
// of 4 us gives up too early and costs the DSD 5 %.)
#ifndef STK_PACE_SLACK
#define STK_PACE_SLACK 3
#endif
#ifndef STK_PACE_LIMIT_NS
#define STK_PACE_LIMIT_NS 12000
#endif
constexpr unsigned int kPaceSlack = STK_PACE_SLACK;  // pairs that may still be busy when a round starts
constexpr unsigned long long kPaceLimitNs = STK_PACE_LIMIT_NS;
__device__ __forceinline__ void pace_gate(const unsigned int* pace, unsigned int target) {
  const unsigned long long t0 = globaltimer_ns();
  while (*reinterpret_cast<const volatile unsigned int*>(pace) < target) {
    if (globaltimer_ns() - t0 > kPaceLimitNs) return;
    __nanosleep(100);
  }
}

// kF8: 8-bit float operands (kind::f8f6f4); a stage then covers 128 of K, i.e. a whole sparse block.
template <bool kTrain, bool kF8 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPThreads, 1)
bsmm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX,
                 const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);

  const uint32_t staging_base = smem_base + kPStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPStages * kStageBytes + 2 * kOutStageBytes);
  const uint32_t bars_base = staging_base + 2 * kOutStageBytes;
  auto full_bar = [&](int s) { return bars_base + 8u * s; };
  auto empty_bar = [&](int s) { return bars_base + 8u * (kPStages + s); };
  auto tfull_bar = [&](int a) { return bars_base + 8u * (2 * kPStages + a); };
  auto tempty_bar = [&](int a) { return bars_base + 8u * (2 * kPStages + 2 + a); };
  volatile uint32_t* stage_flags = reinterpret_cast<volatile uint32_t*>(bars + kPNumBars);
  uint32_t* tmem_slot = const_cast<uint32_t*>(stage_flags) + kPStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epilogue_go = abort_flag + 1;  // [2], one per epilogue group

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());  // 0 = leader
  const int pair_id = static_cast<int>(cluster_id_x());
  const int num_pairs = static_cast<int>(num_clusters_x());

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(full_bar(s), 1);   // leader's copy is the one in use: its producer's arrive + bytes of both CTAs
      mbar_init(empty_bar(s), 1);  // one multicast commit per phase
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);   // one multicast commit per tile
      mbar_init(tempty_bar(a), 2 * kPEpilogueWarps);  // leader's copy: the epilogue warps of both CTAs
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kPTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched only this SM pair; from here on global memory is read.  With a
  // programmatic dependent launch this is where the kernel waits for the one before it in the stream,
  // and the next kernel may be scheduled onto SMs as this grid drains (its set-up then overlaps our
  // tail).
  pdl_launch_dependents();
  pdl_wait();
  const int num_items = p.plan != nullptr ? __ldg(p.plan) * p.inner : p.num_items;

  if (warp == 0 || warp == kPProducerBWarp) {
    // ------------------------------------------------------------------ TMA producers (both CTAs)
    // Warp 0 fetches this CTA's A tiles, warp 6 its B tiles; each walks the metadata on its own, so
    // that neither issue stream has to carry the other's instructions.  One lane works.
    if (lane == 0) {
      const bool is_a = warp == 0;
      const CUtensorMap* tm = is_a ? &tmA : &tmB;
      const int mn_major = is_a ? p.a_mn : p.b_mn;
      const uint32_t dst0 = smem_base + (is_a ? 0 : kOperandTileBytes);
      const uint32_t leader_full0 = map_to_cta(full_bar(0), 0);
      const bool arms = is_a && rank == 0;  // this thread arms the leader's barrier and tags the stage
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // One pipeline stage of this operand: the tile at (mn_elem, k_elem).
      auto produce = [&](int mn_elem, int k_elem, uint32_t flags) {
        ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
        if (!ok) return;
        if (arms) {
          stage_flags[stage] = flags;
          mbar_arrive_expect_tx(full_bar(stage), 2 * kStageBytes);
        }
        load_operand_pair(tm, dst0 + stage * kStageBytes, leader_full0 + 8u * stage, mn_major, mn_elem,
                          k_elem, kF8);
        if (++stage == kPStages) {
          stage = 0;
          phase ^= 1u;
        }
      };
      // Is this thread's operand the sparse one (DSD: A, DDS: B)?
      const bool sparse_side = (p.mode == kModeDSD) == is_a;
      const bool paced = arms && p.pace != nullptr;  // this thread keeps the pair in step with the others
      unsigned int round = 0;
      for (int item = pair_id; item < num_items && ok; item += num_pairs, ++round) {
        if (paced && round > 0 && round * static_cast<unsigned int>(num_pairs) > kPaceSlack)
          pace_gate(p.pace, round * static_cast<unsigned int>(num_pairs) - kPaceSlack);
        if (p.mode == kModeSDD) {
          const PairItem it = decode_item(p, item);
          TileWalker w;
          w.init(p, it.r, it.inner, it.part);
          int u, blk[2][2];
          while (ok && w.next(u, blk)) {
            const int mn_elem = ((is_a ? it.r : 2 * u) + rank) * kBlk;
            for (int ks = 0; ks < p.k_steps && ok; ++ks)
              produce(mn_elem, ks * (kF8 ? 2 * kBK : kBK),
                      (ks == 0 ? kFlagFirst : 0u) | (ks == p.k_steps - 1 ? kFlagLast : 0u));
          }
        } else {
          const PairItem it = decode_item(p, item);
          MergeWalker w;
          w.init(p, it.r, it.part);
          uint32_t first = kFlagFirst;
          while (ok && !w.empty()) {
            int kpos, blk_a, blk_b;
            w.next(kpos, blk_a, blk_b);
            const uint32_t last = w.empty() ? kFlagLast : 0u;
            int mn_elem, k_elem;
            if (sparse_side) {
              // this CTA's block of the pair, or an out-of-range coordinate that reads as zeros
              const int my_blk = rank ? blk_b : blk_a;
              const int row0 = my_blk == kNoBlock ? p.zero_coord : my_blk * kBlk;
              mn_elem = mn_major ? 0 : row0;
              k_elem = mn_major ? row0 : 0;
            } else {
              mn_elem = it.inner * 2 * kBlk + rank * kBlk;
              k_elem = kpos * kBlk;
            }
            if constexpr (kF8) {
              produce(mn_elem, k_elem, first | last);  // one stage holds the block's whole K
            } else {
              produce(mn_elem, k_elem, first);
              if (ok) produce(mn_elem, k_elem + kBK, last);
            }
            first = 0u;
          }
        }
        if (paced) {
          const unsigned int done = atomicAdd(p.pace, 1u) + 1u;
          if (done == static_cast<unsigned int>(num_items)) atomicExch(p.pace, 0u);  // ready for the next launch
        }
      }
      // The leader tells its MMA issuer that the stream is over.
      if (arms && ok) {
        if (mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
          // Unlike a real stage, whose barrier only completes when its bytes have landed (long after
          // the tag was written), this arrival completes the phase at once: the tag has to be
          // visible first.  (Without the fence the MMA issuer, probing the barrier at that moment, was
          // seen to read the slot's old tag - once in some thousand launches of tiny products - take the
          // slot for a stage and wait for ever for the next.)
          stage_flags[stage] = kFlagEnd;
          __threadfence_block();
          mbar_arrive(full_bar(stage));
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && lane == 0) {
      const uint32_t idesc =
          kF8 ? make_idesc_f8(p.a_mn, p.b_mn, 256, 256) : make_idesc_f16(p.fmt, p.a_mn, p.b_mn, 256, 256);
      const uint32_t a_lo0 = smem_desc_lo(smem_base, p.a_mn ? kOperandTileBytes / 2 : 16u);
      const uint32_t b_lo0 = smem_desc_lo(smem_base + kOperandTileBytes, p.b_mn ? kOperandTileBytes / 2 : 16u);
      constexpr uint32_t kMnStep = (kF8 ? 2u : 1u) * kUmmaK * 128u;  // see bsmm_kernel
      const uint32_t a_kstep = (p.a_mn ? kMnStep : kUmmaK * 2u) >> 4;
      const uint32_t b_kstep = (p.b_mn ? kMnStep : kUmmaK * 2u) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      // The tensor pipe queues only an MMA or two ahead of the one it executes, so whatever this
      // thread does between the last MMA of a stage and the first of the next (a barrier poll costs
      // over a hundred cycles even when the phase is complete) shows up as idle tensor cycles.  The
      // next stage's barrier is therefore probed, and its flags read, between the MMAs of the
      // current stage; the blocking wait only runs when that probe found the operands missing.
      bool ready = false;
      uint32_t flags = 0;
      while (true) {
        if (!ready) {
          const bool got = mbar_wait(full_bar(stage), phase, abort_flag);
          if (!got) break;
          flags = stage_flags[stage];
        }
        if (flags & kFlagEnd) break;
        if (flags & kFlagFirst) {
          if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kPAccCols);
        const uint32_t a_lo = a_lo0 + stage * (kStageBytes >> 4);
        const uint32_t b_lo = b_lo0 + stage * (kStageBytes >> 4);
        const int next_stage = stage + 1 == kPStages ? 0 : stage + 1;
        const uint32_t next_phase = stage + 1 == kPStages ? phase ^ 1u : phase;
        umma_pair<kF8>(d_tmem, smem_desc_join(a_lo), smem_desc_join(b_lo), idesc, (flags & kFlagFirst) ? 0u : 1u);
        umma_pair<kF8>(d_tmem, smem_desc_join(a_lo + a_kstep), smem_desc_join(b_lo + b_kstep), idesc, 1u);
        ready = mbar_test_wait(full_bar(next_stage), next_phase);
        const uint32_t next_flags = stage_flags[next_stage];  // not waited for here; only used if `ready`
        umma_pair<kF8>(d_tmem, smem_desc_join(a_lo + 2 * a_kstep), smem_desc_join(b_lo + 2 * b_kstep), idesc, 1u);
        umma_pair<kF8>(d_tmem, smem_desc_join(a_lo + 3 * a_kstep), smem_desc_join(b_lo + 3 * b_kstep), idesc, 1u);
        umma_commit_pair(empty_bar(stage), 3);  // frees the stage in both CTAs
        if (flags & kFlagLast) {
          umma_commit_pair(tfull_bar(acc), 3);  // accumulator halves ready in both CTAs
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        }
        stage = next_stage;
        phase = next_phase;
        flags = next_flags;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int quarter = warp & 3;  // a warp may only read TMEM lanes 32*(warp%4) .. +31
    const int row = quarter * 32 + lane;
    const int group = warp > kPProducerBWarp ? 1 : 0;
    const bool issuer = lane == 0 && (warp == 2 || warp == kPProducerBWarp + 1);  // issues the group's TMA stores
    const uint32_t staging = staging_base + group * kOutStageBytes;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t leader_tempty[2] = {map_to_cta(tempty_bar(0), 0), map_to_cta(tempty_bar(1), 0)};
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // Waits for the accumulator; returns its TMEM address for this warp.
    // The warps of a group meet at hardware barriers while draining, so all four must take the
    // same decision: one thread reads the abort flag between two barriers, the group follows it.
    auto acquire = [&](uint32_t& t_addr) {
      mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
      epilogue_sync(group);
      if (issuer) epilogue_go[group] = (*abort_flag == 0) ? 1 : 0;
      epilogue_sync(group);
      ok = epilogue_go[group] != 0;
      if (ok) tc_fence_after();
      t_addr = tmem_base + lane_base + static_cast<uint32_t>(acc * kPAccCols);
    };
    auto release = [&]() {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    };
    uint16_t* out = static_cast<uint16_t*>(p.out);
    for (int item = pair_id; item < num_items && ok; item += num_pairs) {
      if (p.mode == kModeSDD) {
        const PairItem it = decode_item(p, item);
        TileWalker w;
        w.init(p, it.r, it.inner, it.part);
        int u, blk[2][2];
        while (ok && w.next(u, blk)) {
          uint32_t t_addr;
          acquire(t_addr);
          if (!ok) break;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int pb = blk[rank][h];
            if (pb != kNoBlock)
              drain_to_output<kTrain>(t_addr, h * kBlk, kBlk, p.fmt, p.epilogue, &tmC, 0, pb * kBlk,
                                      staging, row, group, group, 2, issuer,
                                      EpilogueAux{&tmX, static_cast<const uint16_t*>(p.aux)});
          }
          release();
        }
      } else {
        const PairItem it = decode_item(p, item);
        MergeWalker w;
        w.init(p, it.r, it.part);
        // This CTA's 128 output rows and the 256 output columns of the supertile.  In a single-row
        // item the other CTA's rows belong to another item.
        const int tile_row = (p.mode == kModeDSD ? it.r + rank : 2 * it.inner + rank) * kBlk;
        const int tile_col = (p.mode == kModeDSD ? 2 * it.inner : it.r) * kBlk;
        const bool rows_valid =
            tile_row < p.out_rows && (p.mode != kModeDSD || it.part == 0 || rank == 0);
        // (DDS: a single block column's item owns 128 output columns, not 256.)
        const int ncols =
            min((p.mode == kModeDDS && it.part == 1) ? kBlk : 2 * kBlk, p.out_cols - tile_col);
        uint16_t* dst = out + (static_cast<long long>(tile_row) + row) * p.ldc + tile_col;
        if (w.empty()) {
          if (rows_valid && group == 0) {
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
            for (int c = 0; c < ncols; c += 8) *reinterpret_cast<uint4*>(dst + c) = z;
          }
          continue;
        }
        uint32_t t_addr;
        acquire(t_addr);
        if (!ok) break;
        if (rows_valid)
          drain_to_output(t_addr, 0, ncols, p.fmt, p.epilogue, &tmC, tile_col, tile_row, staging, row,
                          group, group, 2, issuer);
        release();
      }
    }
    if (issuer) tma_store_wait_all<0>();  // every output tile has left shared memory and landed
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while its peer may still touch its barriers or TMEM
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kPTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) report_status(STK_ERR_DEVICE_TIMEOUT);
}

// ====================================================================== host side

struct PairDeviceInfo {
  int max_pairs = 0;
};

static int pair_device_info(PairDeviceInfo** out) {
  static PairDeviceInfo infos[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return STK_ERR_LAUNCH;
  PairDeviceInfo& d = infos[dev];
  if (d.max_pairs == 0) {
    if (cudaFuncSetAttribute(bsmm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kPSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(bsmm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kPSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(bsmm_pair_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kPSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return STK_ERR_LAUNCH;
    }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2)
      return STK_ERR_LAUNCH;
    // How many CTA pairs can be resident at once (a pair must sit in one GPC).
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(sms / 2 * 2));
    cfg.blockDim = dim3(kPThreads);
    cfg.dynamicSmemBytes = kPSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, bsmm_pair_kernel<false>, &cfg) != cudaSuccess || clusters < 1) {
      cudaGetLastError();
      clusters = sms / 2;
    }
    d.max_pairs = clusters < sms / 2 ? clusters : sms / 2;
  }
  *out = &d;
  return STK_OK;
}

// Pace counters: zero between launches (the kernel resets the one it used), one per launch in flight,
// handed out in turn.  A pair kernel occupies every SM, so no more than two or three launches ever
// overlap on a device; 32 counters are never all in use.
constexpr int kPaceSlots = 32;
static __device__ unsigned int g_pair_pace[kPaceSlots];

// The counter of the next launch on the current device (nullptr when pacing is compiled out).
static int next_pace_counter(unsigned int** out) {
  *out = nullptr;
  if (!kPacePairs) return STK_OK;
  static unsigned int* base[64] = {};
  static unsigned int turn[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return STK_ERR_LAUNCH;
  if (base[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_pair_pace) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return STK_ERR_LAUNCH;
    }
    base[dev] = static_cast<unsigned int*>(ptr);
  }
  *out = base[dev] + (__atomic_fetch_add(&turn[dev], 1u, __ATOMIC_RELAXED) % kPaceSlots);
  return STK_OK;
}

static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                       const CUtensorMap& tmX, const PairParams& params, cudaStream_t stream) {
  PairDeviceInfo* d = nullptr;
  int rc = pair_device_info(&d);
  if (rc != STK_OK) return rc;
  PairParams p = params;
  if ((rc = next_pace_counter(&p.pace)) != STK_OK) return rc;
  const int pairs = p.num_items < d->max_pairs ? p.num_items : d->max_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  cfg.blockDim = dim3(kPThreads);
  cfg.dynamicSmemBytes = kPSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = kUseDependentLaunch ? 1 : 0;
  if (p.in8 && p.epilogue >= kEpilogueGeluKeep) return STK_ERR_BAD_DIMS;
  const cudaError_t err =
      p.in8 ? cudaLaunchKernelEx(&cfg, bsmm_pair_kernel<false, true>, tmA, tmB, tmC, tmX, p)
      : p.epilogue >= kEpilogueGeluKeep ? cudaLaunchKernelEx(&cfg, bsmm_pair_kernel<true>, tmA, tmB, tmC, tmX, p)
                                        : cudaLaunchKernelEx(&cfg, bsmm_pair_kernel<false>, tmA, tmB, tmC, tmX, p);
  return err == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

}  // namespace stk
