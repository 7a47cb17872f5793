// DSD with one block row of op(S) times 256 dense columns per CTA (a 128x256 output tile), and DDS
// with 256 dense rows times one block column of op(S) (a 256x128 output tile).
//
// Why: the 128x128 kernel moves 32 KiB of operands into shared memory and reads 32 KiB back out of
// it per 128x128x64 of MMA work; operand writes and tensor-pipe reads share the shared-memory
// bandwidth, and at that ratio the tensor pipe is busy a third of the time.  The CTA-pair kernel
// halves the traffic but needs neighbouring block rows with similar block lists.  This kernel keeps
// the sparse tile for two dense tiles with ONE tcgen05.mma of N = 256 per K step: 48 KiB written and
// 48 KiB read per 128x256x64, three quarters of the 128x128 kernel's traffic per FLOP, for any
// topology.  DDS runs as the transposed product: the sparse tile is the MMA's A operand (its 128
// block columns are the accumulator's lanes), the 256 dense rows are the N side, and the epilogue
// writes the accumulator transposed (for one dense row a warp's 32 lanes hold 32 neighbouring
// output columns; staged through shared memory and stored by TMA).  Structure (roles, barriers, probe-ahead MMA loop, staged
// TMA-store epilogue for DSD) is that of bsmm_sm100.cuh; the reference semantics are those of
// _dsd_kernel / _dds_kernel, stk/backend/triton_kernels.py:83-145, 160-220.
#pragma once
#include "bsmm_sm100.cuh"

namespace stk {

constexpr int kRStages = 4;
constexpr int kRStageBytes = 3 * kOperandTileBytes;  // sparse tile, two dense tiles (contiguous: N = 256)
constexpr int kRTmemCols = 512;                      // two 256-column fp32 accumulators
constexpr int kRNumBars = 2 * kRStages + 4;
constexpr int kRSmemBytes = kRStages * kRStageBytes + 2 * kOutStageBytes + kRNumBars * 8 + 32 + 1024;

// Tile order of the DSD / DDS row kernel.  A tile is (list, panel): one block row of op(S) (DSD) or
// block column (DDS) against 256 dense columns / rows.  With the panel running fastest, the CTAs
// resident at one time cover a few lists times ALL panels, i.e. they sweep the whole dense operand,
// and so does every later wave: at 8192^3 and half the blocks present the dense operand was read
// from DRAM 14 times.  The lists are therefore taken in groups of `raster_group`; inside a group the
// panel is the OUTER index and the list the inner one, so that the CTAs resident at one time share one
// or two panels of the dense operand while the group's sparse blocks (chosen to fit in the L2) are
// re-read from the L2 panel after panel.  (The reference gets a similar effect from tl.swizzle2d,
// stk/backend/triton_kernels.py:94-99.)
__device__ __forceinline__ void row_tile(const BsmmParams& p, int tile, int& list, int& panel) {
  const int num_lists = p.num_tiles / p.tiles_inner;
  const int per_group = p.raster_group * p.tiles_inner;
  const int g = tile / per_group, rem = tile - g * per_group;
  const int first = g * p.raster_group;
  const int lists_here = min(p.raster_group, num_lists - first);
  panel = rem / lists_here;
  list = first + (rem - panel * lists_here);
}

__global__ void __launch_bounds__(kThreads, 1)
bsmm_row_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, const BsmmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);

  const uint32_t staging = smem_base + kRStages * kRStageBytes;  // two 16 KiB output staging tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kRStages * kRStageBytes + 2 * kOutStageBytes);
  const uint32_t bars_base = staging + 2 * kOutStageBytes;
  auto full_bar = [&](int s) { return bars_base + 8u * s; };
  auto empty_bar = [&](int s) { return bars_base + 8u * (kRStages + s); };
  auto tfull_bar = [&](int a) { return bars_base + 8u * (2 * kRStages + a); };
  auto tempty_bar = [&](int a) { return bars_base + 8u * (2 * kRStages + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kRNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epilogue_go = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kRTmemCols);
    tmem_relinquish();
  }
  // nothing above read global memory: with a programmatic dependent launch the kernel before this
  // one in the stream may still be running up to here
  pdl_launch_dependents();
  pdl_wait();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Tile t: list (block row of op(S) for DSD, block column for DDS) t / tiles_inner, dense
  // columns (DSD) or rows (DDS) (t % tiles_inner) * 256 .. +256.
  const bool dds = p.mode == kModeDDS;
  const CUtensorMap* tmS = dds ? &tmB : &tmA;  // sparse / dense operand, whichever side it is on
  const CUtensorMap* tmD = dds ? &tmA : &tmB;
  const int s_mn = dds ? p.b_mn : p.a_mn, d_mn = dds ? p.a_mn : p.b_mn;
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    int ok = 1;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      row_tile(p, tile, tm, tn);
      const int j0 = p.offsets[tm], j1 = p.offsets[tm + 1];
      for (int jb = j0; jb < j1 && ok; jb += 32) {
        // The warp fetches the metadata of up to 32 blocks at once, then replays it.
        const int j = jb + lane;
        int my_col = 0, my_blk = 0;
        if (j < j1) {
          my_col = p.col_idx[j];
          my_blk = p.blk_idx ? p.blk_idx[j] : j;
        }
        const int cnt = min(32, j1 - jb);
        for (int i = 0; i < cnt && ok; ++i) {
          const int col = __shfl_sync(0xffffffffu, my_col, i);
          const int blk = __shfl_sync(0xffffffffu, my_blk, i);
          for (int ks = 0; ks < 2 && ok; ++ks) {
            if (lane == 0) {
              if (mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                const uint32_t a_dst = smem_base + stage * kRStageBytes;
                const int s_mn_elem = s_mn ? 0 : blk * kBlk;
                const int s_k_elem = s_mn ? blk * kBlk + ks * kBK : ks * kBK;
                const int d_k_elem = col * kBlk + ks * kBK;
                mbar_arrive_expect_tx(full_bar(stage), kRStageBytes);
                load_operand(tmS, a_dst, full_bar(stage), s_mn, s_mn_elem, s_k_elem);
                // 256 dense columns / rows: two loads of 128, landing back to back (those past
                // the end of the matrix read as zeros)
                load_operand(tmD, a_dst + kOperandTileBytes, full_bar(stage), d_mn, tn * 2 * kBlk,
                             d_k_elem);
                load_operand(tmD, a_dst + 2 * kOperandTileBytes, full_bar(stage), d_mn,
                             tn * 2 * kBlk + kBlk, d_k_elem);
              } else {
                ok = 0;
              }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (++stage == kRStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // the MMA's A operand is the sparse tile, its B operand the 256-wide dense tile
      const uint32_t idesc = make_idesc_f16(p.fmt, s_mn, d_mn, 2 * kBlk);
      const uint32_t a_lo0 = smem_desc_lo(smem_base, s_mn ? kOperandTileBytes / 2 : 16u);
      const uint32_t b_lo0 = smem_desc_lo(smem_base + kOperandTileBytes, d_mn ? kOperandTileBytes / 2 : 16u);
      const uint32_t a_kstep = (s_mn ? kUmmaK * 128u : kUmmaK * 2u) >> 4;
      const uint32_t b_kstep = (d_mn ? kUmmaK * 128u : kUmmaK * 2u) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      bool ready = false;  // the next stage's barrier is probed between the MMAs of the current one
      int nk_next = 0;
      if (static_cast<int>(blockIdx.x) < p.num_tiles) {
        int tm, tn;
        row_tile(p, blockIdx.x, tm, tn);
        nk_next = 2 * (p.offsets[tm + 1] - p.offsets[tm]);
      }
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        const int nk = nk_next;
        if (tile + static_cast<int>(gridDim.x) < p.num_tiles) {  // fetched while this tile's MMAs are issued
          int tm, tn;
          row_tile(p, tile + gridDim.x, tm, tn);
          nk_next = 2 * (p.offsets[tm + 1] - p.offsets[tm]);
        }
        if (nk == 0) continue;  // the epilogue writes zeros; no accumulator is used
        ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * 2 * kBlk);
        uint32_t accumulate = 0;
        for (int ks = 0; ks < nk; ++ks) {
          if (!ready) {
            ok = mbar_wait(full_bar(stage), phase, abort_flag);
            if (!ok) break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * (kRStageBytes >> 4);
          const uint32_t b_lo = b_lo0 + stage * (kRStageBytes >> 4);
          const int next_stage = stage + 1 == kRStages ? 0 : stage + 1;
          const uint32_t next_phase = stage + 1 == kRStages ? phase ^ 1u : phase;
          umma_f16(d_tmem, smem_desc_join(a_lo), smem_desc_join(b_lo), idesc, accumulate);
          umma_f16(d_tmem, smem_desc_join(a_lo + a_kstep), smem_desc_join(b_lo + b_kstep), idesc, 1u);
          ready = mbar_test_wait(full_bar(next_stage), next_phase);
          umma_f16(d_tmem, smem_desc_join(a_lo + 2 * a_kstep), smem_desc_join(b_lo + 2 * b_kstep), idesc, 1u);
          umma_f16(d_tmem, smem_desc_join(a_lo + 3 * a_kstep), smem_desc_join(b_lo + 3 * b_kstep), idesc, 1u);
          accumulate = 1u;
          umma_commit(empty_bar(stage));  // the stage is free once these MMAs have read it
          stage = next_stage;
          phase = next_phase;
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));  // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // a warp may only read TMEM lanes 32*(warp%4) .. +31
    const int row = quarter * 32 + lane;
    const bool issuer = threadIdx.x == 64;  // first epilogue thread issues the TMA stores
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      row_tile(p, tile, tm, tn);
      const int nk = 2 * (p.offsets[tm + 1] - p.offsets[tm]);
      const int col0 = tn * 2 * kBlk;  // DSD: first dense column; DDS: first dense row
      const int ncols = min(2 * kBlk, (dds ? p.out_rows : p.out_cols) - col0);
      uint16_t* out = static_cast<uint16_t*>(p.out);
      if (nk == 0) {
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
        if (!dds) {
          uint16_t* out_row = out + (static_cast<long long>(tm) * kBlk + row) * p.ldc + col0;
          for (int c = 0; c < ncols; c += 8) *reinterpret_cast<uint4*>(out_row + c) = z;
        } else {
          for (int r = row; r < ncols; r += kBlk) {
            uint16_t* out_row = out + (static_cast<long long>(col0) + r) * p.ldc + tm * kBlk;
            for (int c = 0; c < kBlk; c += 8) *reinterpret_cast<uint4*>(out_row + c) = z;
          }
        }
        continue;
      }
      // The four warps meet at a hardware barrier while draining, so they must all take the same
      // decision: one thread reads the abort flag between two barriers, the others follow it.
      mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
      epilogue_sync(0);
      if (issuer) *epilogue_go = (*abort_flag == 0) ? 1 : 0;
      epilogue_sync(0);
      ok = *epilogue_go != 0;
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                              static_cast<uint32_t>(acc * 2 * kBlk);
      if (!dds) {
        drain_to_output(t_addr, 0, ncols, p.fmt, p.epilogue, &tmC, col0, tm * kBlk, staging, row, 0, 0,
                        1, issuer);
      } else {
        // Accumulator lane = output column tm*128 + row, accumulator column = dense row col0 + c: the
        // tile is written transposed.  128 dense rows at a time go through two staging tiles of
        // [128 dense rows][64 output columns] in the 128-byte-swizzle layout (warps of TMEM lane
        // quarters 0-1 fill the first, 2-3 the second; for one dense row a warp's lanes write 64
        // contiguous bytes), and leave with one TMA store each; rows past the matrix are clipped.
        const uint32_t my_stage = staging + (quarter >> 1) * kOutStageBytes;
        const int col_in_half = (quarter & 1) * 32 + lane;  // this thread's column inside the 64-column half
        for (int c0 = 0; c0 < ncols; c0 += kBlk) {
          if (issuer) tma_store_wait_read<0>();  // the previous stores are done reading the tiles
          epilogue_sync(0);
#pragma unroll 1
          for (int c = 0; c < kBlk; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32(t_addr + c0 + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float f = __uint_as_float(v[i]);
              const uint16_t h = p.fmt == STK_BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(f))
                                                   : __half_as_ushort(__float2half_rn(f));
              const int r = c + i;  // dense row inside the 128-row chunk = row of the staging tile
              const uint32_t addr = my_stage + r * 128 + ((((col_in_half >> 3) ^ (r & 7))) << 4) + (col_in_half & 7) * 2;
              asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(h) : "memory");
            }
          }
          fence_proxy_async_smem();
          epilogue_sync(0);
          if (issuer) {
            tma_store_2d(&tmC, staging, tm * kBlk, col0 + c0);
            tma_store_2d(&tmC, staging + kOutStageBytes, tm * kBlk + 64, col0 + c0);
            tma_store_commit();
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kRTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) report_status(STK_ERR_DEVICE_TIMEOUT);
}

// SDD on the same tile shape: two blocks of one block row share the row's lhs panel, their two rhs
// panels sit side by side as the N = 256 operand, and the two halves of the accumulator go to the two
// blocks.  Work item i = blocks 2i and 2i + 1 of the (row-major) block list: one tile if they lie in
// the same block row, else one half-used tile for each (a static enumeration, no prefix sums; a block
// row of L blocks wastes at most one half tile).  Reference semantics: _sdd_kernel,
// stk/backend/triton_kernels.py:34-68.
struct RowSddItem {
  int tiles;       // 1 or 2
  int row[2];      // block row of each tile
  int col[2][2];   // block columns of each tile's halves (second half: -1 if unused)
  int blk[2][2];   // where each half goes in the output
};
__device__ __forceinline__ RowSddItem row_sdd_item(const BsmmParams& p, int item) {
  RowSddItem it;
  const int j0 = 2 * item, j1 = 2 * item + 1;
  const int r0 = p.row_idx[j0], c0 = p.col_idx[j0];
  it.tiles = 1;
  it.row[0] = r0;
  it.col[0][0] = c0;
  it.blk[0][0] = j0;
  it.col[0][1] = it.blk[0][1] = -1;
  it.row[1] = 0;
  it.col[1][0] = it.col[1][1] = it.blk[1][0] = it.blk[1][1] = -1;
  if (j1 < p.nnz) {
    const int r1 = p.row_idx[j1], c1 = p.col_idx[j1];
    if (r1 == r0) {
      it.col[0][1] = c1;
      it.blk[0][1] = j1;
    } else {
      it.tiles = 2;
      it.row[1] = r1;
      it.col[1][0] = c1;
      it.blk[1][0] = j1;
    }
  }
  return it;
}

template <bool kTrain>
__global__ void __launch_bounds__(kThreads, 1)
bsmm_row_sdd_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX,
                    const BsmmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);

  const uint32_t staging = smem_base + kRStages * kRStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kRStages * kRStageBytes + kOutStageBytes);
  const uint32_t bars_base = staging + kOutStageBytes;
  auto full_bar = [&](int s) { return bars_base + 8u * s; };
  auto empty_bar = [&](int s) { return bars_base + 8u * (kRStages + s); };
  auto tfull_bar = [&](int a) { return bars_base + 8u * (2 * kRStages + a); };
  auto tempty_bar = [&](int a) { return bars_base + 8u * (2 * kRStages + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kRNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epilogue_go = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kRTmemCols);
    tmem_relinquish();
  }
  // nothing above read global memory: with a programmatic dependent launch the kernel before this
  // one in the stream may still be running up to here
  pdl_launch_dependents();
  pdl_wait();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.num_tiles && ok; item += gridDim.x) {
        const RowSddItem it = row_sdd_item(p, item);
        for (int t = 0; t < it.tiles && ok; ++t) {
          const bool both = it.col[t][1] >= 0;
          for (int ks = 0; ks < p.k_steps && ok; ++ks) {
            ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
            if (!ok) break;
            const uint32_t a_dst = smem_base + stage * kRStageBytes;
            // an unused second half is not fetched: its accumulator columns are never stored
            mbar_arrive_expect_tx(full_bar(stage), (both ? 3 : 2) * kOperandTileBytes);
            load_operand(&tmA, a_dst, full_bar(stage), p.a_mn, it.row[t] * kBlk, ks * kBK);
            load_operand(&tmB, a_dst + kOperandTileBytes, full_bar(stage), p.b_mn, it.col[t][0] * kBlk,
                         ks * kBK);
            if (both)
              load_operand(&tmB, a_dst + 2 * kOperandTileBytes, full_bar(stage), p.b_mn,
                           it.col[t][1] * kBlk, ks * kBK);
            if (++stage == kRStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(p.fmt, p.a_mn, p.b_mn, 2 * kBlk);
      const uint32_t a_lo0 = smem_desc_lo(smem_base, p.a_mn ? kOperandTileBytes / 2 : 16u);
      const uint32_t b_lo0 = smem_desc_lo(smem_base + kOperandTileBytes, p.b_mn ? kOperandTileBytes / 2 : 16u);
      const uint32_t a_kstep = (p.a_mn ? kUmmaK * 128u : kUmmaK * 2u) >> 4;
      const uint32_t b_kstep = (p.b_mn ? kUmmaK * 128u : kUmmaK * 2u) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      bool ready = false;  // the next stage's barrier is probed between the MMAs of the current one
      // tiles of an item: 2 iff its two blocks lie in different block rows (fetched one item ahead)
      auto tiles_of = [&](int item) {
        const int j1 = 2 * item + 1;
        return (j1 < p.nnz && p.row_idx[j1] != p.row_idx[j1 - 1]) ? 2 : 1;
      };
      int tiles_next = static_cast<int>(blockIdx.x) < p.num_tiles ? tiles_of(blockIdx.x) : 0;
      for (int item = blockIdx.x; item < p.num_tiles && ok; item += gridDim.x) {
        const int tiles = tiles_next;
        if (item + static_cast<int>(gridDim.x) < p.num_tiles) tiles_next = tiles_of(item + gridDim.x);
        for (int t = 0; t < tiles && ok; ++t) {
          ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag);
          if (!ok) break;
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * 2 * kBlk);
          uint32_t accumulate = 0;
          for (int ks = 0; ks < p.k_steps; ++ks) {
            if (!ready) {
              ok = mbar_wait(full_bar(stage), phase, abort_flag);
              if (!ok) break;
            }
            tc_fence_after();
            const uint32_t a_lo = a_lo0 + stage * (kRStageBytes >> 4);
            const uint32_t b_lo = b_lo0 + stage * (kRStageBytes >> 4);
            const int next_stage = stage + 1 == kRStages ? 0 : stage + 1;
            const uint32_t next_phase = stage + 1 == kRStages ? phase ^ 1u : phase;
            umma_f16(d_tmem, smem_desc_join(a_lo), smem_desc_join(b_lo), idesc, accumulate);
            umma_f16(d_tmem, smem_desc_join(a_lo + a_kstep), smem_desc_join(b_lo + b_kstep), idesc, 1u);
            ready = mbar_test_wait(full_bar(next_stage), next_phase);
            umma_f16(d_tmem, smem_desc_join(a_lo + 2 * a_kstep), smem_desc_join(b_lo + 2 * b_kstep), idesc, 1u);
            umma_f16(d_tmem, smem_desc_join(a_lo + 3 * a_kstep), smem_desc_join(b_lo + 3 * b_kstep), idesc, 1u);
            accumulate = 1u;
            umma_commit(empty_bar(stage));
            stage = next_stage;
            phase = next_phase;
          }
          if (!ok) break;
          umma_commit(tfull_bar(acc));
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const bool issuer = threadIdx.x == 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < p.num_tiles && ok; item += gridDim.x) {
      const RowSddItem it = row_sdd_item(p, item);
      for (int t = 0; t < it.tiles && ok; ++t) {
        mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
        epilogue_sync(0);
        if (issuer) *epilogue_go = (*abort_flag == 0) ? 1 : 0;
        epilogue_sync(0);
        ok = *epilogue_go != 0;
        if (!ok) break;
        tc_fence_after();
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                static_cast<uint32_t>(acc * 2 * kBlk);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (it.blk[t][h] >= 0)
            drain_to_output<kTrain>(t_addr, h * kBlk, kBlk, p.fmt, p.epilogue, &tmC, 0,
                                    it.blk[t][h] * kBlk, staging, row, 0, 0, 1, issuer,
                                    EpilogueAux{&tmX, static_cast<const uint16_t*>(p.aux)});
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    if (issuer) tma_store_wait_all<0>();
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kRTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) report_status(STK_ERR_DEVICE_TIMEOUT);
}

static int launch_row(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                      const CUtensorMap& tmX, const BsmmParams& p, cudaStream_t stream) {
  DeviceInfo* d = nullptr;
  const int rc = device_info(&d);
  if (rc != STK_OK) return rc;
  static bool opted_in[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return STK_ERR_LAUNCH;
  if (!opted_in[dev]) {
    if (cudaFuncSetAttribute(bsmm_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kRSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(bsmm_row_sdd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kRSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(bsmm_row_sdd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kRSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return STK_ERR_LAUNCH;
    }
    opted_in[dev] = true;
  }
  const int grid = p.num_tiles < d->sms ? p.num_tiles : d->sms;
  cudaError_t err;
  if (p.mode != kModeSDD)
    err = launch_dependent(bsmm_row_kernel, grid, kThreads, kRSmemBytes, stream, tmA, tmB, tmC, p);
  else if (p.epilogue >= kEpilogueGeluKeep)
    err = launch_dependent(bsmm_row_sdd_kernel<true>, grid, kThreads, kRSmemBytes, stream, tmA, tmB, tmC, tmX, p);
  else
    err = launch_dependent(bsmm_row_sdd_kernel<false>, grid, kThreads, kRSmemBytes, stream, tmA, tmB, tmC, tmX, p);
  return err == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

}  // namespace stk
