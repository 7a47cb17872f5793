// DSD / DDS on CTA pairs with the sparse operand REUSED across two dense tiles: 256x512 (DSD) or
// 512x256 (DDS) of output per work item.
//
// Why: the 256x256 pair kernel needs 32 KiB of operands per CTA for every 128x256x64 of MMA work,
// and one SM ingests at most ~68 B/clk through TMA - as much as the MMAs consume, so the two never
// overlap perfectly.  Here every pipeline stage carries one sparse tile S and TWO dense tiles D0, D1
// (48 KiB per CTA) and feeds two MMAs per K step, acc0 += S*D0 and acc1 += S*D1: 24 KiB per
// 128x256x64, which leaves the operand fetch well below the tensor rate.  The price: both halves
// of tensor memory hold one item's accumulators, so the epilogue of an item only overlaps the next
// item's operand fetch, not its MMAs - worth it when the K loops are long (many blocks per list).
//
// Structure, barriers and the merge of the two block lists are those of bsmm_pair_sm100.cuh.
#pragma once
#include "bsmm_pair_sm100.cuh"

namespace stk {

constexpr int kWStages = 4;
constexpr int kWStageBytes = 3 * kOperandTileBytes;  // S, D0, D1
constexpr int kWNumBars = 2 * kWStages + 3;          // full, empty, tfull, tempty[2]
constexpr int kWSmemBytes =
    kWStages * kWStageBytes + 2 * kOutStageBytes + kWNumBars * 8 + kWStages * 4 + 32 + 1024;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPThreads, 1)
bsmm_wide_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);

  const uint32_t staging_base = smem_base + kWStages * kWStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kWStages * kWStageBytes + 2 * kOutStageBytes);
  const uint32_t bars_base = staging_base + 2 * kOutStageBytes;
  auto full_bar = [&](int s) { return bars_base + 8u * s; };
  auto empty_bar = [&](int s) { return bars_base + 8u * (kWStages + s); };
  const uint32_t tfull_bar = bars_base + 8u * (2 * kWStages);
  auto tempty_bar = [&](int a) { return bars_base + 8u * (2 * kWStages + 1 + a); };
  volatile uint32_t* stage_flags = reinterpret_cast<volatile uint32_t*>(bars + kWNumBars);
  uint32_t* tmem_slot = const_cast<uint32_t*>(stage_flags) + kWStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epilogue_go = abort_flag + 1;  // [2], one per epilogue group

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const int pair_id = static_cast<int>(cluster_id_x());
  const int num_pairs = static_cast<int>(num_clusters_x());
  const bool dsd = p.mode == kModeDSD;  // sparse operand is A (DSD) or B (DDS)

  if (threadIdx.x == 0) {
    for (int s = 0; s < kWStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    for (int a = 0; a < 2; ++a) mbar_init(tempty_bar(a), kPEpilogueWarps);  // one group of each CTA
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
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 || warp == kPProducerBWarp) {
    // ---------------------------------------------------------------- TMA producers (both CTAs)
    // Warp 0 fetches the sparse tile of every stage, warp 6 the two dense tiles.
    if (lane == 0) {
      const bool sparse_side = warp == 0;
      const CUtensorMap* tm = (sparse_side == dsd) ? &tmA : &tmB;
      const int mn_major = (sparse_side == dsd) ? p.a_mn : p.b_mn;
      const uint32_t dst0 = smem_base + (sparse_side ? 0 : kOperandTileBytes);
      const uint32_t leader_full0 = map_to_cta(full_bar(0), 0);
      const bool arms = sparse_side && rank == 0;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = pair_id; item < p.num_items && ok; item += num_pairs) {
        const int outer = item / p.inner, inner = item - outer * p.inner;
        MergeWalker w;
        w.init(p, 2 * outer);
        uint32_t first = kFlagFirst;
        while (ok && !w.empty()) {
          int kpos, blk_a, blk_b;
          w.next(kpos, blk_a, blk_b);
          const uint32_t last = w.empty() ? kFlagLast : 0u;
          int mn_elem, k_elem;
          if (sparse_side) {
            const int my_blk = rank ? blk_b : blk_a;
            const int row0 = my_blk == kNoBlock ? p.zero_coord : my_blk * kBlk;
            mn_elem = mn_major ? 0 : row0;
            k_elem = mn_major ? row0 : 0;
          } else {
            mn_elem = inner * 4 * kBlk + rank * kBlk;  // D0; D1 is 256 further
            k_elem = kpos * kBlk;
          }
          for (int ks = 0; ks < 2 && ok; ++ks) {
            ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
            if (!ok) break;
            if (arms) {
              stage_flags[stage] = ks == 0 ? first : last;
              mbar_arrive_expect_tx(full_bar(stage), 2 * kWStageBytes);
            }
            const uint32_t dst = dst0 + stage * kWStageBytes;
            const uint32_t bar = leader_full0 + 8u * stage;
            load_operand_pair(tm, dst, bar, mn_major, mn_elem, k_elem + ks * kBK);
            if (!sparse_side)
              load_operand_pair(tm, dst + kOperandTileBytes, bar, mn_major, mn_elem + 2 * kBlk,
                                k_elem + ks * kBK);
            if (++stage == kWStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          first = 0u;
        }
      }
      if (arms && ok) {
        if (mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
          stage_flags[stage] = kFlagEnd;
          mbar_arrive(full_bar(stage));
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA only)
    if (rank == 0 && lane == 0) {
      const uint32_t idesc = make_idesc_f16(p.fmt, p.a_mn, p.b_mn, 256, 256);
      const int s_mn = dsd ? p.a_mn : p.b_mn, d_mn = dsd ? p.b_mn : p.a_mn;
      const uint32_t s_lo0 = smem_desc_lo(smem_base, s_mn ? kOperandTileBytes / 2 : 16u);
      const uint32_t d_lo0 = smem_desc_lo(smem_base + kOperandTileBytes, d_mn ? kOperandTileBytes / 2 : 16u);
      const uint32_t s_kstep = (s_mn ? kUmmaK * 128u : kUmmaK * 2u) >> 4;
      const uint32_t d_kstep = (d_mn ? kUmmaK * 128u : kUmmaK * 2u) >> 4;
      int stage = 0;
      uint32_t phase = 0, tile_phase = 0;
      // As in the pair kernel: the next stage's barrier is probed between the MMAs of this one.
      bool ready = false;
      uint32_t flags = 0;
      while (true) {
        if (!ready) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) break;
          flags = stage_flags[stage];
        }
        if (flags & kFlagEnd) break;
        if (flags & kFlagFirst) {
          if (!mbar_wait(tempty_bar(0), tile_phase ^ 1u, abort_flag)) break;
          if (!mbar_wait(tempty_bar(1), tile_phase ^ 1u, abort_flag)) break;
        }
        tc_fence_after();
        const uint32_t s_lo = s_lo0 + stage * (kWStageBytes >> 4);
        const uint32_t d_lo = d_lo0 + stage * (kWStageBytes >> 4);
        const int next_stage = stage + 1 == kWStages ? 0 : stage + 1;
        const uint32_t next_phase = stage + 1 == kWStages ? phase ^ 1u : phase;
        uint32_t accumulate = (flags & kFlagFirst) ? 0u : 1u;
        uint32_t next_flags = 0;
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          const uint64_t s_desc = smem_desc_join(s_lo + k * s_kstep);
          const uint64_t d0 = smem_desc_join(d_lo + k * d_kstep);
          const uint64_t d1 = smem_desc_join(d_lo + (kOperandTileBytes >> 4) + k * d_kstep);
          if (dsd) {
            umma_f16_pair(tmem_base, s_desc, d0, idesc, accumulate);
            umma_f16_pair(tmem_base + kPAccCols, s_desc, d1, idesc, accumulate);
          } else {
            umma_f16_pair(tmem_base, d0, s_desc, idesc, accumulate);
            umma_f16_pair(tmem_base + kPAccCols, d1, s_desc, idesc, accumulate);
          }
          accumulate = 1u;
          if (k == 1) {
            ready = mbar_test_wait(full_bar(next_stage), next_phase);
            next_flags = stage_flags[next_stage];  // only used if `ready`
          }
        }
        umma_commit_pair(empty_bar(stage), 3);
        if (flags & kFlagLast) {
          umma_commit_pair(tfull_bar, 3);
          tile_phase ^= 1u;
        }
        stage = next_stage;
        phase = next_phase;
        flags = next_flags;
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    // Group g (warps 2..5 / 7..10) drains accumulator g: the output tile of dense tile D_g.
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int group = warp > kPProducerBWarp ? 1 : 0;
    const bool issuer = lane == 0 && (warp == 2 || warp == kPProducerBWarp + 1);
    const uint32_t staging = staging_base + group * kOutStageBytes;
    const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                            static_cast<uint32_t>(group * kPAccCols);
    const uint32_t leader_tempty = map_to_cta(tempty_bar(group), 0);
    uint32_t tile_phase = 0;
    bool ok = true;
    uint16_t* out = static_cast<uint16_t*>(p.out);
    for (int item = pair_id; item < p.num_items && ok; item += num_pairs) {
      const int outer = item / p.inner, inner = item - outer * p.inner;
      MergeWalker w;
      w.init(p, 2 * outer);
      const int tile_row = dsd ? (2 * outer + rank) * kBlk : ((2 * inner + group) * 2 + rank) * kBlk;
      const int tile_col = dsd ? (2 * inner + group) * 2 * kBlk : outer * 2 * kBlk;
      const bool rows_valid = tile_row < p.out_rows;
      const int ncols = min(2 * kBlk, p.out_cols - tile_col);  // may be <= 0 for a missing D1
      if (w.empty()) {
        if (rows_valid && ncols > 0) {
          uint16_t* dst = out + (static_cast<long long>(tile_row) + row) * p.ldc + tile_col;
          const uint4 z = make_uint4(0u, 0u, 0u, 0u);
          for (int c = 0; c < ncols; c += 8) *reinterpret_cast<uint4*>(dst + c) = z;
        }
        continue;
      }
      mbar_wait(tfull_bar, tile_phase, abort_flag);
      epilogue_sync(group);
      if (issuer) epilogue_go[group] = (*abort_flag == 0) ? 1 : 0;
      epilogue_sync(group);
      ok = epilogue_go[group] != 0;
      if (!ok) break;
      tc_fence_after();
      if (rows_valid && ncols > 0)
        drain_to_output(t_addr, 0, ncols, p.fmt, p.epilogue, &tmC, tile_col, tile_row, staging, row, group,
                        0, 1, issuer);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tempty);
      tile_phase ^= 1u;
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
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kPTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) report_status(STK_ERR_DEVICE_TIMEOUT);
}

static int launch_wide(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                       const PairParams& p, cudaStream_t stream) {
  PairDeviceInfo* d = nullptr;
  const int rc = pair_device_info(&d);
  if (rc != STK_OK) return rc;
  static bool opted_in[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return STK_ERR_LAUNCH;
  if (!opted_in[dev]) {
    if (cudaFuncSetAttribute(bsmm_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kWSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return STK_ERR_LAUNCH;
    }
    opted_in[dev] = true;
  }
  const int pairs = p.num_items < d->max_pairs ? p.num_items : d->max_pairs;
  bsmm_wide_kernel<<<2 * pairs, kPThreads, kWSmemBytes, stream>>>(tmA, tmB, tmC, p);
  return cudaGetLastError() == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

}  // namespace stk
