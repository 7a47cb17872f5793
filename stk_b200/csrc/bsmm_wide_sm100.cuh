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
// The epilogue is therefore built to let go of the accumulators as early as possible: every thread
// stores its row straight from registers (32-byte stores, fire and forget), so between two reads of
// tensor memory there is a conversion and nothing to wait for - no staging tile whose previous TMA
// store has to have drained first.
//
// Structure, barriers, work-item table, pacing and the merge of the two block lists are those of
// bsmm_pair_sm100.cuh.
#pragma once
#include "bsmm_pair_sm100.cuh"

namespace stk {

constexpr int kWStages = 4;
#ifndef STK_WIDE_STAGGER
#define STK_WIDE_STAGGER 1
#endif
constexpr bool kWStagger = STK_WIDE_STAGGER != 0;
constexpr int kWStageBytes = 3 * kOperandTileBytes;  // S, D0, D1
constexpr int kWNumBars = 2 * kWStages + 3;          // full, empty, tfull, tempty[2]
constexpr int kWSmemBytes = kWStages * kWStageBytes + kWNumBars * 8 + kWStages * 4 + 32 + 1024;

// One epilogue group moves `ncols` accumulator columns (a multiple of 64) of its TMEM lanes to the
// output: thread = one output row, 64 columns = 128 bytes per step.
__device__ __forceinline__ void drain_rows_direct(uint32_t t_addr, int ncols, int fmt, uint16_t* dst_row) {
  const bool aligned32 = (reinterpret_cast<uintptr_t>(dst_row) & 31u) == 0;
  for (int c = 0; c < ncols; c += 64) {
    uint32_t r0[32], r1[32];
    tmem_ld_32x32(t_addr + c, r0);
    tmem_ld_32x32(t_addr + c + 32, r1);
    tmem_ld_wait();
    uint32_t packed[32];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float a0 = __uint_as_float(r0[2 * i]), a1 = __uint_as_float(r0[2 * i + 1]);
      const float b0 = __uint_as_float(r1[2 * i]), b1 = __uint_as_float(r1[2 * i + 1]);
      if (fmt == STK_BF16) {
        const __nv_bfloat162 va = __floats2bfloat162_rn(a0, a1), vb = __floats2bfloat162_rn(b0, b1);
        packed[i] = *reinterpret_cast<const uint32_t*>(&va);
        packed[16 + i] = *reinterpret_cast<const uint32_t*>(&vb);
      } else {
        const __half2 va = __floats2half2_rn(a0, a1), vb = __floats2half2_rn(b0, b1);
        packed[i] = *reinterpret_cast<const uint32_t*>(&va);
        packed[16 + i] = *reinterpret_cast<const uint32_t*>(&vb);
      }
    }
    uint16_t* dst = dst_row + c;
    if (aligned32) {
#pragma unroll
      for (int v = 0; v < 4; ++v)
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 16 * v),
                     "r"(packed[8 * v]), "r"(packed[8 * v + 1]), "r"(packed[8 * v + 2]), "r"(packed[8 * v + 3]),
                     "r"(packed[8 * v + 4]), "r"(packed[8 * v + 5]), "r"(packed[8 * v + 6]), "r"(packed[8 * v + 7])
                     : "memory");
    } else {
#pragma unroll
      for (int v = 0; v < 8; ++v)
        *reinterpret_cast<uint4*>(dst + 8 * v) =
            make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
    }
  }
}

// kF8: 8-bit float operands (kind::f8f6f4): a stage covers 128 of K, i.e. one sparse block.
template <bool kF8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPThreads, 1)
bsmm_wide_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kWStages * kWStageBytes);
  const uint32_t bars_base = smem_base + kWStages * kWStageBytes;
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
    for (int a = 0; a < 2; ++a) mbar_init(tempty_bar(a), 2 * kPEpilogueWarps);  // the epilogue warps of both CTAs
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
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
  pdl_launch_dependents();
  pdl_wait();  // nothing above read global memory
  const int num_items = p.plan != nullptr ? __ldg(p.plan) * p.inner : p.num_items;

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
      const bool paced = arms && p.pace != nullptr;
      unsigned int round = 0;
      for (int item = pair_id; item < num_items && ok; item += num_pairs, ++round) {
        if (paced && round > 0 && round * static_cast<unsigned int>(num_pairs) > kPaceSlack)
          pace_gate(p.pace, round * static_cast<unsigned int>(num_pairs) - kPaceSlack);
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
            const int my_blk = rank ? blk_b : blk_a;
            const int row0 = my_blk == kNoBlock ? p.zero_coord : my_blk * kBlk;
            mn_elem = mn_major ? 0 : row0;
            k_elem = mn_major ? row0 : 0;
          } else {
            mn_elem = it.inner * 4 * kBlk + rank * kBlk;  // D0; D1 is 256 further
            k_elem = kpos * kBlk;
          }
          constexpr int kStageK = kF8 ? 2 * kBK : kBK;  // K elements per stage
          for (int ks = 0; ks < kBlk / kStageK && ok; ++ks) {
            ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
            if (!ok) break;
            if (arms) {
              stage_flags[stage] = (ks == 0 ? first : 0u) | (ks == kBlk / kStageK - 1 ? last : 0u);
              mbar_arrive_expect_tx(full_bar(stage), 2 * kWStageBytes);
            }
            const uint32_t dst = dst0 + stage * kWStageBytes;
            const uint32_t bar = leader_full0 + 8u * stage;
            load_operand_pair(tm, dst, bar, mn_major, mn_elem, k_elem + ks * kStageK, kF8);
            if (!sparse_side)
              load_operand_pair(tm, dst + kOperandTileBytes, bar, mn_major, mn_elem + 2 * kBlk,
                                k_elem + ks * kStageK, kF8);
            if (++stage == kWStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          first = 0u;
        }
        if (paced) {
          const unsigned int done = atomicAdd(p.pace, 1u) + 1u;
          if (done == static_cast<unsigned int>(num_items)) atomicExch(p.pace, 0u);
        }
      }
      if (arms && ok) {
        if (mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
          stage_flags[stage] = kFlagEnd;
          __threadfence_block();  // the tag before the arrival that completes the phase at once (see the pair kernel)
          mbar_arrive(full_bar(stage));
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA only)
    if (rank == 0 && lane == 0) {
      const uint32_t idesc =
          kF8 ? make_idesc_f8(p.a_mn, p.b_mn, 256, 256) : make_idesc_f16(p.fmt, p.a_mn, p.b_mn, 256, 256);
      const int s_mn = dsd ? p.a_mn : p.b_mn, d_mn = dsd ? p.b_mn : p.a_mn;
      const uint32_t s_lo0 = smem_desc_lo(smem_base, s_mn ? kOperandTileBytes / 2 : 16u);
      const uint32_t d_lo0 = smem_desc_lo(smem_base + kOperandTileBytes, d_mn ? kOperandTileBytes / 2 : 16u);
      constexpr uint32_t kMnStep = (kF8 ? 2u : 1u) * kUmmaK * 128u;  // see bsmm_kernel
      const uint32_t s_kstep = (s_mn ? kMnStep : kUmmaK * 2u) >> 4;
      const uint32_t d_kstep = (d_mn ? kMnStep : kUmmaK * 2u) >> 4;
      int stage = 0;
      uint32_t phase = 0, tile_phase = 0;
      // As in the pair kernel: the next stage's barrier is probed between the MMAs of this one.
      bool ready = false;
      uint32_t flags = 0;
      // The MMAs of one K step (64) of the stage: which = 0 / 1 for one accumulator, 2 for both.
      auto issue = [&](int st, int which, uint32_t accumulate, bool probe, int probe_stage, uint32_t probe_phase,
                       bool& probe_ready, uint32_t& probe_flags) {
        const uint32_t s_lo = s_lo0 + st * (kWStageBytes >> 4);
        const uint32_t d_lo = d_lo0 + st * (kWStageBytes >> 4);
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          const uint64_t s_desc = smem_desc_join(s_lo + k * s_kstep);
          const uint64_t d0 = smem_desc_join(d_lo + k * d_kstep);
          const uint64_t d1 = smem_desc_join(d_lo + (kOperandTileBytes >> 4) + k * d_kstep);
          if (which != 1) {
            if (dsd) umma_pair<kF8>(tmem_base, s_desc, d0, idesc, accumulate);
            else umma_pair<kF8>(tmem_base, d0, s_desc, idesc, accumulate);
          }
          if (which != 0) {
            if (dsd) umma_pair<kF8>(tmem_base + kPAccCols, s_desc, d1, idesc, accumulate);
            else umma_pair<kF8>(tmem_base + kPAccCols, d1, s_desc, idesc, accumulate);
          }
          accumulate = 1u;
          if (probe && k == 1) {
            probe_ready = mbar_test_wait(full_bar(probe_stage), probe_phase);
            probe_flags = stage_flags[probe_stage];  // only used if `probe_ready`
          }
        }
      };
      bool unused_ready = false;
      uint32_t unused_flags = 0;
      bool alive = true;
      while (alive) {
        if (!ready) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) break;
          flags = stage_flags[stage];
        }
        if (flags & kFlagEnd) break;
        if (flags & kFlagFirst) {
          // Head of an item.  The epilogue hands back accumulator 0 first, then accumulator 1: the
          // first stages' MMAs into accumulator 0 are issued while accumulator 1 is still being
          // drained, their MMAs into accumulator 1 follow (a stage is released after both).
          if (!mbar_wait(tempty_bar(0), tile_phase ^ 1u, abort_flag)) break;
          if (!kWStagger && !mbar_wait(tempty_bar(1), tile_phase ^ 1u, abort_flag)) break;
          tc_fence_after();
          uint32_t head_flags[kWStages];
          int n_head = 0, st = stage;
          uint32_t ph = phase, fl = flags;
          while (true) {
            issue(st, kWStagger ? 0 : 2, n_head == 0 ? 0u : 1u, false, 0, 0, unused_ready, unused_flags);
            head_flags[n_head++] = fl;
            if (!kWStagger || (fl & kFlagLast) || n_head == kWStages) break;
            st = st + 1 == kWStages ? 0 : st + 1;
            if (st == 0) ph ^= 1u;
            if (!mbar_wait(full_bar(st), ph, abort_flag)) { alive = false; break; }
            fl = stage_flags[st];
            tc_fence_after();
          }
          if (!alive) break;
          if (!mbar_wait(tempty_bar(1), tile_phase ^ 1u, abort_flag)) break;
          tc_fence_after();
          for (int i = 0; i < n_head; ++i) {
            if (kWStagger) issue(stage, 1, i == 0 ? 0u : 1u, false, 0, 0, unused_ready, unused_flags);
            umma_commit_pair(empty_bar(stage), 3);
            if (head_flags[i] & kFlagLast) {
              umma_commit_pair(tfull_bar, 3);
              tile_phase ^= 1u;
            }
            if (++stage == kWStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          ready = false;
          continue;
        }
        tc_fence_after();
        const int next_stage = stage + 1 == kWStages ? 0 : stage + 1;
        const uint32_t next_phase = stage + 1 == kWStages ? phase ^ 1u : phase;
        uint32_t next_flags = 0;
        issue(stage, 2, 1u, true, next_stage, next_phase, ready, next_flags);
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
    // Accumulator a holds the output tile of dense tile D_a.  Both groups (warps 2..5 / 7..10) drain
    // accumulator 0 first - group g its columns [128 g, 128 g + 128) - and hand it back, then
    // accumulator 1: the MMA issuer starts the next item on accumulator 0 in the meantime.
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int group = warp > kPProducerBWarp ? 1 : 0;
    const bool issuer = lane == 0 && (warp == 2 || warp == kPProducerBWarp + 1);
    const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                            static_cast<uint32_t>(group * kBlk);
    const uint32_t leader_tempty[2] = {map_to_cta(tempty_bar(0), 0), map_to_cta(tempty_bar(1), 0)};
    uint32_t tile_phase = 0;
    bool ok = true;
    uint16_t* out = static_cast<uint16_t*>(p.out);
    for (int item = pair_id; item < num_items && ok; item += num_pairs) {
      const PairItem it = decode_item(p, item);
      MergeWalker w;
      w.init(p, it.r, it.part);
      const bool has_blocks = !w.empty();
      if (has_blocks) {
        mbar_wait(tfull_bar, tile_phase, abort_flag);
        epilogue_sync(group);
        if (issuer) epilogue_go[group] = (*abort_flag == 0) ? 1 : 0;
        epilogue_sync(group);
        ok = epilogue_go[group] != 0;
        if (!ok) break;
        tc_fence_after();
      }
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        const int tile_row = dsd ? (it.r + rank) * kBlk : ((2 * it.inner + a) * 2 + rank) * kBlk;
        const int tile_col = dsd ? (2 * it.inner + a) * 2 * kBlk : it.r * kBlk;
        // (a single-list item: DSD - the other CTA's rows belong to another item; DDS - it owns 128 columns)
        const bool rows_valid = tile_row < p.out_rows && (!dsd || it.part == 0 || rank == 0);
        // this group's share of the tile's columns; none for a missing D1 or the far half of a single column
        const int ncols = min((!dsd && it.part == 1) ? kBlk : 2 * kBlk, p.out_cols - tile_col);
        const int mine = min(kBlk, ncols - group * kBlk);
        uint16_t* dst = out + (static_cast<long long>(tile_row) + row) * p.ldc + tile_col + group * kBlk;
        if (!has_blocks) {
          if (rows_valid) {
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
            for (int c = 0; c < mine; c += 8) *reinterpret_cast<uint4*>(dst + c) = z;
          }
          continue;
        }
        if (rows_valid && mine > 0)
          drain_rows_direct(t_addr + static_cast<uint32_t>(a * kPAccCols), mine, p.fmt, dst);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_tempty[a]);
      }
      if (has_blocks) tile_phase ^= 1u;
    }
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

static int launch_wide(const CUtensorMap& tmA, const CUtensorMap& tmB, const PairParams& params,
                       cudaStream_t stream) {
  PairDeviceInfo* d = nullptr;
  int rc = pair_device_info(&d);
  if (rc != STK_OK) return rc;
  static bool opted_in[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return STK_ERR_LAUNCH;
  if (!opted_in[dev]) {
    if (cudaFuncSetAttribute(bsmm_wide_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kWSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(bsmm_wide_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kWSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return STK_ERR_LAUNCH;
    }
    opted_in[dev] = true;
  }
  PairParams p = params;
  if ((rc = next_pace_counter(&p.pace)) != STK_OK) return rc;
  const int pairs = p.num_items < d->max_pairs ? p.num_items : d->max_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  cfg.blockDim = dim3(kPThreads);
  cfg.dynamicSmemBytes = kWSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = kUseDependentLaunch ? 1 : 0;
  const cudaError_t err = p.in8 ? cudaLaunchKernelEx(&cfg, bsmm_wide_kernel<true>, tmA, tmB, p)
                                : cudaLaunchKernelEx(&cfg, bsmm_wide_kernel<false>, tmA, tmB, p);
  return err == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

}  // namespace stk
