// Block-sparse matmul for sm_100a: SDD, DSD and DDS at 128x128 blocks, fp16/bf16 operands,
// fp32 accumulation in tensor memory.
//
// One persistent, warp-specialised kernel serves the three operations.  Every output tile is
// 128x128; what differs between the operations is only how a tile's K loop is enumerated from
// the blocked CSR-COO metadata and where its two operand tiles live:
//
//   SDD  tile p        : A = lhs rows of block-row r_p,           B = rhs columns of block-col c_p,
//                        K loop over the dense inner dimension.
//   DSD  tile (i, n)   : K loop over the blocks j of block-row i: A = data[blk(j)] (or its transpose),
//                        B = rhs rows col(j)*128.., columns n*128..
//   DDS  tile (m, n)   : K loop over the blocks j of block-column n: A = lhs rows m*128.., columns col(j)*128..,
//                        B = data[blk(j)] (or its transpose).
//
// Operand tiles are fetched by TMA with the 128-byte swizzle into a multi-stage shared-memory ring and
// consumed by tcgen05.mma straight from shared memory.  A transposed operand is never copied: it is a
// different tensor map plus the "MN-major" bit of the instruction / shared-memory descriptors.
//
// Warp roles (192 threads): warp 0 = TMA producer (also walks the metadata), warp 1 = MMA issuer and
// TMEM owner, warps 2..5 = epilogue (TMEM -> registers -> 16-bit -> swizzled staging tile -> TMA
// store).  Two TMEM accumulators let the epilogue of tile t overlap the main loop of tile t+1.
//
// The semantics follow stk/backend/triton_kernels.py of the reference (_sdd_kernel :34-68,
// _dsd_kernel :83-145, _dds_kernel :160-220 and their launchers :222-379).
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/stk_b200.h"
#include "index.cuh"
#include "sm100_ptx.cuh"
#include "status.cuh"

namespace stk {

constexpr int kBlk = 128;                       // sparse block edge = tile edge
constexpr int kBK = 64;                         // K elements per pipeline stage (one 128-byte swizzle row)
constexpr int kUmmaK = 16;                      // K of one tcgen05.mma for 16-bit operands
constexpr int kStages = 6;
constexpr int kOperandTileBytes = kBlk * kBK * 2;  // 16 KiB
constexpr int kStageBytes = 2 * kOperandTileBytes;
constexpr int kThreads = 192;
constexpr int kTmemCols = 256;                  // two 128-column fp32 accumulators
constexpr int kNumBars = 2 * kStages + 4;
constexpr int kSmemBytes =
    kStages * kStageBytes + kBlk * 64 * 2 + kNumBars * 8 + 32 + 1024;  // stages, output staging tile, barriers, slack

enum : int { kModeSDD = 0, kModeDSD = 1, kModeDDS = 2 };

// Optional activation applied to the fp32 accumulator before it is rounded and stored.
// kEpilogueGeluKeep: `out` gets the product itself and the auxiliary tensor GeLU of it (a training
// step needs both).  kEpilogueGeluGrad: `out` = product * GeLU'(auxiliary tensor), the auxiliary
// tensor holding the pre-activations (the backward of GeLU fused into the product that yields the
// gradient of the activations).  The auxiliary tensor has the layout of `out` (SDD only).
enum : int { kEpilogueNone = 0, kEpilogueGelu = 1, kEpilogueGeluKeep = 2, kEpilogueGeluGrad = 3 };

// GeLU in its exact form x * Phi(x) (torch.nn.functional.gelu's default), written as
//   gelu(x) = max(x, 0) - |x| * Phi(-|x|),   Phi(-a) = 2^(-q(a)),
// with q a degree-7 minimax fit of -log2(Phi(-a)) on [0, 5.8] (|error of q| < 5e-6, so the result is
// within 7e-6 relative of the exact value wherever that is not below fp16's smallest subnormal, and
// within 6e-7 absolute everywhere; q keeps growing beyond the fitted range, so the tail goes to
// zero).  Eleven instructions per element, one of them a special-function one: the epilogue warps
// share their schedulers with the TMA producers and the MMA issuer, and the longer forms (erff, or
// erfc as t * P(t) * exp(-z^2) with a reciprocal and an exponential) slowed the main loop down.
// |x| is clamped at 8 inside (Phi(-8) = 6e-16), so that +-infinity give +infinity and -0.
__device__ __forceinline__ float gelu_erf(float x) {
  const float a = fminf(fabsf(x), 8.0f);
  float q = fmaf(1.8287723e-06f, a, -6.149571e-05f);
  q = fmaf(q, a, 0.00092985336f);
  q = fmaf(q, a, -0.008505761f);
  q = fmaf(q, a, 0.053956695f);
  q = fmaf(q, a, 0.45846686f);
  q = fmaf(q, a, 1.1512504f);
  q = fmaf(q, a, 0.9999953f);
  float h;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(h) : "f"(-q));
  return fmaf(-a, h, fmaxf(x, 0.0f));
}

// d/dx of the same GeLU: Phi(x) + x * phi(x), Phi from the same fit, phi(x) = 2^(-x^2 / (2 ln 2)) / sqrt(2 pi).
__device__ __forceinline__ float gelu_erf_grad(float x) {
  const float a = fminf(fabsf(x), 8.0f);
  float q = fmaf(1.8287723e-06f, a, -6.149571e-05f);
  q = fmaf(q, a, 0.00092985336f);
  q = fmaf(q, a, -0.008505761f);
  q = fmaf(q, a, 0.053956695f);
  q = fmaf(q, a, 0.45846686f);
  q = fmaf(q, a, 1.1512504f);
  q = fmaf(q, a, 0.9999953f);
  float h, e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(h) : "f"(-q));                       // Phi(-|x|)
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(a * a * -0.72134752044f));  // exp(-x^2 / 2)
  const float cdf = x < 0.0f ? h : 1.0f - h;
  return fmaf(copysignf(a, x) * 0.3989422804f, e, cdf);
}

// The auxiliary tensor of the epilogues that have one: its tensor map (stores) and its address (loads).
struct EpilogueAux {
  const CUtensorMap* tm;
  const uint16_t* ptr;
};

struct BsmmParams {
  int mode;
  int a_mn;        // 1: A tile is M-contiguous in memory (transposed operand), 0: K-contiguous
  int b_mn;        // 1: B tile is N-contiguous in memory, 0: K-contiguous
  int fmt;         // STK_F16 / STK_BF16: format of the 16-bit operands, and of the output always
  int in8;         // 1: the operands are 8-bit floats (e4m3), both K-major; a stage then holds 128 of K
  int epilogue;    // kEpilogueNone / kEpilogueGelu
  int num_tiles;
  int tiles_inner; // DSD: number of N tiles (n runs fastest); DDS: number of M tiles (m runs fastest)
  int k_steps;     // SDD: ceil(K / 64)
  IndexArray row_idx;       // SDD
  IndexArray col_idx;       // SDD: block column; DSD/DDS: position of block j along K, in blocks
  const int32_t* offsets;   // DSD/DDS: K-loop segment of every block-row / block-column
  const int32_t* blk_idx;   // DSD/DDS: index into data of block j, or nullptr for the identity
  void* out;
  long long ldc;            // DSD/DDS: leading dimension of out in elements
  int out_cols;             // row kernel (bsmm_row_sm100.cuh), DSD: dense columns of the output
  int out_rows;             // row kernel, DDS: dense rows of the output
  int nnz;                  // row kernel, SDD: number of blocks
  int raster_group;         // row kernel, DSD / DDS: lists per tile-order group (see row_tile)
  const void* aux;          // SDD with kEpilogueGeluKeep / kEpilogueGeluGrad: the auxiliary tensor
};

struct TileInfo {
  int tm, tn;   // DSD/DDS tile coordinates (in tiles); SDD: block row / block column
  int j0, j1;   // DSD/DDS: segment of the metadata arrays
  int nk;       // number of 64-wide K steps
};

__device__ __forceinline__ TileInfo tile_info(const BsmmParams& p, int tile) {
  TileInfo t;
  if (p.mode == kModeSDD) {
    t.tm = p.row_idx[tile];
    t.tn = p.col_idx[tile];
    t.j0 = t.j1 = 0;
    t.nk = p.k_steps;
  } else {
    const int outer = tile / p.tiles_inner;
    const int inner = tile - outer * p.tiles_inner;
    if (p.mode == kModeDSD) {
      t.tm = outer;
      t.tn = inner;
      t.j0 = p.offsets[t.tm];
      t.j1 = p.offsets[t.tm + 1];
    } else {
      t.tn = outer;
      t.tm = inner;
      t.j0 = p.offsets[t.tn];
      t.j1 = p.offsets[t.tn + 1];
    }
    t.nk = (p.in8 ? 1 : 2) * (t.j1 - t.j0);  // a block is 128 of K: two stages of 16-bit operands, one of 8-bit
  }
  return t;
}

// One operand tile (128 rows of M or N by 64 of K) into a stage buffer, one TMA instruction.
//   K-major : 2-D box {64 (K), 128 (M/N)} at (k_elem, mn_elem).
//   MN-major: 3-D box {64 (M/N), 64 (K), 2 (groups of 64 M/N)} at (0, k_elem, mn_elem / 64); the two
//             groups land 8 KiB apart, which is the leading byte offset of the UMMA descriptor.
//   8-bit MN-major (bytes8): 128 elements of M/N fill a swizzle row, so the tile is one 2-D box
//             {128 (M/N), 128 (K)} at (mn_elem, k_elem).
__device__ __forceinline__ void load_operand(const CUtensorMap* tm, uint32_t smem_dst, uint32_t bar,
                                             int mn_major, int mn_elem, int k_elem, bool bytes8 = false) {
  if (!mn_major) {
    tma_load_2d(smem_dst, tm, bar, k_elem, mn_elem);
  } else if (bytes8) {
    tma_load_2d(smem_dst, tm, bar, mn_elem, k_elem);
  } else {
    tma_load_3d(smem_dst, tm, bar, 0, k_elem, mn_elem >> 6);
  }
}

constexpr int kOutStageBytes = kBlk * 64 * 2;  // one 128-row x 64-column 16-bit output sub-tile

// Barrier among the 128 threads of one epilogue group (hardware barriers 1 and 2; 0 is __syncthreads).
__device__ __forceinline__ void epilogue_sync(int group) {
  asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory");
}

// One epilogue group (four warps, 128 threads) moves its share of `ncols` accumulator columns (a
// multiple of 64, starting at TMEM column `col0`) to the output: the 64-column sub-tiles `first`,
// `first + step`, ...  `group` names the group's hardware barrier.  TMEM -> registers -> optional activation -> 16-bit -> the group's 128x64
// staging tile in shared memory (128-byte swizzle, conflict-free 16-byte stores) -> one TMA store.
// The two inference forms (product, or GeLU of it), kept apart from the training forms below: folded
// into one template the compiler scheduled this path with 37 more registers and the fused GeLU step
// ran 5 % slower.
__device__ __forceinline__ void drain_to_output_plain(uint32_t t_addr, int col0, int ncols, int fmt,
                                                int epilogue, const CUtensorMap* tmC, int out_x,
                                                int out_y, uint32_t staging, int row, int group,
                                                int first, int step, bool issuer) {
  for (int c = first * 64; c < ncols; c += step * 64) {
    if (issuer) tma_store_wait_read<0>();  // the group's previous store is done reading the tile
    epilogue_sync(group);
    uint32_t r0[32], r1[32];
    tmem_ld_32x32(t_addr + col0 + c, r0);
    tmem_ld_32x32(t_addr + col0 + c + 32, r1);
    tmem_ld_wait();
    uint32_t packed[32];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float a0 = __uint_as_float(r0[2 * i]), a1 = __uint_as_float(r0[2 * i + 1]);
      float b0 = __uint_as_float(r1[2 * i]), b1 = __uint_as_float(r1[2 * i + 1]);
      if (epilogue == kEpilogueGelu) {
        a0 = gelu_erf(a0);
        a1 = gelu_erf(a1);
        b0 = gelu_erf(b0);
        b1 = gelu_erf(b1);
      }
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
    const uint32_t row_addr = staging + row * 128;
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      const uint32_t addr = row_addr + ((ch ^ (row & 7)) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(packed[4 * ch]),
                   "r"(packed[4 * ch + 1]), "r"(packed[4 * ch + 2]), "r"(packed[4 * ch + 3])
                   : "memory");
    }
    fence_proxy_async_smem();
    epilogue_sync(group);
    if (issuer) {
      tma_store_2d(tmC, staging, out_x + c, out_y);
      tma_store_commit();
    }
  }
}

// kEpi: kEpilogueNone covers the two inference forms (`gelu` chooses at run time, one copy of the
// code for both), kEpilogueGeluKeep / kEpilogueGeluGrad are the training forms.
template <int kEpi>
__device__ __forceinline__ void drain_to_output_as(uint32_t t_addr, int col0, int ncols, int fmt,
                                                   bool gelu, const CUtensorMap* tmC, int out_x, int out_y,
                                                   uint32_t staging, int row, int group, int first,
                                                   int step, bool issuer, EpilogueAux aux) {
  for (int c = first * 64; c < ncols; c += step * 64) {
    if (issuer) tma_store_wait_read<0>();  // the group's previous store is done reading the tile
    epilogue_sync(group);
    uint32_t r0[32], r1[32];
    tmem_ld_32x32(t_addr + col0 + c, r0);
    tmem_ld_32x32(t_addr + col0 + c + 32, r1);
    tmem_ld_wait();
    if constexpr (kEpi == kEpilogueGeluGrad) {
      // this thread's 64 pre-activations: 128 contiguous bytes of the auxiliary tensor (SDD: rows of 128)
      const uint4* src = reinterpret_cast<const uint4*>(
          aux.ptr + (static_cast<long long>(out_y) + row) * kBlk + out_x + c);
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        const uint4 w = __ldg(src + v);
        const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float2 pre;
          if (fmt == STK_BF16) pre = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[k]));
          else pre = __half22float2(*reinterpret_cast<const __half2*>(&words[k]));
          const int e = v * 8 + k * 2;  // element index 0..63 within the sub-tile
          uint32_t* r = e < 32 ? r0 : r1;
          const int o = e & 31;
          r[o] = __float_as_uint(__uint_as_float(r[o]) * gelu_erf_grad(pre.x));
          r[o + 1] = __float_as_uint(__uint_as_float(r[o + 1]) * gelu_erf_grad(pre.y));
        }
      }
    }
    // one pass per output tensor: kEpilogueGeluKeep stores the product, then its activation
    constexpr int kPasses = kEpi == kEpilogueGeluKeep ? 2 : 1;
#pragma unroll
    for (int pass = 0; pass < kPasses; ++pass) {
      const bool activate = kEpi == kEpilogueNone ? gelu : pass == 1;
      if (pass == 1) {
        if (issuer) tma_store_wait_read<0>();
        epilogue_sync(group);
      }
      uint32_t packed[32];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float a0 = __uint_as_float(r0[2 * i]), a1 = __uint_as_float(r0[2 * i + 1]);
        float b0 = __uint_as_float(r1[2 * i]), b1 = __uint_as_float(r1[2 * i + 1]);
        if (activate) {
          a0 = gelu_erf(a0);
          a1 = gelu_erf(a1);
          b0 = gelu_erf(b0);
          b1 = gelu_erf(b1);
        }
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
      const uint32_t row_addr = staging + row * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint32_t addr = row_addr + ((ch ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(packed[4 * ch]),
                     "r"(packed[4 * ch + 1]), "r"(packed[4 * ch + 2]), "r"(packed[4 * ch + 3])
                     : "memory");
      }
      fence_proxy_async_smem();
      epilogue_sync(group);
      if (issuer) {
        tma_store_2d(pass == 1 ? aux.tm : tmC, staging, out_x + c, out_y);
        tma_store_commit();
      }
    }
  }
}

// kTrain: whether the two training epilogues can occur in this kernel instantiation; the kernels are
// compiled twice so that the inference forms keep the short epilogue code.
template <bool kTrain = false>
__device__ __forceinline__ void drain_to_output(uint32_t t_addr, int col0, int ncols, int fmt,
                                                int epilogue, const CUtensorMap* tmC, int out_x,
                                                int out_y, uint32_t staging, int row, int group,
                                                int first, int step, bool issuer,
                                                EpilogueAux aux = EpilogueAux{nullptr, nullptr}) {
  // the epilogue kind is a compile-time parameter of the body: the plain and GeLU forms keep their
  // short code whatever the two training forms need
  if constexpr (!kTrain) {
    drain_to_output_plain(t_addr, col0, ncols, fmt, epilogue, tmC, out_x, out_y, staging, row, group, first,
                          step, issuer);
  } else if (epilogue == kEpilogueGeluKeep) {
    drain_to_output_as<kEpilogueGeluKeep>(t_addr, col0, ncols, fmt, false, tmC, out_x, out_y, staging, row,
                                          group, first, step, issuer, aux);
  } else {
    drain_to_output_as<kEpilogueGeluGrad>(t_addr, col0, ncols, fmt, false, tmC, out_x, out_y, staging, row,
                                          group, first, step, issuer, aux);
  }
}

// kF8: the operands are 8-bit floats (tcgen05.mma kind::f8f6f4, 32 of K per instruction); the byte
// geometry of a stage is the same (128 rows of 128 bytes per operand, four MMAs), only the K it covers
// doubles.
template <bool kTrain, bool kF8 = false>
__global__ void __launch_bounds__(kThreads, 1)
bsmm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX,
            const BsmmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);

  const uint32_t staging = smem_base + kStages * kStageBytes;  // 128 x 64 output tile, 1024-aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + kOutStageBytes);
  const uint32_t bars_base = staging + kOutStageBytes;
  auto full_bar = [&](int s) { return bars_base + 8u * s; };
  auto empty_bar = [&](int s) { return bars_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bars_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bars_base + 8u * (2 * kStages + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epilogue_go = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
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
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
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
    int stage = 0;
    uint32_t phase = 0;
    int ok = 1;
    auto produce = [&](int a_mn_elem, int a_k_elem, int b_mn_elem, int b_k_elem) {
      if (lane == 0) {
        if (mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kOperandTileBytes;
          mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
          load_operand(&tmA, a_dst, full_bar(stage), p.a_mn, a_mn_elem, a_k_elem, kF8);
          load_operand(&tmB, b_dst, full_bar(stage), p.b_mn, b_mn_elem, b_k_elem, kF8);
        } else {
          ok = 0;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1u;
      }
    };
    constexpr int kStageK = kF8 ? 2 * kBK : kBK;        // K elements per stage
    constexpr int kStagesPerBlock = kBlk / kStageK;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
      const TileInfo t = tile_info(p, tile);
      if (p.mode == kModeSDD) {
        for (int ks = 0; ks < t.nk && ok; ++ks)
          produce(t.tm * kBlk, ks * kStageK, t.tn * kBlk, ks * kStageK);
      } else {
        for (int jb = t.j0; jb < t.j1 && ok; jb += 32) {
          // The warp fetches the metadata of up to 32 blocks at once, then replays it.
          const int j = jb + lane;
          int my_col = 0, my_blk = 0;
          if (j < t.j1) {
            my_col = p.col_idx[j];
            my_blk = p.blk_idx ? p.blk_idx[j] : j;
          }
          const int cnt = min(32, t.j1 - jb);
          for (int i = 0; i < cnt && ok; ++i) {
            const int col = __shfl_sync(0xffffffffu, my_col, i);
            const int blk = __shfl_sync(0xffffffffu, my_blk, i);
            for (int ks = 0; ks < kStagesPerBlock && ok; ++ks) {
              if (p.mode == kModeDSD) {
                // sparse A, dense B
                const int a_mn_elem = p.a_mn ? 0 : blk * kBlk;
                const int a_k_elem = p.a_mn ? blk * kBlk + ks * kStageK : ks * kStageK;
                produce(a_mn_elem, a_k_elem, t.tn * kBlk, col * kBlk + ks * kStageK);
              } else {
                // dense A, sparse B
                const int b_mn_elem = p.b_mn ? 0 : blk * kBlk;
                const int b_k_elem = p.b_mn ? blk * kBlk + ks * kStageK : ks * kStageK;
                produce(t.tm * kBlk, col * kBlk + ks * kStageK, b_mn_elem, b_k_elem);
              }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = kF8 ? make_idesc_f8(p.a_mn, p.b_mn, kBlk) : make_idesc_f16(p.fmt, p.a_mn, p.b_mn, kBlk);
      // Descriptor low words of stage 0 and their step per 16 elements of K and per stage.
      const uint32_t a_lo0 = smem_desc_lo(smem_base, p.a_mn ? kOperandTileBytes / 2 : 16u);
      const uint32_t b_lo0 = smem_desc_lo(smem_base + kOperandTileBytes, p.b_mn ? kOperandTileBytes / 2 : 16u);
      // bytes between the operand slices of two consecutive MMAs: 32 bytes along a K-major row, or the
      // rows of one MMA's K (16 for 16-bit, 32 for 8-bit operands) x 128 bytes in an MN-major tile
      constexpr uint32_t kMnStep = (kF8 ? 2u : 1u) * kUmmaK * 128u;
      const uint32_t a_kstep = (p.a_mn ? kMnStep : kUmmaK * 2u) >> 4;
      const uint32_t b_kstep = (p.b_mn ? kMnStep : kUmmaK * 2u) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // The tensor pipe does not run ahead of this thread: every cycle it stalls between two MMAs
      // (a barrier poll whose result it needs, a metadata load) is an idle tensor cycle.  So the
      // next stage's barrier is probed (not waited for) between the MMAs of the current stage, and
      // the next tile's metadata is fetched while the current tile's MMAs are issued.
      bool ready = false;
      TileInfo t_next = {};
      if (static_cast<int>(blockIdx.x) < p.num_tiles) t_next = tile_info(p, blockIdx.x);
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        const TileInfo t = t_next;
        if (tile + static_cast<int>(gridDim.x) < p.num_tiles) t_next = tile_info(p, tile + gridDim.x);
        if (t.nk == 0) continue;  // the epilogue writes zeros; no accumulator is used
        ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kBlk);
        uint32_t accumulate = 0;
        for (int ks = 0; ks < t.nk; ++ks) {
          if (!ready) {
            ok = mbar_wait(full_bar(stage), phase, abort_flag);
            if (!ok) break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * (kStageBytes >> 4);
          const uint32_t b_lo = b_lo0 + stage * (kStageBytes >> 4);
          const int next_stage = stage + 1 == kStages ? 0 : stage + 1;
          const uint32_t next_phase = stage + 1 == kStages ? phase ^ 1u : phase;
          umma<kF8>(d_tmem, smem_desc_join(a_lo), smem_desc_join(b_lo), idesc, accumulate);
          umma<kF8>(d_tmem, smem_desc_join(a_lo + a_kstep), smem_desc_join(b_lo + b_kstep), idesc, 1u);
          ready = mbar_test_wait(full_bar(next_stage), next_phase);
          umma<kF8>(d_tmem, smem_desc_join(a_lo + 2 * a_kstep), smem_desc_join(b_lo + 2 * b_kstep), idesc, 1u);
          umma<kF8>(d_tmem, smem_desc_join(a_lo + 3 * a_kstep), smem_desc_join(b_lo + 3 * b_kstep), idesc, 1u);
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
      const TileInfo t = tile_info(p, tile);
      uint16_t* out_row;
      if (p.mode == kModeSDD) {
        out_row = static_cast<uint16_t*>(p.out) + static_cast<long long>(tile) * (kBlk * kBlk) +
                  row * kBlk;
      } else {
        out_row = static_cast<uint16_t*>(p.out) +
                  (static_cast<long long>(t.tm) * kBlk + row) * p.ldc +
                  static_cast<long long>(t.tn) * kBlk;
      }
      uint4* out_vec = reinterpret_cast<uint4*>(out_row);
      if (t.nk == 0) {
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < kBlk / 8; ++i) out_vec[i] = z;
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
                              static_cast<uint32_t>(acc * kBlk);
      // TMEM -> registers -> 16-bit -> swizzled staging tile -> TMA store, 64 columns at a time
      if (p.mode == kModeSDD)
        drain_to_output<kTrain>(t_addr, 0, kBlk, p.fmt, p.epilogue, &tmC, 0, tile * kBlk, staging, row,
                                0, 0, 1, issuer, EpilogueAux{&tmX, static_cast<const uint16_t*>(p.aux)});
      else
        drain_to_output(t_addr, 0, kBlk, p.fmt, p.epilogue, &tmC, t.tn * kBlk, t.tm * kBlk, staging,
                        row, 0, 0, 1, issuer);
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
    // Something never arrived.  Give copies and MMAs still in flight time to land before the
    // shared and tensor memory they target is released, then report.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) report_status(STK_ERR_DEVICE_TIMEOUT);
}

// ====================================================================== host side

static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

// cuTensorMapEncodeTiled wants a CUDA context current on the calling thread.  A thread that has made no runtime
// call that binds one yet (a freshly started autograd worker whose first work is one of these products: its
// allocations came out of a cache) gets CUDA_ERROR_INVALID_CONTEXT; binding the thread's device's primary
// context and encoding again is what any later runtime call would have done.
template <typename... Args>
static CUresult encode_tiled(PFN_cuTensorMapEncodeTiled_v12000 fn, Args... args) {
  CUresult r = fn(args...);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) r = fn(args...);
  }
  return r;
}

// The driver's answer to the last tensor-map encoding of this thread (a CUresult; 0 = success), for
// stk_b200_last_tensor_map_error.
static thread_local int g_last_encode_result = 0;

// Tensor map of a 2-D tensor of 16-bit elements (STK_F16 / STK_BF16) or bytes (STK_F8E4M3): `inner`
// contiguous elements per row, `outer` rows, `ld` elements between rows; boxes of 128 bytes x
// box_outer with the 128-byte swizzle.
static int encode_map(CUtensorMap* tm, const void* base, int dtype, int64_t inner, int64_t outer,
                      int64_t ld, int box_outer) {
  PFN_cuTensorMapEncodeTiled_v12000 fn = get_encode_fn();
  if (fn == nullptr) return STK_ERR_DRIVER;
  const bool bytes = dtype == STK_F8E4M3;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * (bytes ? 1u : 2u)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(bytes ? 2 * kBK : kBK), static_cast<cuuint32_t>(box_outer)};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult r =
      encode_tiled(fn, tm, bytes ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                   : dtype == STK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
         2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  g_last_encode_result = static_cast<int>(r);
  return r == CUDA_SUCCESS ? STK_OK : STK_ERR_TENSOR_MAP;
}

// Tensor map of an operand whose contiguous dimension is M/N (`mn` elements per row, `k` rows, `ld`
// elements between rows), described in three dimensions {64, k, mn/64} with boxes {64, 64, 2}.
static int encode_map(CUtensorMap* tm, const void* base, int dtype, int64_t inner, int64_t outer,
                      int64_t ld, int box_outer);
static int encode_map_mn_major(CUtensorMap* tm, const void* base, int dtype, int64_t mn, int64_t k,
                               int64_t ld) {
  // bytes: 128 elements of M/N are one swizzle row, the tile is a plain 2-D box {128 M/N, 128 K}
  if (dtype == STK_F8E4M3) return encode_map(tm, base, dtype, mn, k, ld, kBlk);
  PFN_cuTensorMapEncodeTiled_v12000 fn = get_encode_fn();
  if (fn == nullptr) return STK_ERR_DRIVER;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(kBK), static_cast<cuuint64_t>(k),
                              static_cast<cuuint64_t>(mn / kBK)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2u, static_cast<cuuint64_t>(kBK) * 2u};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(kBK), 2u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUresult r =
      encode_tiled(fn, tm, dtype == STK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
         3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  g_last_encode_result = static_cast<int>(r);
  return r == CUDA_SUCCESS ? STK_OK : STK_ERR_TENSOR_MAP;
}

// Dense operand with logical shape [mn, k] (the A convention: rows = M; for B pass mn = N):
//   k_contig = 1: K is contiguous in memory  -> K-major tile, box {64 K, 128 MN}
//   k_contig = 0: M/N is contiguous          -> MN-major tile, box {64 MN, 64 K, 2}
static int encode_dense(CUtensorMap* tm, const void* base, int dtype, int64_t mn, int64_t k,
                        int64_t ld, int k_contig) {
  return k_contig ? encode_map(tm, base, dtype, k, mn, ld, kBlk)
                  : encode_map_mn_major(tm, base, dtype, mn, k, ld);
}

// Sparse values viewed as a [nnz*128, 128] row-major tensor.
//   as_stored_k_contig = 1: the block's columns are the K of the product -> K-major
//   as_stored_k_contig = 0: the block's columns are the M/N of the product -> MN-major
static int encode_sparse(CUtensorMap* tm, const void* data, int dtype, int64_t nnz, int k_contig) {
  return k_contig ? encode_map(tm, data, dtype, kBlk, nnz * kBlk, kBlk, kBlk)
                  : encode_map_mn_major(tm, data, dtype, kBlk, nnz * kBlk, kBlk);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct DeviceInfo {
  int sms = 0;
  bool smem_opted_in = false;
};

static int device_info(DeviceInfo** out) {
  static DeviceInfo infos[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return STK_ERR_LAUNCH;
  DeviceInfo& d = infos[dev];
  if (d.sms == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return STK_ERR_LAUNCH;
    d.sms = sms;
  }
  if (!d.smem_opted_in) {
    if (cudaFuncSetAttribute(bsmm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
            cudaSuccess ||
        cudaFuncSetAttribute(bsmm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(bsmm_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return STK_ERR_LAUNCH;
    }
    d.smem_opted_in = true;
  }
  *out = &d;
  return STK_OK;
}

// Launch with programmatic stream serialization: the kernel's set-up (barriers, TMEM allocation) may
// overlap the tail of the kernel before it in the stream; it waits (griddepcontrol.wait) before its
// first global read.
template <typename... Params, typename... Args>
static cudaError_t launch_dependent(void (*kernel)(Params...), int grid, int block, int smem_bytes,
                                    cudaStream_t stream, const Args&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(static_cast<unsigned>(block));
  cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// tmX: tensor map of the auxiliary tensor of the SDD epilogues that have one (else any valid map).
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                  const CUtensorMap& tmX, const BsmmParams& p, cudaStream_t stream) {
  DeviceInfo* d = nullptr;
  const int rc = device_info(&d);
  if (rc != STK_OK) return rc;
  const int grid = p.num_tiles < d->sms ? p.num_tiles : d->sms;
  if (p.in8 && p.epilogue >= kEpilogueGeluKeep) return STK_ERR_BAD_DIMS;
  const cudaError_t err =
      p.in8 ? launch_dependent(bsmm_kernel<false, true>, grid, kThreads, kSmemBytes, stream, tmA, tmB, tmC, tmX, p)
      : p.epilogue >= kEpilogueGeluKeep
          ? launch_dependent(bsmm_kernel<true>, grid, kThreads, kSmemBytes, stream, tmA, tmB, tmC, tmX, p)
          : launch_dependent(bsmm_kernel<false>, grid, kThreads, kSmemBytes, stream, tmA, tmB, tmC, tmX, p);
  return err == cudaSuccess ? STK_OK : STK_ERR_LAUNCH;
}

static int check_dense(const void* ptr, int64_t ld, int64_t min_ld) {
  if (ptr == nullptr) return STK_ERR_NULL_POINTER;
  if (!aligned16(ptr) || ld < min_ld || (ld % 8) != 0) return STK_ERR_BAD_LAYOUT;
  return STK_OK;
}

}  // namespace stk

