// NVFP4 path of the value MLP: second layer + scalar head with 4-bit operands and block scales.
//
// NVFP4 = E2M1 elements (1 sign, 2 exponent, 1 mantissa bit; magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6), one unsigned
// E4M3 scale factor per block of 16 consecutive K elements, and one float32 scale per tensor:
//     x[k] ~ e2m1[k] * sf[k / 16] * tensor_scale.
// The tensor core multiplies the block scales in (tcgen05.mma kind::mxf4nvf4, block16): one instruction covers
// 128 x 256 x 64 and reads, besides the two shared-memory operands, 4 scale factors per A row and per B row from
// tensor memory.  The two tensor scales are folded into the epilogue's per-column factor.
//
// Layouts.  Elements: two per byte, even K in the low nibble, row-major [rows, K / 2] bytes; a 128-byte row of a
// TMA box (128-byte swizzle) therefore holds one K-block of 256 elements = four MMA steps.  Scale factors: the
// tensor core wants, per MMA step and per group of 128 rows, a 512-byte chunk in which row r = r0 + 32 * r1 keeps
// its four factors at byte r0 * 16 + r1 * 4 (32 "lanes" of 16 bytes: what tcgen05.cp 32x128b.warpx4 copies from
// shared into tensor memory, lane r0, 32-bit column r1, replicated over the four lane quadrants).  Global memory
// holds them in the order the kernel consumes them, so that one bulk copy per pipeline stage brings a K-block's
// factors: A: [row tile of 128][K-block][step 0..3][512 B]; B: [column chunk of 128][K-block][step 0..3][512 B].
//
// First-layer activations are produced in e4m3 by the fused layer-1 kernel and re-quantised to NVFP4 by
// k_quant_h1_nvfp4 (block maximum -> E4M3 scale, elements -> E2M1, written in the layouts above).
//
// Tensor memory: the factors need columns of their own, so two accumulators of 256 columns (the scheme of the 8- and
// 16-bit kernels) do not fit the 512.  A single 256-column accumulator cannot overlap its epilogue with the next tile's
// MMAs and measured 1.85 PFLOP/s; the kernel therefore works on 128 x 128 tiles with two accumulators of 128 columns.
//
// What bounds these kernels is not the tensor core but operand traffic from L2: streaming both operands per 128 x 128
// tile is 9 KB per million multiply-adds (the e4m3 CTA-pair kernel needs 8) and measured 0.8 ms for layer 2, no
// faster than e4m3.  With 4-bit operands a whole row tile of A (128 rows x K = 1024: 64 KB, plus 8 KB of factors) fits
// shared memory, so it is loaded ONCE per row tile and kept for all column chunks, double-buffered so that the next
// row tile arrives while this one is multiplied; only the weights stream (16 KB + 2 KB of factors per stage).  A's
// factors stay in tensor memory for the row tile as well.  Columns: 2 x 128 accumulators, 2 x 64 for A's factors,
// 4 x 16 for the weight stages' factors.
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mgbs.h"
#include "mgbs_nvfp4.cuh"
#include "mgbs_tc.cuh"

namespace mgbs {

constexpr int F4_BK = 256;                   // elements per 128-byte K-block row
constexpr int F4_STEPS = 4;                  // MMA steps (64 elements) per K-block
constexpr int F4_BN = 128;                   // accumulator columns per tile
constexpr int F4_MAX_KB = 4;                 // K-blocks of a resident A tile (K <= 1024)
constexpr int F4_B_BYTES = F4_BN * 128;      // 16 KB: 128 weight rows x one K-block
constexpr int F4_SFA_BYTES = F4_STEPS * 512;             // 2 KB per K-block
constexpr int F4_SFB_BYTES = F4_STEPS * 512;             // 2 KB per K-block
constexpr int F4_A_BUF = F4_MAX_KB * (A_BYTES + F4_SFA_BYTES);  // 72 KB: data of all K-blocks, then their factors
constexpr int F4_STAGE_BYTES = F4_B_BYTES + F4_SFB_BYTES;       // 18 KB
constexpr int F4_STAGES = 4;
constexpr int F4_THREADS = 192;              // TMA warp, MMA warp, four epilogue warps
constexpr int F4_SMEM = 2 * F4_A_BUF + F4_STAGES * F4_STAGE_BYTES + 1024 + 512;
constexpr uint32_t F4_SFA_BASE = 2 * F4_BN;                       // A's factors: 2 buffers x 64 columns
constexpr uint32_t F4_SFB_BASE = F4_SFA_BASE + 2 * 16 * F4_MAX_KB; // weight stages' factors: 4 x 16 columns

// Instruction descriptor of kind::mxf4nvf4: A and B format E2M1 (code 1, bits 7-9 / 10-12), both K-major, N >> 3 in
// bits 17-22, scale format UE4M3 (bit 23 = 0), M >> 4 in bits 24-28, scale-factor ids 0, K = 64 (bit 31 = 0).
constexpr uint32_t kIdescNvfp4 = (1u << 7) | (1u << 10) | ((uint32_t)(F4_BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void tc_mma_nvfp4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t sfa_tmem,
                                             uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(kIdescNvfp4), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// Shared-memory descriptor of one 512-byte scale-factor chunk: 32 rows of 16 bytes, no swizzle, 8-row groups 128
// bytes apart (stride byte offset 128 >> 4 = 8), descriptor version 1.
__device__ __forceinline__ uint64_t make_desc_sf(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3fffu) | (8ull << 32) | (1ull << 46);
}

// 32 lanes x 128 bits from shared memory into 4 tensor-memory columns, replicated into all four lane quadrants
__device__ __forceinline__ void tc_cp_sf(uint32_t dst_tmem, uint64_t src_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(dst_tmem), "l"(src_desc) : "memory");
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// q[row] (+)= sum_n relu(acc[row, n] * col_scale[n] + bias[n]) * w_out[n],   acc = (A * sfA) (B * sfB)^T
__global__ void __launch_bounds__(F4_THREADS, 1)
k_mlp_head_nvfp4(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Nvfp4HeadArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* a_buf = smem;                         // 2 x 72 KB
  uint8_t* b_ring = smem + 2 * F4_A_BUF;         // 4 x 18 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(b_ring + F4_STAGES * F4_STAGE_BYTES);
  // bars: b_full[S], b_empty[S], a_full[2], a_empty[2], tmem_full[2], tmem_empty[2], drain; then the tmem base word
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * F4_STAGES + 9);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (F4_STAGES + s); };
  auto afull_bar = [&](int b) { return bar0 + 8u * (2 * F4_STAGES + b); };
  auto aempty_bar = [&](int b) { return bar0 + 8u * (2 * F4_STAGES + 2 + b); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * F4_STAGES + 4 + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * F4_STAGES + 6 + b); };
  const uint32_t drain_bar = bar0 + 8u * (2 * F4_STAGES + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int64_t rows = (int64_t)(*g.count_dev);
  if (rows > g.row_limit) rows = g.row_limit;
  if (rows < 0) rows = 0;
  const int num_mtiles = (int)((rows + BM - 1) / BM);
  const int n_chunks = g.n_total / F4_BN;
  const int k_blocks = g.k_total / F4_BK;  // <= F4_MAX_KB (checked by the launcher)

  if (threadIdx.x == 0) {
    for (int s = 0; s < F4_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(afull_bar(b), 1); mbar_init(aempty_bar(b), 1);
      mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 4);
    }
    mbar_init(drain_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_base_slot);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t a_it = 0;   // row tiles whose A load has been issued
      bool ok = true;
      // one row tile of A: K-blocks of 16 KB through the tensor map, then the tile's factors as one contiguous copy
      auto load_a = [&](int mt) -> bool {
        const uint32_t ab = a_it & 1u;
        if (!mbar_wait(aempty_bar(ab), ((a_it >> 1) & 1u) ^ 1u, g.err, ERR_WAIT_EMPTY)) return false;
        const uint32_t dst = smem_u32(a_buf + ab * F4_A_BUF);
        mbar_expect_tx(afull_bar(ab), (uint32_t)k_blocks * (A_BYTES + F4_SFA_BYTES));
        for (int kb = 0; kb < k_blocks; ++kb) tma_load_2d(dst + kb * A_BYTES, &tmA, kb * 128, mt * BM, afull_bar(ab));
        bulk_load(dst + F4_MAX_KB * A_BYTES, g.sfa + (int64_t)mt * k_blocks * F4_SFA_BYTES, (uint32_t)k_blocks * F4_SFA_BYTES,
                  afull_bar(ab));
        ++a_it;
        return true;
      };
      if ((int)blockIdx.x < num_mtiles) ok = load_a(blockIdx.x);
      for (int mt = blockIdx.x; mt < num_mtiles && ok; mt += gridDim.x) {
        for (int nc = 0; nc < n_chunks && ok; ++nc) {
          // the next row tile's A goes out once this tile's weights are on their way: by then the MMAs of the
          // previous row tile have retired and released the buffer it takes, so this thread does not stall
          if (nc == (n_chunks > 1 ? 1 : 0) && mt + (int)gridDim.x < num_mtiles) ok = load_a(mt + gridDim.x);
          for (int kb = 0; kb < k_blocks && ok; ++kb) {
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, g.err, ERR_WAIT_EMPTY)) { ok = false; break; }
            const uint32_t sb = smem_u32(b_ring + stage * F4_STAGE_BYTES);
            mbar_expect_tx(full_bar(stage), F4_STAGE_BYTES);
            tma_load_2d(sb, &tmB, kb * 128, nc * F4_BN, full_bar(stage));   // x in bytes: 128 per K-block
            bulk_load(sb + F4_B_BYTES, g.sfb + (((int64_t)(nc >> 1) * k_blocks + kb) * 2 + (nc & 1)) * F4_SFB_BYTES, F4_SFB_BYTES,
                      full_bar(stage));
            if (++stage == F4_STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_it = 0, a_it = 0;
      bool ok = true;
      for (int mt = blockIdx.x; mt < num_mtiles && ok; mt += gridDim.x, ++a_it) {
        const uint32_t ab = a_it & 1u;
        if (!mbar_wait(afull_bar(ab), (a_it >> 1) & 1u, g.err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(a_buf + ab * F4_A_BUF);
        const uint32_t sfa_t = tmem_base + F4_SFA_BASE + ab * (16u * F4_MAX_KB);
        // A's factors for the whole row tile: 4 columns per MMA step
        for (int kb = 0; kb < k_blocks; ++kb)
#pragma unroll
          for (int k = 0; k < F4_STEPS; ++k)
            tc_cp_sf(sfa_t + 16u * kb + 4u * k, make_desc_sf(sa + F4_MAX_KB * A_BYTES + (uint32_t)(kb * F4_STEPS + k) * 512u));
        for (int nc = 0; nc < n_chunks && ok; ++nc, ++acc_it) {
          const uint32_t b = acc_it & 1u;
          if (!mbar_wait(tempty_bar(b), ((acc_it >> 1) & 1u) ^ 1u, g.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + b * F4_BN;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, g.err, ERR_WAIT_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sb = smem_u32(b_ring + stage * F4_STAGE_BYTES);
            const uint32_t sfb_t = tmem_base + F4_SFB_BASE + (uint32_t)stage * 16u;
#pragma unroll
            for (int k = 0; k < F4_STEPS; ++k) tc_cp_sf(sfb_t + 4u * k, make_desc_sf(sb + F4_B_BYTES + 512u * k));
            const uint64_t adesc = make_desc_sw128(sa + kb * A_BYTES);
            const uint64_t bdesc = make_desc_sw128(sb);
#pragma unroll
            for (int k = 0; k < F4_STEPS; ++k) {
              // one step = 64 elements = 32 bytes inside the swizzle row: +2 in (address >> 4)
              tc_mma_nvfp4(d_tmem, adesc + 2u * k, bdesc + 2u * k, sfa_t + 16u * kb + 4u * k, sfb_t + 4u * k, (kb | k) != 0 ? 1u : 0u);
            }
            tc_commit(empty_bar(stage));
            if (++stage == F4_STAGES) { stage = 0; phase ^= 1u; }
          }
          if (ok) tc_commit(tfull_bar(b));
        }
        if (ok) tc_commit(aempty_bar(ab));  // every MMA that read this A buffer has retired when this arrives
      }
      tc_commit(drain_bar);
      mbar_wait(drain_bar, 0, g.err, ERR_WAIT_DRAIN);
    }
  } else {
    const int quad = warp & 3;            // TMEM lane quadrant this warp may read
    uint32_t acc_it = 0;
    bool ok = true;
    for (int mt = blockIdx.x; mt < num_mtiles && ok; mt += gridDim.x) {
      const int64_t row = (int64_t)mt * BM + quad * 32 + lane;
      const bool row_ok = row < rows;
      float rowsum = 0.f;
      for (int nc = 0; nc < n_chunks && ok; ++nc, ++acc_it) {
        const uint32_t b = acc_it & 1u;
        if (!mbar_wait(tfull_bar(b), (acc_it >> 1) & 1u, g.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + b * F4_BN;
#pragma unroll 1
        for (int c0 = 0; c0 < F4_BN; c0 += 32) {
          uint32_t v[32];
          tc_ld32(taddr + c0, v);
          tc_wait_ld();
          const int n0 = nc * F4_BN + c0;
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 bq = __ldg(reinterpret_cast<const float4*>(g.bias + n0) + j4);
            const float4 wq = __ldg(reinterpret_cast<const float4*>(g.w_out + n0) + j4);
            const float4 cq = __ldg(reinterpret_cast<const float4*>(g.col_scale + n0) + j4);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4]), cq.x, bq.x), 0.f), wq.x, rowsum);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4 + 1]), cq.y, bq.y), 0.f), wq.y, rowsum);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4 + 2]), cq.z, bq.z), 0.f), wq.z, rowsum);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4 + 3]), cq.w, bq.w), 0.f), wq.w, rowsum);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(b));
      }
      if (row_ok && ok) {
        if (g.accumulate_q) g.out_q[row] += rowsum;
        else g.out_q[row] = rowsum;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// The same head with 256-column accumulator tiles.
//
// What bounds the kernel above is not the tensor core but the one thread that feeds it: per K-block it waits on a
// barrier, copies the weight factors into tensor memory, issues four MMAs and commits - several hundred cycles -
// while four 128 x 128 x 64 MMAs at the FP4 rate keep the tensor core busy for only 256.  Here an MMA covers 256
// columns (512 cycles per K-block), and the factor copies move to a thread of their own that signals the MMA thread
// through one barrier per stage, so the MMA thread's loop is a wait, four MMAs and a commit.  The price is tensor
// memory: 256 accumulator columns + 64 for A's factors + 4 x 32 for the weight stages' factors leave no room for a
// second accumulator, so the epilogue (sixteen warps, four per lane quadrant) does not overlap the MMAs of the next
// chunk; and shared memory: four weight stages of 36 KB leave room for one A tile, whose K-blocks are therefore
// released one by one during the last column chunk and refilled for the next row tile behind the MMAs.
// Warps: 0 = TMA, 1 = MMA + TMEM owner, 2 = factor copies, 4..19 = epilogue.
// ------------------------------------------------------------------------------------------------
constexpr int F4W_BN = 256;
constexpr int F4W_B_BYTES = F4W_BN * 128;                    // 32 KB: 256 weight rows x one K-block
constexpr int F4W_SFB_BYTES = 2 * F4_STEPS * 512;            // 4 KB: two groups of 128 weight rows
constexpr int F4W_STAGE_BYTES = F4W_B_BYTES + F4W_SFB_BYTES;  // 36 KB
constexpr int F4W_STAGES = 4;
constexpr int F4W_A_BUF = F4_MAX_KB * (A_BYTES + F4_SFA_BYTES);  // 72 KB
constexpr int F4W_THREADS = 640;                             // 4 service warps + 16 epilogue warps
constexpr int F4W_SMEM = F4W_A_BUF + F4W_STAGES * F4W_STAGE_BYTES + 1024 + 2048;
constexpr uint32_t F4W_SFA_BASE = F4W_BN;                         // 64 columns: 16 per K-block
constexpr uint32_t F4W_SFB_BASE = F4W_SFA_BASE + 16 * F4_MAX_KB;  // 4 stages x 32 columns
constexpr uint32_t kIdescNvfp4W = (1u << 7) | (1u << 10) | ((uint32_t)(F4W_BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void tc_mma_nvfp4_w(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t sfa_tmem,
                                               uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(kIdescNvfp4W), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

__global__ void __launch_bounds__(F4W_THREADS, 1)
k_mlp_head_nvfp4_wide(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Nvfp4HeadArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* a_buf = smem;                      // 4 x 16 KB of data, then 4 x 2 KB of factors
  uint8_t* b_ring = smem + F4W_A_BUF;         // 4 x 36 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(b_ring + F4W_STAGES * F4W_STAGE_BYTES);
  // bars: b_full[4], b_empty[4], sf_ready[4], a_full[4], a_empty[4], t_full, t_empty, drain; the tmem base word;
  // 3 x 128 floats through which the four column quarters of the epilogue meet
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 23);
  float* part = reinterpret_cast<float*>(bars + 24);
  const uint32_t bar0 = smem_u32(bars);
  auto bfull_bar = [&](int s) { return bar0 + 8u * s; };
  auto bempty_bar = [&](int s) { return bar0 + 8u * (4 + s); };
  auto sfready_bar = [&](int s) { return bar0 + 8u * (8 + s); };
  auto afull_bar = [&](int kb) { return bar0 + 8u * (12 + kb); };
  auto aempty_bar = [&](int kb) { return bar0 + 8u * (16 + kb); };
  const uint32_t tfull_bar = bar0 + 8u * 20, tempty_bar = bar0 + 8u * 21, drain_bar = bar0 + 8u * 22;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int64_t rows = (int64_t)(*g.count_dev);
  if (rows > g.row_limit) rows = g.row_limit;
  if (rows < 0) rows = 0;
  const int num_mtiles = (int)((rows + BM - 1) / BM);
  const int n_chunks = g.n_total / F4W_BN;
  const int k_blocks = g.k_total / F4_BK;  // <= F4_MAX_KB (checked by the launcher)

  if (threadIdx.x == 0) {
    for (int s = 0; s < 20; ++s) mbar_init(bar0 + 8u * s, 1);
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 16);
    mbar_init(drain_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_base_slot);
  const uint32_t sa = smem_u32(a_buf);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, tile_it = 0;
      bool ok = true;
      for (int mt = blockIdx.x; mt < num_mtiles && ok; mt += gridDim.x, ++tile_it) {
        for (int nc = 0; nc < n_chunks && ok; ++nc) {
          for (int kb = 0; kb < k_blocks && ok; ++kb) {
            if (!mbar_wait(bempty_bar(stage), phase ^ 1u, g.err, ERR_WAIT_EMPTY)) { ok = false; break; }
            if (nc == 0) {
              // this row tile's K-block of A: its slot was released by the MMAs of the previous tile's last chunk,
              // which also released the weight stage just waited for (four stages = four K-blocks per chunk), so
              // this wait does not hold the weight stream up
              if (!mbar_wait(aempty_bar(kb), (tile_it & 1u) ^ 1u, g.err, ERR_WAIT_EMPTY)) { ok = false; break; }
              mbar_expect_tx(afull_bar(kb), A_BYTES + F4_SFA_BYTES);
              tma_load_2d(sa + kb * A_BYTES, &tmA, kb * 128, mt * BM, afull_bar(kb));
              bulk_load(sa + F4_MAX_KB * A_BYTES + kb * F4_SFA_BYTES, g.sfa + ((int64_t)mt * k_blocks + kb) * F4_SFA_BYTES,
                        F4_SFA_BYTES, afull_bar(kb));
            }
            const uint32_t sb = smem_u32(b_ring + stage * F4W_STAGE_BYTES);
            mbar_expect_tx(bfull_bar(stage), F4W_STAGE_BYTES);
            tma_load_2d(sb, &tmB, kb * 128, nc * F4W_BN, bfull_bar(stage));  // 256 rows; x in bytes: 128 per K-block
            bulk_load(sb + F4W_B_BYTES, g.sfb + ((int64_t)nc * k_blocks + kb) * F4W_SFB_BYTES, F4W_SFB_BYTES, bfull_bar(stage));
            if (++stage == F4W_STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 2) {
    // ---- block factors: shared memory -> tensor memory, then one commit per stage for the MMA thread ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, tile_it = 0;
      bool ok = true;
      for (int mt = blockIdx.x; mt < num_mtiles && ok; mt += gridDim.x, ++tile_it) {
        for (int nc = 0; nc < n_chunks && ok; ++nc) {
          for (int kb = 0; kb < k_blocks && ok; ++kb) {
            if (nc == 0) {
              if (!mbar_wait(afull_bar(kb), tile_it & 1u, g.err, ERR_WAIT_FULL)) { ok = false; break; }
              tc_fence_after();
#pragma unroll
              for (int k = 0; k < F4_STEPS; ++k)
                tc_cp_sf(tmem_base + F4W_SFA_BASE + 16u * kb + 4u * k,
                         make_desc_sf(sa + F4_MAX_KB * A_BYTES + (uint32_t)(kb * F4_STEPS + k) * 512u));
            }
            if (!mbar_wait(bfull_bar(stage), phase, g.err, ERR_WAIT_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sb = smem_u32(b_ring + stage * F4W_STAGE_BYTES);
            const uint32_t sfb_t = tmem_base + F4W_SFB_BASE + (uint32_t)stage * 32u;
#pragma unroll
            for (int k = 0; k < F4_STEPS; ++k) {
              // 256 weight rows: the second group of 128 takes the next four columns
              tc_cp_sf(sfb_t + 8u * k, make_desc_sf(sb + F4W_B_BYTES + 512u * k));
              tc_cp_sf(sfb_t + 8u * k + 4u, make_desc_sf(sb + F4W_B_BYTES + F4_SFB_BYTES + 512u * k));
            }
            tc_commit(sfready_bar(stage));  // arrives when the copies above (A's included) have landed
            if (++stage == F4W_STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, chunk_it = 0;
      const uint32_t desc_hi = (uint32_t)(make_desc_sw128(0u) >> 32);
      const uint32_t a_lo0 = (uint32_t)make_desc_sw128(sa);
      const uint32_t b_lo0 = (uint32_t)make_desc_sw128(smem_u32(b_ring));
      bool ok = true;
      for (int mt = blockIdx.x; mt < num_mtiles && ok; mt += gridDim.x) {
        for (int nc = 0; nc < n_chunks && ok; ++nc, ++chunk_it) {
          if (!mbar_wait(tempty_bar, (chunk_it & 1u) ^ 1u, g.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          for (int kb = 0; kb < k_blocks; ++kb) {
            // data and factors of this stage (and, in the first chunk, of A's K-block) are in place
            if (!mbar_wait(sfready_bar(stage), phase, g.err, ERR_WAIT_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t al = a_lo0 + (uint32_t)kb * (A_BYTES >> 4);
            const uint32_t bl = b_lo0 + (uint32_t)stage * (F4W_STAGE_BYTES >> 4);
            const uint32_t sfa_t = tmem_base + F4W_SFA_BASE + 16u * kb;
            const uint32_t sfb_t = tmem_base + F4W_SFB_BASE + (uint32_t)stage * 32u;
#pragma unroll
            for (int k = 0; k < F4_STEPS; ++k) {
              // one step = 64 elements = 32 bytes inside the swizzle row: +2 in (address >> 4)
              tc_mma_nvfp4_w(tmem_base, ((uint64_t)desc_hi << 32) | (al + 2u * k), ((uint64_t)desc_hi << 32) | (bl + 2u * k),
                             sfa_t + 4u * k, sfb_t + 8u * k, (kb | k) != 0 ? 1u : 0u);
            }
            tc_commit(bempty_bar(stage));
            if (nc == n_chunks - 1) tc_commit(aempty_bar(kb));  // the next row tile may take this K-block's slot
            if (++stage == F4W_STAGES) { stage = 0; phase ^= 1u; }
          }
          if (ok) tc_commit(tfull_bar);
        }
      }
      tc_commit(drain_bar);
      mbar_wait(drain_bar, 0, g.err, ERR_WAIT_DRAIN);
    }
  } else if (warp >= 4) {
    const int quad = warp & 3;            // TMEM lane quadrant this warp may read
    const int qtr = (warp - 4) >> 2;      // which 64 of the 256 columns
    uint32_t chunk_it = 0;
    bool ok = true;
    for (int mt = blockIdx.x; mt < num_mtiles && ok; mt += gridDim.x) {
      const int64_t row = (int64_t)mt * BM + quad * 32 + lane;
      const bool row_ok = row < rows;
      float rowsum = 0.f;
      for (int nc = 0; nc < n_chunks && ok; ++nc, ++chunk_it) {
        if (!mbar_wait(tfull_bar, chunk_it & 1u, g.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)qtr * 64u;
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t v[32];
          tc_ld32(taddr + c0, v);
          tc_wait_ld();
          const int n0 = nc * F4W_BN + qtr * 64 + c0;
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 bq = __ldg(reinterpret_cast<const float4*>(g.bias + n0) + j4);
            const float4 wq = __ldg(reinterpret_cast<const float4*>(g.w_out + n0) + j4);
            const float4 cq = __ldg(reinterpret_cast<const float4*>(g.col_scale + n0) + j4);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4]), cq.x, bq.x), 0.f), wq.x, rowsum);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4 + 1]), cq.y, bq.y), 0.f), wq.y, rowsum);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4 + 2]), cq.z, bq.z), 0.f), wq.z, rowsum);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4 + 3]), cq.w, bq.w), 0.f), wq.w, rowsum);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar);
      }
      // the four column quarters of a row meet in shared memory
      if (qtr > 0) part[(qtr - 1) * 128 + quad * 32 + lane] = rowsum;
      asm volatile("bar.sync 1, 512;" ::: "memory");
      if (qtr == 0 && row_ok && ok) {
        const int r = quad * 32 + lane;
        const float total = (rowsum + part[r]) + (part[128 + r] + part[256 + r]);
        if (g.accumulate_q) g.out_q[row] += total;
        else g.out_q[row] = total;
      }
      asm volatile("bar.sync 1, 512;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// e4m3 activations [rows, K] (value = e4m3 * in_scale) -> NVFP4: packed E2M1 [rows, K / 2] and E4M3 block factors in the
// layout of the A operand above.  One thread per (row, block of 16).  factor = e4m3_rn(blockmax / 6 * inv_global),
// element = e2m1_rn(x / (factor / inv_global)); a zero block keeps factor 0 and elements 0.
__global__ void __launch_bounds__(256)
k_quant_h1_nvfp4(const uint8_t* __restrict__ h1_e4m3, const uint32_t* count_dev, int64_t row_limit, int K, float in_scale,
                 float inv_global, uint8_t* __restrict__ out_fp4, uint8_t* __restrict__ out_sf) {
  int64_t rows = (int64_t)(*count_dev);
  if (rows > row_limit) rows = row_limit;
  const int blocks_per_row = K / 16;
  const int k_blocks = K / F4_BK;
  const int64_t total = rows * blocks_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / blocks_per_row;
    const int blk = (int)(i - row * blocks_per_row);
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(h1_e4m3 + row * K + blk * 16));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float x[16];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const __nv_fp8_storage_t b = (__nv_fp8_storage_t)((w[j >> 2] >> (8 * (j & 3))) & 0xffu);
      const __half_raw hr = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
      x[j] = __half2float(__half(hr)) * in_scale;
      amax = fmaxf(amax, fabsf(x[j]));
    }
    const __nv_fp8_storage_t sf8 = __nv_cvt_float_to_fp8(amax * (1.f / 6.f) * inv_global, __NV_SATFINITE, __NV_E4M3);
    const float sf = __half2float(__half(__nv_cvt_fp8_to_halfraw(sf8, __NV_E4M3)));
    const float inv = sf > 0.f ? inv_global / sf : 0.f;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t p0 = __nv_cvt_float2_to_fp4x2(make_float2(x[2 * j] * inv, x[2 * j + 1] * inv), __NV_E2M1, cudaRoundNearest);
      if (j < 4) lo |= (p0 & 0xffu) << (8 * j);
      else hi |= (p0 & 0xffu) << (8 * (j - 4));
    }
    *reinterpret_cast<uint2*>(out_fp4 + row * (K / 2) + blk * 8) = make_uint2(lo, hi);
    const int64_t mt = row >> 7;
    const int r = (int)(row & 127);
    const int col = blk * 16;
    const int kb = col / F4_BK, step = (col % F4_BK) / 64, j4 = (col % 64) / 16;
    out_sf[((mt * k_blocks + kb) * F4_STEPS + step) * 512 + (r & 31) * 16 + (r >> 5) * 4 + j4] = (uint8_t)sf8;
  }
}

int nvfp4_head_smem() { return F4_SMEM; }

int nvfp4_prepare() {
  int rc = (int)cudaFuncSetAttribute(k_mlp_head_nvfp4, cudaFuncAttributeMaxDynamicSharedMemorySize, F4_SMEM);
  if (!rc) rc = (int)cudaFuncSetAttribute(k_mlp_head_nvfp4_wide, cudaFuncAttributeMaxDynamicSharedMemorySize, F4W_SMEM);
  return rc;
}

int launch_quant_h1_nvfp4(const uint8_t* h1_e4m3, const uint32_t* count_dev, int64_t row_limit, int K, float in_scale,
                          float inv_global, uint8_t* out_fp4, uint8_t* out_sf, int sms, cudaStream_t st) {
  if (K % F4_BK != 0) return MGBS_ERR_UNSUPPORTED;
  k_quant_h1_nvfp4<<<sms * 8, 256, 0, st>>>(h1_e4m3, count_dev, row_limit, K, in_scale, inv_global, out_fp4, out_sf);
  return (int)cudaGetLastError();
}

int launch_head_nvfp4(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmBw, const Nvfp4HeadArgs& g, int sms,
                      cudaStream_t st, int wide) {
  if (g.k_total % F4_BK != 0 || g.k_total / F4_BK > F4_MAX_KB || g.n_total % F4_BN != 0) return MGBS_ERR_UNSUPPORTED;
  // the wide kernel pairs its four weight stages with the K-blocks of a chunk: it needs exactly four of them
  if (wide && g.k_total / F4_BK == F4W_STAGES && g.n_total % F4W_BN == 0)
    k_mlp_head_nvfp4_wide<<<sms, F4W_THREADS, F4W_SMEM, st>>>(tmA, tmBw, g);
  else
    k_mlp_head_nvfp4<<<sms, F4_THREADS, F4_SMEM, st>>>(tmA, tmB, g);
  return (int)cudaGetLastError();
}

}  // namespace mgbs
