// Value-network scorer for sm_100a: a 3-layer MLP  one-hot(n*V) -> H -> H -> 1  evaluated on every child state.
// The two H-wide layers are GEMMs on the 5th-generation tensor cores: tcgen05.mma issued by one thread, operands
// staged in shared memory by TMA (128-byte swizzle, K-major), accumulators in tensor memory, epilogues read with
// tcgen05.ld.  The last layer (H -> 1) and the score-key quantisation are fused into the second GEMM's epilogue.
//
// Takes the place of FullBeamNiceStaticBackend::forward and its Turing-era CUTLASS HMMA GEMMs
// (beam_engine.cpp:621-667, beam_kernels.cu:208-344, 970-1038).  Unlike the reference's action-value network on
// parents, this is the value network on children that the benchmark configurations name.
//
// Warp roles of the GEMM kernel (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2..5 = epilogue (one TMEM lane quadrant each).  Every mbarrier wait is bounded: after the limit the
// waiter records an error code in global memory and the CTA drains and exits; nothing spins forever.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <new>

#include <cuda_fp4.h>

#include "mgbs.h"
#include "mgbs_nvfp4.cuh"
#include "mgbs_tc.cuh"

namespace mgbs {

struct GemmArgs {
  const uint32_t* count_dev;  // rows to process (device value)
  int64_t row_offset;         // first row of this launch (micro-batching)
  int64_t row_limit;          // rows of this launch at most
  int32_t n_total;            // output features (multiple of BN)
  int32_t k_total;            // reduction length (multiple of BK)
  const float* bias;          // [n_total]
  const float* col_scale;     // fp8 only: [n_total] dequantisation factor of each output column
  const float* w_out;         // EPI 1: [n_total] weights of the scalar head
  __nv_bfloat16* out_bf16;    // EPI 0: [rows, n_total]
  const __nv_bfloat16* resid = nullptr;  // EPI 0: [rows, n_total] added before the ReLU, or null (may alias out_bf16)
  int32_t gelu = 0;           // EPI 0: GELU instead of ReLU
  float* out_q;               // EPI 1: [rows]
  int32_t accumulate_q;       // EPI 1, 2: add to out_q instead of overwriting (ensemble members after the first)
  int32_t q_cols;             // EPI 2: output columns kept (the fan-out); out_q is [rows, q_cols]
  int* err;
};

// EPI 0: out = bf16(relu(acc + bias (+ resid))).  EPI 1: q[row] (+)= sum_n relu(acc + bias[n]) * w_out[n].
// EPI 2: q[row, n] (+)= acc + bias[n] for n < q_cols (output layer of an action-value network: one value per move).
template <int EPI, int F8>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_mlp_gemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty, [2S+4] drain, then tmem base
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 5);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };
  const uint32_t drain_bar = bar0 + 8u * (2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  int64_t rows = (int64_t)(*g.count_dev) - g.row_offset;
  if (rows > g.row_limit) rows = g.row_limit;
  if (rows < 0) rows = 0;
  const int num_mtiles = (int)((rows + BM - 1) / BM);
  const int n_chunks = g.n_total / BN;
  constexpr int BKE = F8 ? BK8 : BK;  // elements per 128-byte K-block
  const int k_blocks = g.k_total / BKE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 4); }
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
      bool ok = true;
      for (int mt = blockIdx.x; mt < num_mtiles && ok; mt += gridDim.x) {
        const int row0 = (int)(g.row_offset + (int64_t)mt * BM);
        for (int nc = 0; nc < n_chunks && ok; ++nc) {
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, g.err, ERR_WAIT_EMPTY)) { ok = false; break; }
            const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
            mbar_expect_tx(full_bar(stage), STAGE_BYTES);
            tma_load_2d(sa, &tmA, kb * BKE, row0, full_bar(stage));
            tma_load_2d(sa + A_BYTES, &tmB, kb * BKE, nc * BN, full_bar(stage));
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_it = 0;
      bool ok = true;
      for (int mt = blockIdx.x; mt < num_mtiles && ok; mt += gridDim.x) {
        for (int nc = 0; nc < n_chunks && ok; ++nc, ++acc_it) {
          const uint32_t b = acc_it & 1u;
          if (!mbar_wait(tempty_bar(b), ((acc_it >> 1) & 1u) ^ 1u, g.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + b * BN;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, g.err, ERR_WAIT_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
            const uint64_t adesc = make_desc_sw128(sa);
            const uint64_t bdesc = make_desc_sw128(sa + A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // advancing K by one instruction (16 bf16 or 32 e4m3 = 32 bytes) inside the swizzle row: +2 in (address >> 4)
              tc_mma<F8>(d_tmem, adesc + 2u * k, bdesc + 2u * k, (kb | k) != 0 ? 1u : 0u);
            }
            tc_commit(empty_bar(stage));
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
          if (ok) tc_commit(tfull_bar(b));
        }
      }
      // drain: every MMA issued by this thread has retired before TMEM is released
      tc_commit(drain_bar);
      mbar_wait(drain_bar, 0, g.err, ERR_WAIT_DRAIN);
    }
  } else {
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    uint32_t acc_it = 0;
    bool ok = true;
    for (int mt = blockIdx.x; mt < num_mtiles && ok; mt += gridDim.x) {
      const int64_t row_local = (int64_t)mt * BM + quad * 32 + lane;
      const int64_t row = g.row_offset + row_local;
      const bool row_ok = row_local < rows;
      float rowsum = 0.f;
      for (int nc = 0; nc < n_chunks && ok; ++nc, ++acc_it) {
        const uint32_t b = acc_it & 1u;
        if (!mbar_wait(tfull_bar(b), (acc_it >> 1) & 1u, g.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + b * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (EPI == 2 && nc * BN + c0 >= g.q_cols) break;  // columns past the fan-out are padding
          uint32_t v[32];
          tc_ld32(taddr + c0, v);
          tc_wait_ld();
          const int n0 = nc * BN + c0;
          if (EPI == 0) {
            uint32_t packed[16];
            if (g.resid != nullptr && row_ok) {  // each thread reads the 32 values it is about to overwrite
              const uint4* src = reinterpret_cast<const uint4*>(g.resid + row * g.n_total + n0);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 r4 = src[q];
                const uint32_t rw[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rw[t]));
                  v[8 * q + 2 * t] = __float_as_uint(__uint_as_float(v[8 * q + 2 * t]) + f.x);
                  v[8 * q + 2 * t + 1] = __float_as_uint(__uint_as_float(v[8 * q + 2 * t + 1]) + f.y);
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float a0 = __uint_as_float(v[2 * j]) + __ldg(g.bias + n0 + 2 * j);
              const float a1 = __uint_as_float(v[2 * j + 1]) + __ldg(g.bias + n0 + 2 * j + 1);
              const float x0 = g.gelu ? gelu_erf(a0) : fmaxf(a0, 0.f);
              const float x1 = g.gelu ? gelu_erf(a1) : fmaxf(a1, 0.f);
              __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
              packed[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            if (row_ok) {
              uint4* dst = reinterpret_cast<uint4*>(g.out_bf16 + row * g.n_total + n0);
#pragma unroll
              for (int q = 0; q < 4; ++q) dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
            }
          } else if (EPI == 2) {
            if (row_ok) {
              float* qrow = g.out_q + row * g.q_cols;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (n0 + j < g.q_cols) {
                  const float x = __uint_as_float(v[j]) + __ldg(g.bias + n0 + j);
                  if (g.accumulate_q) qrow[n0 + j] += x;
                  else qrow[n0 + j] = x;
                }
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float acc = __uint_as_float(v[j]);
              if (F8) acc *= __ldg(g.col_scale + n0 + j);
              const float x = fmaxf(acc + __ldg(g.bias + n0 + j), 0.f);
              rowsum = fmaf(x, __ldg(g.w_out + n0 + j), rowsum);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(b));
      }
      if (EPI == 1 && row_ok && ok) {
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
// Layer 2 + scalar head on CTA pairs (thread-block clusters of two, tcgen05 cta_group::2).
//
// With one CTA per tile every 128 x 256 x 16 MMA reads 4 KB of A and 8 KB of B from shared memory in the 128
// cycles it takes: 96 of the 128 bytes per clock the shared-memory port gives, and the TMA fills of the next
// K-blocks need 48 KB per four MMAs on top.  The port, not the tensor core, then bounds the kernel at about two
// thirds of the tensor peak.  A pair of CTAs shares B: each CTA loads its own 128 rows of A and HALF of the 256
// weight rows of the chunk, the even CTA issues one MMA of M = 256 that reads both CTAs' shared memory and
// writes each CTA's 128 accumulator rows into that CTA's TMEM.  Per CTA that is 8 KB of operand reads per MMA
// and 32 KB of fills per K-block: two thirds of the traffic.
//
// q[row] (+)= sum_n relu(acc[row, n] * col_scale[n] + bias[n]) * w_out[n]  (col_scale for e4m3 operands only).
// Warps of each CTA: 0 = TMA (own A rows, own half of B; completion bytes are counted on the even CTA's barrier),
// 1 = TMEM allocation, and in the even CTA MMA issue; 2..5 = epilogue for the CTA's own 128 rows.
// Barriers: full[s] lives in the even CTA (its TMA thread arms it with the bytes of both CTAs); empty[s] and
// tmem_full[b] exist in both CTAs and are signalled by multicast commits; tmem_empty[b] lives in the even CTA and
// counts the eight epilogue warps of the pair.
// ------------------------------------------------------------------------------------------------

// A stage holds PAIR_KPS consecutive K-blocks.  The thread that issues the MMAs pays a few hundred cycles per stage
// for the barrier wait, the fence and the commit whatever the stage holds (measured ~600-700 cycles per iteration
// against 512 cycles of tensor work for one K-block of four MMAs), so two K-blocks per stage halve that overhead.
constexpr int PAIR_KPS = 2;
constexpr int PAIR_STAGES = 3;
constexpr int PAIR_STAGE_BYTES = PAIR_KPS * 2 * A_BYTES;  // per K-block: 128 x 128-byte rows of A + 128 rows of B
constexpr int PAIR_SMEM = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256;

template <int F8>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_mlp_head_pair(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PAIR_STAGES * PAIR_STAGE_BYTES);
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * PAIR_STAGES + 5);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (PAIR_STAGES + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * PAIR_STAGES + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * PAIR_STAGES + 2 + b); };
  const uint32_t drain_bar = bar0 + 8u * (2 * PAIR_STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();  // 0 = even CTA (issues the MMAs), 1 = its peer
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs_grid = gridDim.x >> 1;

  int64_t rows = (int64_t)(*g.count_dev) - g.row_offset;
  if (rows > g.row_limit) rows = g.row_limit;
  if (rows < 0) rows = 0;
  const int num_ptiles = (int)((rows + 2 * BM - 1) / (2 * BM));  // tiles of 256 rows
  const int n_chunks = g.n_total / BN;
  constexpr int BKE = F8 ? BK8 : BK;
  const int k_blocks = g.k_total / (BKE * PAIR_KPS);  // stages per N-chunk (k_total is a multiple of 256)

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 8); }
    mbar_init(drain_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    // both CTAs' warp 1 take part; each CTA finds the (same) base address in its own slot
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_base_slot);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int pt = pair_id; pt < num_ptiles && ok; pt += num_pairs_grid) {
        const int row0 = (int)(g.row_offset + (int64_t)pt * 2 * BM + (int64_t)crank * BM);
        for (int nc = 0; nc < n_chunks && ok; ++nc) {
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, g.err, ERR_WAIT_EMPTY)) { ok = false; break; }
            const uint32_t sa = smem_u32(smem + stage * PAIR_STAGE_BYTES);
            if (crank == 0) mbar_expect_tx(full_bar(stage), 2 * PAIR_STAGE_BYTES);  // both CTAs' boxes
#pragma unroll
            for (int j = 0; j < PAIR_KPS; ++j) {
              const int kcol = (kb * PAIR_KPS + j) * BKE;
              tma_load_2d_pair(sa + j * 2 * A_BYTES, &tmA, kcol, row0, full_bar(stage));
              tma_load_2d_pair(sa + j * 2 * A_BYTES + A_BYTES, &tmB, kcol, nc * BN + (int)crank * (BN / 2), full_bar(stage));
            }
            if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && crank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_it = 0;
      bool ok = true;
      for (int pt = pair_id; pt < num_ptiles && ok; pt += num_pairs_grid) {
        for (int nc = 0; nc < n_chunks && ok; ++nc, ++acc_it) {
          const uint32_t b = acc_it & 1u;
          if (!mbar_wait(tempty_bar(b), ((acc_it >> 1) & 1u) ^ 1u, g.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + b * BN;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, g.err, ERR_WAIT_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * PAIR_STAGE_BYTES);
#pragma unroll
            for (int j = 0; j < PAIR_KPS; ++j) {
              const uint64_t adesc = make_desc_sw128(sa + j * 2 * A_BYTES);
              const uint64_t bdesc = make_desc_sw128(sa + j * 2 * A_BYTES + A_BYTES);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k)
                tc_mma_pair<F8>(d_tmem, adesc + 2u * k, bdesc + 2u * k, (kb | j | k) != 0 ? 1u : 0u);
            }
            tc_commit_pair(empty_bar(stage), (uint16_t)3);  // both CTAs may refill this stage
            if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
          }
          if (ok) tc_commit_pair(tfull_bar(b), (uint16_t)3);  // both CTAs' epilogues may read their rows
        }
      }
      tc_commit_pair(drain_bar, (uint16_t)1);
      mbar_wait(drain_bar, 0, g.err, ERR_WAIT_DRAIN);
    }
  } else {
    const int quad = warp & 3;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int pt = pair_id; pt < num_ptiles && ok; pt += num_pairs_grid) {
      const int64_t row_local = (int64_t)pt * 2 * BM + (int64_t)crank * BM + quad * 32 + lane;
      const int64_t row = g.row_offset + row_local;
      const bool row_ok = row_local < rows;
      float rowsum = 0.f;
      for (int nc = 0; nc < n_chunks && ok; ++nc, ++acc_it) {
        const uint32_t b = acc_it & 1u;
        if (!mbar_wait(tfull_bar(b), (acc_it >> 1) & 1u, g.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + b * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          tc_ld32(taddr + c0, v);
          tc_wait_ld();
          const int n0 = nc * BN + c0;
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 bq = __ldg(reinterpret_cast<const float4*>(g.bias + n0) + j4);
            const float4 wq = __ldg(reinterpret_cast<const float4*>(g.w_out + n0) + j4);
            float4 cq = make_float4(1.f, 1.f, 1.f, 1.f);
            if (F8) cq = __ldg(reinterpret_cast<const float4*>(g.col_scale + n0) + j4);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4]), cq.x, bq.x), 0.f), wq.x, rowsum);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4 + 1]), cq.y, bq.y), 0.f), wq.y, rowsum);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4 + 2]), cq.z, bq.z), 0.f), wq.z, rowsum);
            rowsum = fmaf(fmaxf(fmaf(__uint_as_float(v[4 * j4 + 3]), cq.w, bq.w), 0.f), wq.w, rowsum);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_even_cta(tempty_bar(b));
      }
      if (row_ok && ok) {
        if (g.accumulate_q) g.out_q[row] += rowsum;
        else g.out_q[row] = rowsum;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still read its shared memory or signal its barriers
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// Layer 1 with the one-hot operand built in shared memory.
//
// out[row, :] = bf16(relu(onehot(child[row]) * W1^T + b1)).  The A operand is never materialised in global
// memory.  The producer warps build the 128 x 64 bf16 K-blocks of the one-hot matrix straight into the
// 128-byte-swizzled A slots the tensor core reads: with the value-major column order every 16-byte chunk is a byte
// compare of two words of the child row, written with conflict-free 16-byte stores.  When the whole one-hot tile
// fits the six A slots (K <= 384) each K-block is built once per M-tile and reused by the four N-chunks; otherwise
// the slots form a ring and blocks are rebuilt per N-chunk.  Four producer groups each work on every fourth block,
// so four K-blocks are in production at any time and the latency of one block is hidden behind the others.  W1
// K-blocks stream by TMA through a separate 3-stage ring.  The epilogue packs the activated tile to bf16 in
// swizzled staging boxes private to each warp and writes them with TMA stores.
//
// Warps: 0 = TMA (W1), 1 = MMA + TMEM owner, then EW epilogue warps, then 12 - EW one-hot producer warps.
// ------------------------------------------------------------------------------------------------

// max(x, 0) rounded to bf16, two values per 32-bit word (lo in bits 0..15)
__device__ __forceinline__ uint32_t pack_relu_bf16(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}


constexpr int L1_THREADS = 448;
constexpr int L1_A_STAGES = 6;                           // 6 x 16 KB: a whole 128 x 384 one-hot tile when K <= 384
constexpr int L1_B_STAGES = 3;
constexpr int L1_PAIRS = 4;                              // producer warp pairs
constexpr int L1_STAGING = A_BYTES;                      // 16 KB of private 2 KB output boxes of the epilogue warps
constexpr int L1_CHILD_PITCH = MGBS_MAX_STATE_LEN + 4;   // bytes; odd word pitch -> conflict-free row reads
constexpr int L1_MAX_KBLOCKS = 16;
constexpr int L1_SMEM = L1_A_STAGES * A_BYTES + L1_B_STAGES * B_BYTES + L1_STAGING + BM * L1_CHILD_PITCH + 1024 + 512;

struct L1Args {
  const uint8_t* children;   // [rows, stride]
  const uint32_t* count_dev;
  int64_t row_limit;
  int32_t n, stride, V;
  int32_t n_total;           // hidden (multiple of BN)
  int32_t k_total;           // n*V rounded up to the K-block width (64 bf16 / 128 e4m3)
  int32_t k_real;            // onehot_columns(n, V): columns at or past it are padding; MMA steps entirely beyond are skipped
  const float* bias;
  const float* col_scale;    // fp8 only: [n_total] dequantisation factor of each W1 output channel
  float out_inv_scale;       // fp8 only: activations are stored as e4m3(value * out_inv_scale)
  uint8_t* sf_out;           // NVFP4 output only: block factors, [row tile][column chunk][step][512 B]
  float inv_global;          // NVFP4 output only: 1 / tensor scale of the activations
  int* err;
};

// EW = epilogue warps (4 or 8); the other 12 - EW warps of the 14 build the one-hot operand.  With the resident
// tile (K <= 384) production is light and the epilogue is the bottleneck: EW = 8 (two warps per TMEM lane quadrant,
// each taking every other 32-column group of a box).  With the ring (K > 384) production dominates: EW = 4.
// PAIR = 1: thread-block clusters of two (see k_mlp_head_pair).  Each CTA builds the one-hot operand of its own 128
// rows and loads half of each 256-row block of W1; the even CTA issues MMAs of M = 256 over both.  The weight ring
// then holds six half blocks instead of three whole ones, and the shared-memory port carries a third less.
// OUT4 = 1 (with F8 = 1, EW = 8): the activations leave as NVFP4 instead of e4m3 - per row and block of 16 columns
// one E4M3 factor e4m3(blockmax / 6 * inv_global), elements E2M1(x * inv_global / factor), two per byte; tmOut is then
// the packed tensor [rows, n_total / 2] bytes and the factors go to sf_out in the layout the block-scaled GEMM of the
// second layer reads (row r of a 128-row tile at byte (r % 32) * 16 + (r / 32) * 4 of each 512-byte step chunk).
template <int F8, int EW, int PAIR, int OUT4 = 0>
__global__ void __launch_bounds__(L1_THREADS, 1)
k_mlp_l1(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmOut, L1Args g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* a_ring = smem;                                   // 6 x 16 KB, 1024-aligned
  uint8_t* b_ring = a_ring + L1_A_STAGES * A_BYTES;         // 3 x 32 KB, or 6 x 16 KB for CTA pairs
  constexpr int NBS = PAIR ? 2 * L1_B_STAGES : L1_B_STAGES; // stages of the weight ring
  constexpr int BSB = PAIR ? B_BYTES / 2 : B_BYTES;         // bytes per stage
  uint8_t* staging = b_ring + L1_B_STAGES * B_BYTES;        // 16 KB: the epilogue warps' private boxes
  uint8_t* child_s = staging + L1_STAGING;
  uint64_t* bars = reinterpret_cast<uint64_t*>(((uintptr_t)(child_s + BM * L1_CHILD_PITCH) + 7) & ~(uintptr_t)7);
  // barriers: a_full[A], a_empty[A], b_full[NBS], b_empty[NBS], tmem_full[2], tmem_empty[2], drain (A = L1_A_STAGES)
  constexpr int NB = 2 * L1_A_STAGES + 2 * NBS + 5;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + NB);
  const uint32_t bar0 = smem_u32(bars);
  auto a_full = [&](int s) { return bar0 + 8u * s; };
  auto a_empty = [&](int s) { return bar0 + 8u * (L1_A_STAGES + s); };
  auto b_full = [&](int s) { return bar0 + 8u * (2 * L1_A_STAGES + s); };
  auto b_empty = [&](int s) { return bar0 + 8u * (2 * L1_A_STAGES + NBS + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * L1_A_STAGES + 2 * NBS + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * L1_A_STAGES + 2 * NBS + 2 + b); };
  const uint32_t drain_bar = bar0 + 8u * (2 * L1_A_STAGES + 2 * NBS + 4);
  // tile schedule: CTA pairs walk tiles of 256 rows, each CTA taking its half; single CTAs walk tiles of 128 rows
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
  const int tile_first = PAIR ? 2 * (int)(blockIdx.x >> 1) + (int)crank : (int)blockIdx.x;
  const int tile_step = PAIR ? (int)(gridDim.x & ~1u) : (int)gridDim.x;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int64_t rows = (int64_t)(*g.count_dev);
  if (rows > g.row_limit) rows = g.row_limit;
  const int num_mtiles = (int)((rows + BM - 1) / BM);
  const int n_chunks = g.n_total / BN;
  constexpr int BKE = F8 ? BK8 : BK;  // one-hot columns per 128-byte K-block
  const int k_blocks = g.k_total / BKE;
  const bool resident = k_blocks <= L1_A_STAGES;  // one-hot tile stays in shared memory for all N-chunks
  const int blocks_per_tile = resident ? k_blocks : n_chunks * k_blocks;

  if (threadIdx.x == 0) {
    // pairs: a_full, b_full and tmem_empty are used in the even CTA only and count both CTAs' arrivals
    for (int s = 0; s < L1_A_STAGES; ++s) { mbar_init(a_full(s), (PAIR ? 2 : 1) * (12 - EW) / 4); mbar_init(a_empty(s), 1); }
    for (int s = 0; s < NBS; ++s) { mbar_init(b_full(s), 1); mbar_init(b_empty(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), (PAIR ? 2 : 1) * EW); }
    mbar_init(drain_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_base_slot);

  if (warp == 0) {
    // ---- W1 K-blocks by TMA ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int mt = tile_first; mt - (int)crank < num_mtiles && ok; mt += tile_step) {
        for (int nc = 0; nc < n_chunks && ok; ++nc) {
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(b_empty(stage), phase ^ 1u, g.err, ERR_WAIT_EMPTY)) { ok = false; break; }
            if (PAIR) {
              // this CTA's half of the weight block; the bytes of both halves are counted in the even CTA
              if (crank == 0) mbar_expect_tx(b_full(stage), 2 * BSB);
              tma_load_2d_pair(smem_u32(b_ring + stage * BSB), &tmB, kb * BKE, nc * BN + (int)crank * (BN / 2), b_full(stage));
            } else {
              mbar_expect_tx(b_full(stage), B_BYTES);
              tma_load_2d(smem_u32(b_ring + stage * B_BYTES), &tmB, kb * BKE, nc * BN, b_full(stage));
            }
            if (++stage == NBS) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue ----
    // One thread; every instruction of its loop is on the critical path (a lone warp issues dependent instructions
    // several cycles apart, and a K-block of four MMAs keeps the tensor core busy for only ~450 cycles), so the loop
    // carries as little as possible: descriptors are 32-bit adds on a precomputed base, ring positions advance
    // incrementally, and the resident one-hot tile is waited for once per tile, not once per N-chunk.
    if (lane == 0 && crank == 0) {
      constexpr int KSTEP = BKE / (BK / UMMA_K);  // one-hot columns per MMA step: 16 (bf16) or 32 (e4m3)
      const uint32_t desc_hi = (uint32_t)(make_desc_sw128(0u) >> 32);
      const uint32_t a_lo0 = (uint32_t)make_desc_sw128(smem_u32(a_ring));
      const uint32_t b_lo0 = (uint32_t)make_desc_sw128(smem_u32(b_ring));
      // the last K-block is mostly padding (336 one-hot columns in 384): its all-zero steps add nothing
      int last_steps = (g.k_real - (k_blocks - 1) * BKE + KSTEP - 1) / KSTEP;
      last_steps = last_steps < 1 ? 1 : (last_steps > BK / UMMA_K ? BK / UMMA_K : last_steps);
      int sb = 0;
      uint32_t pb = 0, acc_it = 0;
      int sa_t = 0;          // A slot and parity of the current tile's first K-block (resident) / next K-block (ring)
      uint32_t pa_t = 0;
      bool ok = true;
      for (int mt = tile_first; mt < num_mtiles && ok; mt += tile_step) {
        int sa = sa_t;
        uint32_t pa = pa_t;
        for (int nc = 0; nc < n_chunks && ok; ++nc, ++acc_it) {
          const uint32_t b = acc_it & 1u;
          if (!mbar_wait(tempty_bar(b), ((acc_it >> 1) & 1u) ^ 1u, g.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + b * BN;
          if (resident) { sa = sa_t; pa = pa_t; }  // every N-chunk walks the same K-blocks of the tile
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!resident || nc == 0) {            // later N-chunks of a resident tile: already waited for
              if (PAIR) {
                if (!mbar_wait_cluster(a_full(sa), pa, g.err, ERR_WAIT_FULL)) { ok = false; break; }
              } else {
                if (!mbar_wait(a_full(sa), pa, g.err, ERR_WAIT_FULL)) { ok = false; break; }
              }
            }
            if (!mbar_wait(b_full(sb), pb, g.err, ERR_WAIT_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t al = a_lo0 + (uint32_t)sa * (A_BYTES >> 4);
            const uint32_t bl = b_lo0 + (uint32_t)sb * (BSB >> 4);
            const int ksteps = kb == k_blocks - 1 ? last_steps : BK / UMMA_K;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              if (k < ksteps) {
                const uint64_t adesc = ((uint64_t)desc_hi << 32) | (al + 2u * k);
                const uint64_t bdesc = ((uint64_t)desc_hi << 32) | (bl + 2u * k);
                if (PAIR) tc_mma_pair<F8>(d_tmem, adesc, bdesc, (kb | k) != 0 ? 1u : 0u);
                else tc_mma<F8>(d_tmem, adesc, bdesc, (kb | k) != 0 ? 1u : 0u);
              }
            }
            if (PAIR) {
              if (!resident || nc == n_chunks - 1) tc_commit_pair(a_empty(sa), (uint16_t)3);
              tc_commit_pair(b_empty(sb), (uint16_t)3);
            } else {
              if (!resident || nc == n_chunks - 1) tc_commit(a_empty(sa));
              tc_commit(b_empty(sb));
            }
            if (++sb == NBS) { sb = 0; pb ^= 1u; }
            if (++sa == L1_A_STAGES) { sa = 0; pa ^= 1u; }
          }
          if (ok) {
            if (PAIR) tc_commit_pair(tfull_bar(b), (uint16_t)3);
            else tc_commit(tfull_bar(b));
          }
        }
        sa_t = sa;  // resident: the tile's first slot advanced by k_blocks; ring: simply where the walk stopped
        pa_t = pa;
      }
      if (PAIR) tc_commit_pair(drain_bar, (uint16_t)1);
      else tc_commit(drain_bar);
      mbar_wait(drain_bar, 0, g.err, ERR_WAIT_DRAIN);
    }
  } else if (warp < 2 + EW) {
    // ---- epilogue: TMEM -> bias, ReLU, bf16 -> swizzled staging box -> TMA store ----
    const int quad = warp & 3;
    const int sg = EW == 4 ? 0 : (warp - 2) >> 2;     // sub-group: which 32-column groups of a box this warp takes
    const uint32_t r = (uint32_t)(quad * 32 + lane);  // tile row owned by this thread
    uint32_t acc_it = 0, box_it = 0;
    bool ok = true;
    for (int mt = tile_first; mt - (int)crank < num_mtiles && ok; mt += tile_step) {
      const int row0 = mt * BM;
      for (int nc = 0; nc < n_chunks && ok; ++nc, ++acc_it) {
        const uint32_t b = acc_it & 1u;
        if (!mbar_wait(tfull_bar(b), (acc_it >> 1) & 1u, g.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + b * BN;
        if constexpr (OUT4 == 0) {
          // private staging: each warp owns boxes of 32 rows x 64 bytes (64-byte swizzle) for its TMEM lane quadrant,
          // so no barrier between warps is needed and every warp has its own TMA stores in flight.  Four epilogue
          // warps own two boxes each and alternate (filling one overlaps the store reading the other); eight
          // warps own one each and take every other box of the chunk.  A TMA store holds its box for well over a
          // thousand cycles, so what counts is the number of boxes in flight: one 16 KB box shared by eight warps
          // behind two block barriers (the earlier form of the eight-warp epilogue) turned around every 2 300 cycles.
          // (Storing straight from registers with plain global stores measured slower than these TMA stores.)
          constexpr int SUBC = F8 ? 64 : 32;  // output columns per 64-byte box row
          constexpr int NBOX = EW == 4 ? 2 : 1;
          uint8_t* mybuf = staging + (warp - 2) * (NBOX * 2048);
#pragma unroll 1
          for (int gcol = sg * SUBC; gcol < BN; gcol += SUBC * (EW / 4), ++box_it) {
            uint8_t* box = mybuf + (NBOX == 2 ? (box_it & 1u) * 2048 : 0u);
            if (lane == 0) {
              if (NBOX == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
              else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            }
            __syncwarp();
            uint32_t packed[16];
            if (F8) {
#pragma unroll
              for (int sub = 0; sub < 2; ++sub) {
                uint32_t v[32];
                tc_ld32(taddr + gcol + sub * 32, v);
                tc_wait_ld();
                const int n0 = nc * BN + gcol + sub * 32;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float4 cq = __ldg(reinterpret_cast<const float4*>(g.col_scale + n0) + j);
                  const float4 bq = __ldg(reinterpret_cast<const float4*>(g.bias + n0) + j);
                  float x[4];
                  x[0] = fmaxf(fmaf(__uint_as_float(v[4 * j]), cq.x, bq.x), 0.f) * g.out_inv_scale;
                  x[1] = fmaxf(fmaf(__uint_as_float(v[4 * j + 1]), cq.y, bq.y), 0.f) * g.out_inv_scale;
                  x[2] = fmaxf(fmaf(__uint_as_float(v[4 * j + 2]), cq.z, bq.z), 0.f) * g.out_inv_scale;
                  x[3] = fmaxf(fmaf(__uint_as_float(v[4 * j + 3]), cq.w, bq.w), 0.f) * g.out_inv_scale;
                  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(x[0], x[1]), __NV_SATFINITE, __NV_E4M3);
                  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(x[2], x[3]), __NV_SATFINITE, __NV_E4M3);
                  packed[sub * 8 + j] = lo | (hi << 16);
                }
              }
            } else {
              uint32_t v[32];
              tc_ld32(taddr + gcol, v);
              tc_wait_ld();
              const int n0 = nc * BN + gcol;
#pragma unroll
              for (int j4 = 0; j4 < 8; ++j4) {
                const float4 bq = __ldg(reinterpret_cast<const float4*>(g.bias + n0) + j4);
                packed[2 * j4] = pack_relu_bf16(__uint_as_float(v[4 * j4]) + bq.x, __uint_as_float(v[4 * j4 + 1]) + bq.y);
                packed[2 * j4 + 1] = pack_relu_bf16(__uint_as_float(v[4 * j4 + 2]) + bq.z, __uint_as_float(v[4 * j4 + 3]) + bq.w);
              }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              // 64-byte swizzle: 16-byte chunk index ^= (row / 2) mod 4 inside 512-byte atoms
              const uint32_t off = (uint32_t)lane * 64u + (((uint32_t)q ^ (((uint32_t)lane >> 1) & 3u)) << 4);
              *reinterpret_cast<uint4*>(box + off) = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmOut, smem_u32(box), nc * BN + gcol, row0 + quad * 32);
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        } else {
          // NVFP4 output: 32 columns become 16 bytes, so a warp's half of the chunk (128 columns) is one private
          // box of 32 rows x 64 bytes; the block factors go straight to global memory
          uint8_t* box = staging + (warp - 2) * 2048;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
          uint8_t* sf_row = g.sf_out + (((int64_t)mt * n_chunks + nc) * 4) * 512 + (r & 31u) * 16u + (r >> 5) * 4u;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int sub = sg * 4 + i;
            uint32_t v[32];
            tc_ld32(taddr + sub * 32, v);
            tc_wait_ld();
            const int n0 = nc * BN + sub * 32;
            float x[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 cq = __ldg(reinterpret_cast<const float4*>(g.col_scale + n0) + j);
              const float4 bq = __ldg(reinterpret_cast<const float4*>(g.bias + n0) + j);
              x[4 * j] = fmaxf(fmaf(__uint_as_float(v[4 * j]), cq.x, bq.x), 0.f);
              x[4 * j + 1] = fmaxf(fmaf(__uint_as_float(v[4 * j + 1]), cq.y, bq.y), 0.f);
              x[4 * j + 2] = fmaxf(fmaf(__uint_as_float(v[4 * j + 2]), cq.z, bq.z), 0.f);
              x[4 * j + 3] = fmaxf(fmaf(__uint_as_float(v[4 * j + 3]), cq.w, bq.w), 0.f);
            }
            uint32_t packed[4] = {0u, 0u, 0u, 0u};
            uint32_t sf_pair = 0;
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
              float amax = 0.f;
#pragma unroll
              for (int j = 0; j < 16; ++j) amax = fmaxf(amax, x[16 * blk + j]);
              const __nv_fp8_storage_t sf8 = __nv_cvt_float_to_fp8(amax * (1.f / 6.f) * g.inv_global, __NV_SATFINITE, __NV_E4M3);
              const float sf = __half2float(__half(__nv_cvt_fp8_to_halfraw(sf8, __NV_E4M3)));
              const float inv = sf > 0.f ? g.inv_global / sf : 0.f;
#pragma unroll
              for (int jj = 0; jj < 8; ++jj) {
                const uint32_t p2 = __nv_cvt_float2_to_fp4x2(make_float2(x[16 * blk + 2 * jj] * inv, x[16 * blk + 2 * jj + 1] * inv),
                                                             __NV_E2M1, cudaRoundNearest);
                packed[2 * blk + (jj >> 2)] |= (p2 & 0xffu) << (8 * (jj & 3));
              }
              sf_pair |= (uint32_t)sf8 << (8 * blk);
            }
            // 64-byte swizzle: 16-byte chunk index ^= (row / 2) mod 4 inside 512-byte atoms
            const uint32_t off = (uint32_t)lane * 64u + (((uint32_t)i ^ (((uint32_t)lane >> 1) & 3u)) << 4);
            *reinterpret_cast<uint4*>(box + off) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            // blocks 2 * sub and 2 * sub + 1 of the chunk's sixteen: MMA step sub / 2, factors (sub & 1) * 2 and + 1
            // (the odd CTA of a pair also walks the tile after the last one when the tile count is odd: the TMA store
            // clips it, these plain stores must not happen)
            if (mt < num_mtiles) *reinterpret_cast<uint16_t*>(sf_row + (sub >> 1) * 512 + (sub & 1) * 2) = (uint16_t)sf_pair;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmOut, smem_u32(box), nc * (BN / 2) + sg * 64, row0 + quad * 32);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_even_cta(tempty_bar(b));
          else mbar_arrive(tempty_bar(b));
        }
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  } else {
    // ---- one-hot producers: warp pw owns A stage pw and builds K-blocks pw, pw+4, pw+8, ... of the sequence ----
    constexpr int PROD_W = 12 - EW;          // producer warps
    constexpr int WPG = PROD_W / 4;          // warps per producer group (one group works on one K-block)
    constexpr int ROWS_W = BM / WPG;         // tile rows per warp
    const int pw = (warp - 2 - EW) / WPG;    // producer group of this warp
    const int half = (warp - 2 - EW) % WPG;  // rows half*ROWS_W .. of the block
    const int pt = (warp - 2 - EW) * 32 + lane;  // threads 0..127 load the child tile
    const int V = g.V, n = g.n;
    const int groups = (n + 7) >> 3;  // eight-position groups per value in the column order
    uint32_t it_base = 0;           // index of this tile's first K-block in the CTA's K-block sequence
    bool ok = true;
    for (int mt = tile_first; mt - (int)crank < num_mtiles; mt += tile_step, it_base += (uint32_t)blocks_per_tile) {
      // all producer warps have finished reading the previous tile's child rows
      asm volatile("bar.sync 2, %0;" ::"n"(PROD_W * 32) : "memory");
      if (pt < BM) {
        const int64_t row = (int64_t)mt * BM + pt;
        uint32_t* dst = reinterpret_cast<uint32_t*>(child_s + pt * L1_CHILD_PITCH);
        if (row < rows) {
          const uint4* src = reinterpret_cast<const uint4*>(g.children + row * g.stride);
          for (int q = 0; q < (g.stride >> 4); ++q) {
            const uint4 w = __ldg(src + q);
            dst[4 * q] = w.x; dst[4 * q + 1] = w.y; dst[4 * q + 2] = w.z; dst[4 * q + 3] = w.w;
          }
        } else {
          for (int q = 0; q < (g.stride >> 2); ++q) dst[q] = 0u;
        }
      }
      asm volatile("bar.sync 2, %0;" ::"n"(PROD_W * 32) : "memory");
      if (!ok) continue;
      // first K-block of this tile that belongs to this warp
      const uint32_t first = (uint32_t)((pw - (int)(it_base & 3u)) & 3);
      for (uint32_t j = first; j < (uint32_t)blocks_per_tile; j += L1_PAIRS) {
        const uint32_t it = it_base + j;
        const int kb = (int)(j % (uint32_t)k_blocks);
        const int slot = (int)(it % L1_A_STAGES);
        uint8_t* a_stage = a_ring + slot * A_BYTES;
        if (!mbar_wait(a_empty(slot), ((it / L1_A_STAGES) & 1u) ^ 1u, g.err, ERR_WAIT_EMPTY)) { ok = false; break; }
        // One-hot columns are ordered value-major in groups of eight positions (column = value * 8 * groups +
        // position): a 16-byte chunk of a bf16 row is then "which of these eight positions hold value v", a byte
        // compare of two words of the child row - no zeroing pass, no scattered stores.  (e4m3 rows hold two such
        // groups per chunk.)  A quarter warp writes the eight chunks of one row and the four quarters take four
        // consecutive rows, so every store instruction fills four whole 128-byte rows without bank conflicts.
        const int chunk = lane & 7, rsub = lane >> 3;
        constexpr int GPC = F8 ? 2 : 1;                      // position groups per 16-byte chunk
        uint32_t vv[GPC], m0[GPC], m1[GPC];                  // value replicated into four bytes; valid-position masks
        int boff[GPC];                                       // byte offset of the group in the child row
#pragma unroll
        for (int s = 0; s < GPC; ++s) {
          const int c8 = (kb * 8 + chunk) * GPC + s;         // group index in the column order
          const int v = c8 / groups, gidx = c8 - v * groups;
          const int valid = v < V ? (n - 8 * gidx > 8 ? 8 : n - 8 * gidx) : 0;  // positions of the group that exist
          vv[s] = (uint32_t)v * 0x01010101u;
          m0[s] = valid >= 4 ? 0xffffffffu : (valid > 0 ? (1u << (8 * valid)) - 1u : 0u);
          m1[s] = valid >= 8 ? 0xffffffffu : (valid > 4 ? (1u << (8 * (valid - 4))) - 1u : 0u);
          boff[s] = valid > 0 ? 8 * gidx : 0;
        }
#pragma unroll 4
        for (int rb = 0; rb < ROWS_W; rb += 4) {
          const uint32_t row = (uint32_t)(half * ROWS_W + rb + rsub);
          const uint8_t* crow = child_s + row * L1_CHILD_PITCH;
          uint32_t o[4];
#pragma unroll
          for (int s = 0; s < GPC; ++s) {
            const uint32_t w0 = *reinterpret_cast<const uint32_t*>(crow + boff[s]);
            const uint32_t w1 = *reinterpret_cast<const uint32_t*>(crow + boff[s] + 4);
            const uint32_t e0 = __vcmpeq4(w0, vv[s]) & m0[s];  // 0xff in the bytes whose position holds the value
            const uint32_t e1 = __vcmpeq4(w1, vv[s]) & m1[s];
            if (F8) {                                          // e4m3 1.0 = 0x38 per column
              o[2 * s] = e0 & 0x38383838u;
              o[2 * s + 1] = e1 & 0x38383838u;
            } else {                                           // bf16 1.0 = 0x3f80 per column: each byte doubled
              o[0] = __byte_perm(e0, 0u, 0x1100) & 0x3f803f80u;
              o[1] = __byte_perm(e0, 0u, 0x3322) & 0x3f803f80u;
              o[2] = __byte_perm(e1, 0u, 0x1100) & 0x3f803f80u;
              o[3] = __byte_perm(e1, 0u, 0x3322) & 0x3f803f80u;
            }
          }
          *reinterpret_cast<uint4*>(a_stage + swz128(row, (uint32_t)chunk * 16u)) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        if (PAIR) asm volatile("fence.proxy.async;" ::: "memory");
        else asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_even_cta_release(a_full(slot));  // the even CTA's MMAs read this CTA's block too
          else mbar_arrive(a_full(slot));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // neither CTA leaves while its peer may still read its shared memory
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// children [rows, stride] u8 -> one-hot [rows, k_pad] bf16 in the column order of the layer-1 kernels:
// column = value * 8 * groups + position, groups = ceil(n / 8); 8 columns (one position group of one value) per thread
__global__ void __launch_bounds__(256) k_onehot(const uint8_t* __restrict__ children, const uint32_t* count_dev,
                                                int64_t row_offset, int64_t row_limit, int n, int stride, int V,
                                                int k_pad, __nv_bfloat16* __restrict__ x) {
  int64_t rows = (int64_t)(*count_dev) - row_offset;
  if (rows > row_limit) rows = row_limit;
  const int chunks = k_pad / 8;
  const int groups = (n + 7) >> 3;
  const int64_t total = rows * chunks;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / chunks;
    const int c8 = (int)(i - r * chunks);
    const int val = c8 / groups, p0 = (c8 - val * groups) * 8;
    const uint8_t* row = children + (row_offset + r) * stride;
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t acc = 0;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int pos = p0 + 2 * j + h;
        const bool on = val < V && pos < n && __ldg(row + pos) == val;
        acc |= (on ? 0x3f80u : 0u) << (16 * h);  // bf16 1.0
      }
      w[j] = acc;
    }
    *reinterpret_cast<uint4*>(x + (row_offset + r) * k_pad + c8 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// First layer as an embedding sum, for vocabularies too wide for a one-hot contraction (the reference's 120 values
// per position give K = 14400; kernel_fullbeamnice_embed_relu, beam_kernels.cu:208-237, is the same operation):
//   out[row, h] = bf16(act(bias[h] + sum_pos table[(pos * V + state[pos]) * hidden + h])), float32 accumulation.
// One thread owns 8 adjacent columns of one row, so the threads of a row read one contiguous table row per
// position (16 bytes each); the table (n * V * hidden bf16: 44 MB at 120 x 120 x 1536) stays in L2.
__global__ void __launch_bounds__(256) k_embed_relu(const uint8_t* __restrict__ states, const uint32_t* count_dev,
                                                    int64_t row_limit, int n, int stride, int V, int hidden,
                                                    const __nv_bfloat16* __restrict__ table,
                                                    const float* __restrict__ bias, int gelu,
                                                    __nv_bfloat16* __restrict__ out) {
  int64_t rows = (int64_t)(*count_dev);
  if (rows > row_limit) rows = row_limit;
  const int chunks = hidden / 8;
  const int64_t total = rows * chunks;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / chunks;
    const int c0 = (int)(i - r * chunks) * 8;
    const uint8_t* row = states + r * stride;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = __ldg(bias + c0 + j);
#pragma unroll 4
    for (int pos = 0; pos < n; ++pos) {
      int v = __ldg(row + pos);
      v = v < V ? v : V - 1;  // a value outside the vocabulary must not read outside the table
      const uint4 t4 = __ldg(reinterpret_cast<const uint4*>(table + ((int64_t)pos * V + v) * hidden + c0));
      const uint32_t tw[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&tw[t]));
        acc[2 * t] += f.x;
        acc[2 * t + 1] += f.y;
      }
    }
    uint32_t w[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float x0 = gelu ? gelu_erf(acc[2 * t]) : fmaxf(acc[2 * t], 0.f);
      const float x1 = gelu ? gelu_erf(acc[2 * t + 1]) : fmaxf(acc[2 * t + 1], 0.f);
      __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
      w[t] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(out + r * hidden + c0) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// q (mean over ensemble members) -> u32 key = uint32(clamp(q - offset, 0, 300) * 256 + 0.5)
// (kernel_fullbeamnice_q_to_score_key_ring, beam_kernels.cu:341-344)
__global__ void __launch_bounds__(256) k_q_to_key(const float* __restrict__ q, const uint32_t* count_dev, float inv_models,
                                                  float offset, uint32_t* __restrict__ keys) {
  const int64_t rows = *count_dev;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < rows; i += (int64_t)gridDim.x * blockDim.x) {
    float x = q[i] * inv_models - offset;
    x = fminf(fmaxf(x, 0.f), 300.f);
    keys[i] = (uint32_t)(x * 256.f + 0.5f);
  }
}

// Action values [parents, fanout] (summed over ensemble members) -> score keys of the candidates; candidate
// c = parent * fanout + move reads q[c], so the two arrays share one index.
// key_mode 1, 2: the reference's 16-bit "higher is better" scores (QuantizedActionScorer, scorers.py:38-53:
// sigmoid_u16 = round(sigmoid(y) * 65535), float_u16 = round(y), both clamped to 0..65535) turned into keys by
// key = 65535 - score, so that the order of the legacy engine (larger score first) is kept.
__global__ void __launch_bounds__(256) k_qa_to_key(const float* __restrict__ q, const int32_t* parents_dev, int fanout,
                                                   float inv_models, float offset, int key_mode,
                                                   uint32_t* __restrict__ keys) {
  const int64_t total = (int64_t)(*parents_dev) * fanout;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    float x = q[i] * inv_models;
    if (key_mode == 0) {
      x = fminf(fmaxf(x - offset, 0.f), 300.f);
      keys[i] = (uint32_t)(x * 256.f + 0.5f);
    } else {
      if (key_mode == 1) x = 65535.f / (1.f + expf(-x));
      x = fminf(fmaxf(rintf(x), 0.f), 65535.f);
      keys[i] = 65535u - (uint32_t)x;
    }
  }
}

}  // namespace mgbs

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------

struct MgbsMlp {
  MgbsMlpConfig cfg;
  int sms = 148;
  int k1_pad = 0;
  CUtensorMap tm_x, tm_h1;
  CUtensorMap tm_h1w;  // same tensor, store boxes of one warp: 32 rows x 64 bytes, 64-byte swizzle
  CUtensorMap tm_w1[MGBS_MAX_MODELS], tm_w2[MGBS_MAX_MODELS];
  CUtensorMap tm_w2h[MGBS_MAX_MODELS];  // W2 in boxes of 128 rows: the half of a chunk one CTA of a pair loads
  CUtensorMap tm_w1h[MGBS_MAX_MODELS];  // W1 likewise
  CUtensorMap tm_h1q, tm_w2q[MGBS_MAX_MODELS];  // NVFP4: packed activations and weights as byte tensors
  CUtensorMap tm_h1qw;                          // packed activations, store boxes of one warp: 32 rows x 64 bytes
  CUtensorMap tm_w2qw[MGBS_MAX_MODELS];         // packed weights in boxes of 256 rows (the wide head kernel)
  int pair_clusters = 0;                // CTA pairs that can be resident at once (0: pairs unavailable)
  int l1_pair_clusters = 0;             // the same for the layer-1 kernel
  bool head_pair = true;
  bool fused_l1 = true;
  bool fused_quant = true;  // NVFP4: the layer-1 epilogue writes packed 4-bit activations itself
  int l1_ew = 0, l1_pair = -1;  // layer-1 kernel variant: 0 / -1 = chosen by operand type
  bool f4_wide = true;          // NVFP4 head: 256-column tiles (see mgbs_nvfp4.cu)
  bool profile = false;
  cudaEvent_t ev[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
};

using mgbs::make_map;

// Address of the layer-1 kernel instance for (e4m3 operands, epilogue warps, CTA pairs, NVFP4 output).
static const void* l1_variant(int f8, int ew, int pair, int out4) {
  using namespace mgbs;
  if (out4) return pair ? (const void*)k_mlp_l1<1, 8, 1, 1> : (const void*)k_mlp_l1<1, 8, 0, 1>;
#define MGBS_L1_CASE(F, E, P) \
  if (f8 == F && ew == E && pair == P) return (const void*)k_mlp_l1<F, E, P, 0>;
  MGBS_L1_CASE(0, 4, 0) MGBS_L1_CASE(0, 4, 1) MGBS_L1_CASE(0, 8, 0) MGBS_L1_CASE(0, 8, 1)
  MGBS_L1_CASE(1, 4, 0) MGBS_L1_CASE(1, 4, 1) MGBS_L1_CASE(1, 8, 0) MGBS_L1_CASE(1, 8, 1)
#undef MGBS_L1_CASE
  return nullptr;
}
using mgbs::make_map_bf16;

#define MGBS_SC_TRY(expr)       \
  do {                          \
    int _e = (int)(expr);       \
    if (_e != 0) return _e;     \
  } while (0)

extern "C" {

int mgbs_sizeof_mlp_config(void) { return (int)sizeof(MgbsMlpConfig); }

int mgbs_mlp_create(const MgbsMlpConfig* cfg, MgbsMlp** out) {
  if (!cfg || !out) return MGBS_ERR_ARG;
  const MgbsMlpConfig& c = *cfg;
  if (c.state_len < 1 || c.state_len > MGBS_MAX_STATE_LEN || c.num_values < 1 || c.num_values > 256) return MGBS_ERR_ARG;
  if (c.hidden < mgbs::BN || c.hidden % mgbs::BN != 0) return MGBS_ERR_UNSUPPORTED;
  if (c.num_models < 1 || c.num_models > MGBS_MAX_MODELS || c.max_rows < 1) return MGBS_ERR_ARG;
  const int k1 = mgbs::onehot_columns(c.state_len, c.num_values);
  if (c.dtype != 0 && c.dtype != 1 && c.dtype != 2) return MGBS_ERR_ARG;
  const int f4 = c.dtype == 2;
  const int f8 = c.dtype == 1 || f4;  // NVFP4 runs layer 1 on the e4m3 path
  if (f4 && (!c.h1q || !c.sf_h1 || !(c.act4_inv_global > 0.f))) return MGBS_ERR_ARG;
  const int kblk = f8 ? mgbs::BK8 : mgbs::BK;
  const int eb = f8 ? 1 : 2;
  const int k1_pad = (k1 + kblk - 1) / kblk * kblk;
  if (c.k1_pad != k1_pad || k1_pad / kblk > mgbs::L1_MAX_KBLOCKS) return MGBS_ERR_ARG;
  if ((!f8 && !c.x) || !c.h1 || !c.q || !c.err) return MGBS_ERR_ARG;
  if (f8 && !(c.act_inv_scale > 0.f)) return MGBS_ERR_ARG;
  MgbsMlp* m = new (std::nothrow) MgbsMlp();
  if (!m) return MGBS_ERR_STATE;
  m->cfg = c;
  m->k1_pad = k1_pad;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) m->sms = sms;
  }
  const uint64_t rows_pad = ((uint64_t)c.max_rows + mgbs::BM - 1) / mgbs::BM * mgbs::BM;
  int rc = 0;
  if (!f8) rc = make_map(&m->tm_x, c.x, rows_pad, (uint64_t)k1_pad, mgbs::BM, eb);
  if (!rc) rc = make_map(&m->tm_h1, c.h1, rows_pad, (uint64_t)c.hidden, mgbs::BM, eb);
  if (!rc) rc = mgbs::make_map_box(&m->tm_h1w, c.h1, rows_pad, (uint64_t)c.hidden, 32, 64 / eb, eb, 64);
  for (int i = 0; i < c.num_models && !rc; ++i) {
    if (!c.w1[i] || !c.b1[i] || !c.w2[i] || !c.b2[i] || !c.w3[i]) rc = MGBS_ERR_ARG;
    if (!rc && f8 && (!c.s1[i] || !c.s2[i])) rc = MGBS_ERR_ARG;
    if (!rc) rc = make_map(&m->tm_w1[i], c.w1[i], (uint64_t)c.hidden, (uint64_t)k1_pad, mgbs::BN, eb);
    if (!rc) rc = make_map(&m->tm_w1h[i], c.w1[i], (uint64_t)c.hidden, (uint64_t)k1_pad, mgbs::BN / 2, eb);
    if (f4) {
      if (!rc && !c.sf_w2[i]) rc = MGBS_ERR_ARG;
      if (!rc) rc = make_map(&m->tm_w2q[i], c.w2[i], (uint64_t)c.hidden, (uint64_t)c.hidden / 2, 128, 1);
      if (!rc) rc = make_map(&m->tm_w2qw[i], c.w2[i], (uint64_t)c.hidden, (uint64_t)c.hidden / 2, 256, 1);
      continue;
    }
    if (!rc) rc = make_map(&m->tm_w2[i], c.w2[i], (uint64_t)c.hidden, (uint64_t)c.hidden, mgbs::BN, eb);
    if (!rc) rc = make_map(&m->tm_w2h[i], c.w2[i], (uint64_t)c.hidden, (uint64_t)c.hidden, mgbs::BN / 2, eb);
  }
  if (f4 && !rc) rc = make_map(&m->tm_h1q, c.h1q, rows_pad, (uint64_t)c.hidden / 2, mgbs::BM, 1);
  if (f4 && !rc) rc = mgbs::make_map_box(&m->tm_h1qw, c.h1q, rows_pad, (uint64_t)c.hidden / 2, 32, 64, 1, 64);
  if (f4 && !rc) rc = mgbs::nvfp4_prepare();
  if (f8) m->fused_l1 = true;
  if (!rc) rc = (int)cudaFuncSetAttribute(mgbs::k_mlp_gemm<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, mgbs::GEMM_SMEM);
  if (!rc) rc = (int)cudaFuncSetAttribute(mgbs::k_mlp_gemm<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, mgbs::GEMM_SMEM);
  auto l1_smem = [&](const void* fn) {
    if (!rc) rc = (int)cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, mgbs::L1_SMEM);
  };
  for (int v = 0; v < 8; ++v) l1_smem(l1_variant(v & 1, v & 2 ? 8 : 4, (v >> 2) & 1, 0));
  l1_smem(l1_variant(1, 8, 0, 1));
  l1_smem(l1_variant(1, 8, 1, 1));
  if (!rc) rc = (int)cudaFuncSetAttribute(mgbs::k_mlp_gemm<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, mgbs::GEMM_SMEM);
  if (!rc) rc = (int)cudaFuncSetAttribute(mgbs::k_mlp_head_pair<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, mgbs::PAIR_SMEM);
  if (!rc) rc = (int)cudaFuncSetAttribute(mgbs::k_mlp_head_pair<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, mgbs::PAIR_SMEM);
  if (!rc) {
    // how many CTA pairs the device can hold at once: the grid of the pair kernel
    cudaLaunchConfig_t lc;
    memset(&lc, 0, sizeof(lc));
    lc.gridDim = dim3(2 * (m->sms / 2));
    lc.blockDim = dim3(mgbs::GEMM_THREADS);
    lc.dynamicSmemBytes = mgbs::PAIR_SMEM;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    lc.attrs = at;
    lc.numAttrs = 1;
    int nclusters = 0;
    if (cudaOccupancyMaxActiveClusters(&nclusters, mgbs::k_mlp_head_pair<0>, &lc) == cudaSuccess && nclusters > 0)
      m->pair_clusters = nclusters < m->sms / 2 ? nclusters : m->sms / 2;
    else
      (void)cudaGetLastError();
    if (m->pair_clusters < 1) m->head_pair = false;
    lc.blockDim = dim3(mgbs::L1_THREADS);
    lc.dynamicSmemBytes = mgbs::L1_SMEM;
    nclusters = 0;
    if (cudaOccupancyMaxActiveClusters(&nclusters, (const void*)mgbs::k_mlp_l1<1, 8, 1>, &lc) == cudaSuccess && nclusters > 0)
      m->l1_pair_clusters = nclusters < m->sms / 2 ? nclusters : m->sms / 2;
    else
      (void)cudaGetLastError();
  }
  if (rc) { delete m; return rc; }
  *out = m;
  return 0;
}

int mgbs_mlp_destroy(MgbsMlp* m) {
  if (m)
    for (int i = 0; i < 5; ++i)
      if (m->ev[i]) cudaEventDestroy(m->ev[i]);
  delete m;
  return 0;
}

int mgbs_mlp_set_head_mode(MgbsMlp* m, int32_t pair) {
  if (!m) return MGBS_ERR_ARG;
  if (m->cfg.dtype == 2) {  // NVFP4: 1 = the head with 256-column tiles, 0 = 128-column tiles and two accumulators
    m->f4_wide = pair != 0;
    return 0;
  }
  if (pair && m->pair_clusters < 1) return MGBS_ERR_UNSUPPORTED;
  m->head_pair = pair != 0;
  return 0;
}

int mgbs_mlp_set_l1_mode(MgbsMlp* m, int32_t fused) {
  if (!m) return MGBS_ERR_ARG;
  if (m->cfg.dtype == 2) {  // NVFP4: fused = layer-1 epilogue quantises; 0 = e4m3 activations + a separate pass
    m->fused_quant = fused != 0;
    return 0;
  }
  if (m->cfg.dtype != 0 && !fused) return MGBS_ERR_UNSUPPORTED;  // the e4m3 path has no separate one-hot matrix
  m->fused_l1 = fused != 0;
  return 0;
}

int mgbs_mlp_set_l1_variant(MgbsMlp* m, int32_t epilogue_warps, int32_t pair) {
  if (!m) return MGBS_ERR_ARG;
  if ((epilogue_warps != 0 && epilogue_warps != 4 && epilogue_warps != 8) || pair < -1 || pair > 1) return MGBS_ERR_ARG;
  m->l1_ew = epilogue_warps;
  m->l1_pair = pair;
  return 0;
}

int mgbs_mlp_profile(MgbsMlp* m, int32_t on) {
  if (!m) return MGBS_ERR_ARG;
  if (on)
    for (int i = 0; i < 5; ++i)
      if (!m->ev[i]) {
        cudaError_t e = cudaEventCreate(&m->ev[i]);
        if (e != cudaSuccess) return (int)e;
      }
  m->profile = on != 0;
  return 0;
}

int mgbs_mlp_profile_read(MgbsMlp* m, float* ms4) {
  if (!m || !ms4 || !m->ev[0]) return MGBS_ERR_ARG;
  cudaError_t e = cudaEventSynchronize(m->ev[4]);
  if (e != cudaSuccess) return (int)e;
  for (int i = 0; i < 4; ++i) {
    e = cudaEventElapsedTime(&ms4[i], m->ev[i], m->ev[i + 1]);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

int mgbs_mlp_enqueue(void* user, const uint8_t* children, const uint32_t* count_dev, uint32_t* scores, void* stream) {
  MgbsMlp* m = static_cast<MgbsMlp*>(user);
  if (!m || !children || !count_dev || !scores) return MGBS_ERR_ARG;
  using namespace mgbs;
  const MgbsMlpConfig& c = m->cfg;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rows_cap = c.max_rows;
  const int grid_gemm = m->sms;
  const bool prof = m->profile && c.num_models == 1;
  const bool f4 = c.dtype == 2;
  const bool e4 = c.dtype == 1 || f4;  // layer 1 on the e4m3 path
  if (prof) cudaEventRecord(m->ev[0], st);
  if (!m->fused_l1) {
    const int64_t chunks = rows_cap * (m->k1_pad / 8);
    int64_t g = (chunks + 255) / 256;
    if (g > (int64_t)m->sms * 16) g = (int64_t)m->sms * 16;
    k_onehot<<<(int)g, 256, 0, st>>>(children, count_dev, 0, rows_cap, c.state_len, c.state_stride, c.num_values,
                                     m->k1_pad, reinterpret_cast<__nv_bfloat16*>(c.x));
  }
  for (int i = 0; i < c.num_models; ++i) {
    GemmArgs g;
    g.count_dev = count_dev;
    g.row_offset = 0;
    g.row_limit = rows_cap;
    g.n_total = c.hidden;
    g.k_total = m->k1_pad;
    g.bias = c.b1[i];
    g.col_scale = nullptr;
    g.w_out = nullptr;
    g.out_bf16 = reinterpret_cast<__nv_bfloat16*>(c.h1);
    g.out_q = nullptr;
    g.accumulate_q = 0;
    g.err = c.err;
    if (prof) cudaEventRecord(m->ev[1], st);
    bool quant_in_l1 = false;
    if (m->fused_l1) {
      L1Args l;
      l.children = children;
      l.count_dev = count_dev;
      l.row_limit = rows_cap;
      l.n = c.state_len; l.stride = c.state_stride; l.V = c.num_values;
      l.n_total = c.hidden;
      l.k_total = m->k1_pad;
      l.k_real = onehot_columns(c.state_len, c.num_values);
      l.bias = c.b1[i];
      l.col_scale = c.s1[i];
      l.out_inv_scale = c.act_inv_scale;
      l.sf_out = c.sf_h1;
      l.inv_global = c.act4_inv_global;
      l.err = c.err;
      const bool resident = m->k1_pad / (e4 ? BK8 : BK) <= L1_A_STAGES;
      quant_in_l1 = f4 && m->fused_quant && resident;
      // Variant: epilogue warps (the other producer warps build the one-hot operand) and CTA pairs.
      // Defaults by operand type; mgbs_mlp_set_l1_variant overrides them.  The ring form (K > 384) needs the eight
      // producer warps; CTA pairs need a device that can co-schedule them.
      int ew = m->l1_ew ? m->l1_ew : (e4 && resident ? 8 : 4);
      int pair = m->l1_pair >= 0 ? m->l1_pair : 0;  // measured: 0.39 vs 0.41 ms (e4m3), 0.55 vs 0.59-0.63 ms (bf16)
      if (!resident) ew = 4;
      if (!(m->head_pair && m->l1_pair_clusters > 0 && resident)) pair = 0;
      if (quant_in_l1) ew = 8;
      const void* fn = l1_variant(e4 ? 1 : 0, ew, pair, quant_in_l1 ? 1 : 0);
      if (!fn) return MGBS_ERR_STATE;
      const CUtensorMap* tm_b = pair ? &m->tm_w1h[i] : &m->tm_w1[i];
      const CUtensorMap* tm_o = quant_in_l1 ? &m->tm_h1qw : &m->tm_h1w;  // boxes of one warp: 32 rows x 64 bytes
      void* kargs[3] = {(void*)tm_b, (void*)tm_o, (void*)&l};
      cudaLaunchConfig_t lc;
      memset(&lc, 0, sizeof(lc));
      lc.gridDim = dim3(pair ? 2 * m->l1_pair_clusters : grid_gemm);
      lc.blockDim = dim3(L1_THREADS);
      lc.dynamicSmemBytes = L1_SMEM;
      lc.stream = st;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = pair ? 2 : 1; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      lc.attrs = at;
      lc.numAttrs = 1;
      cudaError_t le = cudaLaunchKernelExC(&lc, fn, kargs);
      if (le != cudaSuccess) return (int)le;
    } else {
      k_mlp_gemm<0, 0><<<grid_gemm, GEMM_THREADS, GEMM_SMEM, st>>>(m->tm_x, m->tm_w1[i], g);
    }
    if (prof) cudaEventRecord(m->ev[2], st);
    g.k_total = c.hidden;
    g.bias = c.b2[i];
    g.w_out = c.w3[i];
    g.out_bf16 = nullptr;
    g.out_q = c.q;
    g.accumulate_q = i > 0 ? 1 : 0;
    g.col_scale = c.s2[i];
    if (f4) {
      // e4m3 activations -> NVFP4 (packed elements + block factors) unless the layer-1 epilogue wrote them already,
      // then the block-scaled 4-bit GEMM + head
      if (!quant_in_l1)
      MGBS_SC_TRY(launch_quant_h1_nvfp4(reinterpret_cast<const uint8_t*>(c.h1), count_dev, rows_cap, c.hidden,
                                        1.f / c.act_inv_scale, c.act4_inv_global, reinterpret_cast<uint8_t*>(c.h1q),
                                        c.sf_h1, m->sms, st));
      Nvfp4HeadArgs h;
      h.count_dev = count_dev;
      h.row_limit = rows_cap;
      h.n_total = c.hidden;
      h.k_total = c.hidden;
      h.sfa = c.sf_h1;
      h.sfb = c.sf_w2[i];
      h.bias = c.b2[i];
      h.col_scale = c.s2[i];
      h.w_out = c.w3[i];
      h.out_q = c.q;
      h.accumulate_q = i > 0 ? 1 : 0;
      h.err = c.err;
      MGBS_SC_TRY(launch_head_nvfp4(m->tm_h1q, m->tm_w2q[i], m->tm_w2qw[i], h, m->sms, st, m->f4_wide ? 1 : 0));
    } else if (m->head_pair && m->pair_clusters > 0) {
      cudaLaunchConfig_t lc;
      memset(&lc, 0, sizeof(lc));
      lc.gridDim = dim3(2 * m->pair_clusters);
      lc.blockDim = dim3(GEMM_THREADS);
      lc.dynamicSmemBytes = PAIR_SMEM;
      lc.stream = st;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      lc.attrs = at;
      lc.numAttrs = 1;
      cudaError_t le = c.dtype == 1 ? cudaLaunchKernelEx(&lc, k_mlp_head_pair<1>, m->tm_h1, m->tm_w2h[i], g)
                                    : cudaLaunchKernelEx(&lc, k_mlp_head_pair<0>, m->tm_h1, m->tm_w2h[i], g);
      if (le != cudaSuccess) return (int)le;
    } else if (c.dtype == 1) {
      k_mlp_gemm<1, 1><<<grid_gemm, GEMM_THREADS, GEMM_SMEM, st>>>(m->tm_h1, m->tm_w2[i], g);
    } else {
      k_mlp_gemm<1, 0><<<grid_gemm, GEMM_THREADS, GEMM_SMEM, st>>>(m->tm_h1, m->tm_w2[i], g);
    }
    if (prof) cudaEventRecord(m->ev[3], st);
  }
  {
    int64_t g = (rows_cap + 255) / 256;
    if (g > (int64_t)m->sms * 8) g = (int64_t)m->sms * 8;
    float b3 = 0.f;
    for (int i = 0; i < c.num_models; ++i) b3 += c.b3[i];
    // mean over members of (q_i + b3_i) - offset
    k_q_to_key<<<(int)g, 256, 0, st>>>(c.q, count_dev, 1.f / (float)c.num_models, c.score_offset - b3 / (float)c.num_models, scores);
  }
  if (prof) cudaEventRecord(m->ev[4], st);
  return (int)cudaGetLastError();
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Action-value scorer: one-hot -> hidden1 -> hidden2 -> fanout on the parent rows.
// ------------------------------------------------------------------------------------------------

struct MgbsQmlp {
  MgbsQmlpConfig cfg;
  int sms = 148;
  CUtensorMap tm_h1, tm_h1w, tm_h2, tm_h3;
  CUtensorMap tm_w1[MGBS_MAX_MODELS], tm_w2[MGBS_MAX_MODELS], tm_w3[MGBS_MAX_MODELS];
  CUtensorMap tm_wr[2 * MGBS_MAX_RES_BLOCKS][MGBS_MAX_MODELS];
};

extern "C" {

int mgbs_sizeof_qmlp_config(void) { return (int)sizeof(MgbsQmlpConfig); }

int mgbs_qmlp_create(const MgbsQmlpConfig* cfg, MgbsQmlp** out) {
  if (!cfg || !out) return MGBS_ERR_ARG;
  const MgbsQmlpConfig& c = *cfg;
  if (c.state_len < 1 || c.state_len > MGBS_MAX_STATE_LEN || c.num_values < 1 || c.num_values > 256) return MGBS_ERR_ARG;
  if (c.fanout < 1 || c.fanout > MGBS_MAX_FANOUT) return MGBS_ERR_ARG;
  if (c.hidden1 < mgbs::BN || c.hidden1 % mgbs::BN != 0 || c.hidden2 < mgbs::BN || c.hidden2 % mgbs::BN != 0) return MGBS_ERR_UNSUPPORTED;
  if (c.num_models < 1 || c.num_models > MGBS_MAX_MODELS || c.max_parents < 1) return MGBS_ERR_ARG;
  const int k1 = mgbs::onehot_columns(c.state_len, c.num_values);
  const int k1_pad = (k1 + mgbs::BK - 1) / mgbs::BK * mgbs::BK;
  if (c.embed_sum != 0 && c.embed_sum != 1) return MGBS_ERR_ARG;
  if (c.key_mode < 0 || c.key_mode > 2 || c.activation < 0 || c.activation > 1) return MGBS_ERR_ARG;
  if (c.activation == 1 && !c.embed_sum) return MGBS_ERR_UNSUPPORTED;  // the one-hot contraction kernel is ReLU only
  if (!c.embed_sum && (c.k1_pad != k1_pad || k1_pad / mgbs::BK > mgbs::L1_MAX_KBLOCKS)) return MGBS_ERR_ARG;
  if (c.state_stride < c.state_len || c.state_stride % 16 != 0 || c.state_stride > MGBS_MAX_STATE_LEN) return MGBS_ERR_ARG;
  if (!c.h1 || !c.h2 || !c.q || !c.err) return MGBS_ERR_ARG;
  if (c.num_res_blocks < 0 || c.num_res_blocks > MGBS_MAX_RES_BLOCKS || (c.num_res_blocks > 0 && !c.h3)) return MGBS_ERR_ARG;
  MgbsQmlp* m = new (std::nothrow) MgbsQmlp();
  if (!m) return MGBS_ERR_STATE;
  m->cfg = c;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) m->sms = sms;
  }
  const uint64_t rows_pad = (uint64_t)((c.max_parents + mgbs::BM - 1) / mgbs::BM * mgbs::BM);
  int rc = make_map_bf16(&m->tm_h1, c.h1, rows_pad, (uint64_t)c.hidden1, mgbs::BM);
  if (!rc) rc = mgbs::make_map_box(&m->tm_h1w, c.h1, rows_pad, (uint64_t)c.hidden1, 32, 32, 2, 64);
  if (!rc) rc = make_map_bf16(&m->tm_h2, c.h2, rows_pad, (uint64_t)c.hidden2, mgbs::BM);
  if (!rc && c.num_res_blocks > 0) rc = make_map_bf16(&m->tm_h3, c.h3, rows_pad, (uint64_t)c.hidden2, mgbs::BM);
  for (int i = 0; i < c.num_models && !rc; ++i) {
    if (!(c.embed_sum ? c.w1t[i] : c.w1[i]) || !c.b1[i] || !c.w2[i] || !c.b2[i] || !c.w3[i] || !c.b3[i]) { rc = MGBS_ERR_ARG; break; }
    if (!c.embed_sum) rc = make_map_bf16(&m->tm_w1[i], c.w1[i], (uint64_t)c.hidden1, (uint64_t)k1_pad, mgbs::BN);
    if (!rc) rc = make_map_bf16(&m->tm_w2[i], c.w2[i], (uint64_t)c.hidden2, (uint64_t)c.hidden1, mgbs::BN);
    if (!rc) rc = make_map_bf16(&m->tm_w3[i], c.w3[i], (uint64_t)mgbs::BN, (uint64_t)c.hidden2, mgbs::BN);
    for (int l = 0; l < 2 * c.num_res_blocks && !rc; ++l) {
      if (!c.wr[l][i] || !c.br[l][i]) { rc = MGBS_ERR_ARG; break; }
      rc = make_map_bf16(&m->tm_wr[l][i], c.wr[l][i], (uint64_t)c.hidden2, (uint64_t)c.hidden2, mgbs::BN);
    }
  }
  if (!rc) rc = (int)cudaFuncSetAttribute(mgbs::k_mlp_gemm<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, mgbs::GEMM_SMEM);
  if (!rc) rc = (int)cudaFuncSetAttribute(mgbs::k_mlp_gemm<2, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, mgbs::GEMM_SMEM);
  if (!rc) rc = (int)cudaFuncSetAttribute(mgbs::k_mlp_l1<0, 4, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, mgbs::L1_SMEM);
  if (rc) { delete m; return rc; }
  *out = m;
  return 0;
}

int mgbs_qmlp_destroy(MgbsQmlp* m) {
  delete m;
  return 0;
}

int mgbs_qmlp_enqueue(void* user, const uint8_t* parents, const int32_t* parent_count_dev, uint32_t* cand_scores,
                      void* stream) {
  MgbsQmlp* m = static_cast<MgbsQmlp*>(user);
  if (!m || !parents || !parent_count_dev || !cand_scores) return MGBS_ERR_ARG;
  using namespace mgbs;
  const MgbsQmlpConfig& c = m->cfg;
  cudaStream_t st = (cudaStream_t)stream;
  const uint32_t* count_dev = reinterpret_cast<const uint32_t*>(parent_count_dev);  // never negative
  const int grid = m->sms;
  for (int i = 0; i < c.num_models; ++i) {
    L1Args l;
    l.children = parents;
    l.count_dev = count_dev;
    l.row_limit = c.max_parents;
    l.n = c.state_len; l.stride = c.state_stride; l.V = c.num_values;
    l.n_total = c.hidden1;
    l.k_total = c.k1_pad;
    l.k_real = onehot_columns(c.state_len, c.num_values);
    l.bias = c.b1[i];
    l.col_scale = nullptr;
    l.out_inv_scale = 1.f;
    l.sf_out = nullptr;
    l.inv_global = 0.f;
    l.err = c.err;
    if (c.embed_sum)
      k_embed_relu<<<m->sms * 8, 256, 0, st>>>(parents, count_dev, c.max_parents, c.state_len, c.state_stride, c.num_values,
                                               c.hidden1, reinterpret_cast<const __nv_bfloat16*>(c.w1t[i]), c.b1[i],
                                               c.activation, reinterpret_cast<__nv_bfloat16*>(c.h1));
    else
      k_mlp_l1<0, 4, 0><<<grid, L1_THREADS, L1_SMEM, st>>>(m->tm_w1[i], m->tm_h1w, l);
    GemmArgs g;
    g.count_dev = count_dev;
    g.row_offset = 0;
    g.row_limit = c.max_parents;
    g.n_total = c.hidden2;
    g.k_total = c.hidden1;
    g.bias = c.b2[i];
    g.col_scale = nullptr;
    g.w_out = nullptr;
    g.out_bf16 = reinterpret_cast<__nv_bfloat16*>(c.h2);
    g.out_q = nullptr;
    g.accumulate_q = 0;
    g.q_cols = 0;
    g.gelu = c.activation;
    g.err = c.err;
    k_mlp_gemm<0, 0><<<grid, GEMM_THREADS, GEMM_SMEM, st>>>(m->tm_h1, m->tm_w2[i], g);
    for (int b = 0; b < c.num_res_blocks; ++b) {  // x (in h2) = relu(relu(x Wa^T + ba) Wb^T + bb + x), h3 in between
      g.k_total = c.hidden2;
      g.bias = c.br[2 * b][i];
      g.out_bf16 = reinterpret_cast<__nv_bfloat16*>(c.h3);
      g.resid = nullptr;
      k_mlp_gemm<0, 0><<<grid, GEMM_THREADS, GEMM_SMEM, st>>>(m->tm_h2, m->tm_wr[2 * b][i], g);
      g.bias = c.br[2 * b + 1][i];
      g.out_bf16 = reinterpret_cast<__nv_bfloat16*>(c.h2);
      g.resid = reinterpret_cast<const __nv_bfloat16*>(c.h2);  // in place: A is h3, each thread adds what it overwrites
      k_mlp_gemm<0, 0><<<grid, GEMM_THREADS, GEMM_SMEM, st>>>(m->tm_h3, m->tm_wr[2 * b + 1][i], g);
    }
    g.resid = nullptr;
    g.n_total = BN;  // output layer padded to one 256-column chunk
    g.k_total = c.hidden2;
    g.bias = c.b3[i];
    g.out_bf16 = nullptr;
    g.out_q = c.q;
    g.accumulate_q = i > 0 ? 1 : 0;
    g.q_cols = c.fanout;
    k_mlp_gemm<2, 0><<<grid, GEMM_THREADS, GEMM_SMEM, st>>>(m->tm_h2, m->tm_w3[i], g);
  }
  k_qa_to_key<<<m->sms * 4, 256, 0, st>>>(c.q, parent_count_dev, c.fanout, 1.f / (float)c.num_models, c.score_offset,
                                          c.key_mode, cand_scores);
  return (int)cudaGetLastError();
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free scoring for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the moment they need scores: code running inside a
// stream-ordered region that forbids allocation, plugins whose memory budget is fixed at load time, or callers
// holding locks that an allocating runtime call could take.  For them the scratch that mgbs_mlp_enqueue takes from
// caller-allocated buffers (one-hot activations, first-layer activations, head outputs, the error word and the row
// count) lives in one file-scope device array.  Every device that loads the library holds these bytes until the
// process exits.
// ------------------------------------------------------------------------------------------------

constexpr int kNoAllocMaxRows = MGBS_NOALLOC_MAX_ROWS;
constexpr int kNoAllocMaxK1 = MGBS_NOALLOC_MAX_K1;
constexpr int kNoAllocMaxHidden = MGBS_NOALLOC_MAX_HIDDEN;
constexpr size_t kNaX = (size_t)kNoAllocMaxRows * kNoAllocMaxK1 * 2;          // bf16 one-hot rows
constexpr size_t kNaH1 = (size_t)kNoAllocMaxRows * kNoAllocMaxHidden * 2;     // bf16 first-layer activations
constexpr size_t kNaQ = (size_t)kNoAllocMaxRows * 4;                           // f32 head outputs
constexpr size_t kNaOffX = 0, kNaOffH1 = kNaOffX + kNaX, kNaOffQ = kNaOffH1 + kNaH1, kNaOffWords = kNaOffQ + kNaQ;
constexpr size_t kNaTotal = kNaOffWords + 256;                                 // [0] row count, [1] error word

static __device__ __align__(256) uint8_t g_noalloc_scratch[kNaTotal];

namespace {

constexpr int kMaxDevices = 64;
// Device address of g_noalloc_scratch per device ordinal.  In host code the array's name is only a stand-in for
// the symbol; the address a kernel may use comes from cudaGetSymbolAddress, asked once per device with that
// device current.
uint8_t* g_noalloc_base[kMaxDevices] = {nullptr};

__global__ void k_noalloc_begin(uint32_t* words, uint32_t rows) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    words[0] = rows;  // the row count the kernels read
    words[1] = 0;     // error word starts clean: the array keeps whatever the previous call left
  }
}

}  // namespace

extern "C" int mgbs_mlp_score_noalloc(const MgbsMlpNoAllocArgs* a, const uint8_t* children, int32_t rows,
                                      uint32_t* scores, int32_t* err_out_host, void* stream) {
  using namespace mgbs;
  if (!a || !children || !scores || rows < 0) return MGBS_ERR_ARG;
  if (!a->w1 || !a->b1 || !a->w2 || !a->b2 || !a->w3) return MGBS_ERR_ARG;
  if (a->state_len < 1 || a->state_len > MGBS_MAX_STATE_LEN || a->num_values < 1 || a->num_values > 256) return MGBS_ERR_ARG;
  if (a->state_stride < a->state_len || a->state_stride % 16 != 0) return MGBS_ERR_ARG;
  const int k1_pad = (onehot_columns(a->state_len, a->num_values) + BK - 1) / BK * BK;
  if (a->hidden < BN || a->hidden % BN != 0) return MGBS_ERR_UNSUPPORTED;
  // sizes beyond the static scratch are refused, never truncated
  if (rows > kNoAllocMaxRows || k1_pad > kNoAllocMaxK1 || a->hidden > kNoAllocMaxHidden) return MGBS_ERR_TOO_LARGE;
  if (rows == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  int dev = -1;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return (int)ce;
  if (dev < 0 || dev >= kMaxDevices) return MGBS_ERR_UNSUPPORTED;
  if (!g_noalloc_base[dev]) {
    // first call on this device: resolve the symbol's device address and raise the kernels' shared-memory limit
    void* p = nullptr;
    ce = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (ce != cudaSuccess) return (int)ce;
    ce = cudaFuncSetAttribute(k_mlp_gemm<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    if (ce != cudaSuccess) return (int)ce;
    ce = cudaFuncSetAttribute(k_mlp_gemm<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    if (ce != cudaSuccess) return (int)ce;
    g_noalloc_base[dev] = static_cast<uint8_t*>(p);
  }
  uint8_t* base = g_noalloc_base[dev];
  __nv_bfloat16* x = reinterpret_cast<__nv_bfloat16*>(base + kNaOffX);
  __nv_bfloat16* h1 = reinterpret_cast<__nv_bfloat16*>(base + kNaOffH1);
  float* q = reinterpret_cast<float*>(base + kNaOffQ);
  uint32_t* words = reinterpret_cast<uint32_t*>(base + kNaOffWords);
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);

  // TMA descriptors are host-side objects; encoding them allocates nothing
  CUtensorMap tm_x, tm_h1, tm_w1, tm_w2;
  const uint64_t rows_pad = (uint64_t)kNoAllocMaxRows;  // multiple of 128
  int rc = make_map_bf16(&tm_x, x, rows_pad, (uint64_t)k1_pad, BM);
  if (!rc) rc = make_map_bf16(&tm_h1, h1, rows_pad, (uint64_t)a->hidden, BM);
  if (!rc) rc = make_map_bf16(&tm_w1, a->w1, (uint64_t)a->hidden, (uint64_t)k1_pad, BN);
  if (!rc) rc = make_map_bf16(&tm_w2, a->w2, (uint64_t)a->hidden, (uint64_t)a->hidden, BN);
  if (rc) return rc;

  k_noalloc_begin<<<1, 32, 0, st>>>(words, (uint32_t)rows);
  {
    const int64_t chunks = (int64_t)rows * (k1_pad / 8);
    int64_t g = (chunks + 255) / 256;
    if (g > (int64_t)sms * 16) g = (int64_t)sms * 16;
    k_onehot<<<(int)g, 256, 0, st>>>(children, words, 0, rows, a->state_len, a->state_stride, a->num_values, k1_pad, x);
  }
  GemmArgs g;
  g.count_dev = words;
  g.row_offset = 0;
  g.row_limit = rows;
  g.n_total = a->hidden;
  g.k_total = k1_pad;
  g.bias = a->b1;
  g.col_scale = nullptr;
  g.w_out = nullptr;
  g.out_bf16 = h1;
  g.out_q = nullptr;
  g.accumulate_q = 0;
  g.err = reinterpret_cast<int*>(words + 1);
  k_mlp_gemm<0, 0><<<sms, GEMM_THREADS, GEMM_SMEM, st>>>(tm_x, tm_w1, g);
  g.k_total = a->hidden;
  g.bias = a->b2;
  g.w_out = a->w3;
  g.out_bf16 = nullptr;
  g.out_q = q;
  k_mlp_gemm<1, 0><<<sms, GEMM_THREADS, GEMM_SMEM, st>>>(tm_h1, tm_w2, g);
  {
    int64_t gq = ((int64_t)rows + 255) / 256;
    k_q_to_key<<<(int)gq, 256, 0, st>>>(q, words, 1.f, a->score_offset - a->b3, scores);
  }
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return (int)ce;
  if (err_out_host) {
    // optional: wait for the call and hand back the error word (0 = every bounded wait completed)
    ce = cudaMemcpyAsync(err_out_host, words + 1, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
    if (ce != cudaSuccess) return (int)ce;
  }
  return 0;
}

