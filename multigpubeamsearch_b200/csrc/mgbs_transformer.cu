// Transformer value scorer for sm_100a: an ensemble of pre-LayerNorm encoders (token + position embedding,
// L layers of multi-head self-attention and a GELU feed-forward block, final LayerNorm, mean pooling, scalar head)
// evaluated on every child state.  All projections (QKV, attention output, both feed-forward matrices) run as
// tcgen05 GEMMs fed by TMA with accumulators in tensor memory; LayerNorm, the 54-token attention core and the
// pooling head are bandwidth/latency kernels on the CUDA cores.  States are processed in micro-batches so that the
// activation buffers have a fixed, modest size.
//
// The reference has no transformer scorer; its InferenceBackend interface (beam_engine.cpp:423-668) is the slot
// this fills, through the same mgbs_scorer_fn hook as the MLP.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <new>

#include "mgbs.h"
#include "mgbs_tc.cuh"

namespace mgbs {

// Warps: 0 = TMA, 1 = MMA + TMEM owner, 2..9 = epilogue.  Eight epilogue warps (two per TMEM lane quadrant, each
// taking one 128-column half of the 256-column accumulator) because the GEMMs here have short reductions (K = 256):
// per output tile the epilogue (bias, GELU, bf16 packing) costs more instructions than the tensor core needs cycles.
constexpr int TF_THREADS = 320;
constexpr int TF_STAGES = 3;
constexpr int TF_STAGING = 4 * A_BYTES;  // eight epilogue warps x two private boxes of 32 rows x 128 bytes
constexpr int TF_SMEM = TF_STAGES * STAGE_BYTES + TF_STAGING + 1024 + 256;

enum { TF_EPI_STORE = 0, TF_EPI_STORE_GELU = 1, TF_EPI_RESID = 2 };

struct TfGemmArgs {
  const uint32_t* count_dev;  // states to score (device value)
  int32_t tokens;             // rows per state
  int64_t row_offset;         // first row (state * tokens) of this micro-batch
  int64_t row_limit;          // rows of one micro-batch at most
  int32_t n_total, k_total;   // multiples of BN / BK
  const float* bias;          // [n_total]
  const float* col_scale;     // e4m3 operands: [n_total] = activation scale * weight-row scale
  float out_inv_scale;        // e4m3 output (TF_EPI_STORE_GELU with e4m3 operands): stored value = x * out_inv_scale
  int* err;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// C = A * W^T (+ bias) with A [rows, K] and W [N, K] bf16, K-major, both by TMA.
// TF_EPI_STORE / _GELU: bf16 output through swizzled staging boxes and TMA stores (tmOut: [rows, N] bf16, boxes of 32 rows).
// TF_EPI_RESID: resid[row, n] += acc + bias[n] in float32 through TMA reduce-add (tmOut: [rows, N] float32).
// F8 = 1: both operands e4m3 (kind::f8f6f4, 128-element K-blocks), accumulators multiplied by col_scale; the GELU
// variant then also writes e4m3 (one 128-column box per epilogue half), the plain store variant still writes bf16.
template <int EPI, int F8>
__global__ void __launch_bounds__(TF_THREADS, 1)
k_tf_gemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
          const __grid_constant__ CUtensorMap tmOut, TfGemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + TF_STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + TF_STAGING);
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * TF_STAGES + 5);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (TF_STAGES + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * TF_STAGES + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * TF_STAGES + 2 + b); };
  const uint32_t drain_bar = bar0 + 8u * (2 * TF_STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int64_t rows = (int64_t)(*g.count_dev) * g.tokens - g.row_offset;
  if (rows > g.row_limit) rows = g.row_limit;
  if (rows < 0) rows = 0;
  const int num_mtiles = (int)((rows + BM - 1) / BM);
  const int n_chunks = g.n_total / BN;
  constexpr int BKE = F8 ? BK8 : BK;
  const int k_blocks = g.k_total / BKE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TF_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 8); }
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
        for (int nc = 0; nc < n_chunks && ok; ++nc) {
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, g.err, ERR_WAIT_EMPTY)) { ok = false; break; }
            const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
            mbar_expect_tx(full_bar(stage), STAGE_BYTES);
            tma_load_2d(sa, &tmA, kb * BKE, mt * BM, full_bar(stage));
            tma_load_2d(sa + A_BYTES, &tmB, kb * BKE, nc * BN, full_bar(stage));
            if (++stage == TF_STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, acc_it = 0;
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
            for (int k = 0; k < BK / UMMA_K; ++k)
              tc_mma<F8>(d_tmem, adesc + 2u * k, bdesc + 2u * k, (kb | k) != 0 ? 1u : 0u);
            tc_commit(empty_bar(stage));
            if (++stage == TF_STAGES) { stage = 0; phase ^= 1u; }
          }
          if (ok) tc_commit(tfull_bar(b));
        }
      }
      tc_commit(drain_bar);
      mbar_wait(drain_bar, 0, g.err, ERR_WAIT_DRAIN);
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;              // which 128 columns of the accumulator
    // Each warp stages its 32 rows in two private 4 KB boxes (32 rows x 128 bytes) and alternates between them: no
    // barrier between warps, sixteen TMA operations in flight per CTA.  (A TMA store or reduce holds its box for
    // well over a thousand cycles; with four 16 KB boxes shared by the warps of a column half, behind two barriers
    // per box, the epilogue was what these GEMMs waited for.)
    uint8_t* mybox = staging + (warp - 2) * 8192;
    const uint32_t r = (uint32_t)(quad * 32 + lane);
    uint32_t acc_it = 0, box_it = 0;
    bool ok = true;
    for (int mt = blockIdx.x; mt < num_mtiles && ok; mt += gridDim.x) {
      const int row0 = mt * BM;
      const int64_t row = (int64_t)row0 + r;
      const bool row_ok = row < rows;
      for (int nc = 0; nc < n_chunks && ok; ++nc, ++acc_it) {
        const uint32_t b = acc_it & 1u;
        if (!mbar_wait(tfull_bar(b), (acc_it >> 1) & 1u, g.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + b * BN;
        if (EPI == TF_EPI_RESID) {
          // acc * scale + bias goes to a swizzled float32 box (128 rows x 32 columns) and from there into the
          // residual stream by a TMA reduce-add: the read-modify-write happens in the memory system, in whole
          // 128-byte rows, instead of as 16-byte accesses to 32 different rows per warp instruction
#pragma unroll 1
          for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 32, ++box_it) {
            uint8_t* box = mybox + (box_it & 1u) * 4096;
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
            uint32_t v[32];
            tc_ld32(taddr + c0, v);
            tc_wait_ld();
            const int n0 = nc * BN + c0;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 bq = __ldg(reinterpret_cast<const float4*>(g.bias + n0) + q);
              float4 cq = make_float4(1.f, 1.f, 1.f, 1.f);
              if (F8) cq = __ldg(reinterpret_cast<const float4*>(g.col_scale + n0) + q);
              float4 x;
              x.x = row_ok ? fmaf(__uint_as_float(v[4 * q]), cq.x, bq.x) : 0.f;
              x.y = row_ok ? fmaf(__uint_as_float(v[4 * q + 1]), cq.y, bq.y) : 0.f;
              x.z = row_ok ? fmaf(__uint_as_float(v[4 * q + 2]), cq.z, bq.z) : 0.f;
              x.w = row_ok ? fmaf(__uint_as_float(v[4 * q + 3]), cq.w, bq.w) : 0.f;
              *reinterpret_cast<float4*>(box + swz128((uint32_t)lane, (uint32_t)(q * 16))) = x;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              tma_reduce_add_2d(&tmOut, smem_u32(box), n0, row0 + quad * 32);
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        } else {
          constexpr bool OUT8 = F8 && EPI == TF_EPI_STORE_GELU;   // e4m3 output
          constexpr int BOXC = OUT8 ? 128 : 64;                   // columns per 128-byte box row
#pragma unroll 1
          for (int gcol = half * (BN / 2); gcol < (half + 1) * (BN / 2); gcol += BOXC, ++box_it) {
            uint8_t* box = mybox + (box_it & 1u) * 4096;
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
#pragma unroll
            for (int sub = 0; sub < BOXC / 32; ++sub) {
              uint32_t v[32];
              tc_ld32(taddr + gcol + sub * 32, v);
              tc_wait_ld();
              const int n0 = nc * BN + gcol + sub * 32;
              float x[32];
#pragma unroll
              for (int j4 = 0; j4 < 8; ++j4) {
                const float4 bq = __ldg(reinterpret_cast<const float4*>(g.bias + n0) + j4);
                float4 cq = make_float4(1.f, 1.f, 1.f, 1.f);
                if (F8) cq = __ldg(reinterpret_cast<const float4*>(g.col_scale + n0) + j4);
                x[4 * j4] = fmaf(__uint_as_float(v[4 * j4]), cq.x, bq.x);
                x[4 * j4 + 1] = fmaf(__uint_as_float(v[4 * j4 + 1]), cq.y, bq.y);
                x[4 * j4 + 2] = fmaf(__uint_as_float(v[4 * j4 + 2]), cq.z, bq.z);
                x[4 * j4 + 3] = fmaf(__uint_as_float(v[4 * j4 + 3]), cq.w, bq.w);
              }
              if (EPI == TF_EPI_STORE_GELU) {
#pragma unroll
                for (int j = 0; j < 32; ++j) x[j] = gelu_erf(x[j]);
              }
              if (OUT8) {
                uint32_t packed[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(x[4 * j] * g.out_inv_scale, x[4 * j + 1] * g.out_inv_scale), __NV_SATFINITE, __NV_E4M3);
                  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(x[4 * j + 2] * g.out_inv_scale, x[4 * j + 3] * g.out_inv_scale), __NV_SATFINITE, __NV_E4M3);
                  packed[j] = lo | (hi << 16);
                }
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  const uint32_t off = swz128((uint32_t)lane, (uint32_t)(sub * 32 + q * 16));
                  *reinterpret_cast<uint4*>(box + off) = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
              } else {
                uint32_t packed[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
                  packed[j] = *reinterpret_cast<uint32_t*>(&h);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint32_t off = swz128((uint32_t)lane, (uint32_t)(sub * 64 + q * 16));
                  *reinterpret_cast<uint4*>(box + off) = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
              }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmOut, smem_u32(box), nc * BN + gcol, row0 + quad * 32);
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(b));
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// rows of one micro-batch: min(max(count*tokens - row_offset, 0), row_limit)
__device__ __forceinline__ int64_t tf_rows(const uint32_t* count_dev, int tokens, int64_t row_offset, int64_t row_limit) {
  int64_t rows = (int64_t)(*count_dev) * tokens - row_offset;
  if (rows > row_limit) rows = row_limit;
  return rows < 0 ? 0 : rows;
}

// x[row, :] = tok_emb[value] + pos_emb[position]; row = state * tokens + position.  One warp per row.
__global__ void __launch_bounds__(256) k_tf_embed(const uint8_t* __restrict__ children, const uint32_t* count_dev,
                                                  int tokens, int stride, int d, int64_t row_offset, int64_t row_limit,
                                                  const float* __restrict__ tok_emb, const float* __restrict__ pos_emb,
                                                  float* __restrict__ x) {
  const int64_t rows = tf_rows(count_dev, tokens, row_offset, row_limit);
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    const int64_t grow = row_offset + r;
    const int64_t state = grow / tokens;
    const int pos = (int)(grow - state * tokens);
    const int val = __ldg(children + state * stride + pos);
    const float* te = tok_emb + (int64_t)val * d;
    const float* pe = pos_emb + (int64_t)pos * d;
    for (int c = lane * 4; c < d; c += 128) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(te + c));
      const float4 b = __ldg(reinterpret_cast<const float4*>(pe + c));
      *reinterpret_cast<float4*>(x + r * d + c) = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
    }
  }
}

// y = bf16(LayerNorm(x) * gamma + beta), d = 256: one warp per row, 8 elements per lane.
template <int OUT8>
__global__ void __launch_bounds__(256) k_tf_layernorm(const float* __restrict__ x, const uint32_t* count_dev, int tokens,
                                                      int64_t row_offset, int64_t row_limit,
                                                      const float* __restrict__ gamma, const float* __restrict__ beta,
                                                      void* __restrict__ y_out, float out_inv_scale) {
  constexpr int D = 256;
  const int64_t rows = tf_rows(count_dev, tokens, row_offset, row_limit);
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    const float4 a = *reinterpret_cast<const float4*>(x + r * D + lane * 8);
    const float4 b = *reinterpret_cast<const float4*>(x + r * D + lane * 8 + 4);
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += v[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mu = s * (1.f / D);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[i] -= mu; q += v[i] * v[i]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    const float rstd = rsqrtf(q * (1.f / D) + 1e-5f);
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = v[i] * rstd * __ldg(gamma + lane * 8 + i) + __ldg(beta + lane * 8 + i);
    if (OUT8) {
      uint32_t w[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(o[4 * i] * out_inv_scale, o[4 * i + 1] * out_inv_scale), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(o[4 * i + 2] * out_inv_scale, o[4 * i + 3] * out_inv_scale), __NV_SATFINITE, __NV_E4M3);
        w[i] = lo | (hi << 16);
      }
      *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(y_out) + r * D + lane * 8) = make_uint2(w[0], w[1]);
    } else {
      uint32_t packed[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) packed[i] = pack_bf16(o[2 * i], o[2 * i + 1]);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(y_out) + r * D + lane * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
  }
}

// Self-attention core of one layer: out[row, h*32:(h+1)*32] = softmax(q k^T / sqrt(32)) v per state and head,
// on the tensor cores with warp-level mma (m16n8k16, bf16 in, fp32 accumulate).  A warp owns one (state, head):
// it stages Q, K and V ([token][32], row pitch 40 bf16, so that fragment loads and ldmatrix rows hit distinct
// banks) in shared memory with one batch of 16-byte cp.async copies - every copy of a task is in flight at once,
// the task pays one global-memory latency - then for each block of 16 query rows computes S = Q K^T (8 key
// blocks), a masked softmax in registers, and O = P V with the probabilities re-packed from accumulator layout
// into A fragments and V fragments read transposed by ldmatrix.  Tokens are padded to 64; padded rows are zeroed
// once per warp and padded keys are masked out.
constexpr int TF_MAX_T = 64;
constexpr int TF_ATT_WARPS = 7;   // 15 KB of staging per warp: two CTAs of seven warps per SM
constexpr int TF_QK_PITCH = 40;   // bf16 per row of Q / K / V
constexpr int TF_ATT_WARP_ELEMS = 3 * TF_MAX_T * TF_QK_PITCH;
constexpr int TF_ATT_SMEM = TF_ATT_WARPS * TF_ATT_WARP_ELEMS * 2;

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int OUT8>
__global__ void __launch_bounds__(TF_ATT_WARPS * 32) k_tf_attention(const __nv_bfloat16* __restrict__ qkv,
                                                                    const uint32_t* count_dev, int tokens,
                                                                    int64_t row_offset, int64_t row_limit,
                                                                    void* __restrict__ out_v, float out_inv_scale) {
  constexpr int D = 256, HD = 32, NH = D / HD;
  extern __shared__ __align__(16) uint8_t att_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(att_raw) + (size_t)warp * TF_ATT_WARP_ELEMS;
  __nv_bfloat16* ks = qs + TF_MAX_T * TF_QK_PITCH;
  __nv_bfloat16* vs = ks + TF_MAX_T * TF_QK_PITCH;
  const int64_t rows = tf_rows(count_dev, tokens, row_offset, row_limit);
  const int64_t units = (rows / tokens) * NH;
  const float scale_log2 = 0.17677669529663687f * 1.4426950408889634f;  // 1/sqrt(32) * log2(e)
  // rows tokens..63 of the three matrices stay zero for the whole kernel (the copies below never touch them)
  for (int c = tokens * 4 + lane; c < TF_MAX_T * 4; c += 32) {
    const int t = c >> 2, part = c & 3;
#pragma unroll
    for (int m = 0; m < 3; ++m)
      *reinterpret_cast<uint4*>(qs + m * TF_MAX_T * TF_QK_PITCH + t * TF_QK_PITCH + part * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
  const uint32_t qs_u32 = smem_u32(qs);
  // ldmatrix row address of this lane inside a 16-token x 16-column block of V
  const uint32_t v_lane = smem_u32(vs) + (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * TF_QK_PITCH + (lane >> 4) * 8) * 2);
  for (int64_t u = (int64_t)blockIdx.x * TF_ATT_WARPS + warp; u < units; u += (int64_t)gridDim.x * TF_ATT_WARPS) {
    const int64_t s = u / NH;
    const int h = (int)(u - s * NH);
    const __nv_bfloat16* base = qkv + s * tokens * (3 * D) + h * HD;
    __syncwarp();
    // stage: tokens x {q, k, v} x 4 chunks of 8 bf16
    for (int c = lane; c < tokens * 4; c += 32) {
      const int t = c >> 2, part = c & 3;
      const __nv_bfloat16* src = base + (int64_t)t * 3 * D + part * 8;
      const uint32_t dst = qs_u32 + (uint32_t)((t * TF_QK_PITCH + part * 8) * 2);
#pragma unroll
      for (int m = 0; m < 3; ++m)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)(m * TF_MAX_T * TF_QK_PITCH * 2)), "l"(__cvta_generic_to_global(src + m * D)) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    const int mblocks = (tokens + 15) >> 4;
    for (int mb = 0; mb < mblocks; ++mb) {
      // Q fragments of this 16-row block: two k-steps of 16
      uint32_t qa[2][4];
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const __nv_bfloat16* q0 = qs + (mb * 16 + gid) * TF_QK_PITCH + kk * 16 + 2 * tig;
        qa[kk][0] = *reinterpret_cast<const uint32_t*>(q0);
        qa[kk][1] = *reinterpret_cast<const uint32_t*>(q0 + 8 * TF_QK_PITCH);
        qa[kk][2] = *reinterpret_cast<const uint32_t*>(q0 + 8);
        qa[kk][3] = *reinterpret_cast<const uint32_t*>(q0 + 8 * TF_QK_PITCH + 8);
      }
      float sc[8][4];
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
        sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const __nv_bfloat16* k0 = ks + (nb * 8 + gid) * TF_QK_PITCH + kk * 16 + 2 * tig;
          mma_bf16_16816(sc[nb], qa[kk], *reinterpret_cast<const uint32_t*>(k0), *reinterpret_cast<const uint32_t*>(k0 + 8));
        }
      }
      // masked softmax over keys for rows gid (c0, c1) and gid + 8 (c2, c3); a row is spread over the 4 lanes of a group
      float mx0 = -1e30f, mx1 = -1e30f;
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const bool valid = nb * 8 + 2 * tig + e < tokens;
          sc[nb][e] = valid ? sc[nb][e] * scale_log2 : -1e30f;
          sc[nb][2 + e] = valid ? sc[nb][2 + e] * scale_log2 : -1e30f;
          mx0 = fmaxf(mx0, sc[nb][e]);
          mx1 = fmaxf(mx1, sc[nb][2 + e]);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          sc[nb][e] = exp2f(sc[nb][e] - mx0);
          sc[nb][2 + e] = exp2f(sc[nb][2 + e] - mx1);
          sum0 += sc[nb][e];
          sum1 += sc[nb][2 + e];
        }
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      // O = P V: probabilities of key blocks (2j, 2j+1) form the A fragment of k-step j
      float o[4][4];
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t pa[4];
        pa[0] = pack_bf16(sc[2 * j][0], sc[2 * j][1]);
        pa[1] = pack_bf16(sc[2 * j][2], sc[2 * j][3]);
        pa[2] = pack_bf16(sc[2 * j + 1][0], sc[2 * j + 1][1]);
        pa[3] = pack_bf16(sc[2 * j + 1][2], sc[2 * j + 1][3]);
#pragma unroll
        for (int nb = 0; nb < 4; nb += 2) {
          uint32_t b0, b1, b2, b3;   // V[j*16 .. +15][nb*8 .. +7] and [(nb+1)*8 .. +7], transposed into B fragments
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                       : "r"(v_lane + (uint32_t)((j * 16 * TF_QK_PITCH + nb * 8) * 2)));
          mma_bf16_16816(o[nb], pa, b0, b1);
          mma_bf16_16816(o[nb + 1], pa, b2, b3);
        }
      }
      const float inv0 = 1.f / sum0, inv1 = 1.f / sum1;
      const int r0 = mb * 16 + gid, r1 = r0 + 8;
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        const int col = h * HD + nb * 8 + 2 * tig;
        if (OUT8) {
          uint8_t* out8 = reinterpret_cast<uint8_t*>(out_v);
          if (r0 < tokens)
            *reinterpret_cast<uint16_t*>(out8 + (s * tokens + r0) * D + col) = (uint16_t)__nv_cvt_float2_to_fp8x2(
                make_float2(o[nb][0] * inv0 * out_inv_scale, o[nb][1] * inv0 * out_inv_scale), __NV_SATFINITE, __NV_E4M3);
          if (r1 < tokens)
            *reinterpret_cast<uint16_t*>(out8 + (s * tokens + r1) * D + col) = (uint16_t)__nv_cvt_float2_to_fp8x2(
                make_float2(o[nb][2] * inv1 * out_inv_scale, o[nb][3] * inv1 * out_inv_scale), __NV_SATFINITE, __NV_E4M3);
        } else {
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(out_v);
          if (r0 < tokens) *reinterpret_cast<uint32_t*>(out + (s * tokens + r0) * D + col) = pack_bf16(o[nb][0] * inv0, o[nb][1] * inv0);
          if (r1 < tokens) *reinterpret_cast<uint32_t*>(out + (s * tokens + r1) * D + col) = pack_bf16(o[nb][2] * inv1, o[nb][3] * inv1);
        }
      }
    }
  }
}

// Final LayerNorm, mean over the tokens of a state, scalar head: q[state] (+)= mean_t(LN(x_t)) . w_head.
// One warp per state.
__global__ void __launch_bounds__(256) k_tf_pool_head(const float* __restrict__ x, const uint32_t* count_dev, int tokens,
                                                      int64_t row_offset, int64_t row_limit,
                                                      const float* __restrict__ gamma, const float* __restrict__ beta,
                                                      const float* __restrict__ w_head, int accumulate,
                                                      float* __restrict__ q_out) {
  constexpr int D = 256;
  const int64_t rows = tf_rows(count_dev, tokens, row_offset, row_limit);
  const int64_t states = rows / tokens;
  const int64_t state0 = row_offset / tokens;
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t s = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); s < states; s += warps) {
    float pooled[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) pooled[i] = 0.f;
    for (int t = 0; t < tokens; ++t) {
      const float* xr = x + (s * tokens + t) * D + lane * 8;
      const float4 a = *reinterpret_cast<const float4*>(xr);
      const float4 b = *reinterpret_cast<const float4*>(xr + 4);
      float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) sum += v[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float mu = sum * (1.f / D);
      float var = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { v[i] -= mu; var += v[i] * v[i]; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
      const float rstd = rsqrtf(var * (1.f / D) + 1e-5f);
#pragma unroll
      for (int i = 0; i < 8; ++i) pooled[i] += v[i] * rstd;
    }
    float dot = 0.f;
    const float inv_t = 1.f / (float)tokens;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = lane * 8 + i;
      dot += (pooled[i] * inv_t * __ldg(gamma + c) + __ldg(beta + c)) * __ldg(w_head + c);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) {
      if (accumulate) q_out[state0 + s] += dot;
      else q_out[state0 + s] = dot;
    }
  }
}

__global__ void __launch_bounds__(256) k_tf_q_to_key(const float* __restrict__ q, const uint32_t* count_dev, float inv_models,
                                                     float offset, uint32_t* __restrict__ keys) {
  const int64_t rows = *count_dev;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < rows; i += (int64_t)gridDim.x * blockDim.x) {
    float x = q[i] * inv_models - offset;
    x = fminf(fmaxf(x, 0.f), 300.f);
    keys[i] = (uint32_t)(x * 256.f + 0.5f);
  }
}

}  // namespace mgbs

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------

struct MgbsTf {
  MgbsTfConfig cfg;
  int sms = 148;
  int64_t mb_rows = 0;      // rows of one micro-batch (micro_batch * tokens)
  int64_t mb_rows_pad = 0;  // rounded up to 128
  int n_micro = 0;
  CUtensorMap tm_y, tm_qkv, tm_att, tm_hid;  // activations (load as A operand / store as output)
  CUtensorMap tm_qkv_st, tm_hid_st;          // qkv and hid as store targets: boxes of 32 rows (one warp's rows)
  CUtensorMap tm_x_st;                       // float32 residual stream (reduce-add target), boxes of 32 rows
  CUtensorMap tm_wqkv[MGBS_TF_MAX_ENCODERS][MGBS_TF_MAX_LAYERS], tm_wo[MGBS_TF_MAX_ENCODERS][MGBS_TF_MAX_LAYERS],
      tm_w1[MGBS_TF_MAX_ENCODERS][MGBS_TF_MAX_LAYERS], tm_w2[MGBS_TF_MAX_ENCODERS][MGBS_TF_MAX_LAYERS];
};

extern "C" {

int mgbs_sizeof_tf_config(void) { return (int)sizeof(MgbsTfConfig); }

int mgbs_tf_create(const MgbsTfConfig* cfg, MgbsTf** out) {
  if (!cfg || !out) return MGBS_ERR_ARG;
  const MgbsTfConfig& c = *cfg;
  if (c.d_model != 256 || c.heads != 8) return MGBS_ERR_UNSUPPORTED;
  if (c.ffn < mgbs::BN || c.ffn % mgbs::BN != 0) return MGBS_ERR_UNSUPPORTED;
  if (c.state_len < 1 || c.state_len > mgbs::TF_MAX_T || c.state_stride < c.state_len) return MGBS_ERR_ARG;
  if (c.layers < 1 || c.layers > MGBS_TF_MAX_LAYERS || c.encoders < 1 || c.encoders > MGBS_TF_MAX_ENCODERS) return MGBS_ERR_ARG;
  if (c.max_states < 1 || c.micro_batch < 1) return MGBS_ERR_ARG;
  if (!c.x || !c.y || !c.qkv || !c.att || !c.hid || !c.q || !c.err) return MGBS_ERR_ARG;
  MgbsTf* t = new (std::nothrow) MgbsTf();
  if (!t) return MGBS_ERR_STATE;
  t->cfg = c;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) t->sms = sms;
  }
  t->mb_rows = c.micro_batch * c.state_len;
  t->mb_rows_pad = (t->mb_rows + mgbs::BM - 1) / mgbs::BM * mgbs::BM;
  t->n_micro = (int)((c.max_states + c.micro_batch - 1) / c.micro_batch);
  const uint64_t R = (uint64_t)t->mb_rows_pad;
  if (c.dtype != 0 && c.dtype != 1) { delete t; return MGBS_ERR_ARG; }
  const int eb = c.dtype == 1 ? 1 : 2;  // bytes per GEMM operand element
  int rc = mgbs::make_map(&t->tm_y, c.y, R, 256, mgbs::BM, eb);
  if (!rc) rc = mgbs::make_map_bf16(&t->tm_qkv, c.qkv, R, 768, mgbs::BM);
  if (!rc) rc = mgbs::make_map(&t->tm_att, c.att, R, 256, mgbs::BM, eb);
  if (!rc) rc = mgbs::make_map(&t->tm_hid, c.hid, R, (uint64_t)c.ffn, mgbs::BM, eb);
  if (!rc) rc = mgbs::make_map_bf16(&t->tm_qkv_st, c.qkv, R, 768, 32);
  if (!rc) rc = mgbs::make_map(&t->tm_hid_st, c.hid, R, (uint64_t)c.ffn, 32, eb);
  if (!rc) rc = mgbs::make_map(&t->tm_x_st, c.x, R, 256, 32, 4);
  for (int e = 0; e < c.encoders && !rc; ++e) {
    if (!c.tok_emb[e] || !c.pos_emb[e] || !c.lnf_g[e] || !c.lnf_b[e] || !c.w_head[e]) rc = MGBS_ERR_ARG;
    for (int l = 0; l < c.layers && !rc; ++l) {
      const MgbsTfLayer& L = c.layer[e][l];
      if (!L.ln1_g || !L.ln1_b || !L.wqkv || !L.bqkv || !L.wo || !L.bo || !L.ln2_g || !L.ln2_b || !L.w1 || !L.b1 ||
          !L.w2 || !L.b2)
        rc = MGBS_ERR_ARG;
      if (!rc && c.dtype == 1 && (!L.cs_qkv || !L.cs_o || !L.cs_1 || !L.cs_2)) rc = MGBS_ERR_ARG;
      if (!rc) rc = mgbs::make_map(&t->tm_wqkv[e][l], L.wqkv, 768, 256, mgbs::BN, eb);
      if (!rc) rc = mgbs::make_map(&t->tm_wo[e][l], L.wo, 256, 256, mgbs::BN, eb);
      if (!rc) rc = mgbs::make_map(&t->tm_w1[e][l], L.w1, (uint64_t)c.ffn, 256, mgbs::BN, eb);
      if (!rc) rc = mgbs::make_map(&t->tm_w2[e][l], L.w2, 256, (uint64_t)c.ffn, mgbs::BN, eb);
    }
  }
  auto big_smem = [&](const void* fn, int bytes) {
    if (!rc) rc = (int)cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  };
  big_smem((const void*)mgbs::k_tf_gemm<mgbs::TF_EPI_STORE, 0>, mgbs::TF_SMEM);
  big_smem((const void*)mgbs::k_tf_gemm<mgbs::TF_EPI_STORE_GELU, 0>, mgbs::TF_SMEM);
  big_smem((const void*)mgbs::k_tf_gemm<mgbs::TF_EPI_RESID, 0>, mgbs::TF_SMEM);
  big_smem((const void*)mgbs::k_tf_gemm<mgbs::TF_EPI_STORE, 1>, mgbs::TF_SMEM);
  big_smem((const void*)mgbs::k_tf_gemm<mgbs::TF_EPI_STORE_GELU, 1>, mgbs::TF_SMEM);
  big_smem((const void*)mgbs::k_tf_gemm<mgbs::TF_EPI_RESID, 1>, mgbs::TF_SMEM);
  big_smem((const void*)mgbs::k_tf_attention<0>, mgbs::TF_ATT_SMEM);
  big_smem((const void*)mgbs::k_tf_attention<1>, mgbs::TF_ATT_SMEM);
  if (rc) { delete t; return rc; }
  *out = t;
  return 0;
}

int mgbs_tf_destroy(MgbsTf* t) {
  delete t;
  return 0;
}

int mgbs_tf_enqueue(void* user, const uint8_t* children, const uint32_t* count_dev, uint32_t* scores, void* stream) {
  MgbsTf* t = static_cast<MgbsTf*>(user);
  if (!t || !children || !count_dev || !scores) return MGBS_ERR_ARG;
  using namespace mgbs;
  const MgbsTfConfig& c = t->cfg;
  cudaStream_t st = (cudaStream_t)stream;
  const int T = c.state_len;
  const int ew_grid = t->sms * 8;
  const __nv_bfloat16* qkv = reinterpret_cast<const __nv_bfloat16*>(c.qkv);
  const bool f8 = c.dtype == 1;
  const dim3 gg(t->sms), gb(TF_THREADS);
  for (int mb = 0; mb < t->n_micro; ++mb) {
    const int64_t off = (int64_t)mb * t->mb_rows;
    TfGemmArgs g;
    g.count_dev = count_dev;
    g.tokens = T;
    g.row_offset = off;
    g.row_limit = t->mb_rows;
    g.err = c.err;
    g.col_scale = nullptr;
    g.out_inv_scale = 1.f;
    for (int e = 0; e < c.encoders; ++e) {
      k_tf_embed<<<ew_grid, 256, 0, st>>>(children, count_dev, T, c.state_stride, 256, off, t->mb_rows, c.tok_emb[e],
                                          c.pos_emb[e], c.x);
      for (int l = 0; l < c.layers; ++l) {
        const MgbsTfLayer& L = c.layer[e][l];
        g.n_total = 768; g.k_total = 256; g.bias = L.bqkv;
        if (f8) {
          k_tf_layernorm<1><<<ew_grid, 256, 0, st>>>(c.x, count_dev, T, off, t->mb_rows, L.ln1_g, L.ln1_b, c.y, L.inv_y1);
          g.col_scale = L.cs_qkv;
          k_tf_gemm<TF_EPI_STORE, 1><<<gg, gb, TF_SMEM, st>>>(t->tm_y, t->tm_wqkv[e][l], t->tm_qkv_st, g);
          k_tf_attention<1><<<t->sms * 2, TF_ATT_WARPS * 32, TF_ATT_SMEM, st>>>(qkv, count_dev, T, off, t->mb_rows, c.att, L.inv_att);
        } else {
          k_tf_layernorm<0><<<ew_grid, 256, 0, st>>>(c.x, count_dev, T, off, t->mb_rows, L.ln1_g, L.ln1_b, c.y, 1.f);
          k_tf_gemm<TF_EPI_STORE, 0><<<gg, gb, TF_SMEM, st>>>(t->tm_y, t->tm_wqkv[e][l], t->tm_qkv_st, g);
          k_tf_attention<0><<<t->sms * 2, TF_ATT_WARPS * 32, TF_ATT_SMEM, st>>>(qkv, count_dev, T, off, t->mb_rows, c.att, 1.f);
        }
        g.n_total = 256; g.k_total = 256; g.bias = L.bo;
        if (f8) {
          g.col_scale = L.cs_o;
          k_tf_gemm<TF_EPI_RESID, 1><<<gg, gb, TF_SMEM, st>>>(t->tm_att, t->tm_wo[e][l], t->tm_x_st, g);
          k_tf_layernorm<1><<<ew_grid, 256, 0, st>>>(c.x, count_dev, T, off, t->mb_rows, L.ln2_g, L.ln2_b, c.y, L.inv_y2);
        } else {
          k_tf_gemm<TF_EPI_RESID, 0><<<gg, gb, TF_SMEM, st>>>(t->tm_att, t->tm_wo[e][l], t->tm_x_st, g);
          k_tf_layernorm<0><<<ew_grid, 256, 0, st>>>(c.x, count_dev, T, off, t->mb_rows, L.ln2_g, L.ln2_b, c.y, 1.f);
        }
        g.n_total = c.ffn; g.k_total = 256; g.bias = L.b1;
        if (f8) {
          g.col_scale = L.cs_1; g.out_inv_scale = L.inv_hid;
          k_tf_gemm<TF_EPI_STORE_GELU, 1><<<gg, gb, TF_SMEM, st>>>(t->tm_y, t->tm_w1[e][l], t->tm_hid_st, g);
        } else {
          k_tf_gemm<TF_EPI_STORE_GELU, 0><<<gg, gb, TF_SMEM, st>>>(t->tm_y, t->tm_w1[e][l], t->tm_hid_st, g);
        }
        g.n_total = 256; g.k_total = c.ffn; g.bias = L.b2;
        if (f8) {
          g.col_scale = L.cs_2;
          k_tf_gemm<TF_EPI_RESID, 1><<<gg, gb, TF_SMEM, st>>>(t->tm_hid, t->tm_w2[e][l], t->tm_x_st, g);
        } else {
          k_tf_gemm<TF_EPI_RESID, 0><<<gg, gb, TF_SMEM, st>>>(t->tm_hid, t->tm_w2[e][l], t->tm_x_st, g);
        }
      }
      k_tf_pool_head<<<ew_grid, 256, 0, st>>>(c.x, count_dev, T, off, t->mb_rows, c.lnf_g[e], c.lnf_b[e], c.w_head[e],
                                              e > 0 ? 1 : 0, c.q);
    }
  }
  float bh = 0.f;
  for (int e = 0; e < c.encoders; ++e) bh += c.b_head[e];
  k_tf_q_to_key<<<t->sms * 4, 256, 0, st>>>(c.q, count_dev, 1.f / (float)c.encoders,
                                            c.score_offset - bh / (float)c.encoders, scores);
  return (int)cudaGetLastError();
}

}  // extern "C"
