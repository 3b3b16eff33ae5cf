// tcgen05 / TMA / mbarrier building blocks shared by the scorer kernels (sm_100a): PTX wrappers, shared-memory
// matrix descriptors, instruction descriptors, bounded waits, and the host helper that encodes TMA descriptors.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mgbs.h"

namespace mgbs {

constexpr int BM = 128;       // rows per tile (TMEM lanes)
constexpr int BN = 256;       // accumulator columns per tile
constexpr int BK = 64;        // bf16 elements per 128-byte swizzle row
constexpr int BK8 = 128;      // e4m3 elements per 128-byte swizzle row
constexpr int UMMA_K = 16;    // K of one tcgen05.mma for 16-bit operands
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_SMEM = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t TMEM_COLS = 512;

// Width of the one-hot first-layer operand: columns are ordered value-major in groups of eight positions
// (column = value * 8 * ceil(n / 8) + position), so that eight adjacent columns are one byte-compare of the state row.
inline __host__ __device__ int onehot_columns(int state_len, int num_values) { return num_values * ((state_len + 7) / 8 * 8); }

constexpr int ERR_WAIT_EMPTY = 1, ERR_WAIT_FULL = 2, ERR_WAIT_TMEM_EMPTY = 3, ERR_WAIT_TMEM_FULL = 4, ERR_WAIT_DRAIN = 5;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait that also acquires what other CTAs of the cluster released on this barrier
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded waits: about 1-2 s of polling at most, then report and give up.  The common case - the phase is already
// complete, or completes within the instruction's own wait - is one try_wait and a branch; the polling loop with its
// counter lives out of line so that the callers' loops stay short.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, int* err, int code, int cluster) {
  for (uint32_t it = 0; it < (1u << 24); ++it) {
    if (cluster ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return true;
    if (it > 1024) __nanosleep(64);
  }
  if (err) atomicCAS(err, 0, code);
  return false;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int* err, int code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, err, code, 1);
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, err, code, 0);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; both operands K-major, described by shared-memory matrix descriptors
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// same for e4m3 operands (kind::f8f6f4, K = 32 elements per instruction)
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

template <int F8>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t accumulate);

// ---- CTA pairs (cta_group::2): one thread of the even CTA issues an MMA of M = 256 over both CTAs' shared
// memory (each holds its 128 rows of A and half of B's N rows at the same offsets) into both CTAs' TMEM ----
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared address: the even CTA of the pair

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose completion bytes are counted on the even CTA's barrier (no multicast: each CTA loads its own box)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar & kPeerBitMask)
      : "memory");
}
// arrive on the barrier at this offset in every CTA of the mask once all MMAs issued so far have completed
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(cta_mask) : "memory");
}
// plain arrive on the even CTA's barrier at this offset (from either CTA of the pair)
__device__ __forceinline__ void mbar_arrive_even_cta(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & kPeerBitMask) : "memory");
}
// the same with release semantics at cluster scope: what this thread (and, after a __syncwarp, its warp) wrote to
// its CTA's shared memory is visible to whoever acquires the barrier in the even CTA
__device__ __forceinline__ void mbar_arrive_even_cta_release(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar & kPeerBitMask) : "memory");
}
__device__ __forceinline__ void tc_mma_pair_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_mma_pair_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
// Fields: start address >> 4 (bits 0-13), leading byte offset >> 4 (16-29, unused for swizzled K-major: 1),
// stride byte offset >> 4 (32-45: 1024 >> 4), descriptor version 1 (46-47), layout type SWIZZLE_128B = 2 (61-63).
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor for kind::f16: D = f32 (bits 4-5 = 1), A = B = bf16 (bits 7-9 / 10-12 = 1), both K-major
// (bits 15, 16 = 0), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
constexpr uint32_t kIdescBf16 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
// kind::f8f6f4 with A = B = E4M3 (format code 0), D = f32
constexpr uint32_t kIdescE4m3 = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// pair MMA: M = 256 (128 rows per CTA), N = 256
constexpr uint32_t kIdescBf16Pair = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
constexpr uint32_t kIdescE4m3Pair = (1u << 4) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
template <int F8>
__device__ __forceinline__ void tc_mma_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t acc) {
  if (F8) tc_mma_pair_f8(d, a, b, kIdescE4m3Pair, acc);
  else tc_mma_pair_f16(d, a, b, kIdescBf16Pair, acc);
}

template <>
__device__ __forceinline__ void tc_mma<0>(uint32_t d, uint64_t a, uint64_t b, uint32_t acc) { tc_mma_f16(d, a, b, kIdescBf16, acc); }
template <>
__device__ __forceinline__ void tc_mma<1>(uint32_t d, uint64_t a, uint64_t b, uint32_t acc) { tc_mma_f8(d, a, b, kIdescE4m3, acc); }

__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t byte_in_row) {
  // 128-byte swizzle inside 1024-byte (8-row) atoms: 16-byte chunk index ^= row mod 8
  return row * 128u + (byte_in_row ^ ((row & 7u) << 4));
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}

// element-wise float32 add of a shared-memory box into global memory, performed by the memory system
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}

}  // namespace mgbs

// ---- host: TMA descriptor encoding (driver entry point resolved at run time; no link-time libcuda dependency) ----
namespace mgbs {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
  if (qres != cudaDriverEntryPointSuccess) return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// 2-D row-major [rows, cols] tensor of 2-byte (bf16) or 1-byte (e4m3) elements, box = {128 bytes of columns,
// box_rows}, 128-byte swizzle
inline int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, int elem_bytes) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return MGBS_ERR_STATE;
  if (((uintptr_t)base & 15u) != 0 || (cols * elem_bytes) % 16 != 0) return MGBS_ERR_ARG;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(map, dt, 2,
                   const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : MGBS_ERR_STATE;
}

// general form: box of box_rows x box_cols elements, swizzle 64 or 128 bytes (box_cols * elem_bytes must equal it)
inline int make_map_box(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                        uint32_t box_cols, int elem_bytes, int swizzle_bytes) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return MGBS_ERR_STATE;
  if (((uintptr_t)base & 15u) != 0 || (cols * elem_bytes) % 16 != 0) return MGBS_ERR_ARG;
  if ((int)(box_cols * elem_bytes) != swizzle_bytes || (swizzle_bytes != 64 && swizzle_bytes != 128)) return MGBS_ERR_ARG;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : MGBS_ERR_STATE;
}

inline int make_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  return make_map(map, base, rows, cols, box_rows, 2);
}

// x * Phi(x) with erf from the rational-exponential approximation of Abramowitz & Stegun 7.1.26 (absolute error
// below 1.5e-7 plus ~1e-6 from the approximate reciprocal and exponential: far under half a unit in the last
// place of the bf16 and e4m3 values this feeds).  A dozen instructions, two of them on the special-function unit;
// it matters because the feed-forward epilogue evaluates it once per output element.
__device__ __forceinline__ float gelu_erf(float x) {
  const float z = fabsf(x) * 0.70710678118654752f;
  float t, e;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.f)));
  float p = fmaf(1.061405429f, t, -1.453152027f);
  p = fmaf(p, t, 1.421413741f);
  p = fmaf(p, t, -0.284496736f);
  p = fmaf(p, t, 0.254829592f);
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * z * z));
  const float erf_abs = fmaf(-p * t, e, 1.f);          // erf(|x| / sqrt 2)
  return 0.5f * x + 0.5f * fabsf(x) * erf_abs;         // x/2 (1 + sign(x) erf(|x|/sqrt 2))
}

}  // namespace mgbs
