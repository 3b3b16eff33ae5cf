// Kernels of the per-depth beam-search step for sm_100a.
//
// Data flow of one depth (one rank):
//   frontier rows --k_expand--> candidate arrays (hash, fingerprint, score, back-pointer, optional child rows)
//   [world > 1: k_route buckets candidates by hash owner; the engine exchanges the buckets]
//   band rounds: k_band_hist x levels -> k_band_insert   (dedup into an open-addressing table, best-first bands)
//   final cut:   k_final_hist x levels -> k_emit -> k_finish (exact top-K on (score, hash, fingerprint))
//
// Every kernel has a fixed launch shape and reads its sizes from the device control block, so a whole depth can
// be captured in a CUDA graph.  Capacity problems set status bits; nothing traps and no wait is unbounded
// (there are no spin waits: the table protocol uses only compare-and-swap and max).

#include <cuda_runtime.h>
#include <stdint.h>

#include "mgbs.h"
#include "mgbs_device.cuh"
#include "mgbs_internal.cuh"

namespace mgbs {

// ------------------------------------------------------------------------------------------------
// Expansion: child = gather(parent, generator); hash64; fingerprint64; Hamming distance; goal test.
// Replaces apply_move_table / hash_state_120 / fingerprint_state_120 / hamming_to_central and the expansion
// half of kernel_process_score_slot (beam_kernels.cu:29-103, 528-580).
//
// Both hashes are serial byte chains, so the work is one chain pair per candidate and the kernel is bound by
// instruction issue, not by memory.  A block stages 64 parent rows in shared memory with a row pitch of stride+4
// bytes (odd word pitch: the 32 lanes of a warp read 32 different rows at the same byte offset without bank
// conflicts) and the generator tables next to them; a warp handles 32 parents and TWO moves per pass - two
// independent chain pairs per thread, which the scheduler interleaves - so the table lookups are broadcasts.  The
// 24-byte records of the tile's 64 x fanout candidates are staged in shared memory and copied out afterwards with
// consecutive lanes on consecutive candidates (the candidate index is parent-major, so a warp's own candidates
// lie fanout entries apart).
// ------------------------------------------------------------------------------------------------

template <int WORDS>
struct ExpandSmem {
  static constexpr int kPitchW = WORDS + 1;
  // byte offsets inside the dynamic shared memory block
  static __host__ __device__ constexpr int par() { return 0; }
  static __host__ __device__ constexpr int gen() { return par() + kExpandTile * kPitchW * 4; }
  static __host__ __device__ constexpr int sol() { return gen() + MGBS_MAX_FANOUT * WORDS * 4; }
  static __host__ __device__ constexpr int rec() { return (sol() + WORDS * 4 + 15) / 16 * 16; }
  static __host__ __device__ constexpr int total(int fanout) { return rec() + kExpandTile * fanout * 24; }
};

// The loop over 16-byte groups of the child row is not unrolled: with all groups (and their two interleaved hash
// chains) laid out straight-line the kernel stalled on instruction fetch (2.4 no-instruction stalls per issue);
// rolled it is 12 % faster (0.083 -> 0.073 ms on 786 432 candidates of 54 bytes).
constexpr int kExpandUnroll = 1;
template <int WORDS, int ZOB>
__global__ void __launch_bounds__(kExpandThreads, 3) k_expand(ExpandArgs a) {
  using L = ExpandSmem<WORDS>;
  constexpr int PITCH_W = L::kPitchW;
  extern __shared__ __align__(16) uint8_t expand_smem[];
  uint32_t* par_s = reinterpret_cast<uint32_t*>(expand_smem + L::par());
  uint32_t* gen_s = reinterpret_cast<uint32_t*>(expand_smem + L::gen());
  uint32_t* sol_s = reinterpret_cast<uint32_t*>(expand_smem + L::sol());
  const int G = a.fanout;
  const int tile_cands = kExpandTile * G;
  uint64_t* rec_h = reinterpret_cast<uint64_t*>(expand_smem + L::rec());
  uint64_t* rec_f = rec_h + tile_cands;
  uint32_t* rec_k = reinterpret_cast<uint32_t*>(rec_f + tile_cands);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int n = a.n;
  const int64_t P = a.count_dev ? (int64_t)(*a.count_dev) : a.count;
  if (P <= 0) return;

  // generator tables and solved state, padded to WORDS*4 bytes per row
  for (int i = tid; i < G * WORDS * 4; i += kExpandThreads) {
    int g = i / (WORDS * 4), b = i - g * (WORDS * 4);
    reinterpret_cast<uint8_t*>(gen_s)[i] = b < n ? a.gens[g * n + b] : 0;
  }
  for (int i = tid; i < WORDS * 4; i += kExpandThreads) reinterpret_cast<uint8_t*>(sol_s)[i] = i < n ? a.solved[i] : 0;

  const bool want_score = a.score_mode != MGBS_SCORE_EXTERNAL;
  const int64_t ntiles = (P + kExpandTile - 1) / kExpandTile;
  const uint32_t* fw = reinterpret_cast<const uint32_t*>(a.frontier);
  const ulonglong2* ztab = reinterpret_cast<const ulonglong2*>(a.zobrist);
  const int pairs = (G + 1) >> 1;
  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int64_t p0 = tile * kExpandTile;
    __syncthreads();  // the previous tile's records have been copied out
    for (int i = tid; i < kExpandTile * WORDS; i += kExpandThreads) {
      int r = i / WORDS, w = i - r * WORDS;
      int64_t p = p0 + r;
      par_s[r * PITCH_W + w] = p < P ? fw[p * WORDS + w] : 0u;
    }
    __syncthreads();
    for (int u = warp; u < 2 * pairs; u += kExpandThreads / 32) {
      const int g0 = (u >> 1) << 1;
      const bool two = g0 + 1 < G;
      const int g1 = two ? g0 + 1 : g0;  // an odd fan-out: the last pass repeats its move and drops the copy
      const int pl = ((u & 1) << 5) + lane;
      const int64_t p = p0 + pl;
      if (p >= P) continue;
      const uint8_t* row = reinterpret_cast<const uint8_t*>(par_s + pl * PITCH_W);
      uint64_t h0 = ZOB ? 0ull : kFnvOffset, f0 = ZOB ? 0ull : kGolden;
      uint64_t h1 = h0, f1 = f0;
      int ham0 = 0, ham1 = 0;
      const int64_t c0 = p * G + g0;
      uint4* dst0 = a.children ? reinterpret_cast<uint4*>(a.children + c0 * (int64_t)a.stride) : nullptr;
      uint4* dst1 = (a.children && two) ? reinterpret_cast<uint4*>(a.children + (c0 + 1) * (int64_t)a.stride) : nullptr;
      // 16 bytes of each child at a time: the words are stored as soon as they are complete, so that only
      // eight of them are live (the register count decides how many warps hide the shared-memory latency)
#pragma unroll kExpandUnroll
      for (int q = 0; q < WORDS / 4; ++q) {
        uint32_t cw0[4], cw1[4];
#pragma unroll
        for (int w4 = 0; w4 < 4; ++w4) {
          const int wi = q * 4 + w4;
          const uint32_t gi0 = gen_s[g0 * WORDS + wi];
          const uint32_t gi1 = gen_s[g1 * WORDS + wi];
          const uint32_t sv = sol_s[wi];
          uint32_t acc0 = 0, acc1 = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (wi * 4 + j < n) {
              const uint32_t v0 = row[(gi0 >> (8 * j)) & 0xffu];
              const uint32_t v1 = row[(gi1 >> (8 * j)) & 0xffu];
              if (ZOB) {
                const ulonglong2 z0 = __ldg(ztab + (wi * 4 + j) * a.zobrist_values + (int)v0);
                const ulonglong2 z1 = __ldg(ztab + (wi * 4 + j) * a.zobrist_values + (int)v1);
                h0 ^= z0.x; f0 ^= z0.y;
                h1 ^= z1.x; f1 ^= z1.y;
              } else {
                h0 = (h0 ^ (uint64_t)v0) * kFnvPrime;
                h1 = (h1 ^ (uint64_t)v1) * kFnvPrime;
                f0 ^= (uint64_t)v0 + kGolden + (f0 << 6) + (f0 >> 2);
                f1 ^= (uint64_t)v1 + kGolden + (f1 << 6) + (f1 >> 2);
              }
              const uint32_t s8 = (sv >> (8 * j)) & 0xffu;
              ham0 += (v0 != s8);
              ham1 += (v1 != s8);
              acc0 |= v0 << (8 * j);
              acc1 |= v1 << (8 * j);
            }
          }
          cw0[w4] = acc0;
          cw1[w4] = acc1;
        }
        if (dst0) dst0[q] = make_uint4(cw0[0], cw0[1], cw0[2], cw0[3]);
        if (dst1) dst1[q] = make_uint4(cw1[0], cw1[1], cw1[2], cw1[3]);
      }
      if (ZOB) {
        h0 = finish_zobrist_lo(h0); f0 = finish_zobrist_hi(f0);
        h1 = finish_zobrist_lo(h1); f1 = finish_zobrist_hi(f1);
      } else {
        h0 = finish_hash(h0); f0 = finish_fingerprint(f0);
        h1 = finish_hash(h1); f1 = finish_fingerprint(f1);
      }
      const int s0 = pl * G + g0;
      rec_h[s0] = h0;
      rec_f[s0] = f0;
      if (want_score) rec_k[s0] = a.score_mode == MGBS_SCORE_HAMMING ? (uint32_t)ham0 : (uint32_t)a.uniform_score;
      if (ham0 == 0 && a.ctrl) atomicMin(&a.ctrl->found_payload, pack_payload((uint32_t)p, (uint32_t)a.rank, (uint32_t)g0));
      if (two) {
        rec_h[s0 + 1] = h1;
        rec_f[s0 + 1] = f1;
        if (want_score) rec_k[s0 + 1] = a.score_mode == MGBS_SCORE_HAMMING ? (uint32_t)ham1 : (uint32_t)a.uniform_score;
        if (ham1 == 0 && a.ctrl) atomicMin(&a.ctrl->found_payload, pack_payload((uint32_t)p, (uint32_t)a.rank, (uint32_t)g1));
      }
    }
    __syncthreads();
    // copy-out: consecutive lanes, consecutive candidates; the back-pointer is a function of the index
    const int64_t rows_here = P - p0 < kExpandTile ? P - p0 : kExpandTile;
    const int cnt = (int)rows_here * G;
    const int64_t cbase = p0 * G;
    for (int i = tid; i < cnt; i += kExpandThreads) {
      a.cand_hash[cbase + i] = rec_h[i];
      a.cand_fp[cbase + i] = rec_f[i];
      const int pl = i / G;
      a.cand_payload[cbase + i] = pack_payload((uint32_t)(p0 + pl), (uint32_t)a.rank, (uint32_t)(i - pl * G));
      if (want_score) a.cand_score[cbase + i] = rec_k[i];
    }
  }
}


// Block-wide search of a 2048-bin histogram for the bin where the running count crosses `target`.
// gt = true : first bin with cum_incl >  target   (band: how much fits)
// gt = false: first bin with cum_incl >= target   (final: where the K-th entry lies)
// Returns bin (or -1), the exclusive count before it and its own count.  All threads get the same answer.
struct Cross {
  int bin;
  uint64_t before;
  uint32_t count;
  uint64_t total;
};

__device__ Cross find_crossing(const uint32_t* hist, uint64_t target, bool gt) {
  __shared__ uint64_t warp_sums[kStreamThreads / 32];
  __shared__ int s_bin;
  __shared__ uint64_t s_before;
  __shared__ uint32_t s_count;
  __shared__ uint64_t s_total;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int PER = MGBS_RADIX_BINS / kStreamThreads;  // 8
  uint32_t v[PER];
  uint64_t local = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    v[j] = __ldcg(hist + tid * PER + j);
    local += v[j];
  }
  uint64_t incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint64_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (tid == 0) s_bin = -1;
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  uint64_t base = 0, total = 0;
#pragma unroll
  for (int w = 0; w < kStreamThreads / 32; ++w) {
    uint64_t s = warp_sums[w];
    if (w < warp) base += s;
    total += s;
  }
  uint64_t excl = base + incl - local;
  uint64_t end = excl + local;
  bool mine = gt ? (excl <= target && end > target) : (excl < target && end >= target);
  if (mine) {
    uint64_t c = excl;
    for (int j = 0; j < PER; ++j) {
      uint64_t ci = c + v[j];
      bool hit = gt ? (ci > target) : (ci >= target);
      if (hit) {
        s_bin = tid * PER + j;
        s_before = c;
        s_count = v[j];
        break;
      }
      c = ci;
    }
  }
  if (tid == 0) s_total = total;
  __syncthreads();
  Cross r;
  r.bin = s_bin;
  r.before = s_bin >= 0 ? s_before : 0;
  r.count = s_bin >= 0 ? s_count : 0;
  r.total = s_total;
  __syncthreads();
  return r;
}

__device__ __forceinline__ int digit_bits_at(int key_bits, int bits_done) {
  int left = key_bits - bits_done;
  return left < MGBS_RADIX_BITS ? left : MGBS_RADIX_BITS;
}

__device__ __forceinline__ uint64_t range_end(uint64_t prefix, int key_bits, int bits_done) {
  // first key after the range selected by `prefix` (bits_done decided bits); saturates at ~0
  int left = key_bits - bits_done;
  if (left >= 64) return ~0ull;
  uint64_t span = 1ull << left;
  uint64_t e = prefix + span;
  if (e < prefix) return ~0ull;
  if (key_bits < 64 && e >= (1ull << key_bits)) return ~0ull;
  return e;
}

// Per-rank statistics ride in the tail of every level-0 histogram so that one all-reduce carries them.
__device__ __forceinline__ void read_stats(const uint32_t* hist0, int world, uint64_t& u_tot, uint64_t& u_max,
                                           uint64_t& i_tot, uint32_t& found_any) {
  u_tot = 0; u_max = 0; i_tot = 0;
  for (int r = 0; r < world; ++r) {
    uint64_t u = __ldcg(hist0 + MGBS_RADIX_BINS + r);
    u_tot += u;
    u_max = u > u_max ? u : u_max;
    i_tot += __ldcg(hist0 + MGBS_RADIX_BINS + 16 + r);
  }
  found_any = __ldcg(hist0 + MGBS_RADIX_BINS + 32);
}

constexpr uint32_t kFlagComplete = 1u;  // bands: enough unique entries, or every candidate inserted
constexpr uint32_t kFlagNoRoom = 2u;    // bands: table at its hard limit

__device__ __forceinline__ MgbsRadix radix_zero() {
  MgbsRadix st;
  st.prefix = 0; st.remaining = 0; st.bits_done = 0; st.done = 0; st.flag = 0; st.pad = 0;
  st.result = 0; st.tie_key = 0; st.tie_need = 0; st.kept_below = 0;
  return st;
}

// Initial band state of a round, from the all-reduced statistics: how many candidates (duplicates included)
// the next band may hold.
__device__ MgbsRadix band_initial(const StepArgs& a, const uint32_t* hist0, uint64_t D) {
  MgbsRadix st = radix_zero();
  st.result = D;
  uint64_t u_tot, u_max, i_tot;
  uint32_t found_any;
  read_stats(hist0, a.world, u_tot, u_max, i_tot, found_any);
  st.kept_below = u_tot;
  const uint64_t W = (uint64_t)a.world;
  if (u_tot >= (uint64_t)a.beam || D == ~0ull) {
    st.done = 1;
    st.flag = kFlagComplete;
    return st;
  }
  // hard limit: keep every rank's table below 7/8 full even with a 1/16 owner imbalance
  const uint64_t hard_cap = ((uint64_t)a.hash_capacity * 7) / 8;
  uint64_t hard = u_max < hard_cap ? (hard_cap - u_max) * W : 0;
  hard -= hard / 16;
  // fill target: bring the pool to its target size assuming the unique ratio seen so far
  const uint64_t pool = (uint64_t)a.pool_target * W;
  uint64_t want_unique = pool > u_tot ? pool - u_tot : 0;
  uint64_t num = i_tot, den = u_tot;
  if (den == 0 || num == 0) {  // nothing inserted yet this depth: use last depth's ratio
    num = a.ctrl->rho_num;
    den = a.ctrl->rho_den;
    if (den == 0 || num < den) { num = 1; den = 1; }
  }
  uint64_t n = (want_unique * num + den - 1) / den;
  if (n > hard) n = hard;
  st.remaining = n;
  if (n == 0) { st.done = 1; st.flag = kFlagNoRoom; }
  return st;
}

// Consume one band-level histogram.
__device__ MgbsRadix band_advance(MgbsRadix st, const uint32_t* hist, int key_bits, bool last_level, uint64_t D) {
  if (st.done) return st;
  Cross c = find_crossing(hist, st.remaining, true);
  if (c.bin < 0) {  // everything under this prefix fits
    st.result = range_end(st.prefix, key_bits, (int)st.bits_done);
    st.done = 1;
    return st;
  }
  const int db = digit_bits_at(key_bits, (int)st.bits_done);
  const int shift = key_bits - (int)st.bits_done - db;
  st.prefix |= (uint64_t)c.bin << shift;
  st.bits_done += db;
  st.remaining -= c.before;
  if (last_level || (int)st.bits_done >= key_bits) {
    st.result = st.prefix > D ? st.prefix : D;  // exclude the crossing bin
    st.done = 1;
  }
  return st;
}

__device__ MgbsRadix final_initial(const StepArgs& a, const uint32_t* hist0) {
  MgbsRadix st = radix_zero();
  st.result = ~0ull;
  uint64_t u_tot, u_max, i_tot;
  uint32_t found_any;
  read_stats(hist0, a.world, u_tot, u_max, i_tot, found_any);
  st.kept_below = u_tot;
  const uint64_t B = (uint64_t)a.beam;
  const bool keep_all = (a.select_mode == MGBS_SELECT_LEGACY_STRICT) ? (u_tot < B) : (u_tot <= B);
  if (keep_all || u_tot == 0) { st.done = 1; return st; }
  st.remaining = B;
  return st;
}

__device__ MgbsRadix final_advance(MgbsRadix st, const uint32_t* hist, int key_bits, int select_mode) {
  if (st.done) return st;
  Cross c = find_crossing(hist, st.remaining, false);
  if (c.bin < 0) {  // counts inconsistent (cannot happen): keep everything
    st.result = ~0ull;
    st.done = 1;
    return st;
  }
  const int db = digit_bits_at(key_bits, (int)st.bits_done);
  const int shift = key_bits - (int)st.bits_done - db;
  st.prefix |= (uint64_t)c.bin << shift;
  st.bits_done += db;
  st.remaining -= c.before;
  const bool full_res = (int)st.bits_done >= key_bits;
  if (select_mode == MGBS_SELECT_LEGACY_STRICT) {
    if (full_res) { st.result = st.prefix; st.done = 1; }  // the whole cutoff key is pruned
    return st;
  }
  if (select_mode == MGBS_SELECT_V6_INCLUSIVE) {
    if (full_res || c.count == st.remaining) {
      st.result = range_end(st.prefix, key_bits, (int)st.bits_done);
      st.done = 1;
    }
    return st;
  }
  if (c.count == st.remaining) {  // the whole bin survives
    st.result = range_end(st.prefix, key_bits, (int)st.bits_done);
    st.done = 1;
  } else if (full_res) {
    st.result = st.prefix;
    st.tie_key = st.prefix;
    st.tie_need = st.remaining;
    st.done = 1;
  }
  return st;
}

template <class F>
__device__ __forceinline__ void for_each_candidate(const CandView& cv, F f) {
  for (int b = 0; b < cv.nbuckets; ++b) {
    uint32_t cnt = __ldcg(cv.counts + b);
    if (cnt > cv.cap) cnt = cv.cap;
    const uint32_t rounded = (cnt + 31u) & ~31u;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < rounded; i += gridDim.x * blockDim.x) {
      f((uint64_t)b * cv.cap + i, i < cnt);
    }
  }
}

// The same walk with four items in flight per thread: `load(index)` fetches what an item needs (the loads of a batch
// are independent and issued together), `f(index, valid, item)` consumes it and may use warp-wide operations.
template <class Item, class L, class F>
__device__ __forceinline__ void for_each_candidate_batched(const CandView& cv, L load, F f) {
  const uint32_t stride = gridDim.x * blockDim.x;
  for (int b = 0; b < cv.nbuckets; ++b) {
    uint32_t cnt = __ldcg(cv.counts + b);
    if (cnt > cv.cap) cnt = cv.cap;
    const uint32_t rounded = (cnt + 31u) & ~31u;
    const uint64_t base = (uint64_t)b * cv.cap;
    for (uint32_t i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < rounded; i0 += 4u * stride) {
      Item it[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t i = i0 + (uint32_t)u * stride;
        if (i < cnt) it[u] = load(base + i);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t i = i0 + (uint32_t)u * stride;
        if (i < rounded) f(base + i, i < cnt, it[u]);  // i < rounded is uniform over a warp
      }
    }
  }
}

__device__ __forceinline__ void hist_add(uint32_t* sh, bool in, uint32_t digit) {
  const unsigned m = __ballot_sync(0xffffffffu, in);
  if (in) {
    const unsigned peers = __match_any_sync(m, digit);
    if ((int)(threadIdx.x & 31) == (__ffs(peers) - 1)) atomicAdd(&sh[digit], (uint32_t)__popc(peers));
  }
}

__device__ __forceinline__ void hist_flush(const uint32_t* sh, uint32_t* hist) {
  __syncthreads();
  for (int b = threadIdx.x; b < MGBS_RADIX_BINS; b += blockDim.x) {
    uint32_t v = sh[b];
    if (v) atomicAdd(&hist[b], v);
  }
}

__device__ __forceinline__ void publish_stats(const StepArgs& a) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    // read past the L1 cache: inside the persistent selection kernel other blocks' atomics updated these words
    a.hist[MGBS_RADIX_BINS + a.rank] = __ldcg(&a.ctrl->table_count);
    a.hist[MGBS_RADIX_BINS + 16 + a.rank] = __ldcg(&a.ctrl->inserted_total);
    a.hist[MGBS_RADIX_BINS + 32] = (__ldcg(&a.ctrl->found_payload) != 0xffffffffu) ? 1u : 0u;
  }
}

// A wait for another rank ran out: record it here and tell every rank (their abort words take this depth's epoch),
// so that ranks which never time out themselves - because this rank's flags did arrive - learn that the sums they
// used were partial.
__device__ __forceinline__ void peer_give_up(const StepArgs& a) {
  atomicOr(&a.ctrl->status, MGBS_ST_PEER_TIMEOUT);
  const uint32_t epoch = a.ctrl->epoch;
  for (int r = 0; r < a.world; ++r)
    *reinterpret_cast<volatile uint32_t*>(a.peer.base[r] + a.peer.off_abort) = epoch;
  __threadfence_system();
}

// Sum of one histogram over all ranks through peer-mapped memory, executed by every thread of ONE block: push the
// local histogram into slot [rank] of every rank's exchange area, raise this rank's flag there (value = epoch),
// wait - with a limit - for the flags of all ranks in the own area, and replace the local histogram by the sum.
__device__ void peer_allreduce_block(const StepArgs& a, uint32_t* hist, int slot) {
  const uint32_t epoch = a.ctrl->epoch;
  const int W = a.world;
  const int64_t slot_words = (int64_t)slot * W * MGBS_HIST_STRIDE;
  // every thread keeps its words of the local histogram in registers (independent loads, issued together) and
  // stores them to all peers: stores do not stall, so the push costs one load latency instead of one per word
  constexpr int PER = (MGBS_HIST_STRIDE + kStreamThreads - 1) / kStreamThreads;
  uint32_t mine_v[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = threadIdx.x + j * kStreamThreads;
    mine_v[j] = i < MGBS_HIST_STRIDE ? __ldcg(hist + i) : 0u;
  }
  for (int r = 0; r < W; ++r) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(a.peer.base[r] + a.peer.off_hx) + slot_words + (int64_t)a.rank * MGBS_HIST_STRIDE;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * kStreamThreads;
      if (i < MGBS_HIST_STRIDE) dst[i] = mine_v[j];
    }
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < W) {
    const int r = threadIdx.x;
    volatile uint32_t* f = reinterpret_cast<volatile uint32_t*>(a.peer.base[r] + a.peer.off_hflag) + (int64_t)slot * W + a.rank;
    *f = epoch;
    volatile uint32_t* mine = reinterpret_cast<volatile uint32_t*>(a.peer.base[a.rank] + a.peer.off_hflag) + (int64_t)slot * W + r;
    bool ok = false;
    for (uint32_t it = 0; it < a.peer.poll_limit; ++it) {
      if ((int32_t)(*mine - epoch) >= 0) { ok = true; break; }
      if (it > 1024) __nanosleep(100);
    }
    if (!ok) peer_give_up(a);
  }
  __threadfence_system();
  __syncthreads();
  // sum the W contributions that peers stored into this rank's slots (L2 is the point of coherence for them)
  const uint32_t* src = reinterpret_cast<const uint32_t*>(a.peer.base[a.rank] + a.peer.off_hx) + slot_words;
  uint32_t sum[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) sum[j] = 0u;
  for (int r = 0; r < W; ++r) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * kStreamThreads;
      if (i < MGBS_HIST_STRIDE) sum[j] += __ldcg(src + (int64_t)r * MGBS_HIST_STRIDE + i);
    }
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = threadIdx.x + j * kStreamThreads;
    if (i < MGBS_HIST_STRIDE) hist[i] = sum[j];
  }
  __threadfence();
}

// One-shot all-reduce of a finished histogram over peer-mapped memory.  Called by every thread of every block
// after its contribution was added to the local histogram; the block that arrives last pushes the local
// histogram into slot [rank] of every rank's exchange area, raises its flag there (value = epoch), waits - with a
// limit - for the flags of all ranks in its own area, and replaces the local histogram by the sum.  Consumers then
// read the local histogram exactly as in the NCCL mode.
__device__ void peer_allreduce_hist(const StepArgs& a) {
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(&a.peer.tickets[a.peer.slot], 1u);
    s_last = ((t + 1u) % gridDim.x) == 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  peer_allreduce_block(a, a.hist, a.peer.slot);
}

// Band histogram of one level.  Level 0 needs only the lower bound D; deeper levels first consume the previous
// level's (all-reduced) histogram to learn which prefix to refine.
__global__ void __launch_bounds__(kStreamThreads) k_band_hist(StepArgs a) {
  __shared__ uint32_t sh[MGBS_RADIX_BINS];
  for (int b = threadIdx.x; b < MGBS_RADIX_BINS; b += blockDim.x) sh[b] = 0;
  // an earlier round found the pool complete (from summed statistics, so every rank agrees): nothing left to do,
  // not even the reduction
  if (a.ctrl->halt || a.ctrl->bands_done) return;
  const uint64_t D = a.ctrl->band_lo[a.round];
  MgbsRadix st = radix_zero();
  if (a.level == 0) {
    st.done = (D == ~0ull) ? 1u : 0u;
    publish_stats(a);
  } else {
    if (a.level == 1) st = band_initial(a, a.hist_prev, D);
    else st = a.ctrl->band[a.round][a.level - 1];
    st = band_advance(st, a.hist_prev, a.key_bits, false, D);
    if (blockIdx.x == 0 && threadIdx.x == 0) a.ctrl->band[a.round][a.level] = st;
  }
  __syncthreads();
  if (st.done) {
    // nothing to count; level-0 histograms still carry the per-rank statistics to every rank
    if (a.peer.enabled && a.level == 0) peer_allreduce_hist(a);
    return;
  }
  const int db = digit_bits_at(a.key_bits, (int)st.bits_done);
  const int shift = a.key_bits - (int)st.bits_done - db;
  const uint32_t mask = (1u << db) - 1u;
  const int pshift = a.key_bits - (int)st.bits_done;  // bits below the decided prefix
  const bool any_prefix = st.bits_done != 0;
  const uint64_t pfx = any_prefix ? (st.prefix >> pshift) : 0;
  const int hb = a.hash_bits;
  for_each_candidate(a.cvh, [&](uint64_t i, bool valid) {
    bool in = false;
    uint32_t digit = 0;
    if (valid) {
      const uint64_t s = order_key(__ldg(a.cvh.score + i), __ldg(a.cvh.hash + i), hb);
      in = s >= D && (!any_prefix || (s >> pshift) == pfx);
      digit = (uint32_t)(s >> shift) & mask;
    }
    hist_add(sh, in, digit);
  });
  hist_flush(sh, a.hist);
  if (a.peer.enabled) peer_allreduce_hist(a);
}

// ------------------------------------------------------------------------------------------------
// Dedup table.  32-byte slots {hash, fingerprint, ~best, spare}; 0 = empty in every word.
// Replaces hash_insert_or_update (beam_kernels.cu:374-513): a slot is claimed with one compare-and-swap on the
// hash word and one on the fingerprint word (no BUSY state, so no waiting), the winner among duplicates is kept
// by an atomic max on the complemented (score, back-pointer) word, i.e. the smallest (score, parent, rank, move).
// ------------------------------------------------------------------------------------------------

struct Slot {
  unsigned long long hash;
  unsigned long long fp;
  unsigned long long best_inv;
  unsigned long long spare;
};

__device__ __forceinline__ uint32_t slot_home(uint64_t h, uint64_t cap) {
  // low hash word -> [0, cap): the selection key uses the top hash bits, the owner rank h mod world
  return (uint32_t)(((h & 0xffffffffull) * cap) >> 32);
}

// Returns the number of slots this call claimed (0 = merged into an existing entry, 1 = new entry; 2 only if a
// different state with an equal hash took the fingerprint of a slot this call had just claimed), or -1 when
// the probe limit was reached (the candidate is dropped and counted, as COUNTER_HASH_OVERFLOW is in the reference).
__device__ __forceinline__ int table_insert(Slot* table, uint64_t cap, int probe_limit, uint64_t h, uint64_t f, uint64_t val) {
  uint64_t pos = slot_home(h, cap);
  int claims = 0;
  for (int probe = 0; probe < probe_limit; ++probe) {
    Slot* s = table + pos;
    unsigned long long cur = *reinterpret_cast<volatile unsigned long long*>(&s->hash);
    if (cur == 0ull) {
      cur = atomicCAS(&s->hash, 0ull, (unsigned long long)h);
      if (cur == 0ull) { cur = h; ++claims; }
    }
    if (cur == h) {
      unsigned long long curf = *reinterpret_cast<volatile unsigned long long*>(&s->fp);
      if (curf == 0ull) {
        curf = atomicCAS(&s->fp, 0ull, (unsigned long long)f);
        if (curf == 0ull) curf = f;
      }
      if (curf == f) {
        atomicMax(&s->best_inv, ~(unsigned long long)val);
        return claims;
      }
    }
    pos = pos + 1 == cap ? 0 : pos + 1;
  }
  return -1;
}

// read-only lookup: the slot holding (h, f), or null
__device__ __forceinline__ const Slot* table_find(const Slot* table, uint64_t cap, int probe_limit, uint64_t h, uint64_t f) {
  uint64_t pos = slot_home(h, cap);
  for (int probe = 0; probe < probe_limit; ++probe) {
    const Slot* s = table + pos;
    const ulonglong2 hf = __ldcg(reinterpret_cast<const ulonglong2*>(s));
    if (hf.x == 0ull) return nullptr;
    if (hf.x == h && hf.y == f) return s;
    pos = pos + 1 == cap ? 0 : pos + 1;
  }
  return nullptr;
}

// Insert the band [D, E) of candidates.  The prologue consumes the last band-level histogram to get E.
__global__ void __launch_bounds__(kStreamThreads) k_band_insert(StepArgs a) {
  if (a.ctrl->halt) return;
  const uint64_t D = a.ctrl->band_lo[a.round];
  if (a.ctrl->bands_done) {  // set by an earlier round of this depth
    if (blockIdx.x == 0 && threadIdx.x == 0) a.ctrl->band_lo[a.round + 1] = D;
    return;
  }
  MgbsRadix st;
  if (a.levels == 1) st = band_initial(a, a.hist_prev, D);
  else st = a.ctrl->band[a.round][a.levels - 1];
  st = band_advance(st, a.hist_prev, a.key_bits, true, D);
  const uint64_t E = st.result;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    a.ctrl->band[a.round][a.levels] = st;
    a.ctrl->band_lo[a.round + 1] = E > D ? E : D;
    if (st.flag & kFlagComplete) {
      a.ctrl->bands_done = 1;
    } else {
      a.ctrl->rounds_used = a.round + 1;
      if (E <= D) atomicOr(&a.ctrl->status, MGBS_ST_BAND_STALL);
    }
  }
  if (E <= D) return;
  Slot* table = reinterpret_cast<Slot*>(a.table);
  const uint64_t cap = (uint64_t)a.hash_capacity;
  const int hb = a.hash_bits;
  uint32_t fresh_total = 0, ins_total = 0, drop_total = 0;
  for_each_candidate(a.cv, [&](uint64_t i, bool valid) {
    int res = -2;  // -2 = not in the band, -1 = dropped, >= 0 = slots claimed
    if (valid) {
      const uint32_t k = __ldg(a.cv.score + i);
      const uint64_t h = __ldg(a.cv.hash + i);
      const uint64_t s = order_key(k, h, hb);
      if (s >= D && s < E) {
        const uint64_t val = ((uint64_t)k << 32) | (uint64_t)__ldg(a.cv.payload + i);
        res = table_insert(table, cap, a.probe_limit, h, __ldg(a.cv.fp + i), val);
      }
    }
    fresh_total += __reduce_add_sync(0xffffffffu, (uint32_t)(res > 0 ? res : 0));
    ins_total += __popc(__ballot_sync(0xffffffffu, res != -2));
    drop_total += __popc(__ballot_sync(0xffffffffu, res == -1));
  });
  if ((threadIdx.x & 31) == 0) {
    if (fresh_total) atomicAdd(&a.ctrl->table_count, fresh_total);
    if (ins_total) atomicAdd(&a.ctrl->inserted_total, ins_total);
    if (drop_total) {
      atomicAdd(&a.ctrl->hash_overflow, drop_total);
      atomicOr(&a.ctrl->status, MGBS_ST_HASH_OVERFLOW);
    }
  }
}

// Final-cut histogram over the occupied table slots.
__global__ void __launch_bounds__(kStreamThreads) k_final_hist(StepArgs a) {
  __shared__ uint32_t sh[MGBS_RADIX_BINS];
  if (a.ctrl->halt) return;
  for (int b = threadIdx.x; b < MGBS_RADIX_BINS; b += blockDim.x) sh[b] = 0;
  MgbsRadix st = radix_zero();
  if (a.level == 0) {
    publish_stats(a);
  } else {
    if (a.level == 1) st = final_initial(a, a.hist_prev);
    else st = a.ctrl->fin[a.level - 1];
    st = final_advance(st, a.hist_prev, a.key_bits, a.select_mode);
    if (blockIdx.x == 0 && threadIdx.x == 0) a.ctrl->fin[a.level] = st;
  }
  __syncthreads();
  if (st.done) {
    // nothing to count; level-0 histograms still carry the per-rank statistics to every rank
    if (a.peer.enabled && a.level == 0) peer_allreduce_hist(a);
    return;
  }
  const int db = digit_bits_at(a.key_bits, (int)st.bits_done);
  const int shift = a.key_bits - (int)st.bits_done - db;
  const uint32_t mask = (1u << db) - 1u;
  const int pshift = a.key_bits - (int)st.bits_done;
  const bool any_prefix = st.bits_done != 0;
  const uint64_t pfx = any_prefix ? (st.prefix >> pshift) : 0;
  const int hb = a.hash_bits;
  const Slot* table = reinterpret_cast<const Slot*>(a.table);
  const uint64_t cap = (uint64_t)a.hash_capacity;
  const uint64_t rounded = (cap + 31ull) & ~31ull;
  for (uint64_t j = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; j < rounded; j += (uint64_t)gridDim.x * blockDim.x) {
    bool in = false;
    uint32_t digit = 0;
    if (j < cap) {
      const ulonglong2 hf = __ldcg(reinterpret_cast<const ulonglong2*>(table + j));
      if (hf.x != 0ull && hf.y != 0ull) {
        const uint64_t best = ~__ldcg(&table[j].best_inv);
        const uint64_t s = order_key((uint32_t)(best >> 32), hf.x, hb);
        in = !any_prefix || (s >> pshift) == pfx;
        digit = (uint32_t)(s >> shift) & mask;
      }
    }
    hist_add(sh, in, digit);
  }
  hist_flush(sh, a.hist);
  if (a.peer.enabled) peer_allreduce_hist(a);
}

// Write one survivor into the next frontier.
__device__ __forceinline__ void emit_row(const StepArgs& a, uint64_t i, uint32_t k, uint64_t h, uint32_t payload, uint32_t pos) {
  if ((int64_t)pos >= a.next_cap) {
    atomicOr(&a.ctrl->status, MGBS_ST_FRONTIER_OVERFLOW);
    return;
  }
  uint4* dst = reinterpret_cast<uint4*>(a.frontier_next + (int64_t)pos * a.stride);
  const int vecs = a.stride >> 4;
  if (a.cv.states) {
    const uint4* src = reinterpret_cast<const uint4*>(a.cv.states + i * (uint64_t)a.stride);
    for (int q = 0; q < vecs; ++q) dst[q] = __ldg(src + q);
  } else if (a.peer.enabled) {
    // the record travelled without its state: fetch the parent row from the rank that expanded it (its current
    // frontier is mapped here; nobody writes that buffer before the next depth's histograms have been summed over
    // all ranks) with 16-byte loads, then apply the move
    uint32_t parent, rank, move;
    unpack_payload(payload, parent, rank, move);
    const uint4* src = reinterpret_cast<const uint4*>(a.peer.base[rank] + a.off_frontier_cur + (int64_t)parent * a.stride);
    uint32_t row[MGBS_MAX_STATE_LEN / 4];
    for (int q = 0; q < vecs; ++q) {
      const uint4 v = __ldcg(src + q);
      row[4 * q] = v.x; row[4 * q + 1] = v.y; row[4 * q + 2] = v.z; row[4 * q + 3] = v.w;
    }
    const uint8_t* g = a.gens + (int64_t)move * a.n;
    for (int q = 0; q < vecs; ++q) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t acc = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int idx = q * 16 + j * 4 + b;
          if (idx < a.n) {
            const uint32_t sidx = __ldg(g + idx);
            acc |= ((row[sidx >> 2] >> (8 * (sidx & 3u))) & 0xffu) << (8 * b);
          }
        }
        w[j] = acc;
      }
      dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
    // regenerate the child from its parent row (world = 1: the parent is local)
    uint32_t parent, rank, move;
    unpack_payload(payload, parent, rank, move);
    const uint8_t* src = a.frontier_cur + (int64_t)parent * a.stride;
    const uint8_t* g = a.gens + (int64_t)move * a.n;
    for (int q = 0; q < vecs; ++q) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t acc = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int idx = q * 16 + j * 4 + b;
          if (idx < a.n) acc |= (uint32_t)__ldg(src + __ldg(g + idx)) << (8 * b);
        }
        w[j] = acc;
      }
      dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  if (a.next_score) a.next_score[pos] = k;
  if (a.next_hash) a.next_hash[pos] = h;
  const int32_t depth = a.ctrl->depth;
  // the rows form a ring: hosts that archive every layer after its step need one row, the others size it to
  // the deepest search
  if (a.history && a.history_depths > 0) a.history[(int64_t)(depth % a.history_depths) * a.frontier_cap + pos] = payload;
}


// Survivors: every candidate below the cut that is the winner of its table entry.  Winners whose key equals the
// cut key go to the tie list; k_finish keeps the smallest (hash, fingerprint) among them.
__global__ void __launch_bounds__(kStreamThreads) k_emit(StepArgs a) {
  if (a.ctrl->halt) return;
  MgbsRadix st;
  if (a.levels == 1) st = final_initial(a, a.hist_prev);
  else st = a.ctrl->fin[a.levels - 1];
  st = final_advance(st, a.hist_prev, a.key_bits, a.select_mode);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    a.ctrl->fin[a.levels] = st;
    a.ctrl->threshold_key = st.result;
  }
  const uint64_t T = st.result;
  const bool ties = st.tie_need > 0;
  const uint64_t tie_key = st.tie_key;
  const Slot* table = reinterpret_cast<const Slot*>(a.table);
  const uint64_t cap = (uint64_t)a.hash_capacity;
  const int hb = a.hash_bits;
  const int lane = threadIdx.x & 31;
  unsigned long long* seg = a.tie_buf + (int64_t)a.rank * kTieSegWords;
  if (a.cv.states == nullptr) {
    // Survivors are rebuilt from their back-pointers, so everything needed sits in the table entry itself (hash,
    // fingerprint, score and back-pointer of the winner): walk the table's slots instead of the candidates - five
    // times fewer items on one GPU and no lookups.  Tie records then carry the slot index.
    const uint64_t rounded = (cap + 31ull) & ~31ull;
    for (uint64_t j = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; j < rounded; j += (uint64_t)gridDim.x * blockDim.x) {
      bool keep = false, tie = false;
      uint32_t k = 0, payload = 0;
      uint64_t h = 0, f = 0;
      if (j < cap) {
        const ulonglong2 hf = __ldcg(reinterpret_cast<const ulonglong2*>(table + j));
        if (hf.x != 0ull && hf.y != 0ull) {
          const uint64_t best = ~__ldcg(&table[j].best_inv);
          h = hf.x; f = hf.y;
          k = (uint32_t)(best >> 32);
          payload = (uint32_t)best;
          const uint64_t s = order_key(k, h, hb);
          keep = s < T;
          tie = !keep && ties && s == tie_key;
        }
      }
      const unsigned km = __ballot_sync(0xffffffffu, keep);
      if (km) {
        uint32_t base = 0;
        if (lane == 0) base = atomicAdd(&a.ctrl->next_count, (uint32_t)__popc(km));
        base = __shfl_sync(0xffffffffu, base, 0);
        if (keep) emit_row(a, j, k, h, payload, base + __popc(km & ((1u << lane) - 1u)));
      }
      if (tie) {
        const unsigned long long t = atomicAdd(seg, 1ull);
        if (t < MGBS_TIE_CAP) {
          seg[1 + 3 * t] = h;
          seg[2 + 3 * t] = f;
          seg[3 + 3 * t] = j;
        } else {
          atomicOr(&a.ctrl->status, MGBS_ST_TIE_OVERFLOW);
        }
      }
    }
    return;
  }
  for_each_candidate(a.cv, [&](uint64_t i, bool valid) {
    bool keep = false, tie = false;
    uint32_t k = 0, payload = 0;
    uint64_t h = 0, f = 0;
    if (valid) {
      k = __ldg(a.cv.score + i);
      h = __ldg(a.cv.hash + i);
      const uint64_t s = order_key(k, h, hb);
      const bool below = s < T;
      const bool at = ties && s == tie_key;
      if (below || at) {
        payload = __ldg(a.cv.payload + i);
        f = __ldg(a.cv.fp + i);
        const Slot* sl = table_find(table, cap, a.probe_limit, h, f);
        if (sl != nullptr) {
          const uint64_t best = ~__ldcg(&sl->best_inv);
          if (best == (((uint64_t)k << 32) | payload)) { keep = below; tie = !below; }
        }
      }
    }
    const unsigned km = __ballot_sync(0xffffffffu, keep);
    if (km) {
      uint32_t base = 0;
      if (lane == 0) base = atomicAdd(&a.ctrl->next_count, (uint32_t)__popc(km));
      base = __shfl_sync(0xffffffffu, base, 0);
      if (keep) emit_row(a, i, k, h, payload, base + __popc(km & ((1u << lane) - 1u)));
    }
    if (tie) {
      const unsigned long long t = atomicAdd(seg, 1ull);
      if (t < MGBS_TIE_CAP) {
        seg[1 + 3 * t] = h;
        seg[2 + 3 * t] = f;
        seg[3 + 3 * t] = i;
      } else {
        atomicOr(&a.ctrl->status, MGBS_ST_TIE_OVERFLOW);
      }
    }
  });
}

// Summary of the control block for the host (pinned memory), written by the last kernel of every depth launch,
// halted or not; seq goes last, after a system-wide fence.
__device__ __forceinline__ void write_mirror(const StepArgs& a) {
  MgbsCtrl* c = a.ctrl;
  c->launch_seq += 1;
  MgbsMirror* m = a.mirror;
  if (!m) return;
  m->depth = c->depth;
  m->found = c->found;
  m->found_depth = c->found_depth;
  m->frontier_next = c->frontier_count[c->depth & 1];
  m->found_payload = c->found_payload;
  m->status = c->status;
  m->unique_total = c->unique_total;
  m->epoch = c->epoch;
  m->total_candidates = c->total_candidates;
  __threadfence_system();
  m->seq = c->launch_seq;
}

// Resolve ties at the cut key against the tie records of all ranks (tie_all: world segments), one block.
__device__ void resolve_ties(const StepArgs& a, const MgbsRadix& st, const unsigned long long* tie_all) {
  const uint64_t need = st.tie_need;
  if (need == 0) return;
  const unsigned long long* mine = tie_all + (int64_t)a.rank * kTieSegWords;
  uint64_t my_n = mine[0] < MGBS_TIE_CAP ? mine[0] : MGBS_TIE_CAP;
  for (uint64_t t = threadIdx.x; t < my_n; t += blockDim.x) {
    const uint64_t h = mine[1 + 3 * t], f = mine[2 + 3 * t], i = mine[3 + 3 * t];
    uint64_t before = 0;
    for (int r = 0; r < a.world; ++r) {
      const unsigned long long* seg = tie_all + (int64_t)r * kTieSegWords;
      const uint64_t n_r = seg[0] < MGBS_TIE_CAP ? seg[0] : MGBS_TIE_CAP;
      for (uint64_t j = 0; j < n_r; ++j) {
        const uint64_t hj = seg[1 + 3 * j], fj = seg[2 + 3 * j];
        before += (hj < h || (hj == h && fj < f)) ? 1 : 0;
      }
    }
    if (before < need) {
      const uint32_t pos = atomicAdd(&a.ctrl->next_count, 1u);
      if (a.cv.states == nullptr) {  // i is a table slot (see k_emit)
        const uint64_t best = ~__ldcg(&reinterpret_cast<const Slot*>(a.table)[i].best_inv);
        emit_row(a, i, (uint32_t)(best >> 32), h, (uint32_t)best, pos);
      } else {
        emit_row(a, i, __ldg(a.cv.score + i), h, __ldg(a.cv.payload + i), pos);
      }
    }
  }
}

// Thread 0 of one block: close the depth.
__device__ void close_depth(const StepArgs& a, const uint32_t* hist_stats) {
  MgbsCtrl* c = a.ctrl;
  uint64_t u_tot, u_max, i_tot;
  uint32_t found_any;
  read_stats(hist_stats, a.world, u_tot, u_max, i_tot, found_any);
  uint32_t nc = *reinterpret_cast<volatile uint32_t*>(&c->next_count);
  if ((int64_t)nc > a.next_cap) nc = (uint32_t)a.next_cap;
  c->frontier_count[a.parity ^ 1] = (int32_t)nc;
  c->unique_total = (uint32_t)u_tot;
  c->exhausted = u_tot == 0 ? 1u : 0u;
  if (u_tot > 0 && i_tot >= u_tot) { c->rho_num = i_tot; c->rho_den = u_tot; }
  if (u_tot < (uint64_t)a.beam && c->band_lo[a.rounds] != ~0ull)
    atomicOr(&c->status, MGBS_ST_ROUNDS_EXHAUSTED);
  // some rank gave up a wait during this depth and said so: this rank's sums may be partial as well
  if (a.peer.enabled) {
    const uint32_t ab = *reinterpret_cast<volatile uint32_t*>(a.peer.base[a.rank] + a.peer.off_abort);
    if (ab != 0u && (int32_t)(ab - c->epoch) >= 0) atomicOr(&c->status, MGBS_ST_PEER_TIMEOUT);
  }
  if (found_any && !c->found) {
    c->found = 1;
    c->found_depth = c->depth + 1;
  }
  c->total_candidates += c->cand_count;
  c->depth += 1;
  write_mirror(a);
}

// One block: resolve ties at the cut key against the tie records of all ranks, then close the depth.
__global__ void __launch_bounds__(kStreamThreads) k_finish(StepArgs a) {
  if (a.ctrl->halt) {
    if (threadIdx.x == 0) write_mirror(a);
    return;
  }
  const MgbsRadix st = a.ctrl->fin[a.levels];
  resolve_ties(a, st, a.tie_buf);
  __syncthreads();
  if (threadIdx.x == 0) close_depth(a, a.hist_stats);
}

// One thread: open the depth.  auto_halt = the launch belongs to a depth loop that must not run past the end of
// the search (found, nothing left); a failed cross-rank wait halts every later depth in any case, because the ranks
// no longer agree on what they hold.
__global__ void k_depth_begin(MgbsCtrl* c, int parity, int fanout, int64_t cand_cap, unsigned long long* tie_seg,
                              uint32_t* send_counts, uint32_t* recv_counts, int world, int64_t active_limit,
                              int auto_halt, const uint32_t* abort_word) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  if (abort_word) {
    const uint32_t ab = *reinterpret_cast<const volatile uint32_t*>(abort_word);
    if (ab != 0u && (int32_t)(ab - c->epoch) >= 0 && c->epoch != 0u) atomicOr(&c->status, MGBS_ST_PEER_TIMEOUT);
  }
  const bool broken = (c->status & (MGBS_ST_PEER_TIMEOUT | MGBS_ST_GRID_TIMEOUT)) != 0u;
  const bool finished = c->found != 0 || c->exhausted != 0u;
  c->grid_bar = 0;
  if (broken || (auto_halt && finished)) {
    c->halt = 1;
    c->active_rows = 0;
    c->cand_count = 0;
    return;
  }
  c->halt = 0;
  int64_t rows = c->frontier_count[parity];
  if (active_limit > 0 && rows > active_limit) rows = active_limit;
  int64_t cand = rows * fanout;
  if (cand > cand_cap) { cand = cand_cap; rows = cand_cap / fanout; }
  c->active_rows = (int32_t)rows;
  c->cand_count = (uint32_t)cand;
  c->table_count = 0;
  c->next_count = 0;
  c->tie_count = 0;
  c->inserted_total = 0;
  c->hash_overflow = 0;
  c->rounds_used = 0;
  c->bands_done = 0;
  c->found_payload = 0xffffffffu;
  c->epoch += 1;
  c->band_lo[0] = 0;
  tie_seg[0] = 0;
  if (send_counts)
    for (int r = 0; r < world; ++r) send_counts[r] = 0;
  // peer mode: this rank's receive fills of the depth (senders rewrite them after every band they route; no sender
  // can be that far before this rank has contributed to the depth's first histogram sum, which comes later in
  // this stream)
  if (recv_counts)
    for (int r = 0; r < world; ++r) recv_counts[r] = 0;
}

// world > 1: bucket this rank's candidates by owner = hash mod world (beam_kernels.cu:582) into the send arrays.
// Replaces the remote branch of kernel_process_score_slot (beam_kernels.cu:592-608); the local share goes through
// its own bucket as well, so that the owner sees one uniform set of receive buckets.
__global__ void __launch_bounds__(kStreamThreads) k_route(RouteArgs a) {
  if (a.ctrl->halt) return;
  const uint32_t cnt = a.ctrl->cand_count;
  const uint32_t rounded = (cnt + 31u) & ~31u;
  const int lane = threadIdx.x & 31;
  const int vecs = a.stride >> 4;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < rounded; i += gridDim.x * blockDim.x) {
    const bool valid = i < cnt;
    uint64_t h = 0, f = 0;
    uint32_t owner = 0;
    if (valid) {
      h = __ldg(a.hash + i);
      f = __ldg(a.fp + i);
      owner = owner_of(h, f, (uint32_t)a.world, a.hash_mode);
    }
    const unsigned vm = __ballot_sync(0xffffffffu, valid);
    if (!valid) continue;
    const unsigned peers = __match_any_sync(vm, owner);
    const int leader = __ffs(peers) - 1;
    uint32_t base = 0;
    if (lane == leader) base = atomicAdd(&a.send_counts[owner], (uint32_t)__popc(peers));
    base = __shfl_sync(peers, base, leader);
    const uint32_t pos = base + __popc(peers & ((1u << lane) - 1u));
    if (pos >= a.bucket_cap) {
      atomicOr(&a.ctrl->status, MGBS_ST_BUCKET_OVERFLOW);
      continue;
    }
    const uint64_t d = (uint64_t)owner * a.bucket_cap + pos;
    a.s_hash[d] = h;
    a.s_fp[d] = f;
    a.s_score[d] = __ldg(a.score + i);
    a.s_payload[d] = __ldg(a.payload + i);
    const uint4* src = reinterpret_cast<const uint4*>(a.states + (uint64_t)i * a.stride);
    uint4* dst = reinterpret_cast<uint4*>(a.s_states + d * a.stride);
    for (int q = 0; q < vecs; ++q) dst[q] = __ldg(src + q);
  }
}

// MGBS_EXCHANGE_PEER routing of one band.  The band histograms were counted where the candidates were generated
// and summed over ranks, so every rank derives the same band [D, E) here.  Each candidate of this rank inside the
// band goes to its owner as a 24-byte record (hash, fingerprint, score, back-pointer; the owner rebuilds the
// survivors' states from the back-pointers afterwards), appended to bucket [this rank] in the owner's symmetric
// region over NVLink; positions come from this rank's own per-destination cursor, which keeps growing over the
// rounds of a depth, so no remote atomics.  Only ~pool_target * duplicate ratio records cross the links instead of
// every candidate with its state.  The block that finishes last publishes the cursors and this rank's flag
// (epoch * 16 + round) to every owner, then waits - with a limit - until every sender has flagged this rank, so
// that when the kernel ends the receive buckets hold the whole band.
__global__ void __launch_bounds__(kStreamThreads) k_route_band(StepArgs a, RouteArgs r) {
  __shared__ int s_last;
  if (a.ctrl->halt || a.ctrl->bands_done) return;
  const uint64_t D = a.ctrl->band_lo[a.round];
  MgbsRadix st;
  if (a.levels == 1) st = band_initial(a, a.hist_prev, D);
  else st = a.ctrl->band[a.round][a.levels - 1];
  st = band_advance(st, a.hist_prev, a.key_bits, true, D);
  const uint64_t E = st.result;
  if (E <= D) return;  // same decision on every rank: nobody sends, nobody waits
  const uint32_t cnt = a.ctrl->cand_count;
  const uint32_t rounded = (cnt + 31u) & ~31u;
  const int lane = threadIdx.x & 31;
  const int hb = a.hash_bits;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < rounded; i += gridDim.x * blockDim.x) {
    bool in = false;
    uint64_t h = 0;
    uint32_t k = 0, owner = 0;
    uint64_t f = 0;
    if (i < cnt) {
      h = __ldg(r.hash + i);
      k = __ldg(r.score + i);
      const uint64_t s = order_key(k, h, hb);
      in = s >= D && s < E;
      if (in) {
        f = __ldg(r.fp + i);
        owner = owner_of(h, f, (uint32_t)r.world, r.hash_mode);
      }
    }
    const unsigned vm = __ballot_sync(0xffffffffu, in);
    if (!in) continue;
    const unsigned peers = __match_any_sync(vm, owner);
    const int leader = __ffs(peers) - 1;
    uint32_t base = 0;
    if (lane == leader) base = atomicAdd(&r.send_counts[owner], (uint32_t)__popc(peers));
    base = __shfl_sync(peers, base, leader);
    const uint32_t pos = base + __popc(peers & ((1u << lane) - 1u));
    if (pos >= r.bucket_cap) {
      atomicOr(&a.ctrl->status, MGBS_ST_BUCKET_OVERFLOW);
      continue;
    }
    uint8_t* ob = r.peer.base[owner];
    const uint64_t d = (uint64_t)r.rank * r.bucket_cap + pos;
    reinterpret_cast<uint64_t*>(ob + r.off_hash)[d] = h;
    reinterpret_cast<uint64_t*>(ob + r.off_fp)[d] = f;
    reinterpret_cast<uint32_t*>(ob + r.off_score)[d] = k;
    reinterpret_cast<uint32_t*>(ob + r.off_payload)[d] = __ldg(r.payload + i);
  }
  // completion: all of this rank's stores are ordered before its flag
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(&r.peer.tickets[r.peer.slot], 1u);
    s_last = ((t + 1u) % gridDim.x) == 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const uint32_t want = a.ctrl->epoch * 16u + (uint32_t)a.round;
  if ((int)threadIdx.x < r.world) {
    const int q = threadIdx.x;
    uint32_t fill = *reinterpret_cast<volatile uint32_t*>(&r.send_counts[q]);
    if (fill > r.bucket_cap) fill = r.bucket_cap;
    *reinterpret_cast<volatile uint32_t*>(r.peer.base[q] + r.off_counts + 4 * r.rank) = fill;
    __threadfence_system();
    *reinterpret_cast<volatile uint32_t*>(r.peer.base[q] + r.off_route_flag + 4 * r.rank) = want;
    volatile uint32_t* mine = reinterpret_cast<volatile uint32_t*>(r.peer.base[r.rank] + r.off_route_flag + 4 * q);
    bool ok = false;
    for (uint32_t it = 0; it < a.peer.poll_limit; ++it) {
      if ((int32_t)(*mine - want) >= 0) { ok = true; break; }
      if (it > 256) __nanosleep(200);
    }
    if (!ok) peer_give_up(a);
  }
  __threadfence_system();
}

// ------------------------------------------------------------------------------------------------
// Persistent selection kernel: everything after scoring in ONE launch (world 1 and MGBS_EXCHANGE_PEER).
//
// The staged form above needs about twenty launches per depth (per band round: histogram levels + insert; final
// histogram levels; emit; finish), most of them a few microseconds of work behind a launch, and in peer mode every
// cross-rank reduction sits at the end of a launch.  Here the same steps run as phases of one co-resident grid
// (cooperative launch, at most select_blocks_per_sm() blocks per SM) with a block barrier between them; block 0
// does the cross-rank work (histogram sums, band-route handshake, tie exchange) between two barriers.  Every
// decision is taken from histograms in global memory that all blocks read after a barrier, so the blocks agree;
// the arithmetic (band_initial / band_advance / final_initial / final_advance, table_insert, emit_row) is the same
// code the staged kernels call.
//
// The barrier is an arrival counter in the control block, reset when the depth opens; generation g is complete
// when the counter reaches g * gridDim.x.  Its wait is bounded: after grid_poll_limit polls the block sets
// MGBS_ST_GRID_TIMEOUT, and from then on no block waits any more (the depth ends with that status; the host stops).
// ------------------------------------------------------------------------------------------------

__device__ __forceinline__ void grid_barrier(const StepArgs& a, uint32_t& gen) {
  __syncthreads();
  gen += 1u;
  if (threadIdx.x == 0) {
    MgbsCtrl* c = a.ctrl;
    __threadfence();
    atomicAdd(&c->grid_bar, 1u);
    const uint32_t target = gen * gridDim.x;
    volatile uint32_t* bar = &c->grid_bar;
    volatile uint32_t* status = &c->status;
    uint32_t it = 0;
    while ((int32_t)(*bar - target) < 0) {
      if (*status & MGBS_ST_GRID_TIMEOUT) break;
      if (++it > a.grid_poll_limit) { atomicOr(&c->status, MGBS_ST_GRID_TIMEOUT); break; }
      if (it > 32) __nanosleep(40);
    }
    __threadfence();
  }
  __syncthreads();
}

// Count one radix level of the candidates in view cv into the shared histogram and add it to `hist`.
__device__ void count_candidates_level(const CandView& cv, const MgbsRadix& st, uint64_t D, int key_bits, int hash_bits,
                                       uint32_t* sh, uint32_t* hist) {
  for (int b = threadIdx.x; b < MGBS_RADIX_BINS; b += blockDim.x) sh[b] = 0;
  __syncthreads();
  const int db = digit_bits_at(key_bits, (int)st.bits_done);
  const int shift = key_bits - (int)st.bits_done - db;
  const uint32_t mask = (1u << db) - 1u;
  const int pshift = key_bits - (int)st.bits_done;
  const bool any_prefix = st.bits_done != 0;
  const uint64_t pfx = any_prefix ? (st.prefix >> pshift) : 0;
  for_each_candidate(cv, [&](uint64_t i, bool valid) {
    bool in = false;
    uint32_t digit = 0;
    if (valid) {
      const uint64_t s = order_key(__ldg(cv.score + i), __ldg(cv.hash + i), hash_bits);
      in = s >= D && (!any_prefix || (s >> pshift) == pfx);
      digit = (uint32_t)(s >> shift) & mask;
    }
    hist_add(sh, in, digit);
  });
  hist_flush(sh, hist);
}

__device__ void count_table_level(const StepArgs& a, const MgbsRadix& st, uint64_t base, int key_bits, uint32_t* sh,
                                  uint32_t* hist) {
  for (int b = threadIdx.x; b < MGBS_RADIX_BINS; b += blockDim.x) sh[b] = 0;
  __syncthreads();
  const int db = digit_bits_at(key_bits, (int)st.bits_done);
  const int shift = key_bits - (int)st.bits_done - db;
  const uint32_t mask = (1u << db) - 1u;
  const int pshift = key_bits - (int)st.bits_done;
  const bool any_prefix = st.bits_done != 0;
  const uint64_t pfx = any_prefix ? (st.prefix >> pshift) : 0;
  const Slot* table = reinterpret_cast<const Slot*>(a.table);
  const uint64_t cap = (uint64_t)a.hash_capacity;
  const uint64_t rounded = (cap + 31ull) & ~31ull;
  for (uint64_t j = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; j < rounded; j += (uint64_t)gridDim.x * blockDim.x) {
    bool in = false;
    uint32_t digit = 0;
    if (j < cap) {
      const ulonglong2 hf = __ldcg(reinterpret_cast<const ulonglong2*>(table + j));
      if (hf.x != 0ull && hf.y != 0ull) {
        const uint64_t best = ~__ldcg(&table[j].best_inv);
        const uint64_t s = order_key((uint32_t)(best >> 32), hf.x, a.hash_bits) - base;
        in = !any_prefix || (s >> pshift) == pfx;
        digit = (uint32_t)(s >> shift) & mask;
      }
    }
    hist_add(sh, in, digit);
  }
  hist_flush(sh, hist);
}

// Route this rank's candidates of the band [D, E) to their owners' receive buckets (the loop of k_route_band).
__device__ void route_band_body(const StepArgs& a, const RouteArgs& r, uint64_t D, uint64_t E) {
  const uint32_t cnt = a.ctrl->cand_count;
  const uint32_t rounded = (cnt + 31u) & ~31u;
  const int lane = threadIdx.x & 31;
  const int hb = a.hash_bits;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < rounded; i += gridDim.x * blockDim.x) {
    bool in = false;
    uint64_t h = 0, f = 0;
    uint32_t k = 0, owner = 0;
    if (i < cnt) {
      h = __ldg(r.hash + i);
      k = __ldg(r.score + i);
      const uint64_t s = order_key(k, h, hb);
      in = s >= D && s < E;
      if (in) {
        f = __ldg(r.fp + i);
        owner = owner_of(h, f, (uint32_t)r.world, r.hash_mode);
      }
    }
    const unsigned vm = __ballot_sync(0xffffffffu, in);
    if (!in) continue;
    const unsigned peers = __match_any_sync(vm, owner);
    const int leader = __ffs(peers) - 1;
    uint32_t base = 0;
    if (lane == leader) base = atomicAdd(&r.send_counts[owner], (uint32_t)__popc(peers));
    base = __shfl_sync(peers, base, leader);
    const uint32_t pos = base + __popc(peers & ((1u << lane) - 1u));
    if (pos >= r.bucket_cap) {
      atomicOr(&a.ctrl->status, MGBS_ST_BUCKET_OVERFLOW);
      continue;
    }
    uint8_t* ob = r.peer.base[owner];
    const uint64_t d = (uint64_t)r.rank * r.bucket_cap + pos;
    reinterpret_cast<uint64_t*>(ob + r.off_hash)[d] = h;
    reinterpret_cast<uint64_t*>(ob + r.off_fp)[d] = f;
    reinterpret_cast<uint32_t*>(ob + r.off_score)[d] = k;
    reinterpret_cast<uint32_t*>(ob + r.off_payload)[d] = __ldg(r.payload + i);
  }
  __threadfence_system();
}

// One block, after every block's routed records are fenced: publish the cursors and this rank's flag to every
// owner and wait (bounded) until every sender has flagged this rank.
__device__ void route_handshake_block(const StepArgs& a, const RouteArgs& r, int round) {
  const uint32_t want = a.ctrl->epoch * 16u + (uint32_t)round;
  if ((int)threadIdx.x < r.world) {
    const int q = threadIdx.x;
    uint32_t fill = *reinterpret_cast<volatile uint32_t*>(&r.send_counts[q]);
    if (fill > r.bucket_cap) fill = r.bucket_cap;
    *reinterpret_cast<volatile uint32_t*>(r.peer.base[q] + r.off_counts + 4 * r.rank) = fill;
    __threadfence_system();
    *reinterpret_cast<volatile uint32_t*>(r.peer.base[q] + r.off_route_flag + 4 * r.rank) = want;
    volatile uint32_t* mine = reinterpret_cast<volatile uint32_t*>(r.peer.base[r.rank] + r.off_route_flag + 4 * q);
    bool ok = false;
    for (uint32_t it = 0; it < a.peer.poll_limit; ++it) {
      if ((int32_t)(*mine - want) >= 0) { ok = true; break; }
      if (it > 256) __nanosleep(200);
    }
    if (!ok) peer_give_up(a);
  }
  __threadfence_system();
  __syncthreads();
}

// Insert the band [D, E) of the candidates this rank owns (the loop of k_band_insert).
__device__ void insert_band_body(const StepArgs& a, uint64_t D, uint64_t E) {
  Slot* table = reinterpret_cast<Slot*>(a.table);
  const uint64_t cap = (uint64_t)a.hash_capacity;
  const int hb = a.hash_bits;
  uint32_t fresh_total = 0, ins_total = 0, drop_total = 0;
  struct Item { uint32_t k; uint64_t h; };
  for_each_candidate_batched<Item>(
      a.cv,
      [&](uint64_t i) {
        Item it;  // past the L1 cache: in peer mode other ranks appended these records during this kernel
        it.k = __ldcg(a.cv.score + i);
        it.h = __ldcg(a.cv.hash + i);
        return it;
      },
      [&](uint64_t i, bool valid, const Item& it) {
        int res = -2;  // -2 = not in the band, -1 = dropped, >= 0 = slots claimed
        if (valid) {
          const uint64_t s = order_key(it.k, it.h, hb);
          if (s >= D && s < E) {
            const uint64_t val = ((uint64_t)it.k << 32) | (uint64_t)__ldcg(a.cv.payload + i);
            res = table_insert(table, cap, a.probe_limit, it.h, __ldcg(a.cv.fp + i), val);
          }
        }
        fresh_total += __reduce_add_sync(0xffffffffu, (uint32_t)(res > 0 ? res : 0));
        ins_total += __popc(__ballot_sync(0xffffffffu, res != -2));
        drop_total += __popc(__ballot_sync(0xffffffffu, res == -1));
      });
  if ((threadIdx.x & 31) == 0) {
    if (fresh_total) atomicAdd(&a.ctrl->table_count, fresh_total);
    if (ins_total) atomicAdd(&a.ctrl->inserted_total, ins_total);
    if (drop_total) {
      atomicAdd(&a.ctrl->hash_overflow, drop_total);
      atomicOr(&a.ctrl->status, MGBS_ST_HASH_OVERFLOW);
    }
  }
}

// Survivors below the cut straight from the table slots (the table-walk branch of k_emit); ties go to `seg`.
__device__ void emit_table_body(const StepArgs& a, const MgbsRadix& st, uint64_t base, unsigned long long* seg) {
  const uint64_t T = st.result;
  const bool ties = st.tie_need > 0;
  const uint64_t tie_key = st.tie_key;
  const Slot* table = reinterpret_cast<const Slot*>(a.table);
  const uint64_t cap = (uint64_t)a.hash_capacity;
  const int hb = a.hash_bits;
  const int lane = threadIdx.x & 31;
  const uint64_t rounded = (cap + 31ull) & ~31ull;
  for (uint64_t j = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; j < rounded; j += (uint64_t)gridDim.x * blockDim.x) {
    bool keep = false, tie = false;
    uint32_t k = 0, payload = 0;
    uint64_t h = 0, f = 0;
    if (j < cap) {
      const ulonglong2 hf = __ldcg(reinterpret_cast<const ulonglong2*>(table + j));
      if (hf.x != 0ull && hf.y != 0ull) {
        const uint64_t best = ~__ldcg(&table[j].best_inv);
        h = hf.x; f = hf.y;
        k = (uint32_t)(best >> 32);
        payload = (uint32_t)best;
        const uint64_t s = order_key(k, h, hb) - base;  // the cut was selected on keys relative to base
        keep = s < T;
        tie = !keep && ties && s == tie_key;
      }
    }
    const unsigned km = __ballot_sync(0xffffffffu, keep);
    if (km) {
      uint32_t pos0 = 0;
      if (lane == 0) pos0 = atomicAdd(&a.ctrl->next_count, (uint32_t)__popc(km));
      pos0 = __shfl_sync(0xffffffffu, pos0, 0);
      if (keep) emit_row(a, j, k, h, payload, pos0 + __popc(km & ((1u << lane) - 1u)));
    }
    if (tie) {
      const unsigned long long t = atomicAdd(seg, 1ull);
      if (t < MGBS_TIE_CAP) {
        seg[1 + 3 * t] = h;
        seg[2 + 3 * t] = f;
        seg[3 + 3 * t] = j;
      } else {
        atomicOr(&a.ctrl->status, MGBS_ST_TIE_OVERFLOW);
      }
    }
  }
}

// One block: bring every rank's tie records at the cut key together (peer stores + flags, bounded wait).  Only
// called when the cut needs a tie-break, which every rank derives from the same summed histogram.
__device__ void tie_exchange_block(const StepArgs& a, const unsigned long long* my_seg) {
  const uint32_t epoch = a.ctrl->epoch;
  const int W = a.world;
  for (int r = 0; r < W; ++r) {
    unsigned long long* dst = reinterpret_cast<unsigned long long*>(a.peer.base[r] + a.peer.off_tie) + (int64_t)a.rank * kTieSegWords;
    for (int i = threadIdx.x; i < kTieSegWords; i += blockDim.x) dst[i] = my_seg[i];
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < W) {
    const int r = threadIdx.x;
    *(reinterpret_cast<volatile uint32_t*>(a.peer.base[r] + a.peer.off_tie_flag) + a.rank) = epoch;
    volatile uint32_t* mine = reinterpret_cast<volatile uint32_t*>(a.peer.base[a.rank] + a.peer.off_tie_flag) + r;
    bool ok = false;
    for (uint32_t it = 0; it < a.peer.poll_limit; ++it) {
      if ((int32_t)(*mine - epoch) >= 0) { ok = true; break; }
      if (it > 256) __nanosleep(200);
    }
    if (!ok) peer_give_up(a);
  }
  __threadfence_system();
  __syncthreads();
}

// Band histogram over SCORES.  The selection key is the score above the top hash bits, and hashes are uniform, so the
// number of candidates below a key (s, hash prefix x) is count(score < s) + x * count(score == s) up to a binomial
// deviation far inside the tolerance of a band (any pool between the beam and the table's hard limit will do, and
// the statistics after the insert verify it).  One histogram over scores therefore places a band, where a radix
// descent over the whole key needs one pass per 11 bits.  Fine bins: bin 0 = score below the window, bin b in
// 1..2046 = score win_lo + b - 1, bin 2047 = above.  Coarse bins (to find a window when the previous depth's does
// not fit): score >> 9.
__device__ __forceinline__ uint32_t clamp_score(uint32_t k) { return k > 0xfffffu ? 0xfffffu : k; }

__device__ void count_score_window(const CandView& cv, uint64_t D, uint32_t win_lo, bool coarse, int hash_bits,
                                   uint32_t* sh, uint32_t* hist) {
  for (int b = threadIdx.x; b < MGBS_RADIX_BINS; b += blockDim.x) sh[b] = 0;
  __syncthreads();
  struct Item { uint32_t k; uint64_t h; };
  const bool need_hash = D != 0ull && hash_bits != 0;
  for_each_candidate_batched<Item>(
      cv,
      [&](uint64_t i) {
        Item it;
        it.k = __ldg(cv.score + i);
        it.h = need_hash ? __ldg(cv.hash + i) : 0ull;
        return it;
      },
      [&](uint64_t, bool valid, const Item& it) {
        bool in = false;
        uint32_t bin = 0;
        if (valid) {
          const uint32_t k = clamp_score(it.k);
          in = D == 0ull || order_key(k, it.h, hash_bits) >= D;
          if (coarse) {
            bin = k >> 9;
          } else {
            const uint32_t rel = k < win_lo ? 0u : k - win_lo + 1u;
            bin = rel > (uint32_t)(MGBS_RADIX_BINS - 1) ? (uint32_t)(MGBS_RADIX_BINS - 1) : rel;
          }
        }
        hist_add(sh, in, bin);
      });
  hist_flush(sh, hist);
}

// First and last non-empty bin of a 2048-bin histogram (-1, -1 when empty); same answer on every thread.
__device__ void hist_extent(const uint32_t* hist, int& first, int& last) {
  __shared__ int s_first, s_last;
  if (threadIdx.x == 0) { s_first = MGBS_RADIX_BINS; s_last = -1; }
  __syncthreads();
  constexpr int PER = MGBS_RADIX_BINS / kStreamThreads;
  int lo = MGBS_RADIX_BINS, hi = -1;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int b = threadIdx.x * PER + j;
    if (__ldcg(hist + b) != 0u) { lo = b < lo ? b : lo; hi = b; }
  }
  if (hi >= 0) { atomicMin(&s_first, lo); atomicMax(&s_last, hi); }
  __syncthreads();
  first = s_last >= 0 ? s_first : -1;
  last = s_last;
  __syncthreads();
}

// Band bound from a fine score histogram: true = st.result holds the bound, false = the cut score lies outside the
// window (or in its open-ended first / last bin).
__device__ bool band_from_window(MgbsRadix& st, const uint32_t* hist, uint32_t win_lo, int hash_bits, uint64_t D,
                                 uint32_t& cut_score) {
  const Cross c = find_crossing(hist, st.remaining, true);
  if (c.bin < 0) {  // everything that is left fits
    st.result = ~0ull;
    st.done = 1;
    cut_score = 0xffffffffu;
    return true;
  }
  if (c.bin == 0 || c.bin == MGBS_RADIX_BINS - 1) return false;
  const uint64_t sstar = (uint64_t)win_lo + (uint64_t)c.bin - 1ull;
  cut_score = (uint32_t)sstar;
  uint64_t E;
  if (hash_bits == 0) {
    E = sstar;  // score-only order: the level that does not fit whole stays out
  } else {
    const uint64_t full = 1ull << hash_bits;
    const uint64_t lo = (D >> hash_bits) == sstar ? (D & (full - 1ull)) : 0ull;  // the level is partly inserted already
    const uint64_t range = full - lo;
    const uint64_t r = st.remaining - c.before, cnt = c.count;  // r < cnt
    const uint64_t part = (range / cnt) * r + ((range % cnt) * r) / cnt;
    E = (sstar << hash_bits) | (lo + part);
  }
  st.result = E > D ? E : D;
  st.done = 1;
  return true;
}

__device__ __forceinline__ int ceil_log2_u64(uint64_t x) {  // smallest b with 2^b >= x, x >= 1
  return x <= 1ull ? 0 : 64 - __clzll((long long)(x - 1ull));
}

__global__ void __launch_bounds__(kStreamThreads, 2) k_select(StepArgs a, RouteArgs pr) {
  __shared__ uint32_t sh[MGBS_RADIX_BINS];
  MgbsCtrl* c = a.ctrl;
  if (c->halt) {
    if (blockIdx.x == 0 && threadIdx.x == 0) write_mirror(a);
    return;
  }
  const bool peer = a.peer.enabled != 0;
  const bool lead = blockIdx.x == 0 && threadIdx.x == 0;
  const int R = a.rounds;
  constexpr int kBandSlots = 3;  // histograms a band round may use: score window, coarse scores, second window
  uint32_t gen = 0;

  // ---------------- band rounds: dedup the best-scoring candidates into the table ----------------
  uint64_t D = 0;
  int rounds_run = 0;
  uint32_t win_lo = c->win_lo, next_win_lo = c->win_lo;
  uint32_t score_min = 0, score_max = 0xfffffu;
  bool range_known = false;
  while (rounds_run < R) {
    const int round = rounds_run;
    a.round = round;
    uint32_t* hist0 = a.hist_base + (int64_t)(round * kBandSlots) * MGBS_HIST_STRIDE;
    a.hist = hist0;
    // one histogram over the scores of every remaining candidate; it also carries the per-rank statistics
    MgbsRadix st = radix_zero();
    st.done = (D == ~0ull) ? 1u : 0u;
    publish_stats(a);
    if (!st.done) count_score_window(a.cvh, D, win_lo, false, a.hash_bits, sh, hist0);
    grid_barrier(a, gen);
    if (peer) {
      if (blockIdx.x == 0) peer_allreduce_block(a, hist0, round * kBandSlots);
      grid_barrier(a, gen);
    }
    st = band_initial(a, hist0, D);
    const uint32_t* win_hist = hist0;
    uint32_t cut_score = 0xffffffffu;
    if (!st.done && !band_from_window(st, hist0, win_lo, a.hash_bits, D, cut_score)) {
      // the window inherited from the previous depth misses the cut: find the cut's coarse score range, put a
      // window around it and count once more (first depth of a search, or a jump of the scores between depths)
      uint32_t* histc = hist0 + MGBS_HIST_STRIDE;
      count_score_window(a.cvh, D, 0u, true, a.hash_bits, sh, histc);
      grid_barrier(a, gen);
      if (peer) {
        if (blockIdx.x == 0) peer_allreduce_block(a, histc, round * kBandSlots + 1);
        grid_barrier(a, gen);
      }
      const Cross cc = find_crossing(histc, st.remaining, true);
      const uint32_t cb = cc.bin < 0 ? 0u : (uint32_t)cc.bin;
      win_lo = cb * 512u > 767u ? cb * 512u - 767u : 0u;
      uint32_t* hist2 = histc + MGBS_HIST_STRIDE;
      count_score_window(a.cvh, D, win_lo, false, a.hash_bits, sh, hist2);
      grid_barrier(a, gen);
      if (peer) {
        if (blockIdx.x == 0) peer_allreduce_block(a, hist2, round * kBandSlots + 2);
        grid_barrier(a, gen);
      }
      win_hist = hist2;
      if (!band_from_window(st, hist2, win_lo, a.hash_bits, D, cut_score)) {
        st.result = D;  // cannot happen (the window was placed around the cut); ends the round without a band
        st.done = 1;
      }
    }
    if (round == 0) {
      // score range of everything generated this depth: bounds the keys of the final cut
      int b_first, b_last;
      hist_extent(win_hist, b_first, b_last);
      if (b_first >= 1 && b_last >= b_first && b_last <= MGBS_RADIX_BINS - 2) {
        score_min = win_lo + (uint32_t)b_first - 1u;
        score_max = win_lo + (uint32_t)b_last - 1u;
        range_known = true;
      }
      if (cut_score != 0xffffffffu) next_win_lo = cut_score > 1023u ? cut_score - 1023u : 0u;
      else if (range_known) next_win_lo = (score_min + score_max) / 2u > 1023u ? (score_min + score_max) / 2u - 1023u : 0u;
      else next_win_lo = win_lo;
    }
    const uint64_t E = st.result;
    const bool complete = (st.flag & kFlagComplete) != 0u;
    if (lead) {
      c->band[round][0] = st;
      c->band_lo[round + 1] = E > D ? E : D;
      if (complete) {
        c->bands_done = 1;
      } else {
        c->rounds_used = round + 1;
        if (E <= D) atomicOr(&c->status, MGBS_ST_BAND_STALL);
      }
    }
    ++rounds_run;
    if (complete) break;
    if (E > D) {
      if (peer) {
        route_band_body(a, pr, D, E);
        grid_barrier(a, gen);
        if (blockIdx.x == 0) route_handshake_block(a, pr, round);
        grid_barrier(a, gen);
      }
      insert_band_body(a, D, E);
      grid_barrier(a, gen);  // table_count / inserted_total are final before the next statistics are published
      D = E;
    }
  }
  // later entries keep the last bound, so that close_depth sees where the bands stopped
  if (lead)
    for (int r = rounds_run + 1; r <= R; ++r) c->band_lo[r] = D;

  // ---------------- final cut: the key of the beam-th unique entry, by radix select over the table ----------------
  // Every table entry has a score inside [score_min, score_max] and a key below the last band bound, so the select
  // runs on key - base with only as many bits as that range needs (three 11-bit levels where the whole 44-bit key
  // would take four); base and bit count derive from summed histograms, so all blocks and ranks agree.
  uint64_t base = 0;
  int kb = a.key_bits;
  if (range_known) {
    uint64_t top_score = score_max;
    if (D != ~0ull && a.hash_bits > 0 && (D >> a.hash_bits) < top_score) top_score = D >> a.hash_bits;  // keys < D only
    if (D != ~0ull && a.hash_bits == 0 && D > 0 && D - 1 < top_score) top_score = D - 1;
    if (top_score >= score_min) {
      base = (uint64_t)score_min << a.hash_bits;
      kb = ceil_log2_u64(top_score - score_min + 1ull) + a.hash_bits;
      if (kb < 1) kb = 1;
      if (kb > a.key_bits) { kb = a.key_bits; base = 0; }
    }
  }
  const int Lf = (kb + MGBS_RADIX_BITS - 1) / MGBS_RADIX_BITS;
  uint32_t* fin0 = a.hist_base + (int64_t)(R * kBandSlots) * MGBS_HIST_STRIDE;
  a.hist = fin0;
  publish_stats(a);
  MgbsRadix fs = radix_zero();
  count_table_level(a, fs, base, kb, sh, fin0);
  grid_barrier(a, gen);
  if (peer) {
    if (blockIdx.x == 0) peer_allreduce_block(a, fin0, R * kBandSlots);
    grid_barrier(a, gen);
  }
  fs = final_initial(a, fin0);
  for (int l = 1; l < Lf; ++l) {
    uint32_t* hist = fin0 + (int64_t)l * MGBS_HIST_STRIDE;
    fs = final_advance(fs, hist - MGBS_HIST_STRIDE, kb, a.select_mode);
    if (fs.done) break;
    count_table_level(a, fs, base, kb, sh, hist);
    grid_barrier(a, gen);
    if (peer) {
      if (blockIdx.x == 0) peer_allreduce_block(a, hist, R * kBandSlots + l);
      grid_barrier(a, gen);
    }
  }
  if (!fs.done) fs = final_advance(fs, fin0 + (int64_t)(Lf - 1) * MGBS_HIST_STRIDE, kb, a.select_mode);
  if (lead) {
    c->fin[0] = fs;
    c->fin[1].prefix = base;
    c->fin[1].bits_done = (uint32_t)kb;
    c->threshold_key = fs.result == ~0ull ? ~0ull : base + fs.result;
    c->win_lo = next_win_lo;
  }
  unsigned long long* seg = a.tie_buf + (int64_t)a.rank * kTieSegWords;
  emit_table_body(a, fs, base, seg);
  grid_barrier(a, gen);
  if (blockIdx.x != 0) return;
  // ---------------- one block: ties at the cut key, then close the depth ----------------
  const unsigned long long* tie_all = a.tie_buf;
  if (fs.tie_need > 0 && peer) {
    tie_exchange_block(a, seg);
    tie_all = reinterpret_cast<const unsigned long long*>(a.peer.base[a.rank] + a.peer.off_tie);
  }
  resolve_ties(a, fs, tie_all);
  __syncthreads();
  if (threadIdx.x == 0) close_depth(a, fin0);
}

// Copy rows of n bytes between a packed and a padded layout (bytes n..pitch of a padded destination row are zeroed).
__global__ void __launch_bounds__(256) k_repack_rows(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                     int64_t rows, int src_pitch, int dst_pitch, int n) {
  const int64_t total = rows * dst_pitch;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / dst_pitch;
    const int c = (int)(i - r * dst_pitch);
    dst[i] = c < n ? src[r * src_pitch + c] : (uint8_t)0;
  }
}

// After the exchange a bucket may claim more than it holds when the sender overflowed: clamp.
__global__ void k_clamp_counts(uint32_t* counts, int world, uint32_t cap) {
  const int r = threadIdx.x;
  if (r < world && counts[r] > cap) counts[r] = cap;
}

}  // namespace mgbs

// ------------------------------------------------------------------------------------------------
// Launchers (host)
// ------------------------------------------------------------------------------------------------

namespace mgbs {

static inline int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

SymLayout sym_layout(const MgbsConfig& c, int band_levels_effective) {
  SymLayout L;
  const int64_t W = c.world_size, cap = c.bucket_cap;
  int64_t off = 0;
  for (int p = 0; p < 2; ++p) {
    L.hash[p] = off;    off += align256(W * cap * 8);
    L.fp[p] = off;      off += align256(W * cap * 8);
    L.score[p] = off;   off += align256(W * cap * 4);
    L.payload[p] = off; off += align256(W * cap * 4);
    L.counts[p] = off;  off += align256(W * 4);
  }
  for (int p = 0; p < 2; ++p) { L.frontier[p] = off; off += align256(c.frontier_cap * (int64_t)c.state_stride); }
  L.route_flag = off; off += align256(W * 4);
  L.slots = c.band_rounds * (band_levels_effective < 3 ? 3 : band_levels_effective) + MGBS_MAX_LEVELS;
  L.hx = off;         off += align256((int64_t)L.slots * W * MGBS_HIST_STRIDE * 4);
  L.hflag = off;      off += align256((int64_t)L.slots * W * 4);
  L.tie = off;        off += align256(W * (int64_t)kTieSegWords * 8);
  L.tie_flag = off;   off += align256(W * 4);
  L.abort_word = off; off += 256;
  L.total = off;
  return L;
}

static inline int grid_for(int64_t items, int sms) {
  int64_t g = (items + kStreamThreads * 4 - 1) / (kStreamThreads * 4);
  const int64_t cap = (int64_t)sms * 4;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

template <int WORDS, int ZOB>
static int launch_expand_t(const ExpandArgs& a, int grid, cudaStream_t st) {
  const int smem = ExpandSmem<WORDS>::total(a.fanout);
  if (smem > 48 * 1024) {
    cudaError_t ce = cudaFuncSetAttribute(k_expand<WORDS, ZOB>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (ce != cudaSuccess) return (int)ce;
  }
  k_expand<WORDS, ZOB><<<grid, kExpandThreads, smem, st>>>(a);
  return (int)cudaGetLastError();
}

int launch_expand(const ExpandArgs& a, int64_t max_parents, int sms, cudaStream_t st) {
  const int words = a.stride / 4;
  int64_t tiles = (max_parents + kExpandTile - 1) / kExpandTile;
  int grid = (int)(tiles < (int64_t)sms * 6 ? (tiles < 1 ? 1 : tiles) : (int64_t)sms * 6);
  if (a.zobrist) {
    switch (words) {
      case 4: return launch_expand_t<4, 1>(a, grid, st);
      case 8: return launch_expand_t<8, 1>(a, grid, st);
      case 16: return launch_expand_t<16, 1>(a, grid, st);
      case 24: return launch_expand_t<24, 1>(a, grid, st);
      case 32: return launch_expand_t<32, 1>(a, grid, st);
      default: return MGBS_ERR_UNSUPPORTED;
    }
  }
  switch (words) {
    case 4: return launch_expand_t<4, 0>(a, grid, st);
    case 8: return launch_expand_t<8, 0>(a, grid, st);
    case 16: return launch_expand_t<16, 0>(a, grid, st);
    case 24: return launch_expand_t<24, 0>(a, grid, st);
    case 32: return launch_expand_t<32, 0>(a, grid, st);
    default: return MGBS_ERR_UNSUPPORTED;
  }
}

int launch_depth_begin(MgbsCtrl* c, int parity, int fanout, int64_t cand_cap, unsigned long long* tie_seg,
                       uint32_t* send_counts, uint32_t* recv_counts, int world, int64_t active_limit, int auto_halt,
                       const uint32_t* abort_word, cudaStream_t st) {
  k_depth_begin<<<1, 32, 0, st>>>(c, parity, fanout, cand_cap, tie_seg, send_counts, recv_counts, world, active_limit,
                                  auto_halt, abort_word);
  return (int)cudaGetLastError();
}

int launch_band_hist(const StepArgs& a, int64_t items, int sms, cudaStream_t st) {
  k_band_hist<<<grid_for(items, sms), kStreamThreads, 0, st>>>(a);
  return (int)cudaGetLastError();
}

int launch_band_insert(const StepArgs& a, int64_t items, int sms, cudaStream_t st) {
  k_band_insert<<<grid_for(items, sms), kStreamThreads, 0, st>>>(a);
  return (int)cudaGetLastError();
}

int launch_final_hist(const StepArgs& a, int64_t slots, int sms, cudaStream_t st) {
  k_final_hist<<<grid_for(slots, sms), kStreamThreads, 0, st>>>(a);
  return (int)cudaGetLastError();
}

int launch_emit(const StepArgs& a, int64_t items, int sms, cudaStream_t st) {
  k_emit<<<grid_for(items, sms), kStreamThreads, 0, st>>>(a);
  return (int)cudaGetLastError();
}

int launch_finish(const StepArgs& a, cudaStream_t st) {
  k_finish<<<1, kStreamThreads, 0, st>>>(a);
  return (int)cudaGetLastError();
}

int select_blocks_per_sm() {
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_select, kStreamThreads, 0) != cudaSuccess) return 1;
  if (occ > 2) occ = 2;
  return occ < 1 ? 1 : occ;
}

int launch_select(const StepArgs& a, const RouteArgs& r, int sms, bool cooperative, cudaStream_t st) {
  const int grid = sms * select_blocks_per_sm();
  if (cooperative) {
    void* args[2] = {const_cast<StepArgs*>(&a), const_cast<RouteArgs*>(&r)};
    return (int)cudaLaunchCooperativeKernel(reinterpret_cast<void*>(k_select), dim3(grid), dim3(kStreamThreads), args, 0, st);
  }
  k_select<<<grid, kStreamThreads, 0, st>>>(a, r);
  return (int)cudaGetLastError();
}

int launch_route(const RouteArgs& a, int64_t items, int sms, cudaStream_t st) {
  k_route<<<grid_for(items, sms), kStreamThreads, 0, st>>>(a);
  return (int)cudaGetLastError();
}

int launch_route_band(const StepArgs& a, const RouteArgs& r, int64_t items, int sms, cudaStream_t st) {
  k_route_band<<<grid_for(items, sms), kStreamThreads, 0, st>>>(a, r);
  return (int)cudaGetLastError();
}

int launch_repack_rows(const uint8_t* src, uint8_t* dst, int64_t rows, int src_pitch, int dst_pitch, int n, int sms,
                       cudaStream_t st) {
  if (rows <= 0) return 0;
  k_repack_rows<<<grid_for(rows * dst_pitch, sms), 256, 0, st>>>(src, dst, rows, src_pitch, dst_pitch, n);
  return (int)cudaGetLastError();
}

int launch_clamp_counts(uint32_t* counts, int world, uint32_t cap, cudaStream_t st) {
  k_clamp_counts<<<1, 32, 0, st>>>(counts, world, cap);
  return (int)cudaGetLastError();
}

}  // namespace mgbs
