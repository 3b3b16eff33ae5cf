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
// One thread per candidate because both hashes are serial byte chains.  A block stages 64 parent rows in
// shared memory with a row pitch of stride+4 bytes (odd word pitch: the 32 lanes of a warp read 32 different
// rows at the same byte offset without bank conflicts) and the generator tables next to them; a warp handles
// one move for 32 parents, so the table lookups are broadcasts.
// ------------------------------------------------------------------------------------------------


template <int WORDS, int ZOB>
__global__ void __launch_bounds__(kExpandThreads, 3) k_expand(ExpandArgs a) {
  constexpr int PITCH_W = WORDS + 1;
  __shared__ uint32_t par_s[kExpandTile * PITCH_W];
  __shared__ uint32_t gen_s[MGBS_MAX_FANOUT * WORDS];
  __shared__ uint32_t sol_s[WORDS];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int n = a.n;
  const int G = a.fanout;
  const int64_t P = a.count_dev ? (int64_t)(*a.count_dev) : a.count;

  // generator tables and solved state, padded to WORDS*4 bytes per row
  for (int i = tid; i < G * WORDS * 4; i += kExpandThreads) {
    int g = i / (WORDS * 4), b = i - g * (WORDS * 4);
    reinterpret_cast<uint8_t*>(gen_s)[i] = b < n ? a.gens[g * n + b] : 0;
  }
  for (int i = tid; i < WORDS * 4; i += kExpandThreads) reinterpret_cast<uint8_t*>(sol_s)[i] = i < n ? a.solved[i] : 0;

  const int64_t ntiles = (P + kExpandTile - 1) / kExpandTile;
  const uint32_t* fw = reinterpret_cast<const uint32_t*>(a.frontier);
  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int64_t p0 = tile * kExpandTile;
    __syncthreads();
    for (int i = tid; i < kExpandTile * WORDS; i += kExpandThreads) {
      int r = i / WORDS, w = i - r * WORDS;
      int64_t p = p0 + r;
      par_s[r * PITCH_W + w] = p < P ? fw[p * WORDS + w] : 0u;
    }
    __syncthreads();
    for (int u = warp; u < 2 * G; u += kExpandThreads / 32) {
      const int g = u >> 1;
      const int pl = ((u & 1) << 5) + lane;
      const int64_t p = p0 + pl;
      if (p >= P) continue;
      const uint8_t* row = reinterpret_cast<const uint8_t*>(par_s + pl * PITCH_W);
      uint64_t h = ZOB ? 0ull : kFnvOffset, f = ZOB ? 0ull : kGolden;
      const ulonglong2* ztab = reinterpret_cast<const ulonglong2*>(a.zobrist);
      int ham = 0;
      const int64_t c = p * G + g;
      uint4* child_dst = a.children ? reinterpret_cast<uint4*>(a.children + c * (int64_t)a.stride) : nullptr;
      // 16 bytes of the child at a time: the four words are stored as soon as they are complete, so that only
      // four of them are live (the register count decides how many warps hide the shared-memory latency)
#pragma unroll
      for (int q = 0; q < WORDS / 4; ++q) {
        uint32_t cw[4];
#pragma unroll
        for (int w4 = 0; w4 < 4; ++w4) {
          const int wi = q * 4 + w4;
          const uint32_t gi = gen_s[g * WORDS + wi];
          const uint32_t sv = sol_s[wi];
          uint32_t acc = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (wi * 4 + j < n) {
              const uint32_t v = row[(gi >> (8 * j)) & 0xffu];
              if (ZOB) {
                const ulonglong2 z = __ldg(ztab + (wi * 4 + j) * a.zobrist_values + (int)v);
                h ^= z.x;
                f ^= z.y;
              } else {
                h = (h ^ (uint64_t)v) * kFnvPrime;
                f ^= (uint64_t)v + kGolden + (f << 6) + (f >> 2);
              }
              ham += (v != ((sv >> (8 * j)) & 0xffu));
              acc |= v << (8 * j);
            }
          }
          cw[w4] = acc;
        }
        if (child_dst) child_dst[q] = make_uint4(cw[0], cw[1], cw[2], cw[3]);
      }
      if (ZOB) {
        h = finish_zobrist_lo(h);
        f = finish_zobrist_hi(f);
      } else {
        h = finish_hash(h);
        f = finish_fingerprint(f);
      }
      const uint32_t payload = pack_payload((uint32_t)p, (uint32_t)a.rank, (uint32_t)g);
      a.cand_hash[c] = h;
      a.cand_fp[c] = f;
      a.cand_payload[c] = payload;
      if (a.score_mode == MGBS_SCORE_HAMMING) a.cand_score[c] = (uint32_t)ham;
      else if (a.score_mode == MGBS_SCORE_UNIFORM) a.cand_score[c] = (uint32_t)a.uniform_score;
      if (ham == 0 && a.ctrl) atomicMin(&a.ctrl->found_payload, payload);
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
    a.hist[MGBS_RADIX_BINS + a.rank] = a.ctrl->table_count;
    a.hist[MGBS_RADIX_BINS + 16 + a.rank] = a.ctrl->inserted_total;
    a.hist[MGBS_RADIX_BINS + 32] = (a.ctrl->found_payload != 0xffffffffu) ? 1u : 0u;
  }
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
  const uint32_t epoch = a.ctrl->epoch;
  const int W = a.world;
  const int64_t slot_words = (int64_t)a.peer.slot * W * MGBS_HIST_STRIDE;
  // every thread keeps its words of the local histogram in registers (independent loads, issued together) and
  // stores them to all peers: stores do not stall, so the push costs one load latency instead of one per word
  constexpr int PER = (MGBS_HIST_STRIDE + kStreamThreads - 1) / kStreamThreads;
  uint32_t mine_v[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = threadIdx.x + j * kStreamThreads;
    mine_v[j] = i < MGBS_HIST_STRIDE ? __ldcg(a.hist + i) : 0u;
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
    volatile uint32_t* f = reinterpret_cast<volatile uint32_t*>(a.peer.base[r] + a.peer.off_hflag) +
                           (int64_t)a.peer.slot * W + a.rank;
    *f = epoch;
    volatile uint32_t* mine = reinterpret_cast<volatile uint32_t*>(a.peer.base[a.rank] + a.peer.off_hflag) +
                              (int64_t)a.peer.slot * W + r;
    bool ok = false;
    for (uint32_t it = 0; it < (1u << 22); ++it) {
      if ((int32_t)(*mine - epoch) >= 0) { ok = true; break; }
      if (it > 1024) __nanosleep(100);
    }
    if (!ok) atomicOr(&a.ctrl->status, MGBS_ST_PEER_TIMEOUT);
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
    if (i < MGBS_HIST_STRIDE) a.hist[i] = sum[j];
  }
}

// Band histogram of one level.  Level 0 needs only the lower bound D; deeper levels first consume the previous
// level's (all-reduced) histogram to learn which prefix to refine.
__global__ void __launch_bounds__(kStreamThreads) k_band_hist(StepArgs a) {
  __shared__ uint32_t sh[MGBS_RADIX_BINS];
  for (int b = threadIdx.x; b < MGBS_RADIX_BINS; b += blockDim.x) sh[b] = 0;
  // an earlier round found the pool complete (from summed statistics, so every rank agrees): nothing left to do,
  // not even the reduction
  if (a.ctrl->bands_done) return;
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
  if ((int64_t)pos >= a.frontier_cap) {
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

// One block: resolve ties at the cut key against the tie records of all ranks, then close the depth.
__global__ void __launch_bounds__(kStreamThreads) k_finish(StepArgs a) {
  const MgbsRadix st = a.ctrl->fin[a.levels];
  const uint64_t need = st.tie_need;
  if (need > 0) {
    const unsigned long long* mine = a.tie_buf + (int64_t)a.rank * kTieSegWords;
    uint64_t my_n = mine[0] < MGBS_TIE_CAP ? mine[0] : MGBS_TIE_CAP;
    for (uint64_t t = threadIdx.x; t < my_n; t += blockDim.x) {
      const uint64_t h = mine[1 + 3 * t], f = mine[2 + 3 * t], i = mine[3 + 3 * t];
      uint64_t before = 0;
      for (int r = 0; r < a.world; ++r) {
        const unsigned long long* seg = a.tie_buf + (int64_t)r * kTieSegWords;
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
  __syncthreads();
  if (threadIdx.x == 0) {
    MgbsCtrl* c = a.ctrl;
    uint64_t u_tot, u_max, i_tot;
    uint32_t found_any;
    read_stats(a.hist_stats, a.world, u_tot, u_max, i_tot, found_any);
    uint32_t nc = c->next_count;
    if ((int64_t)nc > a.frontier_cap) nc = (uint32_t)a.frontier_cap;
    c->frontier_count[a.parity ^ 1] = (int32_t)nc;
    c->unique_total = (uint32_t)u_tot;
    if (u_tot > 0 && i_tot >= u_tot) { c->rho_num = i_tot; c->rho_den = u_tot; }
    if (u_tot < (uint64_t)a.beam && c->band_lo[a.rounds] != ~0ull)
      atomicOr(&c->status, MGBS_ST_ROUNDS_EXHAUSTED);
    if (found_any && !c->found) {
      c->found = 1;
      c->found_depth = c->depth + 1;
    }
    c->total_candidates += c->cand_count;
    c->depth += 1;
  }
}

// One thread: open the depth.
__global__ void k_depth_begin(MgbsCtrl* c, int parity, int fanout, int64_t cand_cap, unsigned long long* tie_seg,
                              uint32_t* send_counts, uint32_t* recv_counts, int world) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  int64_t cand = (int64_t)c->frontier_count[parity] * fanout;
  if (cand > cand_cap) cand = cand_cap;
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
  if (a.ctrl->bands_done) return;
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
    for (uint32_t it = 0; it < (1u << 22); ++it) {
      if ((int32_t)(*mine - want) >= 0) { ok = true; break; }
      if (it > 256) __nanosleep(200);
    }
    if (!ok) atomicOr(&a.ctrl->status, MGBS_ST_PEER_TIMEOUT);
  }
  __threadfence_system();
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
  L.slots = c.band_rounds * band_levels_effective + MGBS_MAX_LEVELS;
  L.hx = off;         off += align256((int64_t)L.slots * W * MGBS_HIST_STRIDE * 4);
  L.hflag = off;      off += align256((int64_t)L.slots * W * 4);
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

int launch_expand(const ExpandArgs& a, int64_t max_parents, int sms, cudaStream_t st) {
  const int words = a.stride / 4;
  int64_t tiles = (max_parents + kExpandTile - 1) / kExpandTile;
  int grid = (int)(tiles < (int64_t)sms * 6 ? (tiles < 1 ? 1 : tiles) : (int64_t)sms * 6);
  if (a.zobrist) {
    switch (words) {
      case 4: k_expand<4, 1><<<grid, kExpandThreads, 0, st>>>(a); break;
      case 8: k_expand<8, 1><<<grid, kExpandThreads, 0, st>>>(a); break;
      case 16: k_expand<16, 1><<<grid, kExpandThreads, 0, st>>>(a); break;
      case 24: k_expand<24, 1><<<grid, kExpandThreads, 0, st>>>(a); break;
      case 32: k_expand<32, 1><<<grid, kExpandThreads, 0, st>>>(a); break;
      default: return MGBS_ERR_UNSUPPORTED;
    }
    return (int)cudaGetLastError();
  }
  switch (words) {
    case 4: k_expand<4, 0><<<grid, kExpandThreads, 0, st>>>(a); break;
    case 8: k_expand<8, 0><<<grid, kExpandThreads, 0, st>>>(a); break;
    case 16: k_expand<16, 0><<<grid, kExpandThreads, 0, st>>>(a); break;
    case 24: k_expand<24, 0><<<grid, kExpandThreads, 0, st>>>(a); break;
    case 32: k_expand<32, 0><<<grid, kExpandThreads, 0, st>>>(a); break;
    default: return MGBS_ERR_UNSUPPORTED;
  }
  return (int)cudaGetLastError();
}

int launch_depth_begin(MgbsCtrl* c, int parity, int fanout, int64_t cand_cap, unsigned long long* tie_seg,
                       uint32_t* send_counts, uint32_t* recv_counts, int world, cudaStream_t st) {
  k_depth_begin<<<1, 32, 0, st>>>(c, parity, fanout, cand_cap, tie_seg, send_counts, recv_counts, world);
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
