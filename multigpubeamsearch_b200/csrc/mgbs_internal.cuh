// Argument blocks and launcher prototypes shared by the step kernels and the engine.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "mgbs.h"

namespace mgbs {

constexpr int kExpandThreads = 256;
constexpr int kExpandTile = 64;  // parents per block iteration
constexpr int kStreamThreads = 256;

// Tie records of all ranks: world segments of {count, then MGBS_TIE_CAP x (hash, fingerprint, candidate index)}.
constexpr int kTieSegWords = 1 + 3 * MGBS_TIE_CAP;

// Peer-mapped symmetric regions (MGBS_EXCHANGE_PEER).  base[r] is rank r's region as seen from this GPU
// (base[rank] is the local one).  Offsets are the same on every rank.
struct SymLayout {
  int64_t hash[2], fp[2], score[2], payload[2], counts[2];  // receive buckets per frontier parity (records only)
  int64_t frontier[2];  // the two frontier buffers: peers read parent rows from them when they rebuild survivors
  int64_t route_flag;   // [world] u32: sender r finished routing a band (value = epoch * 16 + round)
  int64_t hx;          // [slots][world][MGBS_HIST_STRIDE] u32 histogram exchange
  int64_t hflag;       // [slots][world] u32
  int64_t tie;         // [world][kTieSegWords] u64: tie records of every rank at the cut key (persistent selection)
  int64_t tie_flag;    // [world] u32: rank r's tie records have arrived (value = epoch)
  int64_t abort_word;  // u32: epoch in which some rank gave up a wait and told everybody (0 = never)
  int64_t total;
  int32_t slots;
};

struct PeerCtx {
  uint8_t* base[MGBS_MAX_WORLD];
  int64_t off_hx, off_hflag;
  int64_t off_tie, off_tie_flag, off_abort;
  uint32_t* tickets;
  int32_t enabled;
  int32_t slot;  // histogram slot of this launch
  uint32_t poll_limit;  // polls before a wait for another rank gives up
};

struct ExpandArgs {
  const uint8_t* frontier;
  const int32_t* count_dev;
  int64_t count;
  const uint8_t* gens;
  const uint8_t* solved;
  int32_t n, stride, fanout, rank, score_mode, uniform_score;
  uint8_t* children;
  uint64_t* cand_hash;
  uint64_t* cand_fp;
  uint32_t* cand_score;
  uint32_t* cand_payload;
  MgbsCtrl* ctrl;
  const uint64_t* zobrist;  // MGBS_HASH_ZOBRIST128: [n, zobrist_values, 2]; null = FNV hash + fingerprint
  int32_t zobrist_values;
};

// Candidate view: one or more buckets of `cap` entries with device-side fill counts.
// world = 1: a single bucket (the arrays the expansion wrote).  world > 1: one receive bucket per peer.
struct CandView {
  const uint64_t* hash;
  const uint64_t* fp;
  const uint32_t* score;
  const uint32_t* payload;
  const uint8_t* states;  // rows of `stride` bytes; may be null (world = 1 without materialised children)
  const uint32_t* counts;
  int32_t nbuckets;
  uint32_t cap;
};

struct StepArgs {
  CandView cv;   // candidates this rank owns (world = 1: all of them; world > 1: the receive buckets)
  CandView cvh;  // candidates the band histograms count: cv, or in peer mode the ones this rank generated
                 // (the histograms are summed over ranks, so either partition gives the same sums)
  MgbsCtrl* ctrl;
  uint32_t* hist;             // histogram this kernel fills
  const uint32_t* hist_prev;  // histogram of the previous level, consumed in the prologue
  const uint32_t* hist_stats; // level-0 histogram of the final cut (carries the all-reduced statistics)
  uint8_t* table;
  unsigned long long* tie_buf;
  int64_t hash_capacity;
  int64_t beam;
  int64_t pool_target;
  int64_t frontier_cap;  // row capacity (and history row pitch) of a frontier buffer
  int64_t next_cap;      // rows the next frontier may take: frontier_cap, or the logical next limit
  int32_t world, rank;
  int32_t key_bits, hash_bits;
  int32_t level, levels, round, rounds;
  int32_t select_mode, probe_limit;
  const uint8_t* frontier_cur;
  uint8_t* frontier_next;
  const uint8_t* gens;
  uint32_t* history;
  int64_t history_depths;
  uint32_t* next_score;
  uint64_t* next_hash;
  int32_t n, stride, fanout, parity;
  PeerCtx peer;
  int64_t off_frontier_cur;  // peer mode: offset of the current frontier inside every rank's symmetric region
  // persistent selection kernel (k_select): all histograms of the depth and the level counts
  uint32_t* hist_base;       // [(rounds * band_levels + final_levels)][MGBS_HIST_STRIDE]
  int32_t band_levels, final_levels;
  uint32_t grid_poll_limit;  // polls before the block barrier gives up
  MgbsMirror* mirror;        // pinned host summary, or null
};

struct RouteArgs {
  const uint64_t* hash; const uint64_t* fp; const uint32_t* score; const uint32_t* payload; const uint8_t* states;
  uint64_t* s_hash; uint64_t* s_fp; uint32_t* s_score; uint32_t* s_payload; uint8_t* s_states;
  uint32_t* send_counts;
  MgbsCtrl* ctrl;
  int32_t world, stride;
  uint32_t bucket_cap;
  // peer mode: records go straight into the owner's receive buckets; offsets of the bucket arrays of this parity
  PeerCtx peer;
  int64_t off_hash, off_fp, off_score, off_payload, off_counts, off_route_flag;
  int32_t hash_mode;
  int32_t rank;
};

int launch_expand(const ExpandArgs& a, int64_t max_parents, int sms, cudaStream_t st);
int launch_depth_begin(MgbsCtrl* c, int parity, int fanout, int64_t cand_cap, unsigned long long* tie_seg,
                       uint32_t* send_counts, uint32_t* recv_counts, int world, int64_t active_limit, int auto_halt,
                       const uint32_t* abort_word, cudaStream_t st);
int launch_select(const StepArgs& a, const RouteArgs& r, int sms, bool cooperative, cudaStream_t st);
int select_blocks_per_sm();
int launch_band_hist(const StepArgs& a, int64_t items, int sms, cudaStream_t st);
int launch_band_insert(const StepArgs& a, int64_t items, int sms, cudaStream_t st);
int launch_final_hist(const StepArgs& a, int64_t slots, int sms, cudaStream_t st);
int launch_emit(const StepArgs& a, int64_t items, int sms, cudaStream_t st);
int launch_finish(const StepArgs& a, cudaStream_t st);
int launch_route(const RouteArgs& a, int64_t items, int sms, cudaStream_t st);
int launch_route_band(const StepArgs& a, const RouteArgs& r, int64_t items, int sms, cudaStream_t st);
SymLayout sym_layout(const MgbsConfig& c, int band_levels_effective);
int launch_repack_rows(const uint8_t* src, uint8_t* dst, int64_t rows, int src_pitch, int dst_pitch, int n, int sms,
                       cudaStream_t st);
int launch_clamp_counts(uint32_t* counts, int world, uint32_t cap, cudaStream_t st);

}  // namespace mgbs
