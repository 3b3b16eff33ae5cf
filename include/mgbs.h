/*
 * mgbs.h — C ABI of the B200 beam-search step library (libmgbs_b200.so).
 *
 * Plain C: raw device pointers, sizes, a cudaStream_t passed as void*.  Every
 * function returns 0 on success or a negative MGBS_ERR_* / the CUDA error code
 * (positive) of the failing runtime call; nothing here allocates device memory
 * unless its comment says so.  The caller (the Python BeamEngine mirror, or any
 * host that owns its buffers) allocates every buffer, exactly as the reference's
 * pybind module takes torch tensors allocated by allocate_buffers
 * (beam_engine.py:171-234) and never allocates in the hot path
 * (beam_engine.cpp:674-698).
 *
 * Each entry point names the reference interface it replaces.
 */
#ifndef MGBS_H_
#define MGBS_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MGBS_RADIX_BITS 11
#define MGBS_RADIX_BINS 2048
#define MGBS_HIST_STRIDE 2096 /* 2048 bins + 16 per-rank unique counts + 16 per-rank inserted counts + 16 flags */
#define MGBS_MAX_LEVELS 6
#define MGBS_MAX_ROUNDS 8
#define MGBS_TIE_CAP 256
#define MGBS_MAX_WORLD 16
#define MGBS_MAX_FANOUT 32
#define MGBS_MAX_STATE_LEN 128
#define MGBS_MAX_MODELS 4
#define MGBS_MAX_RES_BLOCKS 4

/* select modes */
#define MGBS_SELECT_EXACT_K 0      /* keep the first beam entries of the (score, hash, fingerprint) order */
#define MGBS_SELECT_V6_INCLUSIVE 1 /* keep score <= T, ties kept (production_v6_dispatcher.py:159-192) */
#define MGBS_SELECT_LEGACY_STRICT 2 /* prune the whole cutoff bin (beam_kernels.cu:657-680, 700) */

/* scorer modes of the expand kernel */
/* candidate exchange / histogram reduction between ranks */
#define MGBS_EXCHANGE_NCCL 0 /* grouped ncclSend/ncclRecv of fixed buckets + ncclAllReduce per histogram */
#define MGBS_EXCHANGE_PEER 1 /* stores into the owner's buckets over NVLink peer mappings + one-shot in-kernel reduction */

#define MGBS_SCORE_EXTERNAL 0 /* scores written later by a scorer kernel */
#define MGBS_SCORE_HAMMING 1  /* mismatches against the solved state (beam_kernels.cu:86-94) */
#define MGBS_SCORE_UNIFORM 2  /* constant score (kernel_uniform_inference, beam_kernels.cu:147) */

/* status bits (MgbsCtrl.status): capacity problems are reported, never trapped
 * (the reference counts them: COUNTER_HASH_OVERFLOW / COUNTER_BUCKET_OVERFLOW,
 * beam_kernels.cu:419-429, 511, 606-608). */
#define MGBS_ST_HASH_OVERFLOW 1u   /* probe limit exhausted, candidate dropped */
#define MGBS_ST_BAND_STALL 2u      /* next sub-bin larger than the free pool; selection incomplete */
#define MGBS_ST_TIE_OVERFLOW 4u    /* more than MGBS_TIE_CAP entries share the cutoff key */
#define MGBS_ST_FRONTIER_OVERFLOW 8u /* survivors beyond the frontier capacity were dropped */
#define MGBS_ST_BUCKET_OVERFLOW 16u /* exchange bucket full, candidate dropped */
#define MGBS_ST_ROUNDS_EXHAUSTED 32u /* fewer than beam unique entries after the last band round */
#define MGBS_ST_PEER_TIMEOUT 64u     /* a bounded wait for another rank's data gave up (here or, by its notice, on a peer) */
#define MGBS_ST_GRID_TIMEOUT 128u    /* a bounded wait between the blocks of the selection kernel gave up */

#define MGBS_ERR_ARG (-1)
#define MGBS_ERR_UNSUPPORTED (-2)
#define MGBS_ERR_NCCL (-3)
#define MGBS_ERR_STATE (-4)
#define MGBS_ERR_TOO_LARGE (-5)
#define MGBS_ERR_PEER_TIMEOUT (-6) /* the depth loop stopped because a cross-rank wait gave up (status has MGBS_ST_PEER_TIMEOUT) */

/* Progress of one radix descent (band threshold or final cut). */
typedef struct MgbsRadix {
  uint64_t prefix;    /* decided key bits, already shifted to their place */
  uint64_t remaining; /* count still to cover inside the prefix range */
  uint32_t bits_done;
  uint32_t done;
  uint32_t flag;     /* band rounds: 1 = complete (enough unique entries or nothing left), 2 = table at its hard limit */
  uint32_t pad;
  uint64_t result;   /* band: exclusive upper bound E.  final: keep every key < result */
  uint64_t tie_key;  /* final: key at the cut whose entries are only partly kept */
  uint64_t tie_need; /* final: how many entries with key == tie_key survive (0 = none/all handled by result) */
  uint64_t kept_below;
} MgbsRadix;

/* Device-resident control block; one per engine.  The host reads it (or a pinned mirror) after a step.
 * It takes the place of the reference's counters[8] / beam_status[8] / threshold_cell[2]
 * (beam_engine_common.hpp:46-68). */
typedef struct MgbsCtrl {
  int32_t depth;             /* depth of the current frontier */
  int32_t frontier_count[2]; /* rows in frontier buffer 0 / 1 */
  int32_t found;             /* 1 once a solved state was seen */
  uint32_t found_payload;    /* smallest back-pointer among solved children of the finding depth */
  int32_t found_depth;       /* depth of the solved state (0 = start state) */
  uint32_t status;           /* MGBS_ST_* bits, sticky until reset */
  uint32_t table_count;      /* unique entries in this rank's table (this depth) */
  uint32_t next_count;       /* rows written to the next frontier (this depth) */
  uint32_t tie_count;
  uint32_t cand_count;       /* candidates generated by this rank this depth */
  uint32_t unique_total;     /* unique entries over all ranks when the final cut was taken */
  uint32_t inserted_total;   /* candidates passed to the table this depth (this rank) */
  uint32_t hash_overflow;    /* candidates dropped at the probe limit (this depth) */
  uint32_t rounds_used;
  uint32_t bands_done;       /* 1 when band rounds are complete */
  uint32_t epoch;            /* depth steps taken since the engine was created; tags cross-rank flags */
  int32_t active_rows;       /* frontier rows this depth expands: min(frontier_count, logical active limit) */
  uint64_t band_lo[MGBS_MAX_ROUNDS + 1];
  uint64_t threshold_key;    /* last final cut: every key below survives */
  uint64_t rho_num;          /* candidates inserted / unique entries of the last depth: the duplicate ratio that */
  uint64_t rho_den;          /* sizes the first band of the next depth */
  uint64_t total_candidates; /* running sum over depths (this rank) */
  uint32_t halt;             /* 1 while a depth runs that opened on a finished search (a failed wait; inside the depth
                              * loop also: found, or nothing left to expand): every kernel of that depth returns at
                              * once and the block stays as it was, so a host that enqueues one depth ahead of what it
                              * has read loses nothing.  exhausted: the last depth produced no state at all */
  uint32_t exhausted;
  uint32_t grid_bar;         /* arrival counter of the selection kernel's block barrier (reset when a depth opens) */
  uint32_t win_lo;           /* lowest score of the 2046-score window the next depth's band histogram is taken over
                              * (the cut score of this depth minus 1023, not below 0) */
  uint64_t launch_seq;       /* depth launches finished since the last reset, halted ones included */
  MgbsRadix band[MGBS_MAX_ROUNDS][MGBS_MAX_LEVELS + 1];
  MgbsRadix fin[MGBS_MAX_LEVELS + 1];
} MgbsCtrl;

/* Static description of one engine: shapes, capacities, knobs and every device buffer.
 * Knob names follow the reference's config dict (beam_engine.py:68-109; EngineConfig::derive,
 * beam_engine.cpp:244-321). */
typedef struct MgbsConfig {
  int32_t state_len;     /* n, bytes per state (reference: 120, compile time) */
  int32_t state_stride;  /* row pitch in bytes, multiple of 16, >= state_len (reference: state_size_bytes 128) */
  int32_t fanout;        /* G (reference: 24, compile time) */
  int32_t world_size;
  int32_t rank;
  int32_t select_mode;   /* MGBS_SELECT_* */
  int32_t score_mode;    /* MGBS_SCORE_* */
  int32_t hash_bits;     /* hash bits in the 64-bit selection key (44 for exact_k; 0 orders by score only) */
  int32_t band_levels;   /* radix levels used to place a band threshold (1..6) */
  int32_t band_rounds;   /* band rounds enqueued per depth (1..MGBS_MAX_ROUNDS) */
  int32_t probe_limit;   /* PROBE_LIMIT */
  int32_t uniform_score; /* score for MGBS_SCORE_UNIFORM */
  int64_t global_beam_width; /* GLOBAL_BEAM_WIDTH */
  int64_t frontier_cap;  /* rows per frontier buffer (k_work: beta*gamma*ceil(beam/world)) */
  int64_t pool_target;   /* per-rank fill target of the table: round(beta * ceil(beam/world)) */
  int64_t hash_capacity; /* slots: frontier_cap / HASH_LOAD_FACTOR */
  int64_t cand_cap;      /* capacity of the candidate arrays on this rank */
  int64_t bucket_cap;    /* world > 1: records per peer bucket (send and recv) */
  int64_t history_depths; /* rows of history kept (max_depth) */
  /* device buffers */
  uint8_t* frontier[2];     /* [frontier_cap, state_stride] ping-pong (beam_current) */
  uint8_t* gens;            /* [fanout, state_len] gather tables (c_action_permutation) */
  uint8_t* solved;          /* [state_len] (c_central_state) */
  uint8_t* children;        /* [cand_cap, state_stride] or NULL when children are not materialised */
  uint64_t* cand_hash;      /* [cand_cap] */
  uint64_t* cand_fp;        /* [cand_cap] */
  uint32_t* cand_score;     /* [cand_cap] */
  uint32_t* cand_payload;   /* [cand_cap] */
  uint8_t* table;           /* [hash_capacity * 32] */
  uint32_t* hist;           /* [(band_rounds*band_levels + MGBS_MAX_LEVELS) * MGBS_HIST_STRIDE] */
  uint64_t* tie_buf;        /* [world * (1 + 3*MGBS_TIE_CAP)] tie records at the cut key, one segment per rank */
  uint32_t* history;        /* [history_depths, frontier_cap] back-pointers, or NULL */
  uint64_t* frontier_hash[2];  /* [frontier_cap] hash of each frontier row, or NULL */
  uint32_t* frontier_score[2]; /* [frontier_cap] score of each frontier row, or NULL */
  MgbsCtrl* ctrl;
  /* world > 1: exchange buffers, [world * bucket_cap] each (send side, then receive side) */
  uint64_t* send_hash; uint64_t* send_fp; uint32_t* send_score; uint32_t* send_payload; uint8_t* send_states;
  uint64_t* recv_hash; uint64_t* recv_fp; uint32_t* recv_score; uint32_t* recv_payload; uint8_t* recv_states;
  uint32_t* send_counts; uint32_t* recv_counts; /* [world] */
  /* MGBS_EXCHANGE_PEER: one region of mgbs_sym_bytes() bytes per rank, zero-filled, laid out identically on every
   * rank and mapped into every peer (mgbs_engine_set_peers); it holds the receive buckets for candidate records
   * (two parities), the per-sender counts and flags, the histogram exchange slots and BOTH FRONTIER BUFFERS:
   * frontier[p] must equal sym + mgbs_sym_frontier_offsets()[p], because owners rebuild the states of survivors
   * from parent rows they read out of the senders' frontiers.  recv_* / send_* arrays above are then unused
   * (send_counts stays: local per-destination cursors).  tickets: [hist slots + 1] uint32, zero-filled, local. */
  int32_t exchange_mode;
  int32_t pad1;
  uint8_t* sym;
  int64_t sym_bytes;
  uint32_t* tickets;
  /* optional [frontier_cap * state_len] bytes: packed staging rows so that host<->device frontier copies are one
   * contiguous transfer plus a repack kernel instead of a strided 2-D copy */
  uint8_t* io_stage;
  /* Hash function of the dedup / owner / tie-break logic.  MGBS_HASH_FNV (default): hash_state_120 +
   * fingerprint_state_120 (beam_kernels.cu:38-59).  MGBS_HASH_ZOBRIST128: the v6 alternative
   * (hash_state128_zobrist, beam_kernels_stream2.cu:28-38): XOR over positions of zobrist[position][value], a table
   * of 128-bit entries {lo, hi} with zobrist_values entries per position, [state_len, zobrist_values, 2] uint64 on
   * the device; lo acts as the hash, hi as the fingerprint, the owner is (hi ^ lo*0x9e3779b97f4a7c15) mod world
   * (owner_from_hash128, beam_kernels_stream3.cu:29-35). */
  int32_t hash_mode;
  int32_t zobrist_values;
  const uint64_t* zobrist;
  /* Optional pinned host memory, sizeof(MgbsMirror) bytes, device-accessible at the same address (cudaHostAlloc /
   * torch pin_memory): the last kernel of every depth writes a summary of the control block there, so that the
   * depth loop (mgbs_engine_search) reads host memory instead of copying the control block and synchronising the
   * stream after every depth (the reference's status() synchronises every stream and makes three device-to-host
   * copies per depth, beam_engine.cpp:1173-1198). */
  struct MgbsMirror* host_mirror;
  /* Bounded waits of the cross-rank kernels give up after this many polls (0 = default 2^22, about a second). */
  int64_t peer_poll_limit;
  /* 0 (default) = selection as one persistent kernel (band rounds, final cut, emit and finish with block barriers
   * in between; world 1 and MGBS_EXCHANGE_PEER); 1 = one launch per stage (always used with MGBS_EXCHANGE_NCCL,
   * whose collectives sit between the stages). */
  int32_t staged_select;
  int32_t pad2;
} MgbsConfig;

/* Summary of the control block written to MgbsConfig.host_mirror by the last kernel of a depth; seq is written
 * last (after a system-wide fence) and equals MgbsCtrl.launch_seq: one more per enqueued depth, halted or not. */
typedef struct MgbsMirror {
  int32_t depth, found, found_depth, frontier_next; /* frontier_next: rows of the frontier the depth produced (this rank) */
  uint32_t found_payload, status, unique_total, epoch;
  uint64_t total_candidates;
  volatile uint64_t seq;
} MgbsMirror;

#define MGBS_HASH_FNV 0
#define MGBS_HASH_ZOBRIST128 1

typedef struct MgbsEngine MgbsEngine; /* opaque */

/* Library version / build info; no reference counterpart. */
int mgbs_version(void);
int mgbs_sizeof_ctrl(void);
int mgbs_sizeof_config(void);

/* Derived sizes (ext.derive_sizes, beam_engine.cpp:1692-1748; EngineConfig::derive :244-321):
 * n_local = ceil(beam/world), k_keep = round(gamma*n_local), k_work = round(beta*k_keep),
 * hash_capacity = max(1024, round(k_work/load)).  out[0..5] = n_local, k_keep, k_work, hash_capacity,
 * pool_target, hist_words. */
int mgbs_derive_sizes(int64_t global_beam_width, int32_t world_size, double gamma, double beta, double hash_load_factor,
                      int32_t band_rounds, int32_t band_levels, int64_t* out6);

/* Engine object: keeps a copy of the config (host memory only; no device allocation).
 * Replaces BeamEngine's constructor (beam_engine.cpp:672-755). */
int mgbs_engine_create(const MgbsConfig* cfg, MgbsEngine** out);
int mgbs_engine_destroy(MgbsEngine* e);

/* Loads NCCL entry points from the given shared object (NULL = already loaded in the process) and joins the
 * communicator.  Replaces BeamEngine::init_nccl (beam_engine.cpp:782-787); unique_id is the 128-byte id from
 * mgbs_nccl_unique_id on rank 0 (get_nccl_unique_id, beam_engine.cpp:2097). */
int mgbs_nccl_unique_id(const char* libnccl_path, uint8_t* out128);
int mgbs_engine_init_nccl(MgbsEngine* e, const char* libnccl_path, const uint8_t* unique_id128);

/* Size of the symmetric region for MGBS_EXCHANGE_PEER and number of ticket words, from the shape fields of cfg. */
int mgbs_sym_bytes(const MgbsConfig* cfg, int64_t* out_bytes, int64_t* out_tickets);
/* Byte offsets of the two frontier buffers inside the symmetric region (same shape fields as mgbs_sym_bytes plus
 * frontier_cap).  No reference counterpart. */
int mgbs_sym_frontier_offsets(const MgbsConfig* cfg, int64_t* out2);
/* Map the peers' symmetric regions: handles = world x 64 bytes (cudaIpcMemHandle_t of the allocation that holds each
 * rank's region), offsets = byte offset of the region inside that allocation.  The reference has no counterpart
 * (it exchanges through NCCL only, beam_engine.cpp:1368-1400). */
int mgbs_engine_set_peers(MgbsEngine* e, const uint8_t* handles, const int64_t* offsets);
/* The same for ranks that live in ONE process (threads, or one thread driving several GPUs with peer access
 * enabled): bases[r] = device pointer of rank r's symmetric region as this GPU addresses it.  No reference
 * counterpart. */
int mgbs_engine_set_peer_pointers(MgbsEngine* e, uint8_t* const* bases);
/* CUDA IPC handle (64 bytes) of the device allocation containing ptr and ptr's offset inside it: what each rank
 * publishes to the others for mgbs_engine_set_peers.  No reference counterpart. */
int mgbs_ipc_export(const void* ptr, uint8_t* handle64, int64_t* offset);

/* Scorer hook for MGBS_SCORE_EXTERNAL: enqueue on `stream` a kernel sequence that reads the first *count_dev
 * rows of `children` ([.., state_stride] bytes) and writes one uint32 score key per row (lower is better).
 * Takes the place of InferenceBackend::forward (beam_engine.cpp:423-668); mgbs_mlp_enqueue has this signature. */
typedef int (*mgbs_scorer_fn)(void* user, const uint8_t* children, const uint32_t* count_dev, uint32_t* scores,
                              void* stream);
int mgbs_engine_set_scorer(MgbsEngine* e, mgbs_scorer_fn fn, void* user);
/* Parent scorer (action values): called instead of the child scorer when set; writes the score key of candidate
 * parent*fanout + move for the first *parent_count_dev rows of the current frontier.  Replaces the reference's
 * scoring of parents before expansion (kernel_process_score_slot reads ring scores [action][parent],
 * beam_kernels.cu:528-560).  Pass fn = NULL to go back to the child scorer. */
typedef int (*mgbs_parent_scorer_fn)(void* user, const uint8_t* parents, const int32_t* parent_count_dev,
                                     uint32_t* cand_scores, void* stream);
int mgbs_engine_set_parent_scorer(MgbsEngine* e, mgbs_parent_scorer_fn fn, void* user);

/* Switch the scorer used by the expansion (MGBS_SCORE_*); drops captured graphs.  Covers begin_uniform_score /
 * set_uniform_score / end_uniform_score (beam_engine.cpp:893-915): the uniform mode is the reference's prepass fill. */
int mgbs_engine_set_score_mode(MgbsEngine* e, int32_t score_mode, int32_t uniform_score);

/* Logical limits of the reference's prepass (set_active_limit / set_next_limit / clear_logical_limits,
 * beam_engine.cpp:1064-1090): active_limit > 0 makes a depth expand at most that many rows of the current frontier;
 * next_limit > 0 caps the next frontier at that many rows and the dedup table at next_limit / load + 1024 slots
 * (load = frontier_cap / hash_capacity), with the pool target scaled alike.  -1 clears a limit.  Drops captured
 * graphs, as the reference invalidates its graph. */
int mgbs_engine_set_logical_limits(MgbsEngine* e, int64_t active_limit, int64_t next_limit);

/* Reset to a one-state frontier on the owning rank (reset_search, beam_engine.cpp:995-1021).  start_is_solved = 1
 * marks the search as found at depth 0 (kernel_check_current_solved, beam_kernels.cu:857-875).  Synchronises. */
int mgbs_engine_reset(MgbsEngine* e, const uint8_t* start_state_host, int32_t active_on_this_rank,
                      int32_t start_is_solved, void* stream);

/* Load `count` rows (state_len bytes each, host memory) as the frontier in buffer `parity` at `depth`; clears the
 * search status.  No reference counterpart as one call (the v6 dispatcher copies a whole frontier to the device
 * every depth, production_v6_dispatcher.py:739-742).  Synchronises. */
int mgbs_engine_load_frontier(MgbsEngine* e, const uint8_t* rows_host, int64_t count, int32_t parity, int32_t depth,
                              void* stream);

/* Copy the frontier in buffer `parity` to host memory as packed rows of state_len bytes (at most capacity_rows);
 * *count_out receives the number of rows.  Synchronises.  Counterpart of the v6 dispatcher's device-to-host copy of
 * the next frontier (production_v6_dispatcher.py:700-706) and of current_state_bytes (beam_engine.cpp:2146). */
int mgbs_engine_read_frontier(MgbsEngine* e, int32_t parity, uint8_t* dst_host, int64_t capacity_rows,
                              int64_t* count_out, void* stream);

/* Enqueue one depth step on the stream: expand+hash(+score) -> [scorer hook] -> [exchange] -> band rounds of
 * dedup inserts -> final cut -> next frontier.  Replaces enqueue_one_depth (beam_engine.cpp:1465-1656).
 * phase: 0 = whole step; 1 = up to and including expansion (then the caller runs its scorer on
 * children -> cand_score); 2 = everything after scoring.  parity = index of the frontier buffer that holds the
 * current frontier.  No host synchronisation, no allocation: safe to capture in a CUDA graph. */
int mgbs_engine_enqueue_depth(MgbsEngine* e, int32_t parity, int32_t phase, void* stream);

/* One depth through a captured CUDA graph, one graph per parity, captured on first use
 * (BeamEngine::step + capture_cuda_graph, beam_engine.cpp:1104-1116, 1658-1672). */
int mgbs_engine_step_graph(MgbsEngine* e, int32_t parity, void* stream);

/* Per-stage timing (enable_step_timers / step_timing, beam_engine.cpp:1035-1062): when on, eager
 * mgbs_engine_enqueue_depth calls record CUDA events between stages; read returns the last step's milliseconds for
 * {clear + expand, scorer, exchange, band rounds, final cut + emit + finish}.  Turning it on drops captured graphs,
 * as enabling timers invalidates the reference's graph. */
int mgbs_engine_profile(MgbsEngine* e, int32_t on);
int mgbs_engine_profile_read(MgbsEngine* e, float* ms5);
/* Per-launch trace of the last profiled step, in enqueue order: clears, expand, scorer, route+exchange, then per band
 * round {histogram levels, insert}, final histogram levels, emit, tie gather + finish.  Returns the interval count. */
int mgbs_engine_trace_read(MgbsEngine* e, float* ms, int32_t capacity);

/* Copy the control block to host memory (status(), beam_engine.cpp:1173-1198); synchronises the stream. */
int mgbs_engine_read_ctrl(MgbsEngine* e, MgbsCtrl* out_host, void* stream);

/* Depth loop: step until found, max_depth or an empty frontier (BeamEngine::search, beam_engine.cpp:1147-1171).
 * out_host receives the final control block.  With MgbsConfig.host_mirror the loop enqueues one depth ahead of the
 * last summary it has read and never synchronises the stream between depths (a depth that opens on a finished
 * search halts on the device).  Returns MGBS_ERR_PEER_TIMEOUT when a cross-rank wait gave up: the status bit is set
 * on every rank that took part, each rank's loop returns, and nothing is left waiting. */
int mgbs_engine_search(MgbsEngine* e, int32_t max_depth, int32_t use_graph, MgbsCtrl* out_host, void* stream);

/* Stage launchers, usable on their own (reference convention: extern "C" launch_<stage>(ptrs, sizes, stream),
 * beam_engine.cpp:55-194). */

/* expand + hash64 + fingerprint64 (+ Hamming / uniform score, + goal test) of `count` parents.
 * Replaces kernel_dummy_inference + the expansion half of kernel_process_score_slot (beam_kernels.cu:107-145,
 * 528-580) and kernel_v6_stream2_hash_goal (beam_kernels_stream2.cu:40).  count_dev (device int32) overrides
 * count when not NULL.  Outputs are parent-major: candidate c = p*fanout + m. */
int mgbs_launch_expand(const uint8_t* frontier, const int32_t* count_dev, int64_t count, const uint8_t* gens,
                       const uint8_t* solved, int32_t state_len, int32_t state_stride, int32_t fanout, int32_t rank,
                       int32_t score_mode, int32_t uniform_score, uint8_t* children, uint64_t* cand_hash,
                       uint64_t* cand_fp, uint32_t* cand_score, uint32_t* cand_payload, MgbsCtrl* ctrl, void* stream);

/* Value-network scorer: ensemble of MLPs  one-hot(state_len*num_values) -> hidden -> hidden -> 1  (ReLU), bf16
 * operands with fp32 accumulation on the tcgen05 tensor cores, scalar head and score key fused into the last
 * GEMM's epilogue.  All buffers are the caller's.  Replaces FullBeamNiceStaticBackend (beam_engine.cpp:556-668)
 * and its activation buffers fb_act1..fb_out (beam_engine.py:223-231). */
typedef struct MgbsMlpConfig {
  int32_t state_len, state_stride, num_values, hidden, num_models;
  /* One-hot column order of the first layer (w1's second axis, and x): column = value * P + position with
   * P = state_len rounded up to a multiple of 8, so that eight adjacent columns are one byte-compare of the state row.
   * k1_pad = num_values * P rounded up to a multiple of 64 (bf16) or 128 (fp8); columns of positions >= state_len and
   * columns >= num_values * P must be zero in w1. */
  int32_t k1_pad;
  int64_t max_rows;     /* capacity in child rows; x, h1 and q hold max_rows rounded up to 128 */
  float score_offset;   /* key = uint32(clamp(q - score_offset, 0, 300) * 256 + 0.5) (beam_kernels.cu:341-344) */
  float b3[MGBS_MAX_MODELS];
  void* x;              /* bf16 [rows_pad, k1_pad] one-hot activations */
  void* h1;             /* bf16 [rows_pad, hidden] */
  float* q;             /* [rows_pad] */
  int32_t* err;         /* device word: first bounded-wait failure code, 0 = none */
  const void* w1[MGBS_MAX_MODELS]; /* bf16 [hidden, k1_pad], zero padded */
  const float* b1[MGBS_MAX_MODELS];
  const void* w2[MGBS_MAX_MODELS]; /* bf16 [hidden, hidden] */
  const float* b2[MGBS_MAX_MODELS];
  const float* w3[MGBS_MAX_MODELS]; /* f32 [hidden] */
  /* dtype 1 (FP8 E4M3, per-channel weight scales): w1/w2 hold e4m3 bytes ([hidden, k1_pad] / [hidden, hidden],
   * k1_pad a multiple of 128), h1 holds e4m3 bytes [rows_pad, hidden], x is unused.
   * s1[n] = scale of W1 row n; s2[n] = act_scale * scale of W2 row n; activations are stored as
   * e4m3(h1 * act_inv_scale) with one per-tensor act_scale. */
  const float* s1[MGBS_MAX_MODELS];
  const float* s2[MGBS_MAX_MODELS];
  int32_t dtype;        /* 0 = bf16 operands, 1 = e4m3 operands, 2 = NVFP4 second layer; fp32 accumulation always */
  float act_inv_scale;
  /* dtype 2 (NVFP4: E2M1 elements, one E4M3 factor per 16 elements, one float32 scale per tensor): layer 1 runs as for
   * dtype 1 (w1, s1, h1, act_inv_scale as above) and its e4m3 activations are re-quantised to NVFP4; layer 2 runs on
   * the block-scaled 4-bit tensor-core path.  w2 then holds packed E2M1 [hidden, hidden / 2] bytes (even K in the low
   * nibble), sf_w2 its block factors in tiles [chunk of 256 rows][K-block of 256][group of 128 rows][step of 64]
   * [512 B: row r at (r % 32) * 16 + (r / 32) * 4 + block], s2[n] = (tensor scale of W2) * (tensor scale of the
   * activations); h1q / sf_h1 are the scorer's own buffers: packed activations [rows_pad, hidden / 2] and their
   * factors [rows_pad / 128][hidden / 256][4][512 B]; act4_inv_global = 1 / (tensor scale of the activations). */
  void* h1q;
  uint8_t* sf_h1;
  const uint8_t* sf_w2[MGBS_MAX_MODELS];
  float act4_inv_global;
  int32_t pad0;
} MgbsMlpConfig;
typedef struct MgbsMlp MgbsMlp;
int mgbs_sizeof_mlp_config(void);
int mgbs_mlp_create(const MgbsMlpConfig* cfg, MgbsMlp** out); /* host object + TMA descriptors; no device allocation */
int mgbs_mlp_destroy(MgbsMlp* m);
/* mgbs_scorer_fn for the engine: children -> score keys for the first *count_dev rows.  Replaces
 * InferenceBackend::forward (beam_engine.cpp:621-667). */
/* Layer-1 implementation: 1 (default) = one-hot operand built in shared memory inside the GEMM and TMA-stored
 * activations; 0 = separate one-hot kernel + plain GEMM with per-thread stores (kept for comparison). */
int mgbs_mlp_set_l1_mode(MgbsMlp* m, int32_t fused);
/* Layer 2 + head implementation: 1 (default where the device can co-schedule CTA pairs) = thread-block clusters of
 * two sharing each weight block (tcgen05 cta_group::2); 0 = one CTA per 128-row tile (kept for comparison).
 * NVFP4 (dtype 2): 1 (default) = 256-column accumulator tiles with the block-factor copies on a thread of their own;
 * 0 = 128-column tiles with two accumulators. */
int mgbs_mlp_set_head_mode(MgbsMlp* m, int32_t pair);
/* Layer-1 kernel variant for tuning: epilogue_warps 4 or 8 of the kernel's 12 worker warps (the others build the
 * one-hot operand; 0 = default for the operand type), pair = thread-block clusters of two sharing the weight tiles
 * (-1 = default).  Every variant computes the same values. */
int mgbs_mlp_set_l1_variant(MgbsMlp* m, int32_t epilogue_warps, int32_t pair);
/* Per-kernel timing for benchmarks (single-member scorers, eager launches only): when on, mgbs_mlp_enqueue records
 * CUDA events between its kernels; mgbs_mlp_profile_read returns the last call's milliseconds for
 * {one-hot, layer-1 GEMM, layer-2 GEMM + head, key}.  Mirrors benchmark_inference (beam_engine.cpp:931-977). */
int mgbs_mlp_profile(MgbsMlp* m, int32_t on);
int mgbs_mlp_profile_read(MgbsMlp* m, float* ms4);
int mgbs_mlp_enqueue(void* mlp, const uint8_t* children, const uint32_t* count_dev, uint32_t* scores, void* stream);

/* Action-value ("Q") scorer: the reference's own scorer contract - one forward pass per PARENT row gives one value per
 * move (scorers.py:1-57: uint8 [B, n] -> [B, fanout]; FullBeamNiceStaticBackend::forward, beam_engine.cpp:621-667:
 * embedding + ReLU, two hidden layers, output layer of width fanout).  Candidate parent*fanout + move takes
 * q[parent][move]; keys as for the value scorers.  Network: one-hot(state_len x num_values) -> hidden1 (ReLU) ->
 * hidden2 (ReLU) -> [residual blocks] -> fanout, bf16 operands, float32 accumulation; hidden1 and hidden2 multiples
 * of 256; ensemble members are averaged.  All buffers are the caller's. */
typedef struct MgbsQmlpConfig {
  int32_t state_len, state_stride, num_values, fanout, hidden1, hidden2, num_models;
  int32_t k1_pad;        /* as MgbsMlpConfig.k1_pad (bf16): num_values * P rounded up to a multiple of 64; same column order */
  int64_t max_parents;   /* capacity in parent rows; h1, h2, q hold max_parents rounded up to 128 rows */
  float score_offset;
  /* 0: key = uint32(clamp(q - score_offset, 0, 300) * 256 + 0.5) (kernel_fullbeamnice_q_to_score_key_ring,
   * beam_kernels.cu:326-346).  1, 2: the 16-bit higher-is-better scores of QuantizedActionScorer (scorers.py:38-53),
   * sigmoid_u16 and float_u16, as key = 65535 - score. */
  int32_t key_mode;
  void* h1;              /* bf16 [rows_pad, hidden1] */
  void* h2;              /* bf16 [rows_pad, hidden2] */
  float* q;              /* f32 [rows_pad, fanout] */
  int32_t* err;
  const void* w1[MGBS_MAX_MODELS];  /* bf16 [hidden1, k1_pad], zero padded */
  const float* b1[MGBS_MAX_MODELS];
  const void* w2[MGBS_MAX_MODELS];  /* bf16 [hidden2, hidden1] */
  const float* b2[MGBS_MAX_MODELS];
  const void* w3[MGBS_MAX_MODELS];  /* bf16 [256, hidden2]: rows >= fanout are zero */
  const float* b3[MGBS_MAX_MODELS]; /* f32 [256]: entries >= fanout are zero */
  /* Residual form (the reference's static network, scripts/static_fullbeamnice_inference.py:146-171 and
   * FullBeamNiceStaticBackend::forward, beam_engine.cpp:621-667): after hidden2, num_res_blocks blocks of
   * x = relu(relu(x Wa^T + ba) Wb^T + bb + x) with square hidden2 x hidden2 layers, then the output layer. */
  int32_t num_res_blocks;           /* 0 .. MGBS_MAX_RES_BLOCKS */
  /* 1: the first layer is an embedding sum over w1t (for vocabularies too wide for the one-hot contraction;
   * kernel_fullbeamnice_embed_relu, beam_kernels.cu:208-237); w1 and k1_pad are then unused. */
  int32_t embed_sum;
  int32_t activation;               /* hidden layers: 0 ReLU, 1 GELU (MLPActionScorer, scorers.py:21-36; embed_sum only) */
  int32_t pad1;
  void* h3;                         /* bf16 [rows_pad, hidden2]: scratch of the residual blocks (num_res_blocks > 0) */
  const void* w1t[MGBS_MAX_MODELS]; /* embed_sum: bf16 [state_len * num_values, hidden1], row = pos * num_values + value */
  const void* wr[2 * MGBS_MAX_RES_BLOCKS][MGBS_MAX_MODELS];  /* bf16 [hidden2, hidden2]: block b uses 2b (first), 2b+1 */
  const float* br[2 * MGBS_MAX_RES_BLOCKS][MGBS_MAX_MODELS]; /* f32 [hidden2] */
} MgbsQmlpConfig;
typedef struct MgbsQmlp MgbsQmlp;
int mgbs_sizeof_qmlp_config(void);
int mgbs_qmlp_create(const MgbsQmlpConfig* cfg, MgbsQmlp** out);
int mgbs_qmlp_destroy(MgbsQmlp* m);
/* mgbs_parent_scorer_fn for the engine (mgbs_engine_set_parent_scorer). */
int mgbs_qmlp_enqueue(void* qmlp, const uint8_t* parents, const int32_t* parent_count_dev, uint32_t* cand_scores,
                      void* stream);

/* Transformer value scorer: ensemble of pre-LayerNorm encoders (one token per state position from a vocabulary of
 * num_values plus a learned position embedding; per layer x += MHA(LN1 x), x += W2 gelu(W1 LN2 x); final LayerNorm,
 * mean pooling over tokens, scalar head).  d_model is fixed at 256 with 8 heads of 32; ffn is a multiple of 256;
 * tokens <= 64.  bf16 or e4m3 GEMM operands (dtype), fp32 accumulation and residual stream.  States are processed in micro-batches of
 * micro_batch states (B_MICRO of the reference, beam_engine.py:71).  All buffers are the caller's.  The reference has no
 * transformer backend; this fills its InferenceBackend slot (beam_engine.cpp:423-668). */
#define MGBS_TF_MAX_ENCODERS 4
#define MGBS_TF_MAX_LAYERS 8
typedef struct MgbsTfLayer {
  const float* ln1_g; const float* ln1_b;
  const void* wqkv;  /* bf16 [768, 256] rows q | k | v */
  const float* bqkv;
  const void* wo;    /* bf16 [256, 256] */
  const float* bo;
  const float* ln2_g; const float* ln2_b;
  const void* w1;    /* bf16 [ffn, 256] */
  const float* b1;
  const void* w2;    /* bf16 [256, ffn] */
  const float* b2;
  /* dtype 1 only: the four matrices above are e4m3 with one scale per output row, and cs_* [rows] f32 hold
   * (activation scale) * (weight-row scale) for the GEMM that consumes them; inv_* = 1 / activation scale of the
   * e4m3 tensor that feeds it (LN1 output, attention output, LN2 output, GELU output). */
  const float* cs_qkv; const float* cs_o; const float* cs_1; const float* cs_2;
  float inv_y1, inv_att, inv_y2, inv_hid;
} MgbsTfLayer;
typedef struct MgbsTfConfig {
  int32_t state_len, state_stride, num_values, d_model, heads, ffn, layers, encoders;
  int64_t max_states;   /* capacity in child rows */
  int64_t micro_batch;  /* states per micro-batch; activation buffers hold micro_batch*state_len rows rounded up to 128 */
  float score_offset;
  float b_head[MGBS_TF_MAX_ENCODERS];
  const float* tok_emb[MGBS_TF_MAX_ENCODERS]; /* f32 [num_values, 256] */
  const float* pos_emb[MGBS_TF_MAX_ENCODERS]; /* f32 [state_len, 256] */
  const float* lnf_g[MGBS_TF_MAX_ENCODERS]; const float* lnf_b[MGBS_TF_MAX_ENCODERS];
  const float* w_head[MGBS_TF_MAX_ENCODERS];  /* f32 [256] */
  MgbsTfLayer layer[MGBS_TF_MAX_ENCODERS][MGBS_TF_MAX_LAYERS];
  float* x;     /* f32 [rows_pad, 256] residual stream */
  void* y;      /* bf16 (dtype 1: e4m3) [rows_pad, 256] normalised activations */
  void* qkv;    /* bf16 [rows_pad, 768] */
  void* att;    /* bf16 (dtype 1: e4m3) [rows_pad, 256] attention output */
  void* hid;    /* bf16 (dtype 1: e4m3) [rows_pad, ffn] */
  float* q;     /* f32 [max_states] */
  int32_t* err;
  int32_t dtype; /* GEMM operand type: 0 = bf16, 1 = e4m3 (float32 accumulation, residual stream and softmax either way) */
  int32_t reserved;
} MgbsTfConfig;
typedef struct MgbsTf MgbsTf;
int mgbs_sizeof_tf_config(void);
int mgbs_tf_create(const MgbsTfConfig* cfg, MgbsTf** out);
int mgbs_tf_destroy(MgbsTf* t);
/* mgbs_scorer_fn for the engine. */
int mgbs_tf_enqueue(void* tf, const uint8_t* children, const uint32_t* count_dev, uint32_t* scores, void* stream);

/* Scoring without any allocation.  No counterpart in the reference.
 *
 * For hosts that cannot allocate device memory when they need scores (allocation-free regions of a serving
 * runtime, plugins with a memory budget fixed at load time): the same kernels as mgbs_mlp_enqueue, for ONE
 * network, with every scratch buffer (one-hot rows, first-layer activations, head outputs, row count, error word)
 * in a static device array inside the library, MGBS_NOALLOC_SCRATCH_BYTES per device that loads the library, held
 * until the process exits.  The caller passes only inputs (device pointers to child rows and weights, laid out as
 * in MgbsMlpConfig) and the output array.  Calls that need more than MGBS_NOALLOC_MAX_ROWS rows, a padded one-hot
 * width above MGBS_NOALLOC_MAX_K1 or more than MGBS_NOALLOC_MAX_HIDDEN hidden units return MGBS_ERR_TOO_LARGE and
 * launch nothing.  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 * The first call on each device resolves the array's device address (cudaGetSymbolAddress) and sets kernel
 * attributes; make that first call outside any stream capture.  All calls share the one array and it keeps what
 * the previous call wrote (the entry point resets the words that must start at zero): two calls whose kernels
 * overlap on the GPU - different streams, or different host threads - race on it.  Serialise them.
 * err_out_host, when not NULL, makes the call wait for its kernels and receives the GEMM error word (0 = clean). */
#define MGBS_NOALLOC_MAX_ROWS 4096
#define MGBS_NOALLOC_MAX_K1 768
#define MGBS_NOALLOC_MAX_HIDDEN 1024
#define MGBS_NOALLOC_SCRATCH_BYTES (4096 * 768 * 2 + 4096 * 1024 * 2 + 4096 * 4 + 256)
typedef struct MgbsMlpNoAllocArgs {
  int32_t state_len, state_stride, num_values, hidden;
  float score_offset, b3;
  const void* w1;  /* bf16 [hidden, k1_pad], zero padded; k1_pad and the column order as in MgbsMlpConfig */
  const float* b1; /* [hidden] */
  const void* w2;  /* bf16 [hidden, hidden] */
  const float* b2; /* [hidden] */
  const float* w3; /* [hidden] */
} MgbsMlpNoAllocArgs;
int mgbs_mlp_score_noalloc(const MgbsMlpNoAllocArgs* args, const uint8_t* children, int32_t rows, uint32_t* scores,
                           int32_t* err_out_host, void* stream);

/* Host-side helpers with the device's exact arithmetic (data_loader.hash_state_cpu, data_loader.py:192-213). */
uint64_t mgbs_hash64_host(const uint8_t* state, int32_t n);
uint64_t mgbs_fingerprint64_host(const uint8_t* state, int32_t n);

#ifdef __cplusplus
}
#endif
#endif /* MGBS_H_ */
