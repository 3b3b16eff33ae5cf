// Host side of the step library: the engine object, the per-depth enqueue order, CUDA-graph capture, and the
// NCCL exchange for world > 1.  Takes the place of BeamEngine::enqueue_one_depth / capture_cuda_graph / search
// (beam_engine.cpp:1465-1672, 1147-1171).  No device memory is allocated here: every buffer comes in through
// MgbsConfig, as the reference's engine takes torch tensors from allocate_buffers.

#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <stdint.h>
#include <string.h>

#include <new>

#include "mgbs.h"
#include "mgbs_device.cuh"
#include "mgbs_internal.cuh"

namespace {

// NCCL is resolved at run time so that the library loads on a host without it (and without a link-time dependency
// on a particular libnccl build).
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  bool ok = false;
};

NcclApi g_nccl;

int load_nccl(const char* path) {
  if (g_nccl.ok) return 0;
  void* h = nullptr;
  if (path && path[0]) h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return MGBS_ERR_NCCL;
  g_nccl.handle = h;
#define MGBS_SYM(field, name)                                          \
  *reinterpret_cast<void**>(&g_nccl.field) = dlsym(h, name);           \
  if (!g_nccl.field) return MGBS_ERR_NCCL;
  MGBS_SYM(GetUniqueId, "ncclGetUniqueId")
  MGBS_SYM(CommInitRank, "ncclCommInitRank")
  MGBS_SYM(CommDestroy, "ncclCommDestroy")
  MGBS_SYM(AllReduce, "ncclAllReduce")
  MGBS_SYM(AllGather, "ncclAllGather")
  MGBS_SYM(Send, "ncclSend")
  MGBS_SYM(Recv, "ncclRecv")
  MGBS_SYM(GroupStart, "ncclGroupStart")
  MGBS_SYM(GroupEnd, "ncclGroupEnd")
#undef MGBS_SYM
  g_nccl.ok = true;
  return 0;
}

}  // namespace

struct MgbsEngine {
  MgbsConfig cfg;
  int sms = 148;
  int key_bits = 64;
  int final_levels = 6;
  ncclComm_t comm = nullptr;
  mgbs_scorer_fn scorer = nullptr;
  void* scorer_user = nullptr;
  mgbs_parent_scorer_fn parent_scorer = nullptr;
  void* parent_scorer_user = nullptr;
  cudaGraphExec_t graph[2][2] = {{nullptr, nullptr}, {nullptr, nullptr}};  // [parity][inside the depth loop]
  int64_t active_limit = -1, next_limit = -1;
  MgbsMirror* mirror_dev = nullptr;  // device address of cfg.host_mirror
  bool coop_ok = true;               // cooperative launch of the selection kernel works (also inside capture)
  MgbsCtrl host_ctrl;
  mgbs::SymLayout sym{};
  uint8_t* peer_base[MGBS_MAX_WORLD] = {nullptr};
  void* peer_opened[MGBS_MAX_WORLD] = {nullptr};
  bool peers_ready = false;
  bool profile = false;
  cudaEvent_t ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t tev[96] = {nullptr};  // per-launch trace (profile mode)
  int trace_n = 0;
};

static void drop_graphs(MgbsEngine* e) {
  for (int p = 0; p < 2; ++p)
    for (int h = 0; h < 2; ++h)
      if (e->graph[p][h]) { cudaGraphExecDestroy(e->graph[p][h]); e->graph[p][h] = nullptr; }
}

#define MGBS_TRY(expr)            \
  do {                            \
    int _e = (int)(expr);         \
    if (_e != 0) return _e;       \
  } while (0)

#define MGBS_NCCL(expr)                              \
  do {                                               \
    if ((expr) != ncclSuccess) return MGBS_ERR_NCCL; \
  } while (0)

extern "C" {

int mgbs_version(void) { return 100; }
int mgbs_sizeof_ctrl(void) { return (int)sizeof(MgbsCtrl); }
int mgbs_sizeof_config(void) { return (int)sizeof(MgbsConfig); }

static int64_t round_half_up(double x) { return (int64_t)(x + 0.5); }

int mgbs_derive_sizes(int64_t global_beam_width, int32_t world_size, double gamma, double beta, double hash_load_factor,
                      int32_t band_rounds, int32_t band_levels, int64_t* out6) {
  if (global_beam_width <= 0 || world_size <= 0 || world_size > MGBS_MAX_WORLD || !out6) return MGBS_ERR_ARG;
  if (gamma < 1.0 || beta < 1.0 || hash_load_factor <= 0.0 || hash_load_factor >= 1.0) return MGBS_ERR_ARG;
  if (band_rounds < 1 || band_rounds > MGBS_MAX_ROUNDS || band_levels < 1 || band_levels > MGBS_MAX_LEVELS) return MGBS_ERR_ARG;
  const int64_t n_local = (global_beam_width + world_size - 1) / world_size;  // beam_engine.cpp:245
  const int64_t k_keep = round_half_up(gamma * (double)n_local);              // :247
  const int64_t k_work = round_half_up(beta * (double)k_keep);                // :249
  int64_t hash_capacity = round_half_up((double)k_work / hash_load_factor);   // :251-252
  if (hash_capacity < 1024) hash_capacity = 1024;
  out6[0] = n_local;
  out6[1] = k_keep;
  out6[2] = k_work;
  out6[3] = hash_capacity;
  out6[4] = round_half_up(beta * (double)n_local);
  // the persistent selection kernel uses up to three histograms per band round whatever band_levels says
  out6[5] = (int64_t)(band_rounds * (band_levels < 3 ? 3 : band_levels) + MGBS_MAX_LEVELS) * MGBS_HIST_STRIDE;
  return 0;
}

uint64_t mgbs_hash64_host(const uint8_t* state, int32_t n) {
  uint64_t h = mgbs::kFnvOffset;
  for (int i = 0; i < n; ++i) h = (h ^ (uint64_t)state[i]) * mgbs::kFnvPrime;
  return mgbs::finish_hash(h);
}

uint64_t mgbs_fingerprint64_host(const uint8_t* state, int32_t n) {
  uint64_t f = mgbs::kGolden;
  for (int i = 0; i < n; ++i) f ^= (uint64_t)state[i] + mgbs::kGolden + (f << 6) + (f >> 2);
  return mgbs::finish_fingerprint(f);
}

int mgbs_engine_create(const MgbsConfig* cfg, MgbsEngine** out) {
  if (!cfg || !out) return MGBS_ERR_ARG;
  const MgbsConfig& c = *cfg;
  if (c.state_len < 1 || c.state_len > MGBS_MAX_STATE_LEN) return MGBS_ERR_ARG;
  if (c.state_stride < c.state_len || (c.state_stride % 16) != 0 || c.state_stride > MGBS_MAX_STATE_LEN) return MGBS_ERR_ARG;
  const int words = c.state_stride / 4;
  if (words != 4 && words != 8 && words != 16 && words != 24 && words != 32) return MGBS_ERR_UNSUPPORTED;
  if (c.fanout < 1 || c.fanout > MGBS_MAX_FANOUT) return MGBS_ERR_ARG;
  if (c.world_size < 1 || c.world_size > MGBS_MAX_WORLD || c.rank < 0 || c.rank >= c.world_size) return MGBS_ERR_ARG;
  if (c.hash_bits < 0 || c.hash_bits > 44) return MGBS_ERR_ARG;
  if (c.band_levels < 1 || c.band_levels > MGBS_MAX_LEVELS || c.band_rounds < 1 || c.band_rounds > MGBS_MAX_ROUNDS) return MGBS_ERR_ARG;
  if (c.probe_limit < 1 || c.global_beam_width < 1) return MGBS_ERR_ARG;
  if (c.frontier_cap < 1 || c.frontier_cap > (1 << 23) || c.hash_capacity < c.frontier_cap) return MGBS_ERR_ARG;
  if (c.cand_cap < c.frontier_cap * c.fanout || c.cand_cap > 0xffffffffll) return MGBS_ERR_ARG;
  if (!c.frontier[0] || !c.frontier[1] || !c.gens || !c.solved || !c.cand_hash || !c.cand_fp || !c.cand_score ||
      !c.cand_payload || !c.table || !c.hist || !c.tie_buf || !c.ctrl)
    return MGBS_ERR_ARG;
  if (c.exchange_mode != MGBS_EXCHANGE_NCCL && c.exchange_mode != MGBS_EXCHANGE_PEER) return MGBS_ERR_ARG;
  if (c.hash_mode != MGBS_HASH_FNV && c.hash_mode != MGBS_HASH_ZOBRIST128) return MGBS_ERR_ARG;
  if (c.hash_mode == MGBS_HASH_ZOBRIST128 && (!c.zobrist || c.zobrist_values < 1 || c.zobrist_values > 256)) return MGBS_ERR_ARG;
  if (c.world_size > 1 && c.exchange_mode == MGBS_EXCHANGE_PEER) {
    if (!c.children || c.bucket_cap < 1 || !c.send_counts || !c.sym || !c.tickets) return MGBS_ERR_ARG;
  } else if (c.world_size > 1) {
    if (!c.children || c.bucket_cap < 1 || !c.send_hash || !c.send_fp || !c.send_score || !c.send_payload ||
        !c.send_states || !c.recv_hash || !c.recv_fp || !c.recv_score || !c.recv_payload || !c.recv_states ||
        !c.send_counts || !c.recv_counts)
      return MGBS_ERR_ARG;
  }
  if (c.select_mode != MGBS_SELECT_EXACT_K && c.hash_bits != 0) return MGBS_ERR_ARG;  // score-only order for the other modes
  MgbsEngine* e = new (std::nothrow) MgbsEngine();
  if (!e) return MGBS_ERR_STATE;
  e->cfg = c;
  e->key_bits = 20 + c.hash_bits;
  e->final_levels = (e->key_bits + MGBS_RADIX_BITS - 1) / MGBS_RADIX_BITS;
  if (e->cfg.band_levels > e->final_levels) e->cfg.band_levels = e->final_levels;
  if (c.world_size > 1 && c.exchange_mode == MGBS_EXCHANGE_PEER) {
    e->sym = mgbs::sym_layout(e->cfg, e->cfg.band_levels);
    if (c.sym_bytes < e->sym.total) { delete e; return MGBS_ERR_ARG; }
    // peers rebuild survivors from parent rows of this rank's frontiers: both buffers must sit inside the region
    for (int p = 0; p < 2; ++p)
      if (c.frontier[p] != c.sym + e->sym.frontier[p]) { delete e; return MGBS_ERR_ARG; }
    e->peer_base[c.rank] = c.sym;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) e->sms = sms;
  }
  if (c.host_mirror) {
    // pinned host memory: the kernels write through the device alias of the same allocation
    void* dptr = nullptr;
    if (cudaHostGetDevicePointer(&dptr, c.host_mirror, 0) != cudaSuccess || !dptr) { cudaGetLastError(); delete e; return MGBS_ERR_ARG; }
    e->mirror_dev = static_cast<MgbsMirror*>(dptr);
    memset(c.host_mirror, 0, sizeof(MgbsMirror));
  }
  memset(&e->host_ctrl, 0, sizeof(MgbsCtrl));
  *out = e;
  return 0;
}

int mgbs_engine_set_logical_limits(MgbsEngine* e, int64_t active_limit, int64_t next_limit) {
  if (!e) return MGBS_ERR_ARG;
  if (active_limit == 0 || next_limit == 0) return MGBS_ERR_ARG;
  e->active_limit = active_limit < 0 ? -1 : (active_limit > e->cfg.frontier_cap ? e->cfg.frontier_cap : active_limit);
  e->next_limit = next_limit < 0 ? -1 : (next_limit > e->cfg.frontier_cap ? e->cfg.frontier_cap : next_limit);
  drop_graphs(e);
  return 0;
}

int mgbs_engine_set_peer_pointers(MgbsEngine* e, uint8_t* const* bases) {
  if (!e || !bases) return MGBS_ERR_ARG;
  const MgbsConfig& c = e->cfg;
  if (c.world_size == 1 || c.exchange_mode != MGBS_EXCHANGE_PEER) return 0;
  for (int r = 0; r < c.world_size; ++r) {
    if (!bases[r]) return MGBS_ERR_ARG;
    e->peer_base[r] = r == c.rank ? c.sym : bases[r];
  }
  e->peers_ready = true;
  drop_graphs(e);
  return 0;
}

int mgbs_engine_destroy(MgbsEngine* e) {
  if (!e) return 0;
  drop_graphs(e);
  if (e->comm && g_nccl.ok) g_nccl.CommDestroy(e->comm);
  for (int i = 0; i < 6; ++i)
    if (e->ev[i]) cudaEventDestroy(e->ev[i]);
  for (int i = 0; i < 96; ++i)
    if (e->tev[i]) cudaEventDestroy(e->tev[i]);
  for (int r = 0; r < MGBS_MAX_WORLD; ++r)
    if (e->peer_opened[r]) cudaIpcCloseMemHandle(e->peer_opened[r]);
  delete e;
  return 0;
}

int mgbs_nccl_unique_id(const char* libnccl_path, uint8_t* out128) {
  if (!out128) return MGBS_ERR_ARG;
  MGBS_TRY(load_nccl(libnccl_path));
  ncclUniqueId id;
  MGBS_NCCL(g_nccl.GetUniqueId(&id));
  static_assert(sizeof(ncclUniqueId) == 128, "unique id is 128 bytes");
  memcpy(out128, &id, 128);
  return 0;
}

int mgbs_engine_init_nccl(MgbsEngine* e, const char* libnccl_path, const uint8_t* unique_id128) {
  if (!e || !unique_id128) return MGBS_ERR_ARG;
  if (e->cfg.world_size == 1) return 0;
  MGBS_TRY(load_nccl(libnccl_path));
  ncclUniqueId id;
  memcpy(&id, unique_id128, 128);
  MGBS_NCCL(g_nccl.CommInitRank(&e->comm, e->cfg.world_size, id, e->cfg.rank));
  return 0;
}

int mgbs_sym_bytes(const MgbsConfig* cfg, int64_t* out_bytes, int64_t* out_tickets) {
  if (!cfg || !out_bytes || !out_tickets) return MGBS_ERR_ARG;
  if (cfg->world_size < 1 || cfg->world_size > MGBS_MAX_WORLD || cfg->bucket_cap < 0 || cfg->state_stride < 16 ||
      cfg->frontier_cap < 0)
    return MGBS_ERR_ARG;
  int key_bits = 20 + cfg->hash_bits;
  int final_levels = (key_bits + MGBS_RADIX_BITS - 1) / MGBS_RADIX_BITS;
  int bl = cfg->band_levels > final_levels ? final_levels : cfg->band_levels;
  mgbs::SymLayout L = mgbs::sym_layout(*cfg, bl);
  *out_bytes = L.total;
  *out_tickets = L.slots + 1;
  return 0;
}

int mgbs_sym_frontier_offsets(const MgbsConfig* cfg, int64_t* out2) {
  if (!cfg || !out2) return MGBS_ERR_ARG;
  int64_t bytes = 0, tickets = 0;
  int rc = mgbs_sym_bytes(cfg, &bytes, &tickets);
  if (rc) return rc;
  int key_bits = 20 + cfg->hash_bits;
  int final_levels = (key_bits + MGBS_RADIX_BITS - 1) / MGBS_RADIX_BITS;
  int bl = cfg->band_levels > final_levels ? final_levels : cfg->band_levels;
  mgbs::SymLayout L = mgbs::sym_layout(*cfg, bl);
  out2[0] = L.frontier[0];
  out2[1] = L.frontier[1];
  return 0;
}

// IPC handle of the allocation that contains ptr, and ptr's byte offset inside it (the region may be a
// sub-allocation of a caching allocator's block).
int mgbs_ipc_export(const void* ptr, uint8_t* handle64, int64_t* offset) {
  if (!ptr || !handle64 || !offset) return MGBS_ERR_ARG;
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  MGBS_TRY(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres));
  if (qres != cudaDriverEntryPointSuccess || !fn) return MGBS_ERR_STATE;
  CUdeviceptr base = 0;
  size_t size = 0;
  if (reinterpret_cast<RangeFn>(fn)(&base, &size, (CUdeviceptr)ptr) != CUDA_SUCCESS) return MGBS_ERR_STATE;
  cudaIpcMemHandle_t h;
  MGBS_TRY(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  memcpy(handle64, &h, 64);
  *offset = (int64_t)((CUdeviceptr)ptr - base);
  return 0;
}

int mgbs_engine_set_peers(MgbsEngine* e, const uint8_t* handles, const int64_t* offsets) {
  if (!e || !handles || !offsets) return MGBS_ERR_ARG;
  const MgbsConfig& c = e->cfg;
  if (c.world_size == 1 || c.exchange_mode != MGBS_EXCHANGE_PEER) return 0;
  for (int r = 0; r < c.world_size; ++r) {
    if (r == c.rank) { e->peer_base[r] = c.sym; continue; }
    cudaIpcMemHandle_t h;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    memcpy(&h, handles + 64 * r, 64);
    void* base = nullptr;
    MGBS_TRY(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    e->peer_opened[r] = base;
    e->peer_base[r] = static_cast<uint8_t*>(base) + offsets[r];
  }
  e->peers_ready = true;
  return 0;
}

int mgbs_engine_set_parent_scorer(MgbsEngine* e, mgbs_parent_scorer_fn fn, void* user) {
  if (!e) return MGBS_ERR_ARG;
  e->parent_scorer = fn;
  e->parent_scorer_user = user;
  drop_graphs(e);
  return 0;
}

int mgbs_engine_set_scorer(MgbsEngine* e, mgbs_scorer_fn fn, void* user) {
  if (!e) return MGBS_ERR_ARG;
  e->scorer = fn;
  e->scorer_user = user;
  drop_graphs(e);
  return 0;
}

int mgbs_engine_profile(MgbsEngine* e, int32_t on) {
  if (!e) return MGBS_ERR_ARG;
  if (on)
    for (int i = 0; i < 6; ++i)
      if (!e->ev[i]) MGBS_TRY(cudaEventCreate(&e->ev[i]));
  if (on)
    for (int i = 0; i < 96; ++i)
      if (!e->tev[i]) MGBS_TRY(cudaEventCreate(&e->tev[i]));
  e->profile = on != 0;
  drop_graphs(e);
  return 0;
}

int mgbs_engine_profile_read(MgbsEngine* e, float* ms5) {
  if (!e || !ms5 || !e->ev[0]) return MGBS_ERR_ARG;
  MGBS_TRY(cudaEventSynchronize(e->ev[5]));
  for (int i = 0; i < 5; ++i) MGBS_TRY(cudaEventElapsedTime(&ms5[i], e->ev[i], e->ev[i + 1]));
  return 0;
}

// Per-launch trace of the last profiled step: ms[i] = time between consecutive trace points (one after every kernel,
// memset or collective enqueued by mgbs_engine_enqueue_depth, in enqueue order); returns the number of intervals.
int mgbs_engine_trace_read(MgbsEngine* e, float* ms, int32_t capacity) {
  if (!e || !ms || e->trace_n < 2) return 0;
  if (cudaEventSynchronize(e->tev[e->trace_n - 1]) != cudaSuccess) return 0;
  int n = 0;
  for (int i = 0; i + 1 < e->trace_n && n < capacity; ++i, ++n)
    if (cudaEventElapsedTime(&ms[n], e->tev[i], e->tev[i + 1]) != cudaSuccess) return n;
  return n;
}

int mgbs_engine_set_score_mode(MgbsEngine* e, int32_t score_mode, int32_t uniform_score) {
  if (!e || score_mode < MGBS_SCORE_EXTERNAL || score_mode > MGBS_SCORE_UNIFORM) return MGBS_ERR_ARG;
  e->cfg.score_mode = score_mode;
  e->cfg.uniform_score = uniform_score;
  drop_graphs(e);
  return 0;
}

int mgbs_engine_reset(MgbsEngine* e, const uint8_t* start_state_host, int32_t active_on_this_rank,
                      int32_t start_is_solved, void* stream) {
  if (!e || !start_state_host) return MGBS_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const MgbsConfig& c = e->cfg;
  MgbsCtrl& h = e->host_ctrl;
  uint32_t epoch = 0;  // cross-rank flags are tagged with it: it must never go back
  MGBS_TRY(cudaMemcpyAsync(&epoch, &c.ctrl->epoch, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
  MGBS_TRY(cudaStreamSynchronize(st));
  memset(&h, 0, sizeof(MgbsCtrl));
  h.epoch = epoch;
  h.frontier_count[0] = active_on_this_rank ? 1 : 0;
  h.found_payload = 0xffffffffu;
  h.rho_num = 1;
  h.rho_den = 1;
  if (start_is_solved) { h.found = 1; h.found_depth = 0; }
  MGBS_TRY(cudaMemcpyAsync(c.ctrl, &h, sizeof(MgbsCtrl), cudaMemcpyHostToDevice, st));
  if (active_on_this_rank) {
    uint8_t row[MGBS_MAX_STATE_LEN];
    memset(row, 0, sizeof(row));
    memcpy(row, start_state_host, (size_t)c.state_len);
    MGBS_TRY(cudaMemcpyAsync(c.frontier[0], row, (size_t)c.state_stride, cudaMemcpyHostToDevice, st));
  }
  MGBS_TRY(cudaStreamSynchronize(st));
  if (c.host_mirror) memset(c.host_mirror, 0, sizeof(MgbsMirror));  // launch_seq restarts at 0 with the control block
  return 0;
}

// Load a whole frontier (rows of state_len bytes, host memory) as the current frontier of buffer `parity`.
int mgbs_engine_load_frontier(MgbsEngine* e, const uint8_t* rows_host, int64_t count, int32_t parity, int32_t depth,
                              void* stream) {
  if (!e || count < 0 || count > e->cfg.frontier_cap || (count > 0 && !rows_host)) return MGBS_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const MgbsConfig& c = e->cfg;
  MgbsCtrl& h = e->host_ctrl;
  uint32_t epoch = 0;
  MGBS_TRY(cudaMemcpyAsync(&epoch, &c.ctrl->epoch, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
  MGBS_TRY(cudaStreamSynchronize(st));
  memset(&h, 0, sizeof(MgbsCtrl));
  h.epoch = epoch;
  h.frontier_count[parity & 1] = (int32_t)count;
  h.depth = depth;
  h.found_payload = 0xffffffffu;
  h.rho_num = 1;
  h.rho_den = 1;
  MGBS_TRY(cudaMemcpyAsync(c.ctrl, &h, sizeof(MgbsCtrl), cudaMemcpyHostToDevice, st));
  if (count > 0 && c.io_stage) {
    MGBS_TRY(cudaMemcpyAsync(c.io_stage, rows_host, (size_t)count * c.state_len, cudaMemcpyHostToDevice, st));
    MGBS_TRY(mgbs::launch_repack_rows(c.io_stage, c.frontier[parity & 1], count, c.state_len, c.state_stride,
                                      c.state_len, e->sms, st));
  } else if (count > 0) {
    MGBS_TRY(cudaMemsetAsync(c.frontier[parity & 1], 0, (size_t)count * c.state_stride, st));
    MGBS_TRY(cudaMemcpy2DAsync(c.frontier[parity & 1], (size_t)c.state_stride, rows_host, (size_t)c.state_len,
                               (size_t)c.state_len, (size_t)count, cudaMemcpyHostToDevice, st));
  }
  MGBS_TRY(cudaStreamSynchronize(st));
  if (c.host_mirror) memset(c.host_mirror, 0, sizeof(MgbsMirror));
  return 0;
}

// Copy the current frontier (buffer `parity`) to host memory as packed rows of state_len bytes; returns the row
// count through *count_out.  dst_host must hold capacity_rows rows; pinned memory makes the copy asynchronous up to
// the final synchronisation.
int mgbs_engine_read_frontier(MgbsEngine* e, int32_t parity, uint8_t* dst_host, int64_t capacity_rows,
                              int64_t* count_out, void* stream) {
  if (!e || !dst_host || !count_out || capacity_rows < 0) return MGBS_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const MgbsConfig& c = e->cfg;
  int32_t cnt = 0;
  MGBS_TRY(cudaMemcpyAsync(&cnt, &c.ctrl->frontier_count[parity & 1], sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  MGBS_TRY(cudaStreamSynchronize(st));
  int64_t n = cnt < 0 ? 0 : cnt;
  if (n > capacity_rows) n = capacity_rows;
  if (n > 0 && c.io_stage) {
    MGBS_TRY(mgbs::launch_repack_rows(c.frontier[parity & 1], c.io_stage, n, c.state_stride, c.state_len, c.state_len,
                                      e->sms, st));
    MGBS_TRY(cudaMemcpyAsync(dst_host, c.io_stage, (size_t)n * c.state_len, cudaMemcpyDeviceToHost, st));
    MGBS_TRY(cudaStreamSynchronize(st));
  } else if (n > 0) {
    MGBS_TRY(cudaMemcpy2DAsync(dst_host, (size_t)c.state_len, c.frontier[parity & 1], (size_t)c.state_stride,
                               (size_t)c.state_len, (size_t)n, cudaMemcpyDeviceToHost, st));
    MGBS_TRY(cudaStreamSynchronize(st));
  }
  *count_out = n;
  return 0;
}

static int allreduce_hist(MgbsEngine* e, uint32_t* hist, cudaStream_t st) {
  if (e->cfg.world_size == 1 || e->cfg.exchange_mode == MGBS_EXCHANGE_PEER) return 0;  // peer mode reduces in-kernel
  if (!e->comm) return MGBS_ERR_STATE;
  MGBS_NCCL(g_nccl.AllReduce(hist, hist, MGBS_HIST_STRIDE, ncclUint32, ncclSum, e->comm, st));
  return 0;
}

static int exchange(MgbsEngine* e, cudaStream_t st) {
  const MgbsConfig& c = e->cfg;
  if (!e->comm) return MGBS_ERR_STATE;
  const size_t cap = (size_t)c.bucket_cap;
  MGBS_NCCL(g_nccl.GroupStart());
  for (int r = 0; r < c.world_size; ++r) {
    MGBS_NCCL(g_nccl.Send(c.send_counts + r, 1, ncclUint32, r, e->comm, st));
    MGBS_NCCL(g_nccl.Recv(c.recv_counts + r, 1, ncclUint32, r, e->comm, st));
    MGBS_NCCL(g_nccl.Send(c.send_hash + r * cap, cap, ncclUint64, r, e->comm, st));
    MGBS_NCCL(g_nccl.Recv(c.recv_hash + r * cap, cap, ncclUint64, r, e->comm, st));
    MGBS_NCCL(g_nccl.Send(c.send_fp + r * cap, cap, ncclUint64, r, e->comm, st));
    MGBS_NCCL(g_nccl.Recv(c.recv_fp + r * cap, cap, ncclUint64, r, e->comm, st));
    MGBS_NCCL(g_nccl.Send(c.send_score + r * cap, cap, ncclUint32, r, e->comm, st));
    MGBS_NCCL(g_nccl.Recv(c.recv_score + r * cap, cap, ncclUint32, r, e->comm, st));
    MGBS_NCCL(g_nccl.Send(c.send_payload + r * cap, cap, ncclUint32, r, e->comm, st));
    MGBS_NCCL(g_nccl.Recv(c.recv_payload + r * cap, cap, ncclUint32, r, e->comm, st));
    MGBS_NCCL(g_nccl.Send(c.send_states + r * cap * c.state_stride, cap * c.state_stride, ncclUint8, r, e->comm, st));
    MGBS_NCCL(g_nccl.Recv(c.recv_states + r * cap * c.state_stride, cap * c.state_stride, ncclUint8, r, e->comm, st));
  }
  MGBS_NCCL(g_nccl.GroupEnd());
  return 0;
}

static int enqueue_depth(MgbsEngine* e, int32_t parity, int32_t phase, int auto_halt, void* stream) {
  if (!e || phase < 0 || phase > 2) return MGBS_ERR_ARG;
  using namespace mgbs;
  cudaStream_t st = (cudaStream_t)stream;
  const MgbsConfig& c = e->cfg;
  parity &= 1;
  const int W = c.world_size;
  const int Lb = c.band_levels, R = c.band_rounds, Lf = e->final_levels;
  unsigned long long* tie_buf = reinterpret_cast<unsigned long long*>(c.tie_buf);
  // logical limits (set_next_limit, beam_engine.cpp:1072-1083): fewer frontier rows, a smaller table and pool
  int64_t frontier_cap_eff = c.frontier_cap, hash_capacity_eff = c.hash_capacity, pool_target_eff = c.pool_target;
  if (e->next_limit > 0 && e->next_limit < c.frontier_cap) {
    frontier_cap_eff = e->next_limit;
    const double inv_load = (double)c.hash_capacity / (double)c.frontier_cap;
    hash_capacity_eff = (int64_t)((double)e->next_limit * inv_load) + 1024;
    if (hash_capacity_eff > c.hash_capacity) hash_capacity_eff = c.hash_capacity;
    pool_target_eff = (int64_t)((double)c.pool_target * (double)e->next_limit / (double)c.frontier_cap);
    if (pool_target_eff < 1) pool_target_eff = 1;
  }

  const bool prof = e->profile && phase == 0;
  if (prof) { cudaEventRecord(e->ev[0], st); e->trace_n = 0; }
#define MGBS_TRACE() do { if (prof && e->trace_n < 96) cudaEventRecord(e->tev[e->trace_n++], st); } while (0)
  MGBS_TRACE();
  if (phase == 0 || phase == 1) {
    const bool peer_mode = W > 1 && c.exchange_mode == MGBS_EXCHANGE_PEER;
    MGBS_TRY(launch_depth_begin(c.ctrl, parity, c.fanout, c.cand_cap, tie_buf + (int64_t)c.rank * kTieSegWords,
                                W > 1 ? c.send_counts : nullptr,
                                peer_mode ? reinterpret_cast<uint32_t*>(c.sym + e->sym.counts[parity]) : nullptr, W,
                                e->active_limit, auto_halt,
                                peer_mode ? reinterpret_cast<const uint32_t*>(c.sym + e->sym.abort_word) : nullptr, st));
    MGBS_TRY(cudaMemsetAsync(c.table, 0, (size_t)hash_capacity_eff * 32, st));
    MGBS_TRY(cudaMemsetAsync(c.hist, 0, (size_t)(R * (Lb < 3 ? 3 : Lb) + MGBS_MAX_LEVELS) * MGBS_HIST_STRIDE * sizeof(uint32_t), st));
    ExpandArgs x;
    x.frontier = c.frontier[parity];
    x.count_dev = &c.ctrl->active_rows;
    x.count = 0;
    x.gens = c.gens;
    x.solved = c.solved;
    x.n = c.state_len; x.stride = c.state_stride; x.fanout = c.fanout; x.rank = c.rank;
    x.score_mode = c.score_mode; x.uniform_score = c.uniform_score;
    // child rows are needed by a child scorer and by the NCCL exchange; with a parent scorer and survivors rebuilt
    // from back-pointers nobody reads them
    const bool rows_unused = c.score_mode == MGBS_SCORE_EXTERNAL && e->parent_scorer != nullptr &&
                             (W == 1 || c.exchange_mode == MGBS_EXCHANGE_PEER);
    x.children = rows_unused ? nullptr : c.children;
    x.cand_hash = c.cand_hash; x.cand_fp = c.cand_fp; x.cand_score = c.cand_score; x.cand_payload = c.cand_payload;
    x.ctrl = c.ctrl;
    x.zobrist = c.hash_mode == MGBS_HASH_ZOBRIST128 ? c.zobrist : nullptr;
    x.zobrist_values = c.zobrist_values;
    MGBS_TRACE();  // depth_begin + clears
    MGBS_TRY(launch_expand(x, c.frontier_cap, e->sms, st));
    MGBS_TRACE();  // expand
    if (prof) cudaEventRecord(e->ev[1], st);
    if (phase == 0 && c.score_mode == MGBS_SCORE_EXTERNAL) {
      if (e->parent_scorer) {
        // action values: one forward pass per parent row gives the scores of all its children
        MGBS_TRY(e->parent_scorer(e->parent_scorer_user, c.frontier[parity], &c.ctrl->active_rows,
                                  c.cand_score, stream));
      } else {
        if (!e->scorer) return MGBS_ERR_STATE;
        MGBS_TRY(e->scorer(e->scorer_user, c.children, &c.ctrl->cand_count, c.cand_score, stream));
      }
    }
    if (phase == 1) return 0;
  }
  if (prof) cudaEventRecord(e->ev[2], st);
  MGBS_TRACE();  // scorer

  StepArgs a;
  memset(&a, 0, sizeof(a));
  RouteArgs pr;  // peer mode: routing of one band
  memset(&pr, 0, sizeof(pr));
  const bool peer = W > 1 && c.exchange_mode == MGBS_EXCHANGE_PEER;
  int64_t items;
  if (W == 1) {
    a.cv.hash = c.cand_hash; a.cv.fp = c.cand_fp; a.cv.score = c.cand_score; a.cv.payload = c.cand_payload;
    a.cv.states = nullptr;  // survivors are rebuilt from parent row + move (k_emit walks the table, not the candidates)
    a.cv.counts = &c.ctrl->cand_count;
    a.cv.nbuckets = 1;
    a.cv.cap = (uint32_t)c.cand_cap;
    items = c.cand_cap;
    a.cvh = a.cv;
  } else if (peer) {
    // nothing moves yet: every band round counts its histograms over this rank's own candidates (the sums over
    // ranks are what matters), then routes just that band to the owners, who insert it
    if (!e->peers_ready) return MGBS_ERR_STATE;
    const SymLayout& L = e->sym;
    pr.hash = c.cand_hash; pr.fp = c.cand_fp; pr.score = c.cand_score; pr.payload = c.cand_payload;
    pr.send_counts = c.send_counts;
    pr.ctrl = c.ctrl;
    pr.world = W; pr.stride = c.state_stride; pr.bucket_cap = (uint32_t)c.bucket_cap;
    pr.rank = c.rank;
    for (int q = 0; q < W; ++q) pr.peer.base[q] = e->peer_base[q];
    pr.peer.enabled = 1;
    pr.peer.tickets = c.tickets;
    pr.peer.slot = L.slots;  // the ticket word after the histogram slots
    pr.off_hash = L.hash[parity]; pr.off_fp = L.fp[parity]; pr.off_score = L.score[parity];
    pr.off_payload = L.payload[parity]; pr.off_counts = L.counts[parity];
    pr.off_route_flag = L.route_flag;
    pr.hash_mode = c.hash_mode;
    a.cvh.hash = c.cand_hash; a.cvh.fp = c.cand_fp; a.cvh.score = c.cand_score; a.cvh.payload = c.cand_payload;
    a.cvh.states = nullptr;
    a.cvh.counts = &c.ctrl->cand_count;
    a.cvh.nbuckets = 1;
    a.cvh.cap = (uint32_t)c.cand_cap;
    a.cv.hash = reinterpret_cast<const uint64_t*>(c.sym + L.hash[parity]);
    a.cv.fp = reinterpret_cast<const uint64_t*>(c.sym + L.fp[parity]);
    a.cv.score = reinterpret_cast<const uint32_t*>(c.sym + L.score[parity]);
    a.cv.payload = reinterpret_cast<const uint32_t*>(c.sym + L.payload[parity]);
    a.cv.states = nullptr;  // survivors are rebuilt from their parents' rows in the senders' frontiers
    a.cv.counts = reinterpret_cast<const uint32_t*>(c.sym + L.counts[parity]);
    a.cv.nbuckets = W;
    a.cv.cap = (uint32_t)c.bucket_cap;
    a.off_frontier_cur = L.frontier[parity];
    items = c.bucket_cap;
    for (int q = 0; q < W; ++q) a.peer.base[q] = e->peer_base[q];
    a.peer.enabled = 1;
    a.peer.tickets = c.tickets;
    a.peer.off_hx = L.hx;
    a.peer.off_hflag = L.hflag;
    a.peer.off_tie = L.tie;
    a.peer.off_tie_flag = L.tie_flag;
    a.peer.off_abort = L.abort_word;
    const uint32_t poll = c.peer_poll_limit > 0 ? (uint32_t)(c.peer_poll_limit > 0x7fffffffll ? 0x7fffffffll : c.peer_poll_limit) : (1u << 22);
    a.peer.poll_limit = poll;
    pr.peer.poll_limit = poll;
    pr.peer.off_abort = L.abort_word;
  } else {
    RouteArgs r;
    memset(&r, 0, sizeof(r));
    r.hash = c.cand_hash; r.fp = c.cand_fp; r.score = c.cand_score; r.payload = c.cand_payload; r.states = c.children;
    r.s_hash = c.send_hash; r.s_fp = c.send_fp; r.s_score = c.send_score; r.s_payload = c.send_payload;
    r.s_states = c.send_states;
    r.send_counts = c.send_counts;
    r.ctrl = c.ctrl;
    r.world = W; r.stride = c.state_stride; r.bucket_cap = (uint32_t)c.bucket_cap;
    r.hash_mode = c.hash_mode;
    MGBS_TRY(launch_route(r, c.cand_cap, e->sms, st));
    MGBS_TRY(exchange(e, st));
    MGBS_TRY(launch_clamp_counts(c.recv_counts, W, (uint32_t)c.bucket_cap, st));
    a.cv.hash = c.recv_hash; a.cv.fp = c.recv_fp; a.cv.score = c.recv_score; a.cv.payload = c.recv_payload;
    a.cv.states = c.recv_states;
    a.cv.counts = c.recv_counts;
    a.cv.nbuckets = W;
    a.cv.cap = (uint32_t)c.bucket_cap;
    items = c.bucket_cap;  // per bucket; kernels loop over buckets
    a.cvh = a.cv;
  }
  if (prof) cudaEventRecord(e->ev[3], st);
  MGBS_TRACE();  // route + exchange
  a.ctrl = c.ctrl;
  a.table = c.table;
  a.tie_buf = tie_buf;
  a.hash_capacity = hash_capacity_eff;
  a.beam = c.global_beam_width;
  a.pool_target = pool_target_eff;
  a.frontier_cap = c.frontier_cap;
  a.next_cap = frontier_cap_eff;
  a.mirror = e->mirror_dev;
  a.hist_base = c.hist;
  a.band_levels = Lb;
  a.final_levels = Lf;
  // the block barrier must outlast a cross-rank wait that one block is in
  a.grid_poll_limit = (peer ? a.peer.poll_limit : 0u) * 2u + (1u << 22);
  a.world = W; a.rank = c.rank;
  a.key_bits = e->key_bits; a.hash_bits = c.hash_bits;
  a.rounds = R;
  a.select_mode = c.select_mode; a.probe_limit = c.probe_limit;
  a.frontier_cur = c.frontier[parity];
  a.frontier_next = c.frontier[parity ^ 1];
  a.gens = c.gens;
  a.history = c.history;
  a.history_depths = c.history_depths;
  a.next_score = c.frontier_score[parity ^ 1];
  a.next_hash = c.frontier_hash[parity ^ 1];
  a.n = c.state_len; a.stride = c.state_stride; a.fanout = c.fanout; a.parity = parity;

  if (!c.staged_select && (W == 1 || peer)) {
    // band rounds, final cut, emit, ties and finish as phases of one co-resident kernel
    a.levels = Lf;
    a.hist_stats = c.hist + (int64_t)(R * Lb) * MGBS_HIST_STRIDE;
    int rc = launch_select(a, pr, e->sms, e->coop_ok, st);
    if (rc != 0 && e->coop_ok) {
      // a runtime that refuses the cooperative launch here (e.g. inside stream capture): the grid is sized to be
      // co-resident anyway and every block barrier wait is bounded, so a plain launch is used from now on
      cudaGetLastError();
      e->coop_ok = false;
      rc = launch_select(a, pr, e->sms, false, st);
    }
    MGBS_TRY(rc);
    MGBS_TRACE();  // selection
    if (prof) { cudaEventRecord(e->ev[4], st); cudaEventRecord(e->ev[5], st); }
    return 0;
  }
  // band rounds: place a threshold by histogram levels, then insert that band into the table
  for (int r = 0; r < R; ++r) {
    a.round = r;
    a.levels = Lb;
    for (int l = 0; l < Lb; ++l) {
      a.level = l;
      a.hist = c.hist + (int64_t)(r * Lb + l) * MGBS_HIST_STRIDE;
      a.peer.slot = r * Lb + l;
      a.hist_prev = l > 0 ? c.hist + (int64_t)(r * Lb + l - 1) * MGBS_HIST_STRIDE : nullptr;
      MGBS_TRY(launch_band_hist(a, peer ? c.cand_cap : items, e->sms, st));
      MGBS_TRY(allreduce_hist(e, a.hist, st));
      MGBS_TRACE();  // band histogram (+ reduction)
    }
    a.hist = nullptr;
    a.hist_prev = c.hist + (int64_t)(r * Lb + Lb - 1) * MGBS_HIST_STRIDE;
    if (peer) {
      MGBS_TRY(launch_route_band(a, pr, c.cand_cap, e->sms, st));
      MGBS_TRACE();  // band route
    }
    MGBS_TRY(launch_band_insert(a, items, e->sms, st));
    MGBS_TRACE();  // band insert
  }
  if (prof) cudaEventRecord(e->ev[4], st);
  // final cut over the table
  uint32_t* fin = c.hist + (int64_t)(R * Lb) * MGBS_HIST_STRIDE;
  a.levels = Lf;
  a.hist_stats = fin;
  for (int l = 0; l < Lf; ++l) {
    a.level = l;
    a.hist = fin + (int64_t)l * MGBS_HIST_STRIDE;
    a.peer.slot = R * Lb + l;
    a.hist_prev = l > 0 ? fin + (int64_t)(l - 1) * MGBS_HIST_STRIDE : nullptr;
    MGBS_TRY(launch_final_hist(a, hash_capacity_eff, e->sms, st));
    MGBS_TRY(allreduce_hist(e, a.hist, st));
    MGBS_TRACE();  // final histogram (+ reduction)
  }
  a.hist = nullptr;
  a.hist_prev = fin + (int64_t)(Lf - 1) * MGBS_HIST_STRIDE;
  MGBS_TRY(launch_emit(a, a.cv.states ? items : hash_capacity_eff, e->sms, st));
  MGBS_TRACE();  // emit
  if (W > 1) {
    if (!e->comm) return MGBS_ERR_STATE;
    MGBS_NCCL(g_nccl.AllGather(tie_buf + (int64_t)c.rank * kTieSegWords, tie_buf, kTieSegWords, ncclUint64, e->comm, st));
  }
  MGBS_TRY(launch_finish(a, st));
  MGBS_TRACE();  // tie all-gather + finish
#undef MGBS_TRACE
  if (prof) cudaEventRecord(e->ev[5], st);
  return 0;
}

int mgbs_engine_enqueue_depth(MgbsEngine* e, int32_t parity, int32_t phase, void* stream) {
  return enqueue_depth(e, parity, phase, 0, stream);
}

// One depth step through a captured CUDA graph (one graph per frontier parity; captured on first use).
// Replaces BeamEngine::step with capture_cuda_graph (beam_engine.cpp:1104-1116, 1658-1672).
static int step_graph(MgbsEngine* e, int32_t parity, int auto_halt, void* stream) {
  if (!e) return MGBS_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  parity &= 1;
  auto_halt = auto_halt ? 1 : 0;
  if (e->profile) return MGBS_ERR_STATE;  // stage events cannot be timed from inside a graph
  for (int attempt = 0; attempt < 2 && !e->graph[parity][auto_halt]; ++attempt) {
    const bool coop_before = e->coop_ok;
    cudaGraph_t g = nullptr;
    MGBS_TRY(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_depth(e, parity, 0, auto_halt, stream);
    cudaError_t ce = cudaStreamEndCapture(st, &g);
    if (rc == 0 && ce == cudaSuccess) {
      ce = cudaGraphInstantiate(&e->graph[parity][auto_halt], g, 0);
      cudaGraphDestroy(g);
      if (ce == cudaSuccess) break;
      e->graph[parity][auto_halt] = nullptr;
    } else if (g) {
      cudaGraphDestroy(g);
    }
    cudaGetLastError();
    // a runtime that cannot capture or instantiate the cooperative selection launch: capture once more with a
    // plain launch (the grid is sized to be co-resident and every block-barrier wait is bounded)
    if (attempt == 0 && coop_before && !e->cfg.staged_select) { e->coop_ok = false; continue; }
    return rc != 0 ? rc : (int)ce;
  }
  return (int)cudaGraphLaunch(e->graph[parity][auto_halt], st);
}

int mgbs_engine_step_graph(MgbsEngine* e, int32_t parity, void* stream) { return step_graph(e, parity, 0, stream); }

int mgbs_engine_read_ctrl(MgbsEngine* e, MgbsCtrl* out_host, void* stream) {
  if (!e || !out_host) return MGBS_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  MGBS_TRY(cudaMemcpyAsync(out_host, e->cfg.ctrl, sizeof(MgbsCtrl), cudaMemcpyDeviceToHost, st));
  MGBS_TRY(cudaStreamSynchronize(st));
  return 0;
}

// Depth loop on the host: step until found, max_depth or an empty frontier (BeamEngine::search,
// beam_engine.cpp:1147-1171).  Every launch of the loop is made with auto_halt: a depth that opens on a finished
// search returns at once on the device and leaves the control block as it was.  That lets the host run ahead: with a
// pinned mirror it enqueues depth d + 1 before it has seen the summary of depth d and reads summaries from host
// memory, so between depths there is neither a copy nor a stream synchronisation; without a mirror it reads the
// control block once per depth.  world > 1: all ranks see the same found flag and the same global counts (both ride
// in summed statistics), so they stop together; a cross-rank wait that gave up ends the loop with an error on
// every rank (the rank that gave up tells the others, and every wait is bounded).
static const uint32_t kFatalBits = MGBS_ST_PEER_TIMEOUT | MGBS_ST_GRID_TIMEOUT;

static int launch_one(MgbsEngine* e, int parity, int use_graph, void* stream) {
  if (use_graph) return step_graph(e, parity, 1, stream);
  return enqueue_depth(e, parity, 0, 1, stream);
}

int mgbs_engine_search(MgbsEngine* e, int32_t max_depth, int32_t use_graph, MgbsCtrl* out_host, void* stream) {
  if (!e || !out_host) return MGBS_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  MGBS_TRY(mgbs_engine_read_ctrl(e, out_host, stream));
  const int W = e->cfg.world_size;
  volatile MgbsMirror* m = e->profile ? nullptr : e->cfg.host_mirror;
  if (!m) {
    while (!out_host->found && out_host->depth < max_depth && !out_host->exhausted && !(out_host->status & kFatalBits)) {
      const int parity = out_host->depth & 1;
      if (W == 1 && out_host->frontier_count[parity] == 0) break;
      MGBS_TRY(launch_one(e, parity, use_graph && !e->profile, stream));
      MGBS_TRY(mgbs_engine_read_ctrl(e, out_host, stream));
    }
    return (out_host->status & kFatalBits) ? MGBS_ERR_PEER_TIMEOUT : 0;
  }
  // run-ahead loop over the pinned summaries.  Every launch that is not halted advances the depth by one, and once
  // one launch halts all later ones do (found, nothing left and a failed wait are sticky), so the frontier parity
  // of launch k is that of depth0 + k without waiting for anything.
  const uint64_t seq0 = out_host->launch_seq;
  const int depth0 = out_host->depth;
  bool stop = out_host->found || out_host->exhausted || (out_host->status & kFatalBits) ||
              (W == 1 && out_host->frontier_count[depth0 & 1] == 0);
  uint64_t issued = 0, seen = 0;
  for (;;) {
    // keep one depth in flight beyond the last summary read, never past max_depth
    while (!stop && issued - seen < 2 && depth0 + (int64_t)issued < (int64_t)max_depth) {
      MGBS_TRY(launch_one(e, (int)((depth0 + issued) & 1), use_graph, stream));
      ++issued;
    }
    if (seen == issued) break;
    // wait for the next summary: host memory only; now and then ask the runtime whether the stream failed
    const uint64_t want = seq0 + seen + 1;
    uint32_t spins = 0;
    while (m->seq < want) {
      if ((++spins & 0xfffu) == 0u) {
        cudaError_t q = cudaStreamQuery(st);
        if (q != cudaSuccess && q != cudaErrorNotReady) return (int)q;
        if (q == cudaSuccess && m->seq < want) return MGBS_ERR_STATE;  // the stream is idle and nothing arrived
      }
    }
    ++seen;
    // the launch after this one may be rewriting the summary right now; every field only ever moves towards
    // "stop" (found, status and exhaustion are sticky), so a mixed read is still a correct reason to stop
    if (m->found || (m->status & kFatalBits) || m->unique_total == 0 || (W == 1 && m->frontier_next == 0)) stop = true;
  }
  MGBS_TRY(mgbs_engine_read_ctrl(e, out_host, stream));
  return (out_host->status & kFatalBits) ? MGBS_ERR_PEER_TIMEOUT : 0;
}

int mgbs_launch_expand(const uint8_t* frontier, const int32_t* count_dev, int64_t count, const uint8_t* gens,
                       const uint8_t* solved, int32_t state_len, int32_t state_stride, int32_t fanout, int32_t rank,
                       int32_t score_mode, int32_t uniform_score, uint8_t* children, uint64_t* cand_hash,
                       uint64_t* cand_fp, uint32_t* cand_score, uint32_t* cand_payload, MgbsCtrl* ctrl, void* stream) {
  if (!frontier || !gens || !solved || !cand_hash || !cand_fp || !cand_payload) return MGBS_ERR_ARG;
  if (score_mode != MGBS_SCORE_EXTERNAL && !cand_score) return MGBS_ERR_ARG;
  if (state_len < 1 || state_stride < state_len || (state_stride % 16) != 0 || state_stride > MGBS_MAX_STATE_LEN) return MGBS_ERR_ARG;
  if (fanout < 1 || fanout > MGBS_MAX_FANOUT || count < 0) return MGBS_ERR_ARG;
  mgbs::ExpandArgs x;
  x.frontier = frontier; x.count_dev = count_dev; x.count = count; x.gens = gens; x.solved = solved;
  x.n = state_len; x.stride = state_stride; x.fanout = fanout; x.rank = rank;
  x.score_mode = score_mode; x.uniform_score = uniform_score;
  x.children = children; x.cand_hash = cand_hash; x.cand_fp = cand_fp; x.cand_score = cand_score;
  x.cand_payload = cand_payload; x.ctrl = ctrl;
  x.zobrist = nullptr; x.zobrist_values = 0;
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return mgbs::launch_expand(x, count_dev ? (int64_t)1 << 22 : count, sms, (cudaStream_t)stream);
}

}  // extern "C"
