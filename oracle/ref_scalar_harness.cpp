// Host harness around the reference's own scalar device functions.  TEST INFRASTRUCTURE ONLY: it exists to
// generate golden vectors for the oracle (tests/golden/make_golden.py) and is never loaded by the product.
//
// The reference keeps its per-state arithmetic in `__device__ __forceinline__` functions inside CUDA sources:
//   beam_kernels.cu:29-103        mix64, hash_state_120, fingerprint_state_120, tie16, make_best_key,
//                                 apply_move_table, hamming_to_central, is_central_state
//   beam_kernels_stream2.cu:8-38  apply_move_state128, is_goal_state128, hash_state128_zobrist
//   beam_kernels_stream3.cu:29-35 owner_from_hash128
//   beam_kernels_stream4.cu:25-33 candidate_better
// They are pure integer functions of their arguments (plus two __constant__ tables), so they compile as plain
// host C++ once the CUDA qualifiers are defined away.  The Makefile beside this file cuts exactly those line
// ranges out of the reference checkout into oracle/_ref/*.inc (git-ignored; no reference source is stored in
// this repository) and this file includes them, together with the reference's own headers
// beam_engine_common.hpp and beam_types.hpp (plain C++ already), and exports them with C linkage.
#include <cstdint>
#include <cstring>

#define __device__
#define __host__
#define __forceinline__ inline
#define __constant__ static
#define __restrict__

#include "beam_engine_common.hpp"  // from the reference checkout (-I)
#include "beam_types.hpp"          // from the reference checkout (-I)

namespace beam_engine {
#include "_ref/legacy_scalar.inc"
}  // namespace beam_engine

namespace beam_v6 {
#include "_ref/v6_stream2_scalar.inc"
#include "_ref/v6_stream3_scalar.inc"
#include "_ref/v6_stream4_scalar.inc"
}  // namespace beam_v6

extern "C" {

int ref_state_len(void) { return beam_engine::STATE_SIZE_BYTES_FIXED; }
int ref_fanout(void) { return beam_engine::FANOUT_FIXED; }

uint64_t ref_mix64(uint64_t x) { return beam_engine::mix64(x); }
uint64_t ref_hash_state_120(const uint8_t* s) { return beam_engine::hash_state_120(s); }
uint64_t ref_fingerprint_state_120(const uint8_t* s) { return beam_engine::fingerprint_state_120(s); }
uint32_t ref_tie16(uint64_t fp) { return beam_engine::tie16(fp); }
uint32_t ref_make_best_key(uint32_t score_q, uint64_t fp) {
  return beam_engine::make_best_key(static_cast<uint16_t>(score_q), fp);
}

// the two __constant__ tables of the legacy kernels (uploaded by upload_action_permutation_table /
// upload_central_state in the reference); loaded = 0 exercises the reference's "table not loaded" branches
void ref_set_action_table(const uint8_t* table, int loaded) {
  if (table) std::memcpy(beam_engine::c_action_permutation, table, sizeof(beam_engine::c_action_permutation));
  beam_engine::c_action_permutation_loaded = static_cast<uint8_t>(loaded);
}
void ref_set_central_state(const uint8_t* state, int loaded) {
  if (state) std::memcpy(beam_engine::c_central_state, state, sizeof(beam_engine::c_central_state));
  beam_engine::c_central_state_loaded = static_cast<uint8_t>(loaded);
}
void ref_apply_move_table(const uint8_t* src, int action, uint8_t* dst) {
  beam_engine::apply_move_table(src, static_cast<uint8_t>(action), dst);
}
int ref_hamming_to_central(const uint8_t* s) { return beam_engine::hamming_to_central(s); }
int ref_is_central_state(const uint8_t* s) { return beam_engine::is_central_state(s) ? 1 : 0; }

// v6: State128 rows (128 bytes), generators [moves][128], zobrist [128 positions][128 values] of {lo, hi}
void ref_apply_move_state128(const uint8_t* parent128, const uint8_t* generators, int move, uint8_t* child128) {
  beam_v6::State128 p;
  std::memcpy(p.v, parent128, 128);
  const beam_v6::State128 c = beam_v6::apply_move_state128(p, generators, static_cast<uint8_t>(move));
  std::memcpy(child128, c.v, 128);
}
int ref_is_goal_state128(const uint8_t* child128, const uint8_t* central128) {
  beam_v6::State128 c;
  std::memcpy(c.v, child128, 128);
  return beam_v6::is_goal_state128(c, central128) ? 1 : 0;
}
void ref_hash_state128_zobrist(const uint8_t* child128, const uint64_t* zobrist_lo_hi, uint64_t* out_lo_hi) {
  beam_v6::State128 c;
  std::memcpy(c.v, child128, 128);
  const beam_v6::Hash128 h =
      beam_v6::hash_state128_zobrist(c, reinterpret_cast<const beam_v6::Hash128*>(zobrist_lo_hi));
  out_lo_hi[0] = h.lo;
  out_lo_hi[1] = h.hi;
}
uint32_t ref_owner_from_hash128(uint64_t hi, uint64_t lo, uint32_t world) {
  return beam_v6::owner_from_hash128(hi, lo, world);
}
int ref_candidate_better(uint32_t score_a, uint64_t parent_a, uint32_t route_a, uint32_t score_b, uint64_t parent_b,
                         uint32_t route_b) {
  beam_v6::CandidateMeta a{}, b{};
  a.score_key = score_a; a.parent_idx = parent_a; a.route_packed = route_a;
  b.score_key = score_b; b.parent_idx = parent_b; b.route_packed = route_b;
  return beam_v6::candidate_better(a, b) ? 1 : 0;
}

// beam_types.hpp host helpers
uint32_t ref_q_to_score_key(float q) { return beam_v6::q_to_score_key_host(q); }
uint32_t ref_pack_route(uint32_t source_rank, uint32_t owner, uint32_t move) {
  return beam_v6::pack_route(static_cast<uint16_t>(source_rank), static_cast<uint8_t>(owner),
                             static_cast<uint8_t>(move));
}
uint64_t ref_pack_stream3_val(uint32_t score_key, uint32_t payload_id) {
  return beam_v6::pack_stream3_val(score_key, payload_id);
}
uint32_t ref_payload_id(uint32_t ring_slot, uint32_t parent_local, uint32_t move, uint32_t b_micro) {
  return beam_v6::payload_id(ring_slot, parent_local, static_cast<uint8_t>(move), b_micro);
}
// threshold_update keeps its "initialised" flag by reference: *initialised is read and written
uint32_t ref_threshold_update(uint32_t current, int* initialised, uint64_t total_survivors, uint64_t beam,
                              uint32_t new_threshold) {
  bool init = *initialised != 0;
  const uint32_t t = beam_v6::threshold_update(current, init, total_survivors, beam, new_threshold);
  *initialised = init ? 1 : 0;
  return t;
}

}  // extern "C"
