// Device/host helpers shared by the step kernels: the reference's hash arithmetic and the record packing.
#pragma once
#include <stdint.h>

#ifdef __CUDACC__
#define MGBS_HD __host__ __device__ __forceinline__
#else
#define MGBS_HD inline
#endif

namespace mgbs {

constexpr uint64_t kFnvOffset = 1469598103934665603ull;  // beam_kernels.cu:39
constexpr uint64_t kFnvPrime = 1099511628211ull;         // beam_kernels.cu:43
constexpr uint64_t kGolden = 0x9e3779b97f4a7c15ull;      // beam_kernels.cu:51
constexpr uint64_t kFpXor = 0xd6e8feb86659fd93ull;       // beam_kernels.cu:56

// murmur3 fmix64 (beam_kernels.cu:29-36)
MGBS_HD uint64_t mix64(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ull;
  x ^= x >> 33;
  return x;
}

// finaliser of hash_state_120 (beam_kernels.cu:45-47): values 0, 1, 2 are table sentinels and move up by 4
MGBS_HD uint64_t finish_hash(uint64_t h) {
  h = mix64(h);
  if (h <= 2ull) h += 4ull;
  return h;
}

// finaliser of fingerprint_state_120 (beam_kernels.cu:56-58)
MGBS_HD uint64_t finish_fingerprint(uint64_t f) {
  f = mix64(f ^ kFpXor);
  if (f == 0ull) f = 4ull;
  return f;
}

// 128-bit Zobrist hash mode (hash_state128_zobrist, beam_kernels_stream2.cu:28-38): the XOR over positions of a
// 128-bit table entry per (position, value).  Its low word takes the place of the 64-bit hash and its high word that
// of the fingerprint; both get the same sentinel remap as above because the dedup table uses 0 as "empty".
MGBS_HD uint64_t finish_zobrist_lo(uint64_t lo) { return lo <= 2ull ? lo + 4ull : lo; }
MGBS_HD uint64_t finish_zobrist_hi(uint64_t hi) { return hi == 0ull ? 4ull : hi; }

// destination rank of a candidate: hash mod world (beam_kernels.cu:582), or for the Zobrist mode
// (hi ^ lo * golden) mod world (owner_from_hash128, beam_kernels_stream3.cu:29-35)
MGBS_HD uint32_t owner_of(uint64_t h, uint64_t f, uint32_t world, int hash_mode) {
  if (hash_mode == MGBS_HASH_ZOBRIST128) return (uint32_t)((f ^ (h * kGolden)) % (uint64_t)world);
  return (uint32_t)(h % (uint64_t)world);
}

// back-pointer: parent row (23 bits) | source rank (4 bits) | move (5 bits); integer order = the duplicate
// tie-break order (parent_idx, source_rank, move) of candidate_better (beam_kernels_stream4.cu:25-33)
constexpr int kMoveBits = 5;
constexpr int kRankBits = 4;

MGBS_HD uint32_t pack_payload(uint32_t parent, uint32_t rank, uint32_t move) {
  return (parent << (kRankBits + kMoveBits)) | (rank << kMoveBits) | move;
}

MGBS_HD void unpack_payload(uint32_t p, uint32_t& parent, uint32_t& rank, uint32_t& move) {
  move = p & ((1u << kMoveBits) - 1u);
  rank = (p >> kMoveBits) & ((1u << kRankBits) - 1u);
  parent = p >> (kRankBits + kMoveBits);
}

// 64-bit selection key: score (at most 20 bits) above the top hash_bits bits of the hash
MGBS_HD uint64_t order_key(uint32_t score, uint64_t h, int hash_bits) {
  uint64_t k = score > 0xfffffu ? 0xfffffull : (uint64_t)score;
  return hash_bits ? ((k << hash_bits) | (h >> (64 - hash_bits))) : k;
}

}  // namespace mgbs
