"""CPU oracle for the per-depth beam-search step (TEST INFRASTRUCTURE, not product code).

This file restates, in numpy, the algorithm of the reference engine
(TryDotAtwo/MultiGPUBeamSearch) for one hot path: expand -> hash -> score ->
dedup -> threshold top-K -> (hash-owner placement) -> next frontier, plus the
depth loop around it.  Only tests, the smoke entry and the benchmark's
``cpu_baseline`` leg may import it; the CUDA product path never does.

Every function cites the reference file:line it follows.  Where the reference
fixes a shape at compile time (state length 120, fan-out 24) the restatement
takes the shape from its arguments; nothing else is generalised.

Parity pin (fixtures under tests/golden/, each with the script that made it):
``hash64`` against outputs of the reference's ``data_loader.hash_state_cpu``
(make_golden.py); ``mix64``, ``hash_state_120``, ``fingerprint_state_120``,
``tie16``, ``make_best_key``, the expansion, the Hamming score, the goal
tests, the v6 128-bit Zobrist hash and owner rule, ``candidate_better``,
``pack_route``, ``q_to_score_key`` and the monotone ``threshold_update``
against the reference's own scalar device and host functions compiled as host
C++ (oracle/Makefile, make_scalar_golden.py); the residual action-value
network, the batch-norm folding, ``MLPActionScorer`` and
``QuantizedActionScorer`` against the reference's Python functions
(make_residual_q_golden.py); the dedup/tie-break rules against the known
answers of the reference's stream3/stream4 smoke tests; the threshold rules
against the reference's ``histogram_threshold`` / ``threshold_update``
examples.  Unpinned: which set survives a whole depth (the reference's own
result depends on the arrival order of its atomics, so it has no single
answer) and the numerics of the value scorers (its weights blob is absent):
for those, parity is unpinned and tests use the deterministic rule stated
here, respectively a stated tolerance against a float32 evaluation.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

U64 = np.uint64
MASK64 = (1 << 64) - 1

# Sentinels of the open-addressing table (beam_engine_common.hpp:70-72, data_loader.py:25-27).
HASH_EMPTY = 0
HASH_BUSY = 1
HASH_TOMBSTONE = 2

FNV_OFFSET = 1469598103934665603  # beam_kernels.cu:39
FNV_PRIME = 1099511628211  # beam_kernels.cu:43
GOLDEN = 0x9E3779B97F4A7C15  # beam_kernels.cu:51
FP_XOR = 0xD6E8FEB86659FD93  # beam_kernels.cu:56

SCORE_MAX_Q = 300.0  # beam_types.hpp:22-27
SCORE_SCALE = 256
SCORE_BIN_COUNT = 76801  # production_v6_dispatcher.py:159-168 (76 800 + 1 bins)
UINT32_MAX = 0xFFFFFFFF

# Packing of the back-pointer carried by every candidate: parent row (23 bits),
# source rank (4 bits), move (5 bits).  Its integer order is the reference's
# duplicate tie-break order (parent_idx, source_rank, move)
# (beam_kernels_stream4.cu:25-33 with route = rank<<16 | owner<<8 | move).
MOVE_BITS = 5
RANK_BITS = 4
PARENT_BITS = 23


def _u64(x) -> np.ndarray:
    return np.asarray(x, dtype=U64)


def mix64(x: np.ndarray) -> np.ndarray:
    """murmur3 fmix64 (beam_kernels.cu:29-36, data_loader.py:182-189)."""
    x = _u64(x).copy()
    with np.errstate(over="ignore"):
        x ^= x >> U64(33)
        x *= U64(0xFF51AFD7ED558CCD)
        x ^= x >> U64(33)
        x *= U64(0xC4CEB9FE1A85EC53)
        x ^= x >> U64(33)
    return x


def hash64(states: np.ndarray) -> np.ndarray:
    """64-bit FNV-1a over the state bytes, fmix64 finaliser, sentinels {0,1,2} moved by +4.

    Follows hash_state_120 (beam_kernels.cu:38-48) and its CPU mirror
    data_loader.hash_state_cpu (data_loader.py:192-213); the byte count is the
    row length instead of the constant 120.
    """
    s = np.ascontiguousarray(states, dtype=np.uint8)
    if s.ndim == 1:
        s = s[None, :]
    h = np.full((s.shape[0],), FNV_OFFSET, dtype=U64)
    prime = U64(FNV_PRIME)
    with np.errstate(over="ignore"):
        for i in range(s.shape[1]):
            h ^= s[:, i].astype(U64)
            h *= prime
    h = mix64(h)
    with np.errstate(over="ignore"):
        h = np.where(h <= U64(HASH_TOMBSTONE), h + U64(4), h)
    return h


def fingerprint64(states: np.ndarray) -> np.ndarray:
    """Independent 64-bit fingerprint (boost-style combine + fmix64), 0 moved to 4.

    Follows fingerprint_state_120 (beam_kernels.cu:50-59).
    """
    s = np.ascontiguousarray(states, dtype=np.uint8)
    if s.ndim == 1:
        s = s[None, :]
    h = np.full((s.shape[0],), GOLDEN, dtype=U64)
    g = U64(GOLDEN)
    with np.errstate(over="ignore"):
        for i in range(s.shape[1]):
            h ^= s[:, i].astype(U64) + g + (h << U64(6)) + (h >> U64(2))
    h = mix64(h ^ U64(FP_XOR))
    h = np.where(h == U64(0), U64(4), h)
    return h


def zobrist_table(state_len: int, num_values: int) -> np.ndarray:
    """[state_len, num_values, 2] uint64 table {lo, hi}: the corner of the reference's production table
    (make_zobrist, production_v6_dispatcher.py:109-113: default_rng(0xC0DEC0DE), shape (128, 128, 2)) that a puzzle
    with this many positions and values indexes."""
    rng = np.random.default_rng(0xC0DEC0DE)
    z = rng.integers(0, np.iinfo(np.uint64).max, size=(128, 128, 2), dtype=np.uint64)
    return np.ascontiguousarray(z[:state_len, :num_values, :])


def hash128_zobrist(states: np.ndarray, table: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """(lo, hi) = XOR over positions of table[p, state[p]] (hash_state128_zobrist, beam_kernels_stream2.cu:28-38;
    CPU mirror tests/stream2_reference_smoke.py:41-48).  lo takes the role of hash64 and hi that of
    fingerprint64 in the engine, with the same remap of the dedup table's sentinel values (0, 1, 2 -> +4 for lo;
    0 -> 4 for hi)."""
    s = np.ascontiguousarray(states, dtype=np.uint8)
    if s.ndim == 1:
        s = s[None, :]
    lo = np.zeros((s.shape[0],), dtype=U64)
    hi = np.zeros((s.shape[0],), dtype=U64)
    for p in range(s.shape[1]):
        e = table[p][s[:, p].astype(np.int64)]
        lo ^= e[:, 0]
        hi ^= e[:, 1]
    lo = np.where(lo <= U64(HASH_TOMBSTONE), lo + U64(4), lo)
    hi = np.where(hi == U64(0), U64(4), hi)
    return lo, hi


def owner_from_hash128(hi: np.ndarray, lo: np.ndarray, world_size: int) -> np.ndarray:
    """(hi ^ lo * golden) mod world (owner_from_hash128, beam_kernels_stream3.cu:29-35;
    production_v6_dispatcher.py:116-119)."""
    with np.errstate(over="ignore"):
        mixed = _u64(hi) ^ (_u64(lo) * U64(GOLDEN))
    return (mixed % U64(world_size)).astype(np.int64)


def tie16(fp: np.ndarray) -> np.ndarray:
    """beam_kernels.cu:61-63."""
    fp = _u64(fp)
    return ((fp ^ (fp >> U64(32))) & U64(0xFFFF)).astype(np.uint32)


def make_best_key(score_q: np.ndarray, fp: np.ndarray) -> np.ndarray:
    """Legacy slot key: score in the high half, tie16(fingerprint) below (beam_kernels.cu:65-67)."""
    return (np.asarray(score_q, dtype=np.uint32) << np.uint32(16)) | tie16(fp)


def owner_rank(h: np.ndarray, world_size: int) -> np.ndarray:
    """Destination rank of a candidate: hash mod world (beam_kernels.cu:582, data_loader.py:216-219)."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    return (_u64(h) % U64(world_size)).astype(np.int64)


def expand(frontier: np.ndarray, generators: np.ndarray) -> np.ndarray:
    """All P*G children, parent-major (child index c = p*G + m): child[i] = parent[gen[m][i]].

    Follows apply_move_table (beam_kernels.cu:69-76) and data_loader.apply_action_cpu
    (data_loader.py:141-148): a gather of the parent through the generator; no
    inverse-move masking (beam_kernels.cu:528-580 expands every lane).
    """
    f = np.ascontiguousarray(frontier, dtype=np.uint8)
    g = np.asarray(generators, dtype=np.int64)
    p, n = f.shape
    out = f[:, g]  # [P, G, n]
    return np.ascontiguousarray(out.reshape(p * g.shape[0], n))


def hamming(states: np.ndarray, solved: np.ndarray) -> np.ndarray:
    """Number of positions that differ from the solved state (beam_kernels.cu:86-94)."""
    return (np.asarray(states, dtype=np.uint8) != np.asarray(solved, dtype=np.uint8)[None, :]).sum(axis=1).astype(np.uint32)


def legacy_hamming_q(ham: np.ndarray) -> np.ndarray:
    """Legacy u16 score of the built-in Hamming scorer, higher is better (beam_kernels.cu:133-143)."""
    ham = np.asarray(ham, dtype=np.int64)
    raw = np.maximum(65535 - ham * 512, 1)
    raw = np.where(ham == 0, 65535, raw)
    return raw.astype(np.uint16)


def q_to_score_key(q: np.ndarray, offset: float = 0.0) -> np.ndarray:
    """u32 key = uint32(clamp(q - offset, 0, 300) * 256 + 0.5), lower is better.

    Follows kernel_fullbeamnice_q_to_score_key_ring (beam_kernels.cu:341-344) and
    q_to_score_key_host (beam_types.hpp:103-106); float32 arithmetic as on the device.
    """
    x = np.asarray(q, dtype=np.float32) - np.float32(offset)
    x = np.minimum(np.maximum(x, np.float32(0.0)), np.float32(SCORE_MAX_Q))
    return (x * np.float32(SCORE_SCALE) + np.float32(0.5)).astype(np.uint32)


def pack_payload(parent: np.ndarray, rank: np.ndarray, move: np.ndarray) -> np.ndarray:
    parent = np.asarray(parent, dtype=np.uint32)
    rank = np.asarray(rank, dtype=np.uint32)
    move = np.asarray(move, dtype=np.uint32)
    return (parent << np.uint32(RANK_BITS + MOVE_BITS)) | (rank << np.uint32(MOVE_BITS)) | move


def unpack_payload(payload: np.ndarray) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    payload = np.asarray(payload, dtype=np.uint32)
    move = payload & np.uint32((1 << MOVE_BITS) - 1)
    rank = (payload >> np.uint32(MOVE_BITS)) & np.uint32((1 << RANK_BITS) - 1)
    parent = payload >> np.uint32(RANK_BITS + MOVE_BITS)
    return parent, rank, move


def order_key(score_key: np.ndarray, h: np.ndarray, hash_bits: int = 44) -> np.ndarray:
    """64-bit selection key: score in the top (64-hash_bits) bits, top hash bits below.

    The exact-K rule orders candidates by (score, hash, fingerprint); this key
    is that order truncated to 64 bits.  hash_bits = 0 gives the pure score order.
    """
    k = np.asarray(score_key, dtype=U64)
    if hash_bits == 0:
        return k
    return (k << U64(hash_bits)) | (_u64(h) >> U64(64 - hash_bits))


# ----------------------------------------------------------------------------------------------
# Threshold rules
# ----------------------------------------------------------------------------------------------

def v6_histogram_threshold(scores: Sequence[int], keep_count: int) -> int:
    """Smallest key whose cumulative count reaches keep_count, else UINT32_MAX.

    Follows histogram_threshold (production_v6_dispatcher.py:159-168).
    """
    scores = np.asarray(scores, dtype=np.int64)
    if scores.size == 0:
        return UINT32_MAX
    hist = np.bincount(scores, minlength=max(int(scores.max()) + 1, SCORE_BIN_COUNT))
    cum = np.cumsum(hist)
    idx = int(np.searchsorted(cum, keep_count, side="left"))
    return idx if idx < hist.size else UINT32_MAX


def v6_threshold_update(current: int, initialised: bool, total: int, beam: int, new: int) -> Tuple[int, bool]:
    """Monotone threshold: unset until enough survivors, then never relaxes.

    Follows threshold_update (beam_types.hpp:125-134) and allreduce_score_threshold
    (production_v6_dispatcher.py:171-192).
    """
    if (not initialised) and total < beam:
        return UINT32_MAX, False
    if total >= beam:
        return min(int(current), int(new)), True
    return int(current), bool(initialised)


def legacy_threshold(scores_hi: Sequence[int], beam: int, bins: int = 65536) -> Tuple[bool, int]:
    """Largest bin b with count(score >= b) >= beam, scanning from the top (higher is better).

    Follows kernel_compute_threshold (beam_kernels.cu:657-680): returns (valid, threshold).
    """
    hist = np.bincount(np.asarray(scores_hi, dtype=np.int64), minlength=bins)
    acc = 0
    for b in range(bins - 1, -1, -1):
        acc += int(hist[b])
        if acc >= beam:
            return True, b
    return False, 0


def balance_targets(keep: int, world: int) -> Tuple[np.ndarray, np.ndarray]:
    """Balanced placement of global survivor g: rank = min(g*W // K, W-1), local = g - ceil(K*rank / W).

    Follows production_v6_dispatcher.py:584-588.
    """
    g = np.arange(keep, dtype=np.int64)
    if keep == 0:
        return g, g
    rank = np.minimum(g * world // keep, world - 1)
    local = g - (keep * rank + world - 1) // world
    return rank, local


# ----------------------------------------------------------------------------------------------
# Dedup
# ----------------------------------------------------------------------------------------------

def dedup_by_key(keys: Sequence, sort_vals: Sequence) -> Dict:
    """Winner per key = minimum sort value.

    Follows the v6 rule: local stage keeps the min (score_key, payload_id)
    (beam_kernels_stream3.cu:97-105), owner stage the min (score_key, parent_idx,
    route) (beam_kernels_stream4.cu:25-33).
    """
    best: Dict = {}
    for k, v in zip(keys, sort_vals):
        if k not in best or v < best[k]:
            best[k] = v
    return best


@dataclass
class Unique:
    states: np.ndarray  # [U, n] uint8
    h: np.ndarray  # [U] uint64
    fp: np.ndarray  # [U] uint64
    score: np.ndarray  # [U] uint32 (lower is better)
    payload: np.ndarray  # [U] uint32 winner back-pointer
    hash_collisions: int  # distinct states sharing (hash, fingerprint)


def dedup_exact(children: np.ndarray, score: np.ndarray, payload: np.ndarray,
                h: Optional[np.ndarray] = None, fp: Optional[np.ndarray] = None) -> Unique:
    """Dedup by exact state bytes; winner = min (score, parent, rank, move).

    The engine identifies states by (hash64, fingerprint64) (beam_kernels.cu:485);
    the oracle uses the bytes and counts how many distinct states the engine
    would have merged.  Duplicates are only merged within one depth: the table
    is cleared at the start of every depth (beam_engine.cpp:1483).
    """
    c = np.ascontiguousarray(children, dtype=np.uint8)
    n = c.shape[1]
    if h is None:
        h = hash64(c)
    if fp is None:
        fp = fingerprint64(c)
    if c.shape[0] == 0:
        z = np.zeros((0,), dtype=np.uint32)
        return Unique(c, _u64([]), _u64([]), z, z, 0)
    rows = c.view(np.dtype((np.void, n))).ravel()
    _, inverse = np.unique(rows, return_inverse=True)
    inverse = inverse.ravel()
    val = (np.asarray(score, dtype=U64) << U64(32)) | np.asarray(payload, dtype=U64)
    order = np.lexsort((val, inverse))
    first = np.ones(order.size, dtype=bool)
    first[1:] = inverse[order][1:] != inverse[order][:-1]
    win = order[first]
    pair = np.stack([h[win], fp[win]], axis=1)
    distinct_pairs = np.unique(pair, axis=0).shape[0]
    return Unique(c[win], h[win], fp[win], np.asarray(score, dtype=np.uint32)[win],
                  np.asarray(payload, dtype=np.uint32)[win], int(win.size - distinct_pairs))


# ----------------------------------------------------------------------------------------------
# Selection
# ----------------------------------------------------------------------------------------------

def select(u: Unique, beam: int, mode: str = "exact_k") -> np.ndarray:
    """Indices (into the unique set) that survive.

    exact_k       sort by (score, hash, fingerprint), keep the first min(beam, U).
    v6_inclusive  T = smallest key with cumulative count >= beam; keep score <= T, ties kept
                  (production_v6_dispatcher.py:159-192; beam_kernels_stream4.cu:35-54).
    legacy_strict in the legacy orientation (q = 65535 - score, higher is better):
                  T = largest bin with count(q >= T) >= beam, prune q <= T
                  (beam_kernels.cu:657-680, 700); with fewer than beam candidates nothing is pruned.
    For identical scores: legacy_strict is a subset of exact_k, which is a subset of v6_inclusive.
    """
    n = u.score.size
    if mode == "exact_k":
        order = np.lexsort((u.fp, u.h, u.score))
        return np.sort(order[: min(beam, n)])
    if mode == "v6_inclusive":
        if n < beam:
            return np.arange(n)
        t = v6_histogram_threshold(u.score, beam)
        return np.nonzero(u.score <= t)[0]
    if mode == "legacy_strict":
        q = 65535 - np.minimum(u.score.astype(np.int64), 65535)
        valid, t = legacy_threshold(q, beam)
        if not valid:
            return np.arange(n)
        return np.nonzero(q > t)[0]
    raise ValueError(f"unknown select mode {mode!r}")


# ----------------------------------------------------------------------------------------------
# Scorers
# ----------------------------------------------------------------------------------------------

def one_hot(states: np.ndarray, num_values: int) -> np.ndarray:
    """One-hot with column index pos*V + value, float32."""
    s = np.asarray(states, dtype=np.int64)
    c, n = s.shape
    x = np.zeros((c, n * num_values), dtype=np.float32)
    x[np.arange(c)[:, None], np.arange(n)[None, :] * num_values + s] = 1.0
    return x


def mlp_forward(states: np.ndarray, weights: Sequence[Dict[str, np.ndarray]], num_values: int) -> np.ndarray:
    """float32 value MLP on one-hot states; an ensemble (list of weight dicts) is averaged.

    Layer shapes as in scorers.py:21-36 (Linear stacks), ReLU between layers,
    scalar output per state.  w1 [H1, n*V], w2 [H2, H1], w3 [H2].
    """
    x = one_hot(states, num_values)
    out = np.zeros((x.shape[0],), dtype=np.float32)
    for w in weights:
        h1 = np.maximum(x @ w["w1"].T.astype(np.float32) + w["b1"].astype(np.float32), 0.0)
        h2 = np.maximum(h1 @ w["w2"].T.astype(np.float32) + w["b2"].astype(np.float32), 0.0)
        out += (h2 @ w["w3"].astype(np.float32) + np.float32(w["b3"])).astype(np.float32)
    return (out / np.float32(len(weights))).astype(np.float32)


def mlp_action_values(parents: np.ndarray, weights: Sequence[Dict[str, np.ndarray]], num_values: int) -> np.ndarray:
    """float32 action-value MLP on one-hot PARENT states: [P, n] -> [P, fanout], ensemble members averaged.

    The reference's scorer contract (scorers.py:1-57: one forward pass per parent, one value per move;
    FullBeamNiceStaticBackend::forward, beam_engine.cpp:621-667: embedding + ReLU, hidden layers with ReLU, output
    layer of width fanout).  w1 [H1, n*V], w2 [H2, H1], w3 [fanout, H2], b3 [fanout].  Candidate p*fanout + m takes
    out[p, m].
    """
    x = one_hot(parents, num_values)
    out = None
    for w in weights:
        h1 = np.maximum(x @ w["w1"].T.astype(np.float32) + w["b1"].astype(np.float32), 0.0)
        h2 = np.maximum(h1 @ w["w2"].T.astype(np.float32) + w["b2"].astype(np.float32), 0.0)
        q = (h2 @ w["w3"].T.astype(np.float32) + w["b3"].astype(np.float32)).astype(np.float32)
        out = q if out is None else out + q
    return (out / np.float32(len(weights))).astype(np.float32)


def fold_bn_linear(weight: np.ndarray, bias: np.ndarray, bn_weight: np.ndarray, bn_bias: np.ndarray,
                   running_mean: np.ndarray, running_var: np.ndarray, eps: float = 1e-5) -> Tuple[np.ndarray, np.ndarray]:
    """Batch norm (inference form) folded into the linear layer before it: y = bn(x W^T + b) = x W'^T + b'.

    Follows _fold_bn_linear (scripts/static_fullbeamnice_inference.py:59-71): scale = gamma / sqrt(var + eps),
    W' = W * scale per output row, b' = (b - mean) * scale + beta; float32.
    """
    scale = (bn_weight.astype(np.float32) / np.sqrt(running_var.astype(np.float32) + np.float32(eps))).astype(np.float32)
    w = (weight.astype(np.float32) * scale[:, None]).astype(np.float32)
    b = ((bias.astype(np.float32) - running_mean.astype(np.float32)) * scale + bn_bias.astype(np.float32)).astype(np.float32)
    return w, b


def residual_q_forward(states: np.ndarray, w: Dict[str, np.ndarray]) -> np.ndarray:
    """float32 forward pass of the reference's static action-value network: [P, n] uint8 -> [P, outputs].

    Follows static_forward_q (scripts/static_fullbeamnice_inference.py:146-171) and
    FullBeamNiceStaticBackend::forward (beam_engine.cpp:621-667): the first layer is an embedding sum
    x[h] = relu(embed_bias[h] + sum_pos embed_w_t[pos * num_classes + state[pos]][h]) over state_size positions
    (rows shorter than state_size are padded with value 0), then relu(x @ hidden_w_t + hidden_bias), then the
    residual blocks x = relu(relu(x @ fc1 + b1) @ fc2 + b2 + x), then x @ out_w_t + out_bias.  Weight matrices are
    stored transposed ([in, out]) as in the reference's dictionary.  The number of residual blocks is the number of
    res{i}_fc1_w_t keys (two in the reference).
    """
    s = np.asarray(states, dtype=np.int64)
    size, classes = int(w["state_size"]), int(w["num_classes"])
    if s.shape[1] < size:
        s = np.concatenate([s, np.zeros((s.shape[0], size - s.shape[1]), dtype=np.int64)], axis=1)
    tokens = s + (np.arange(size, dtype=np.int64) * classes)[None, :]
    table = np.asarray(w["embed_w_t"], dtype=np.float32)
    x = table[tokens.reshape(-1)].reshape(s.shape[0], size, -1).sum(axis=1, dtype=np.float32)
    x = np.maximum(x + np.asarray(w["embed_bias"], dtype=np.float32), 0.0)
    x = np.maximum(x @ np.asarray(w["hidden_w_t"], dtype=np.float32) + np.asarray(w["hidden_bias"], dtype=np.float32), 0.0)
    block = 0
    while f"res{block}_fc1_w_t" in w:
        r = x
        x = np.maximum(x @ np.asarray(w[f"res{block}_fc1_w_t"], np.float32) + np.asarray(w[f"res{block}_fc1_bias"], np.float32), 0.0)
        x = np.maximum(x @ np.asarray(w[f"res{block}_fc2_w_t"], np.float32) + np.asarray(w[f"res{block}_fc2_bias"], np.float32) + r, 0.0)
        block += 1
    return (x @ np.asarray(w["out_w_t"], np.float32) + np.asarray(w["out_bias"], np.float32)).astype(np.float32)


def residual_q_scores_u16(q: np.ndarray, action_perm: np.ndarray, score_scale: float = 1024.0,
                          score_bias: float = 65535.0) -> np.ndarray:
    """Legacy int16-wrapped scores of static_forward_scores (scripts/static_fullbeamnice_inference.py:174-178):
    columns reordered by action_perm, clamp(round(score_bias - q * score_scale), 0, 65535), then viewed as int16."""
    qc = np.asarray(q, dtype=np.float32)[:, np.asarray(action_perm, dtype=np.int64)]
    sc = np.clip(np.rint(np.float32(score_bias) - qc * np.float32(score_scale)), 0.0, 65535.0).astype(np.int32)
    return np.where(sc >= 32768, sc - 65536, sc).astype(np.int16)


def action_scorer_forward(states: np.ndarray, layers: Sequence[Tuple[np.ndarray, np.ndarray]],
                          value_scale: float = 119.0) -> np.ndarray:
    """float32 forward pass of the reference's MLPActionScorer (scorers.py:21-36): bytes / value_scale, then
    Linear + exact (erf) GELU per hidden layer and a last Linear.  ``layers`` = [(W [out, in], b), ...]."""
    from math import erf
    x = np.asarray(states, dtype=np.float32) / np.float32(value_scale)
    verf = np.vectorize(erf, otypes=[np.float64])
    for i, (wm, bv) in enumerate(layers):
        x = (x @ np.asarray(wm, np.float32).T + np.asarray(bv, np.float32)).astype(np.float32)
        if i + 1 < len(layers):
            x = (0.5 * x.astype(np.float64) * (1.0 + verf(x.astype(np.float64) / np.sqrt(2.0)))).astype(np.float32)
    return x


def quantized_action_scores(y: np.ndarray, score_mode: str = "sigmoid_u16") -> np.ndarray:
    """16-bit scores of QuantizedActionScorer (scorers.py:38-53) as unsigned values 0..65535, larger is better
    (the reference returns the same bits as int16)."""
    y = np.asarray(y, dtype=np.float32)
    if score_mode == "sigmoid_u16":
        y = (np.float32(1.0) / (np.float32(1.0) + np.exp(-y))).astype(np.float32) * np.float32(65535.0)
    elif score_mode != "float_u16":
        raise ValueError("unsupported score_mode")
    return np.clip(np.rint(y), 0.0, 65535.0).astype(np.uint32)


Scorer = Callable[[np.ndarray], np.ndarray]  # children [C, n] -> uint32 keys (lower is better)


def hamming_scorer(solved: np.ndarray) -> Scorer:
    return lambda children: hamming(children, solved)


# ----------------------------------------------------------------------------------------------
# Depth step and search
# ----------------------------------------------------------------------------------------------

@dataclass
class StepResult:
    states: np.ndarray  # [K, n] next frontier (sorted by (score, hash, fp))
    score: np.ndarray  # [K]
    h: np.ndarray
    fp: np.ndarray
    payload: np.ndarray  # winner back-pointer (parent, rank, move) packed
    candidates: int  # P*G generated this depth
    unique: int
    found_child: bool  # some generated child equals the solved state (beam_kernels.cu:455-460)
    found_payloads: np.ndarray  # back-pointers of all generated children that are solved
    hash_collisions: int
    threshold: int = UINT32_MAX


def depth_step(frontiers: Sequence[np.ndarray], generators: np.ndarray, solved: np.ndarray, scorer: Scorer,
               beam: int, mode: str = "exact_k",
               score_override: Optional[Sequence[np.ndarray]] = None,
               hasher: Optional[Callable[[np.ndarray], Tuple[np.ndarray, np.ndarray]]] = None) -> StepResult:
    """One depth over a frontier held by W ranks (frontiers[r] = rows on rank r; W = 1 for one GPU).

    Steps 1-4 of the reference step: expand every parent by every generator,
    hash/fingerprint/score every child, test every child for the goal
    (beam_kernels.cu:455-460, beam_kernels_stream2.cu:84-100), merge duplicates
    (winner = min (score, parent, rank, move)), select globally.
    The owner partition (hash mod W) does not change the surviving set, so it
    is applied by the caller when it needs per-rank placement.
    score_override[r] replaces the scorer output for rank r's candidates (used
    to feed device-computed neural scores into the selection logic).
    """
    gens = np.asarray(generators, dtype=np.int64)
    g = gens.shape[0]
    all_c, all_k, all_p = [], [], []
    for r, f in enumerate(frontiers):
        f = np.ascontiguousarray(f, dtype=np.uint8)
        if f.shape[0] == 0:
            continue
        c = expand(f, gens)
        k = scorer(c) if score_override is None else np.asarray(score_override[r], dtype=np.uint32)
        pidx = np.repeat(np.arange(f.shape[0], dtype=np.uint32), g)
        mv = np.tile(np.arange(g, dtype=np.uint32), f.shape[0])
        all_c.append(c)
        all_k.append(np.asarray(k, dtype=np.uint32))
        all_p.append(pack_payload(pidx, np.full_like(pidx, r), mv))
    n = np.asarray(solved).shape[0]
    if not all_c:
        z32 = np.zeros((0,), dtype=np.uint32)
        return StepResult(np.zeros((0, n), np.uint8), z32, _u64([]), _u64([]), z32, 0, 0, False, z32, 0)
    c = np.concatenate(all_c)
    k = np.concatenate(all_k)
    p = np.concatenate(all_p)
    is_goal = (c == np.asarray(solved, dtype=np.uint8)[None, :]).all(axis=1)
    # hasher: children -> (hash, fingerprint); default hash64 / fingerprint64, or the Zobrist pair.  The hash only
    # decides the order among equal scores (and the owner), never which states are duplicates of each other.
    hh, ff = hasher(c) if hasher is not None else (None, None)
    u = dedup_exact(c, k, p, hh, ff)
    keep = select(u, beam, mode)
    order = keep[np.lexsort((u.fp[keep], u.h[keep], u.score[keep]))]
    thr = int(u.score[order].max()) if order.size else UINT32_MAX
    return StepResult(u.states[order], u.score[order], u.h[order], u.fp[order], u.payload[order],
                      int(c.shape[0]), int(u.score.size), bool(is_goal.any()), p[is_goal], u.hash_collisions, thr)


def place_by_owner(res: StepResult, world: int) -> List[np.ndarray]:
    """Owner-resident placement: survivor rows live on rank hash mod W (beam_kernels.cu:582)."""
    own = owner_rank(res.h, world)
    return [res.states[own == r] for r in range(world)]


@dataclass
class SearchResult:
    found: bool
    depth: int  # depth at which the solved state is in the frontier (0 = start state solved)
    frontier_sizes: List[int] = field(default_factory=list)
    candidates: List[int] = field(default_factory=list)
    frontiers: List[np.ndarray] = field(default_factory=list)  # per depth, sorted rows (if keep_frontiers)
    path: Optional[List[int]] = None  # moves from the start state to the solved state
    hash_collisions: int = 0


def sorted_rows(states: np.ndarray) -> np.ndarray:
    """Rows in lexicographic byte order: the canonical form for set comparison."""
    s = np.ascontiguousarray(states, dtype=np.uint8)
    if s.shape[0] == 0:
        return s
    keys = tuple(s[:, i] for i in range(s.shape[1] - 1, -1, -1))
    return s[np.lexsort(keys)]


def search(start: np.ndarray, generators: np.ndarray, solved: np.ndarray, scorer: Scorer, beam: int,
           max_depth: int, mode: str = "exact_k", world: int = 1, keep_frontiers: bool = False) -> SearchResult:
    """Depth loop: stop when found, when depth == max_depth, or when the frontier is empty.

    Follows BeamEngine::search (beam_engine.cpp:1147-1171): before each step the
    frontier is tested for the goal (kernel_check_current_solved,
    beam_kernels.cu:857-875); a goal hit among generated children is reported
    at the following depth.  With world > 1 the frontier is placed on ranks by
    hash owner and every rank expands its own rows; the surviving set does not
    depend on world.  Back-pointers are kept per depth so the move sequence can
    be rebuilt (history walk-back, beam_engine.cpp:1200-1219).
    """
    solved = np.asarray(solved, dtype=np.uint8)
    start = np.asarray(start, dtype=np.uint8)[None, :]
    fronts = [start if owner_rank(hash64(start), world)[0] == r else start[:0] for r in range(world)]
    res = SearchResult(False, 0)
    payloads: List[List[np.ndarray]] = []  # payloads[d][r][i]: back-pointer of row i on rank r of the depth d+1 frontier

    def walk_back(depth: int, r: int, i: int) -> List[int]:
        moves: List[int] = []
        for d in range(depth, 0, -1):
            pp, pr, pm = unpack_payload(np.asarray([payloads[d - 1][r][i]]))
            moves.append(int(pm[0]))
            r, i = int(pr[0]), int(pp[0])
        return moves[::-1]

    for depth in range(max_depth + 1):
        allrows = np.concatenate(fronts)
        res.frontier_sizes.append(int(allrows.shape[0]))
        if keep_frontiers:
            res.frontiers.append(sorted_rows(allrows))
        if depth == 0 and (allrows == solved[None, :]).all(axis=1).any():
            res.found, res.depth, res.path = True, 0, []
            return res
        if depth == max_depth or allrows.shape[0] == 0:
            res.depth = depth
            return res
        step = depth_step(fronts, generators, solved, scorer, beam, mode)
        res.candidates.append(step.candidates)
        res.hash_collisions += step.hash_collisions
        if step.found_child:
            # goal test on every generated child, whether or not it survives selection
            pp, pr, pm = unpack_payload(np.asarray([step.found_payloads.min()]))
            res.found, res.depth = True, depth + 1
            res.path = walk_back(depth, int(pr[0]), int(pp[0])) + [int(pm[0])]
            return res
        own = owner_rank(step.h, world)
        fronts = [step.states[own == r] for r in range(world)]
        payloads.append([step.payload[own == r] for r in range(world)])
    return res


def replay(start: np.ndarray, generators: np.ndarray, moves: Sequence[int]) -> np.ndarray:
    """Apply a move sequence to a state (data_loader.apply_actions_cpu, data_loader.py:151-155)."""
    s = np.asarray(start, dtype=np.uint8)
    g = np.asarray(generators, dtype=np.int64)
    for m in moves:
        s = s[g[int(m)]]
    return s


# ----------------------------------------------------------------------------------------------
# Transformer value scorer (float32 evaluation used by tolerance tests)
# ----------------------------------------------------------------------------------------------

def _layer_norm(x: np.ndarray, g: np.ndarray, b: np.ndarray, eps: float = 1e-5) -> np.ndarray:
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return ((x - mu) / np.sqrt(var + np.float32(eps)) * g + b).astype(np.float32)


def _gelu(x: np.ndarray) -> np.ndarray:
    from scipy.special import erf
    return (0.5 * x * (1.0 + erf(x / np.sqrt(2.0)))).astype(np.float32)


def round_e4m3(x: np.ndarray) -> np.ndarray:
    """Round to the nearest e4m3 value (4 exponent bits, 3 mantissa bits, bias 7: largest finite 448, smallest
    normal 2^-6, subnormal step 2^-9), ties to even, saturating."""
    a = np.minimum(np.abs(np.asarray(x, dtype=np.float64)), 448.0)
    e = np.maximum(np.floor(np.log2(np.maximum(a, 2.0 ** -30))), -6.0)
    step = np.exp2(e - 3.0)
    return (np.sign(x) * np.minimum(np.rint(a / step) * step, 448.0)).astype(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bfloat16 value (ties to even), returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) & np.uint64(0xFFFF0000)
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(x))


E2M1_MIDPOINTS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def round_e2m1(x: np.ndarray) -> np.ndarray:
    """Round to the nearest E2M1 value (magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6), ties to the even code, saturating."""
    a = np.abs(np.asarray(x, dtype=np.float64))
    code = np.searchsorted(E2M1_MIDPOINTS, a, side="left")  # midpoints strictly below |x|
    tie = (code < 7) & (a == E2M1_MIDPOINTS[np.minimum(code, 6)])
    code = np.where(tie & (code % 2 == 1), code + 1, code)
    return (np.sign(x) * E2M1_VALUES[code]).astype(np.float32)


def quantize_nvfp4(x: np.ndarray, tensor_scale: float) -> np.ndarray:
    """NVFP4 model of a [rows, K] matrix, K a multiple of 16: per block of 16 consecutive K elements one E4M3 factor
    e4m3(blockmax / 6 / tensor_scale), elements E2M1(x / (factor * tensor_scale)); returns the de-quantised matrix."""
    x = np.asarray(x, dtype=np.float32)
    r, k = x.shape
    b = x.reshape(r, k // 16, 16)
    amax = np.abs(b).max(axis=2)
    sf = round_e4m3(amax / np.float32(6.0) / np.float32(tensor_scale))
    step = (sf * np.float32(tensor_scale))[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(step > 0, round_e2m1(np.where(step > 0, b / np.where(step > 0, step, 1.0), 0.0)), 0.0)
    return (q * step).reshape(r, k).astype(np.float32)


def nvfp4_tensor_scale(max_abs: float) -> float:
    """Tensor scale that maps the largest block factor to the top of the E4M3 range: max|x| / (6 * 448)."""
    return float(max(max_abs, 1e-30) / (6.0 * 448.0))


def mlp_forward_nvfp4_model(states: np.ndarray, weights: Sequence[Dict[str, np.ndarray]], num_values: int,
                            act_bound: float, via_e4m3: bool = False) -> np.ndarray:
    """float32 evaluation of the value MLP on the operands the NVFP4 scorer uses: first-layer weights in e4m3 with one
    scale per output channel, then activations and second-layer weights in NVFP4.  via_e4m3: the activations pass
    through e4m3 storage (per-tensor scale act_bound / 448) before they are re-quantised, as the scorer's two-pass
    form does.  Mean over ensemble members."""
    x = one_hot(states, num_values)
    out = np.zeros((x.shape[0],), dtype=np.float64)
    for w in weights:
        w1q, s1 = _e4m3_rows(np.asarray(w["w1"], np.float32))
        h1 = np.maximum(x @ (w1q * s1[:, None]).T + w["b1"][None, :], 0.0).astype(np.float32)
        if via_e4m3:
            h1 = _e4m3_tensor(h1, act_bound)
        h1q = quantize_nvfp4(h1, nvfp4_tensor_scale(act_bound))
        w2 = np.asarray(w["w2"], np.float32)
        w2q = quantize_nvfp4(w2, nvfp4_tensor_scale(float(np.abs(w2).max())))
        h2 = np.maximum(h1q @ w2q.T + w["b2"][None, :], 0.0)
        out += h2.astype(np.float64) @ np.asarray(w["w3"], np.float64) + float(w["b3"])
    return (out / len(weights)).astype(np.float32)


def _e4m3_rows(w: np.ndarray):
    """Per-row e4m3 quantisation of a matrix: (rounded w / scale, scale[rows])."""
    scale = (np.maximum(np.abs(w).max(axis=1), 1e-30) / 448.0).astype(np.float32)
    return round_e4m3(w / scale[:, None]), scale


def _e4m3_tensor(x: np.ndarray, bound: float) -> np.ndarray:
    """Per-tensor e4m3 quantisation with scale bound / 448, returned de-scaled."""
    scale = np.float32(bound / 448.0)
    return round_e4m3(x * np.float32(1.0 / scale)) * scale


def transformer_forward(states: np.ndarray, encoders: Sequence[Dict], heads: int = 8, e4m3: bool = False) -> np.ndarray:
    """float32 pre-LayerNorm transformer encoder ensemble on token states; mean over members.

    One token per state position (vocabulary = value range) plus a learned position embedding; each layer is
    x += MHA(LN1(x)); x += W2 gelu(W1 LN2(x)) (the layout of nn.TransformerEncoderLayer(norm_first=True,
    activation="gelu")); a final LayerNorm, mean pooling over tokens and a linear head give one scalar per state.

    ``e4m3=True`` models 8-bit GEMM operands: the four matrices of a layer rounded to e4m3 with one scale per
    output row, and the three GEMM inputs (LayerNorm output, attention output, GELU output) rounded to e4m3 with
    one scale per tensor taken from a bound that holds for every input: a LayerNorm row has L2 norm sqrt(d)
    before its gain, so |row . w + b| <= (sqrt(d) max|gain| + |shift|_2) |w|_2 + |b|.  This mode also rounds q, k, v
    and the unnormalised softmax weights to bfloat16, as the device stores them, because a rounded-operand model
    is discontinuous: a 1e-3 difference upstream moves some e4m3 roundings by a whole step.
    """
    s = np.asarray(states, dtype=np.int64)
    c, t = s.shape
    out = np.zeros((c,), dtype=np.float32)
    for w in encoders:
        d = w["tok_emb"].shape[1]
        hd = d // heads
        x = (w["tok_emb"][s] + w["pos_emb"][None, :t, :]).astype(np.float32)  # [C, T, d]
        for L in w["layers"]:
            mats = {k: L[k].astype(np.float32) for k in ("wqkv", "wo", "w1", "w2")}
            if e4m3:
                n1 = np.sqrt(d) * np.abs(L["ln1_g"]).max() + np.linalg.norm(L["ln1_b"])
                n2 = np.sqrt(d) * np.abs(L["ln2_g"]).max() + np.linalg.norm(L["ln2_b"])
                b_att = (np.linalg.norm(L["wqkv"][2 * d:].astype(np.float64), axis=1) * n1 + np.abs(L["bqkv"][2 * d:])).max()
                b_hid = (np.linalg.norm(L["w1"].astype(np.float64), axis=1) * n2 + np.abs(L["b1"])).max()
                for k in mats:
                    qw, sc = _e4m3_rows(mats[k])
                    mats[k] = qw * sc[:, None]
            y = _layer_norm(x, L["ln1_g"], L["ln1_b"])
            if e4m3:
                y = _e4m3_tensor(y, n1)
            qkv = y @ mats["wqkv"].T + L["bqkv"]
            if e4m3:
                qkv = round_bf16(qkv.astype(np.float32))
            q, k, v = (qkv[..., i * d:(i + 1) * d].reshape(c, t, heads, hd).transpose(0, 2, 1, 3) for i in range(3))
            att = (q @ k.transpose(0, 1, 3, 2)) / np.float32(np.sqrt(hd))
            att = att - att.max(axis=-1, keepdims=True)
            att = np.exp(att)
            if e4m3:
                o = (round_bf16(att.astype(np.float32)) @ v) / att.sum(axis=-1, keepdims=True)
                o = _e4m3_tensor(o.transpose(0, 2, 1, 3).reshape(c, t, d), b_att)
            else:
                att = att / att.sum(axis=-1, keepdims=True)
                o = (att @ v).transpose(0, 2, 1, 3).reshape(c, t, d)
            x = (x + o @ mats["wo"].T + L["bo"]).astype(np.float32)
            y = _layer_norm(x, L["ln2_g"], L["ln2_b"])
            if e4m3:
                y = _e4m3_tensor(y, n2)
            hdn = _gelu(y @ mats["w1"].T + L["b1"])
            if e4m3:
                hdn = _e4m3_tensor(hdn, b_hid)
            x = (x + hdn @ mats["w2"].T + L["b2"]).astype(np.float32)
        y = _layer_norm(x, w["lnf_g"], w["lnf_b"]).mean(axis=1)
        out += (y @ w["w_head"] + np.float32(w["b_head"])).astype(np.float32)
    return (out / np.float32(len(encoders))).astype(np.float32)
