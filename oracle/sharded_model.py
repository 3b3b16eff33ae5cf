"""CPU model of the sharded selection protocol (TEST INFRASTRUCTURE).

Restates, with numpy and any torch.distributed backend (gloo on CPU), what the ranks of the CUDA engine do between
expansion and the next frontier: route candidates to their hash owner (all of them first, or band by band once the
band bounds are known from histograms counted where the candidates were generated), insert best-first bands into a
bounded per-rank table, and take the exact global top-K from all-reduced radix histograms.  It exists so that the
multi-rank logic (owner routing, band sizing from all-reduced statistics, identical thresholds on every rank, tie
resolution across ranks) is exercised without GPUs.  The reference's counterpart is the exchange + threshold logic
of enqueue_one_depth (beam_engine.cpp:1368-1463) and the v6 dispatcher's all-gathered threshold
(production_v6_dispatcher.py:159-192).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Tuple

import numpy as np

from . import beam_oracle as bo

RADIX_BITS = 11
BINS = 1 << RADIX_BITS
U64 = np.uint64
MAXKEY = (1 << 64) - 1


@dataclass
class Candidates:
    states: np.ndarray
    h: np.ndarray
    fp: np.ndarray
    score: np.ndarray
    payload: np.ndarray


def route(c: Candidates, world: int) -> List[Candidates]:
    """Bucket candidates by owner = hash mod world (beam_kernels.cu:582)."""
    own = bo.owner_rank(c.h, world)
    return [Candidates(c.states[own == r], c.h[own == r], c.fp[own == r], c.score[own == r], c.payload[own == r])
            for r in range(world)]


def _digit_bits(key_bits: int, done: int) -> int:
    return min(RADIX_BITS, key_bits - done)


def _range_end(prefix: int, key_bits: int, done: int) -> int:
    left = key_bits - done
    if left >= 64:
        return MAXKEY
    e = prefix + (1 << left)
    if e > MAXKEY or (key_bits < 64 and e >= (1 << key_bits)):
        return MAXKEY
    return e


def _hist(keys: np.ndarray, mask: np.ndarray, key_bits: int, prefix: int, done: int) -> np.ndarray:
    db = _digit_bits(key_bits, done)
    shift = key_bits - done - db
    k = keys[mask]
    if done:
        pshift = key_bits - done
        k = k[(k >> U64(pshift)) == U64(prefix >> pshift)]
    digit = ((k >> U64(shift)) & U64((1 << db) - 1)).astype(np.int64)
    return np.bincount(digit, minlength=BINS).astype(np.int64)


def _concat(parts: List[Candidates]) -> Candidates:
    return Candidates(*(np.concatenate([getattr(c, f) for c in parts]) for f in ("states", "h", "fp", "score", "payload")))


def sharded_select(local: Candidates, beam: int, world: int, pool_target: int, hash_capacity: int,
                   allreduce_sum: Callable[[np.ndarray], np.ndarray], allgather: Callable[[object], list],
                   hash_bits: int = 44, band_levels: int = 3, max_rounds: int = 8,
                   band_exchange: Callable[[List[Candidates]], List[Candidates]] = None):
    """Survivors on this rank.

    Routed-first form (``band_exchange`` None): ``local`` holds the candidates this rank OWNS (already exchanged);
    returns (indices into ``local``, stats).

    Band-routed form (``band_exchange`` given): ``local`` holds the candidates this rank GENERATED, whoever owns
    them.  The band histograms are counted over them - their sum over ranks is the same as over any other
    partition of the candidates - and after each band bound is known, only the candidates inside that band travel:
    ``band_exchange(parts)`` sends parts[r] to rank r and returns what the ranks sent here.  Returns
    (owned candidates received over all rounds, indices into them, stats).

    ``allreduce_sum`` sums an int64 array over ranks, ``allgather`` gathers a Python object from every rank.
    """
    key_bits = 20 + hash_bits
    keys = bo.order_key(local.score, local.h, hash_bits).astype(U64)
    gen_keys, generated = keys, local
    owned_parts: List[Candidates] = []
    owned_n = 0
    if band_exchange is not None:
        local = Candidates(local.states[:0], local.h[:0], local.fp[:0], local.score[:0], local.payload[:0])
        keys = keys[:0]
    table = {}  # (h, fp) -> (score<<32 | payload), local candidate index of the winner
    inserted = 0
    D = 0
    rho = (1, 1)
    rounds = 0
    stats = {"stalls": 0}
    for _ in range(max_rounds):
        counts = np.array(allgather((len(table), inserted)), dtype=np.int64)
        u_tot, u_max, i_tot = int(counts[:, 0].sum()), int(counts[:, 0].max()), int(counts[:, 1].sum())
        if u_tot >= beam or D == MAXKEY:
            break
        hard_cap = hash_capacity * 7 // 8
        hard = max(hard_cap - u_max, 0) * world
        hard -= hard // 16
        want = max(pool_target * world - u_tot, 0)
        num, den = (i_tot, u_tot) if (i_tot and u_tot) else rho
        n = min((want * num + den - 1) // den, hard)
        if n == 0:
            stats["stalls"] += 1
            break
        # radix descent on all-reduced histograms: largest E with count([D, E)) <= n
        prefix, done, remaining, E = 0, 0, n, None
        in_range = gen_keys >= U64(D)
        for level in range(band_levels):
            hist = allreduce_sum(_hist(gen_keys, in_range, key_bits, prefix, done))
            cum = np.cumsum(hist)
            cross = int(np.searchsorted(cum, remaining, side="right"))
            if cross >= BINS:
                E = _range_end(prefix, key_bits, done)
                break
            db = _digit_bits(key_bits, done)
            shift = key_bits - done - db
            remaining -= int(cum[cross - 1]) if cross else 0
            prefix |= cross << shift
            done += db
            if level == band_levels - 1 or done >= key_bits:
                E = max(prefix, D)
        if E <= D:
            stats["stalls"] += 1
            break
        if band_exchange is not None:
            sel = (gen_keys >= U64(D)) & (gen_keys < U64(E))
            part = Candidates(generated.states[sel], generated.h[sel], generated.fp[sel], generated.score[sel],
                              generated.payload[sel])
            got = _concat(band_exchange(route(part, world)))
            owned_parts.append(got)
            band = np.arange(owned_n, owned_n + got.h.shape[0])
            owned_n += got.h.shape[0]
            local = _concat(owned_parts)
            keys = bo.order_key(local.score, local.h, hash_bits).astype(U64)
        else:
            band = np.nonzero((keys >= U64(D)) & (keys < U64(E)))[0]
        for i in band:
            k = (int(local.h[i]), int(local.fp[i]))
            val = (int(local.score[i]) << 32) | int(local.payload[i])
            if k not in table or val < table[k][0]:
                table[k] = (val, int(i))
        inserted += band.size
        D = E
        rounds += 1
    stats["rounds"] = rounds
    # final cut over table entries
    win_idx = np.array([v[1] for v in table.values()], dtype=np.int64)
    wkeys = keys[win_idx] if win_idx.size else keys[:0]
    u_tot = int(allreduce_sum(np.array([win_idx.size], dtype=np.int64))[0])
    if u_tot <= beam:
        return (local, np.sort(win_idx), stats) if band_exchange is not None else (np.sort(win_idx), stats)
    prefix, done, remaining = 0, 0, beam
    T, tie_key, tie_need = MAXKEY, None, 0
    while True:
        hist = allreduce_sum(_hist(wkeys, np.ones(wkeys.shape, bool), key_bits, prefix, done))
        cum = np.cumsum(hist)
        cross = int(np.searchsorted(cum, remaining, side="left"))
        db = _digit_bits(key_bits, done)
        shift = key_bits - done - db
        remaining -= int(cum[cross - 1]) if cross else 0
        prefix |= cross << shift
        done += db
        if int(hist[cross]) == remaining:
            T = _range_end(prefix, key_bits, done)
            break
        if done >= key_bits:
            T, tie_key, tie_need = prefix, prefix, remaining
            break
    keep = win_idx[wkeys < U64(T)]
    if tie_need:
        mine = win_idx[wkeys == U64(tie_key)]
        records = [(int(local.h[i]), int(local.fp[i])) for i in mine]
        everyone = sorted(x for part in allgather(records) for x in part)
        cutoff = set(everyone[:tie_need])
        keep = np.concatenate([keep, np.array([i for i, r in zip(mine, records) if r in cutoff], dtype=np.int64)])
    return (local, np.sort(keep), stats) if band_exchange is not None else (np.sort(keep), stats)

