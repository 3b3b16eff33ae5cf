"""Host-side views of the engine's packed records."""

from __future__ import annotations

MOVE_BITS = 5
RANK_BITS = 4


def pack_payload(parent, rank, move):
    """Back-pointer word: parent row (23 bits) | source rank (4 bits) | move (5 bits); ints or numpy arrays."""
    import numpy as np
    if isinstance(parent, np.ndarray):
        p, r, m = (np.asarray(x, dtype=np.uint32) for x in (parent, rank, move))
        return (p << np.uint32(RANK_BITS + MOVE_BITS)) | (r << np.uint32(MOVE_BITS)) | m
    return ((int(parent) << (RANK_BITS + MOVE_BITS)) | (int(rank) << MOVE_BITS) | int(move)) & 0xFFFFFFFF


def unpack_payload(payload):
    """(parent, rank, move) of a back-pointer word; works on ints and numpy arrays."""
    move = payload & ((1 << MOVE_BITS) - 1)
    rank = (payload >> MOVE_BITS) & ((1 << RANK_BITS) - 1)
    parent = payload >> (RANK_BITS + MOVE_BITS)
    return parent, rank, move


def order_key(score: int, h: int, hash_bits: int = 24) -> int:
    """The 64-bit selection key of the engine: score above the top ``hash_bits`` bits of the 64-bit hash."""
    k = min(int(score), 0xFFFFF)
    return ((k << hash_bits) | (int(h) >> (64 - hash_bits))) if hash_bits else k
