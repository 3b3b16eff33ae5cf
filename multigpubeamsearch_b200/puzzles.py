"""Seeded synthetic puzzles: generator tables, solved states, scrambles and scorer weights.

The reference ships one puzzle as data files (state length 120, 24 moves, read by
data_loader.py:35-128).  The engine here takes the shape at run time, and the
workloads it is measured on are synthetic Cayley graphs of the same kind: a move
is a fixed permutation applied as a gather, ``child[i] = parent[table[m][i]]``
(data_loader.py:141-148, beam_kernels.cu:69-76).

Everything is derived from integer seeds so that the engine, the CPU oracle and the
benchmark see identical inputs.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import numpy as np


@dataclass(frozen=True)
class Puzzle:
    name: str
    state_len: int
    num_values: int
    generators: np.ndarray  # [G, n] uint8 gather tables
    solved: np.ndarray  # [n] uint8
    scramble_seed: int

    @property
    def fanout(self) -> int:
        return int(self.generators.shape[0])

    def action_table_bytes(self) -> bytes:
        """Row-major fanout x state_len table, as BeamEngine.set_action_permutation_table takes it."""
        return np.ascontiguousarray(self.generators, dtype=np.uint8).tobytes(order="C")

    def scramble(self, index: int, length: int) -> np.ndarray:
        """Scramble ``index``: ``length`` uniform random moves from the solved state (no inverse avoidance)."""
        rng = np.random.default_rng(self.scramble_seed + int(index))
        moves = rng.integers(0, self.fanout, size=int(length))
        s = self.solved.copy()
        for m in moves:
            s = s[self.generators[int(m)].astype(np.int64)]
        return s

    def scramble_moves(self, index: int, length: int) -> np.ndarray:
        rng = np.random.default_rng(self.scramble_seed + int(index))
        return rng.integers(0, self.fanout, size=int(length))


def _with_inverses(tables: List[np.ndarray]) -> np.ndarray:
    inv = [np.argsort(t) for t in tables]
    return np.stack(tables + inv, axis=0).astype(np.uint8)


def lrx(n: int = 16) -> Puzzle:
    """S_n under L (cyclic left shift), R (cyclic right shift), X (swap positions 0 and 1)."""
    i = np.arange(n)
    left = (i + 1) % n
    right = (i - 1) % n
    swap = i.copy()
    swap[0], swap[1] = 1, 0
    gens = np.stack([left, right, swap], axis=0).astype(np.uint8)
    return Puzzle(f"lrx{n}", n, n, gens, i.astype(np.uint8), scramble_seed=1000)


def random_cycles(state_len: int, num_values: int, base_generators: int, cycles: int, cycle_len: int,
                  gen_seed: int, scramble_seed: int, name: str) -> Puzzle:
    """Random generator set: each base generator is a product of disjoint cycles on distinct positions,
    followed by the inverses of all base generators.  solved[p] = p // (state_len / num_values)."""
    rng = np.random.default_rng(gen_seed)
    tables: List[np.ndarray] = []
    for _ in range(base_generators):
        pos = rng.permutation(state_len)[: cycles * cycle_len]
        tbl = np.arange(state_len)
        for c in range(cycles):
            cyc = pos[c * cycle_len:(c + 1) * cycle_len]
            for j in range(cycle_len):
                tbl[cyc[j]] = cyc[(j + 1) % cycle_len]
        tables.append(tbl)
    per_value = state_len // num_values
    solved = (np.arange(state_len) // per_value).astype(np.uint8)
    return Puzzle(name, state_len, num_values, _with_inverses(tables), solved, scramble_seed)


def puzzle54() -> Puzzle:
    """n = 54, values 0..5 (9 each), 12 generators: 6 products of five 4-cycles + inverses."""
    return random_cycles(54, 6, 6, 5, 4, gen_seed=54012, scramble_seed=2000, name="rand54")


def puzzle96() -> Puzzle:
    """n = 96, values 0..7 (12 each), 18 generators: 9 products of eight 3-cycles + inverses."""
    return random_cycles(96, 8, 9, 8, 3, gen_seed=96018, scramble_seed=5000, name="rand96")


def by_name(name: str) -> Puzzle:
    if name.startswith("lrx"):
        return lrx(int(name[3:] or 16))
    if name == "rand54":
        return puzzle54()
    if name == "rand96":
        return puzzle96()
    raise ValueError(f"unknown puzzle {name!r}")


def zobrist_table(state_len: int, num_values: int) -> np.ndarray:
    """[state_len, num_values, 2] uint64 Zobrist table {lo, hi} for the 128-bit hash mode: the corner of the
    reference's production table (production_v6_dispatcher.py:109-113, numpy default_rng(0xC0DEC0DE), shape
    (128, 128, 2)) that this puzzle indexes."""
    rng = np.random.default_rng(0xC0DEC0DE)
    z = rng.integers(0, np.iinfo(np.uint64).max, size=(128, 128, 2), dtype=np.uint64)
    return np.ascontiguousarray(z[:state_len, :num_values, :])


def mlp_weights(in_features: int, hidden: int = 1024, seed: int = 7000, model_idx: int = 0,
                std: float = 0.02) -> Dict[str, np.ndarray]:
    """Random-init value MLP in_features -> hidden -> hidden -> 1 (Gaussian std 0.02, zero biases), float32.

    Drawn with numpy's PCG64 so that no torch build detail enters the numbers."""
    rng = np.random.default_rng(seed + model_idx)
    return {
        "w1": (rng.standard_normal((hidden, in_features)) * std).astype(np.float32),
        "b1": np.zeros((hidden,), dtype=np.float32),
        "w2": (rng.standard_normal((hidden, hidden)) * std).astype(np.float32),
        "b2": np.zeros((hidden,), dtype=np.float32),
        "w3": (rng.standard_normal((hidden,)) * std).astype(np.float32),
        "b3": np.float32(0.0),
    }


def q_mlp_weights(in_features: int, fanout: int, hidden1: int = 1024, hidden2: int = 512, seed: int = 7500,
                  model_idx: int = 0, std: float = 0.02) -> Dict[str, np.ndarray]:
    """Random-init action-value MLP in_features -> hidden1 -> hidden2 -> fanout (Gaussian std 0.02, zero biases)."""
    rng = np.random.default_rng(seed + model_idx)
    return {
        "w1": (rng.standard_normal((hidden1, in_features)) * std).astype(np.float32),
        "b1": np.zeros((hidden1,), dtype=np.float32),
        "w2": (rng.standard_normal((hidden2, hidden1)) * std).astype(np.float32),
        "b2": np.zeros((hidden2,), dtype=np.float32),
        "w3": (rng.standard_normal((fanout, hidden2)) * std).astype(np.float32),
        "b3": np.zeros((fanout,), dtype=np.float32),
    }


def transformer_weights(tokens: int, vocab: int, d_model: int = 256, layers: int = 4, ffn: int = 1024,
                        seed: int = 8000, model_idx: int = 0, std: float = 0.02) -> Dict:
    """Random-init pre-LayerNorm encoder: Gaussian std 0.02 matrices and embeddings, zero biases, LayerNorm 1/0."""
    rng = np.random.default_rng(seed + model_idx)

    def g(*shape):
        return (rng.standard_normal(shape) * std).astype(np.float32)

    def z(*shape):
        return np.zeros(shape, dtype=np.float32)

    def ones(*shape):
        return np.ones(shape, dtype=np.float32)

    return {
        "tok_emb": g(vocab, d_model), "pos_emb": g(tokens, d_model),
        "layers": [{
            "ln1_g": ones(d_model), "ln1_b": z(d_model), "wqkv": g(3 * d_model, d_model), "bqkv": z(3 * d_model),
            "wo": g(d_model, d_model), "bo": z(d_model), "ln2_g": ones(d_model), "ln2_b": z(d_model),
            "w1": g(ffn, d_model), "b1": z(ffn), "w2": g(d_model, ffn), "b2": z(d_model),
        } for _ in range(layers)],
        "lnf_g": ones(d_model), "lnf_b": z(d_model), "w_head": g(d_model), "b_head": np.float32(0.0),
    }
