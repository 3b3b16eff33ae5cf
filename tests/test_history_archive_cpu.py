"""CPU test of the history archive: layers, checkpoint files, resume, path walk-back.

The archive is driven by a CPU model of the engine (the numpy oracle's depth step behind the five members the archive
uses), with a history ring of ONE layer, so every walk-back has to come from the archive."""

import json

import numpy as np
import pytest

from oracle import beam_oracle as bo
from multigpubeamsearch_b200 import puzzles
from multigpubeamsearch_b200.history_archive import CPUHistoryArchive, MANIFEST
from multigpubeamsearch_b200.solver import replay


class OracleEngine:
    def __init__(self, pz, beam, **extra):
        self.pz, self.beam = pz, beam
        self.cfg = {"rank": 0, "world_size": 1, "global_beam_width": beam, "state_len": pz.state_len,
                    "state_size_bytes": pz.state_len, "fanout": pz.fanout, "beta": 1.2, "gamma": 1.05,
                    "select_mode": "exact_k", "hash_bits": 24, "inference_backend": "dummy", **extra}
        self.rows = np.zeros((0, pz.state_len), np.uint8)
        self.depth = 0
        self.last_layer = np.zeros((0,), np.uint32)

    def reset_search(self, start):
        self.rows, self.depth = np.asarray(start, np.uint8)[None, :].copy(), 0

    def step(self):
        res = bo.depth_step([self.rows], self.pz.generators, self.pz.solved, bo.hamming_scorer(self.pz.solved), self.beam)
        self.rows, self.last_layer, self.depth = res.states, res.payload.astype(np.uint32), self.depth + 1

    def status(self):
        return {"depth": self.depth, "current_size": self.rows.shape[0]}

    def frontier(self):
        return self.rows.copy()

    def history_layer(self, depth, count):
        assert depth == self.depth - 1, "the model keeps one layer only"
        return self.last_layer[:count].copy()

    def load_frontier(self, rows, depth=0):
        self.rows, self.depth = np.asarray(rows, np.uint8).copy(), int(depth)


def _run(engine, archive, upto):
    while engine.depth < upto:
        engine.step()
        archive.after_step(engine.depth, engine.status()["current_size"])


def test_archive_checkpoint_resume_and_walk_back(tmp_path):
    pz = puzzles.puzzle54()
    start = pz.scramble(3, 30)
    # uninterrupted run
    e0 = OracleEngine(pz, 64)
    e0.reset_search(start)
    a0 = CPUHistoryArchive(e0, str(tmp_path / "a"), sample_id=7, checkpoint=False)
    a0.start_new()
    _run(e0, a0, 8)
    # interrupted at depth 5, resumed by a fresh engine and archive
    e1 = OracleEngine(pz, 64)
    e1.reset_search(start)
    a1 = CPUHistoryArchive(e1, str(tmp_path / "b"), sample_id=7, checkpoint=True)
    a1.start_new()
    _run(e1, a1, 5)
    a1.finish()
    root = tmp_path / "b" / "sample_7"
    assert json.loads((root / MANIFEST).read_text())["depth"] == 5
    (root / "layer_00005_rank0.npy.tmp").write_bytes(b"torn write of a run that died")  # must be ignored
    e2 = OracleEngine(pz, 64)
    a2 = CPUHistoryArchive(e2, str(tmp_path / "b"), sample_id=7, checkpoint=True)
    assert a2.try_resume() == 5 and e2.depth == 5
    _run(e2, a2, 8)
    a2.finish()
    assert np.array_equal(e2.frontier(), e0.frontier())
    assert len(a2.layers) == 8 and all(np.array_equal(x, y) for x, y in zip(a2.layers, a0.layers))
    # every row of the last frontier is reached by replaying its archived path from the start state
    final = e2.frontier()
    for i in (0, final.shape[0] // 2, final.shape[0] - 1):
        moves = a2.path_to(8, i)
        assert len(moves) == 8 and np.array_equal(replay(start, pz.generators, moves), final[i])
    entry = a2.history_entry(7, 0)
    assert entry["valid"] == 1 and entry["action"] == a2.path_to(8, 0)[-1]
    assert a2.history_entry(8, 0)["valid"] == 0
    # old frontier files are dropped, layers are all kept
    assert not (root / "frontier_00003_rank0.npy").exists() and (root / "layer_00000_rank0.npy").exists()


def test_archive_rejects_a_checkpoint_of_another_configuration(tmp_path):
    pz = puzzles.puzzle54()
    e = OracleEngine(pz, 64)
    e.reset_search(pz.scramble(1, 20))
    a = CPUHistoryArchive(e, str(tmp_path), checkpoint=True)
    a.start_new()
    _run(e, a, 2)
    a.finish()
    other = CPUHistoryArchive(OracleEngine(pz, 128), str(tmp_path), checkpoint=True)
    with pytest.raises(ValueError):
        other.try_resume()
    assert CPUHistoryArchive(OracleEngine(pz, 64), str(tmp_path / "nothing_here"), checkpoint=True).try_resume() is None
    with pytest.raises(ValueError):  # layers must be recorded in order
        a2 = CPUHistoryArchive(e, str(tmp_path / "x"), checkpoint=False)
        a2.start_new()
        a2.after_step(3, 10)
