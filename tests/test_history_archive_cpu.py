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
    (root / "transition_depth0005_rank0000.parent_idx.bin.tmp").write_bytes(b"torn write of a run that died")  # must be ignored
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
    assert not (root / "frontier_depth0003_rank0000.bin").exists()
    assert not (root / "frontier_depth0003_rank0000.json").exists()
    assert (root / "transition_depth0000_rank0000.parent_idx.bin").exists()
    # the manifest is published before the frontier it replaces is dropped: the last two frontiers are there
    assert (root / "frontier_depth0008_rank0000.bin").exists() and (root / "frontier_depth0007_rank0000.bin").exists()


def _write_reference_layout(root, sample_id, cfg, n_local, max_depth, frontiers, layers):
    """A checkpoint directory written the way the reference's CPUHistoryArchive writes it
    (cpu_history_archive.py:199-211, 243-318): raw .bin arrays beside small .json files, manifest last."""
    import hashlib
    d = root / f"sample_{sample_id}"
    d.mkdir(parents=True)
    size = cfg["state_size_bytes"]
    depth = len(layers)
    rows = frontiers[depth]
    padded = np.zeros((rows.shape[0], size), np.uint8)
    padded[:, : rows.shape[1]] = rows
    padded.tofile(d / f"frontier_depth{depth:04d}_rank0000.bin")
    (d / f"frontier_depth{depth:04d}_rank0000.json").write_text(json.dumps({"depth": depth, "rank": 0, "count": int(rows.shape[0])}))
    for t, layer in enumerate(layers):
        parent, rank, move = bo.unpack_payload(layer)
        prefix = str(d / f"transition_depth{t:04d}_rank0000")
        parent.astype(np.int32).tofile(prefix + ".parent_idx.bin")
        rank.astype(np.uint8).tofile(prefix + ".parent_rank.bin")
        move.astype(np.uint8).tofile(prefix + ".action.bin")
        np.ones(layer.shape[0], np.uint8).tofile(prefix + ".valid.bin")
        (d / f"transition_depth{t:04d}_rank0000.json").write_text(json.dumps({"depth": t, "rank": 0, "count": int(layer.shape[0])}))
    payload = {"backend": "cpu", "beta": float(cfg["beta"]), "fanout": int(cfg["fanout"]),
               "global_beam_width": int(cfg["global_beam_width"]), "hash_load_factor": float(cfg["hash_load_factor"]),
               "n_local": int(n_local), "state_size_bytes": int(size), "world_size": 1}
    config_hash = hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":")).encode("utf-8")).hexdigest()
    (d / MANIFEST).write_text(json.dumps({
        "sample_id": str(sample_id), "depth": depth, "rank_count": 1, "world_size": 1, "n_local": n_local,
        "global_beam_width": int(cfg["global_beam_width"]), "max_depth": max_depth, "config_hash": config_hash,
        "complete_layer_depth": depth, "complete": True}, indent=2))


def test_resume_from_a_directory_in_the_reference_layout(tmp_path):
    pz = puzzles.puzzle54()
    start = pz.scramble(4, 30)
    extra = {"hash_load_factor": 0.45, "max_depth": 12, "state_size_bytes": 64}
    # ground truth: an uninterrupted run
    e0 = OracleEngine(pz, 64, **extra)
    e0.reset_search(start)
    a0 = CPUHistoryArchive(e0, str(tmp_path / "truth"), sample_id=1, checkpoint=False)
    a0.start_new()
    frontiers = {0: e0.frontier()}
    while e0.depth < 7:
        e0.step()
        a0.after_step(e0.depth, e0.status()["current_size"])
        frontiers[e0.depth] = e0.frontier()
    # a checkpoint at depth 4 written by hand in the reference's layout, then resumed and run on
    _write_reference_layout(tmp_path / "ref", 1, e0.cfg, 64, 12, frontiers, a0.layers[:4])
    e1 = OracleEngine(pz, 64, **extra)
    a1 = CPUHistoryArchive(e1, str(tmp_path / "ref"), sample_id=1, checkpoint=True)
    assert a1.try_resume() == 4 and e1.depth == 4
    assert np.array_equal(e1.frontier(), frontiers[4])
    _run(e1, a1, 7)
    a1.finish()
    assert np.array_equal(e1.frontier(), frontiers[7])
    assert all(np.array_equal(x, y) for x, y in zip(a1.layers, a0.layers)) and len(a1.layers) == 7
    moves = a1.path_to(7, 0)
    assert np.array_equal(replay(start, pz.generators, moves), frontiers[7][0])
    # and what this archive wrote afterwards carries the reference's manifest keys
    m = json.loads((tmp_path / "ref" / "sample_1" / MANIFEST).read_text())
    assert {"sample_id", "depth", "rank_count", "world_size", "n_local", "global_beam_width", "max_depth",
            "config_hash", "complete_layer_depth", "complete"} <= set(m)
    assert m["depth"] == 7 and m["n_local"] == 64 and len(m["config_hash"]) == 64


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


def _archive_rank(rank, world, port, root, out_q):
    """One gloo rank: every rank runs the same oracle steps over the per-rank frontiers and keeps its own share."""
    import os

    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pz = puzzles.puzzle54()
        start = pz.scramble(5, 25)

        class ShardEngine(OracleEngine):
            def __init__(self):
                super().__init__(pz, 96, rank=rank, world_size=world)
                self.fronts = None

            def reset_search(self, s):
                owner = int(bo.owner_rank(bo.hash64(s[None, :]), world)[0])
                self.fronts = [s[None, :].copy() if r == owner else s[:0][None, :].reshape(0, pz.state_len) for r in range(world)]
                self.rows, self.depth = self.fronts[rank], 0

            def step(self):
                res = bo.depth_step(self.fronts, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), self.beam)
                own = bo.owner_rank(res.h, world)
                self.fronts = [res.states[own == r] for r in range(world)]
                self.rows, self.last_layer = self.fronts[rank], res.payload[own == rank].astype(np.uint32)
                self.depth += 1

        e = ShardEngine()
        e.reset_search(start)
        a = CPUHistoryArchive(e, root, sample_id=0, checkpoint=True, barrier=dist.barrier)
        a.start_new()
        _run(e, a, 6)
        a.finish()

        def exchange(value, src):
            box = [value]
            dist.broadcast_object_list(box, src=int(src))
            return box[0]

        # walk back from row 0 of the LAST rank's frontier: every rank takes part, all get the same moves
        target_rank = world - 1
        target = exchange(e.fronts[target_rank][0] if rank == target_rank else None, target_rank)
        moves = a.path_to(6, 0, rank=target_rank, exchange=exchange)
        ok = len(moves) == 6 and np.array_equal(replay(start, pz.generators, moves), target)
        out_q.put((rank, ok, len(a.layers)))
    finally:
        dist.destroy_process_group()


def test_archive_walk_back_across_two_gloo_ranks(tmp_path):
    import socket

    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_archive_rank, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    got = sorted(q.get(timeout=10) for _ in range(2))
    assert got == [(0, True, 6), (1, True, 6)], got
    m = json.loads((tmp_path / "sample_0" / MANIFEST).read_text())
    assert m["depth"] == 6 and m["world_size"] == 2
    assert m["rank_count"] == 2 and m["complete_layer_depth"] == 6
    assert (tmp_path / "sample_0" / "transition_depth0005_rank0001.action.bin").exists()
