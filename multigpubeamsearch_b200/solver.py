"""Per-sample solver loop over the engine: prepass fill, scored depth steps, per-depth log, path reconstruction.

Counterpart of the reference's production driver (scripts/solve_testcsv_2gpu.py:220-579, 615-736) reduced to what the
hot path needs: reset on the owner rank, a "uniform fill" prepass that expands without scoring while the frontier is
still smaller than the beam (scripts/solve_testcsv_2gpu.py:266-348, 450-496), scored steps through the captured
graph, a status check after every depth (the reference asserts on its overflow counters, :414-415), a
DEPTH_TUNING-style JSON record per depth (:96-136, 344-412), and a history walk-back that also works when the
frontier is sharded over ranks (scripts/fullbeamnice_current_solver_2gpu.py:97-114: one broadcast per hop).
"""

from __future__ import annotations

import ctypes as C
import json
import time
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from .beam_engine import BeamEngine
from .puzzles import Puzzle
from .records import unpack_payload

NO_PAYLOAD = 0xFFFFFFFF


def replay(start: np.ndarray, generators: np.ndarray, moves: Sequence[int]) -> np.ndarray:
    """Apply a move sequence on the host (data_loader.apply_actions_cpu, data_loader.py:151-155)."""
    s = np.asarray(start, dtype=np.uint8)
    g = np.asarray(generators, dtype=np.int64)
    for m in moves:
        s = s[g[int(m)]]
    return s


def _world(engine: BeamEngine) -> int:
    return int(engine.cfg["world_size"])


def reconstruct_path(engine: BeamEngine) -> Optional[List[int]]:
    """Moves from the start state to the solved state after a successful search; collective when world > 1.

    The finding rank is the lowest rank that generated a solved child; every hop asks the rank that holds the parent
    row for that row's back-pointer (history_entry, beam_engine.cpp:1200-1219)."""
    c = engine._read_ctrl()
    if not c.found:
        return None
    if c.found_depth == 0:
        return []
    world, rank = _world(engine), int(engine.cfg["rank"])
    if world == 1:
        return engine.reconstruct_path()
    mine = int(c.found_payload)
    payloads: List[Any] = [None] * world
    dist.all_gather_object(payloads, mine)
    finders = [r for r, p in enumerate(payloads) if p != NO_PAYLOAD]
    if not finders:
        return None
    parent, prank, move = unpack_payload(payloads[finders[0]])
    moves = [int(move)]
    hist = engine.buffers["history_payload"]
    if c.found_depth - 1 > hist.shape[0]:
        raise RuntimeError(f"the device keeps {hist.shape[0]} history layers but the path has {c.found_depth - 1}: "
                           "pass a CPUHistoryArchive to solve_one, or size history_rows / max_depth to the search")
    for d in range(c.found_depth - 2, -1, -1):
        box = [None]
        if rank == prank:
            box[0] = int(hist[d % hist.shape[0], int(parent)].item()) & 0xFFFFFFFF
        dist.broadcast_object_list(box, src=int(prank))
        parent, prank, move = unpack_payload(box[0])
        moves.append(int(move))
    return moves[::-1]


def reconstruct_path_from_archive(engine: BeamEngine, archive) -> Optional[List[int]]:
    """The same walk-back over a CPUHistoryArchive (the device then keeps only a small ring of history rows)."""
    c = engine._read_ctrl()
    if not c.found:
        return None
    if c.found_depth == 0:
        return []
    world = _world(engine)
    payloads: List[Any] = [int(c.found_payload)]
    if world > 1:
        payloads = [None] * world
        dist.all_gather_object(payloads, int(c.found_payload))
    finders = [p for p in payloads if p != NO_PAYLOAD]
    if not finders:
        return None
    parent, prank, move = unpack_payload(finders[0])

    def exchange(value, src):
        box = [value]
        dist.broadcast_object_list(box, src=int(src))
        return box[0]

    head = archive.path_to(int(c.found_depth) - 1, int(parent), int(prank), exchange if world > 1 else None)
    return head + [int(move)]


def solve_one(engine: BeamEngine, puzzle: Puzzle, start: np.ndarray, max_depth: int, sample_id: int = 0,
              prepass: bool = True, depth_log: Optional[List[Dict[str, Any]]] = None, archive=None) -> Dict[str, Any]:
    """Search one start state; returns {id, found, depth, path, valid, status_bits, wall_ms, depths_prepass}.

    With ``archive`` (a history_archive.CPUHistoryArchive over this engine) every depth's back-pointers are copied
    to the host after its step - and checkpointed, if the archive was built with checkpoint=True - and the path is
    rebuilt from the archive."""
    start = np.ascontiguousarray(start, dtype=np.uint8)
    world, rank = _world(engine), int(engine.cfg["rank"])
    n = int(engine.cfg["state_len"])
    owner = engine.owner_of(start)
    t0 = time.perf_counter()
    engine.reset_search(bytes(start), active_on_this_rank=(owner == rank))
    if archive is not None:
        archive.start_new()
    beam = int(engine.cfg["global_beam_width"])
    fanout = int(engine.cfg["fanout"])
    st = engine.status()
    in_prepass = False
    depths_prepass = 0
    bits = 0
    while not st["found"] and st["depth"] < max_depth:
        size = torch.tensor([st["current_size"]], dtype=torch.int64, device=engine.buffers["ctrl"].device)
        if world > 1:
            dist.all_reduce(size)
        total = int(size.item())
        if total == 0:
            break
        # prepass: while even keeping every child cannot exceed the beam, scores cannot change the outcome
        want_prepass = prepass and total * fanout <= beam
        if want_prepass and not in_prepass:
            engine.begin_uniform_score(0)
            in_prepass = True
        elif not want_prepass and in_prepass:
            engine.end_uniform_score()
            in_prepass = False
        t_step = time.perf_counter()
        engine.step()
        st = engine.status()
        bits |= st["status_bits"]
        if archive is not None:
            archive.after_step(st["depth"], st["current_size"])
        depths_prepass += int(in_prepass)
        if depth_log is not None and rank == 0:
            depth_log.append({
                "tag": "DEPTH_TUNING", "id": sample_id, "depth": st["depth"], "prepass": in_prepass,
                "frontier_in": total, "candidates": total * fanout, "unique": st["counters"][3],
                "table_inserts_rank0": st["counters"][1], "band_rounds": st["counters"][5],
                "status_bits": st["status_bits"], "wall_ms": (time.perf_counter() - t_step) * 1e3,
            })
    if in_prepass:
        engine.end_uniform_score()
    if archive is not None:
        archive.finish_pending()
    path = None
    if st["found"]:
        path = reconstruct_path_from_archive(engine, archive) if archive is not None else reconstruct_path(engine)
    valid = bool(path is not None and np.array_equal(replay(start, puzzle.generators, path), puzzle.solved))
    return {
        "id": sample_id, "found": bool(st["found"]), "depth": int(st["found_depth"] if st["found"] else st["depth"]),
        "path": path, "valid": valid, "status_bits": bits, "wall_ms": (time.perf_counter() - t0) * 1e3,
        "depths_prepass": depths_prepass,
    }


def solve_many(engine: BeamEngine, puzzle: Puzzle, starts: Sequence[np.ndarray], max_depth: int,
               log_path: Optional[str] = None) -> Dict[str, Any]:
    """Solve a list of start states; writes one JSON line per depth and per sample to ``log_path`` on rank 0
    (SAMPLE_RESULT / DEPTH_TUNING markers of the reference's driver) and returns the run summary."""
    rank = int(engine.cfg["rank"])
    results = []
    fh = open(log_path, "w") if (log_path and rank == 0) else None
    try:
        for i, s in enumerate(starts):
            log: List[Dict[str, Any]] = []
            r = solve_one(engine, puzzle, s, max_depth, sample_id=i, depth_log=log)
            results.append(r)
            if fh:
                for row in log:
                    fh.write(json.dumps(row) + "\n")
                fh.write(json.dumps({"tag": "SAMPLE_RESULT", **{k: v for k, v in r.items()}}) + "\n")
    finally:
        if fh:
            fh.close()
    solved = sum(1 for r in results if r["found"] and r["valid"])
    return {"tag": "RUN_SUMMARY", "samples": len(results), "solved": solved,
            "invalid_paths": sum(1 for r in results if r["found"] and not r["valid"]),
            "status_bits": int(np.bitwise_or.reduce([r["status_bits"] for r in results])) if results else 0,
            "results": results}
