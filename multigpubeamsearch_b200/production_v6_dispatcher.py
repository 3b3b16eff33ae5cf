"""Task-level dispatcher with the reference's v6 interface over the B200 engine.

Counterpart of ``ProductionV6Dispatcher`` (production_v6_dispatcher.py:195-868): one object per rank, built once,
``run_task(task_id, state, max_depth, global_beam_width_effective) -> ProductionV6Result`` per start state, result
fields and per-depth rows with the reference's names (production_v6_dispatcher.py:62-74, 870-916).

What differs underneath: the reference drives every micro-batch from Python (host copy of the frontier, stream-2
hash kernel, two CUB sorts, an NCCL exchange with two host syncs, a Python dictionary merge of the survivors, a
host-side histogram over pickled score lists, two ``all_to_all_single`` calls with host regrouping in between).
Here a depth is one captured graph of the engine (expand + hash + score + dedup + threshold + exchange + next
frontier on the device); the dispatcher only reads the small control block after each depth and rebuilds the path
from the device's back-pointers at the end.  The v6 selection rule is kept: ``select_mode="v6_inclusive"`` keeps
every candidate whose score key is at most the key of the beam-th survivor (ties kept), the duplicate winner is the
smallest (score, parent, rank, move) (beam_kernels_stream4.cu:25-33), hashing is the 128-bit Zobrist XOR with the
``(hi ^ lo * golden) mod world`` owner rule (beam_kernels_stream2.cu:28-38, beam_kernels_stream3.cu:29-35).  Exact
top-K (this engine's default) is available with ``select_mode="exact_k"``.

The reference refuses anything but two T4s, B_MICRO 8192 and its 120-byte puzzle (production_v6_dispatcher.py:39-48,
77-98); here the puzzle comes in as an argument and B_MICRO only sizes the scorer's micro-batches.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from . import beam_engine as be
from .puzzles import Puzzle
from .solver import reconstruct_path, replay

UINT32_MAX = 0xFFFFFFFF
SCORE_BIN_COUNT = 76801  # production_v6_dispatcher.py:25


@dataclass
class ProductionV6Result:
    """Fields of the reference's result record (production_v6_dispatcher.py:62-74)."""
    task_id: int
    status: str                      # "solved" | "unsolved" | "max_depth_reached"
    path: str                        # move names joined by "." (append_move_to_path, :140-142)
    depth_rows: List[Dict[str, Any]]
    solved_depth: int = -1
    solved_rank: int = -1
    solved_parent_idx: int = -1
    solved_move: int = -1
    raw_solved_record_exists: bool = False
    path_replay_valid: bool = False
    path_failure_reason: str = ""
    status_bits: int = 0             # this engine's capacity/timeout bits over the task (0 = clean)


def move_names(fanout: int) -> List[str]:
    """Default names m0, m1, ... (the reference reads its 24 names from puzzle_info.json, data_loader.py:35-60)."""
    return [f"m{i}" for i in range(fanout)]


def append_move_to_path(path: str, move_name: str) -> str:
    return move_name if not path else f"{path}.{move_name}"


def replay_path_to_central(puzzle: Puzzle, names: Sequence[str], state: np.ndarray, path: str):
    """(valid, length, reason) - the reference's path check (production_v6_dispatcher.py:1254-1266)."""
    if not path:
        return False, 0, "empty_path"
    moves = path.split(".")
    index = {n: i for i, n in enumerate(names)}
    invalid = [m for m in moves if m not in index]
    if invalid:
        return False, len(moves), f"invalid_moves={invalid[:4]}"
    if not np.array_equal(replay(state, puzzle.generators, [index[m] for m in moves]), puzzle.solved):
        return False, len(moves), "replay_not_central"
    return True, len(moves), ""


class ProductionV6Dispatcher:
    def __init__(self, rank: int, world_size: int, device: torch.device, *, beam_width: int, b_micro: int = 8192,
                 puzzle: Optional[Puzzle] = None, scorer=None, action_names: Optional[Sequence[str]] = None,
                 max_depth: int = 100, select_mode: str = "v6_inclusive", hash_mode: str = "zobrist128",
                 **cfg_overrides: Any) -> None:
        from . import puzzles as _puzzles
        self.rank, self.world_size = int(rank), int(world_size)
        self.device = torch.device(device)
        self.beam_width, self.b_micro = int(beam_width), int(b_micro)
        if self.b_micro < 1:
            raise RuntimeError(f"invalid_config: B_MICRO must be positive, got {b_micro}")
        self.puzzle = puzzle if puzzle is not None else _puzzles.puzzle54()
        self.action_names = list(action_names) if action_names is not None else move_names(self.puzzle.fanout)
        if len(self.action_names) != self.puzzle.fanout:
            raise RuntimeError("one action name per generator is required")
        torch.cuda.set_device(self.device)
        # score-only orders (v6_inclusive) need room for a whole score level in the pool: a wider BETA by default
        beta = cfg_overrides.pop("beta", 2.0 if select_mode != "exact_k" else 1.2)
        cfg = be.config_for_puzzle(
            self.puzzle, world_size=self.world_size, rank=self.rank, global_beam_width=self.beam_width,
            b_micro=self.b_micro, max_depth=int(max_depth), select_mode=select_mode, hash_mode=hash_mode, beta=beta,
            hash_load_factor=cfg_overrides.pop("hash_load_factor", 0.45),
            probe_limit=cfg_overrides.pop("probe_limit", 256), **cfg_overrides)
        self.ext, self.cfg, self.buffers, self.engine = be.configure_engine(self.puzzle, cfg=cfg, scorer=scorer)
        self.final_capacity = int(self.ext.derive_sizes(self.cfg)["n_local"])

    def close(self) -> None:
        self.engine.close()

    # -- one task --------------------------------------------------------------------------------------------------
    def _global(self, value: int) -> int:
        if self.world_size == 1:
            return int(value)
        t = torch.tensor([int(value)], dtype=torch.int64, device=self.device)
        dist.all_reduce(t)
        return int(t.item())

    def run_task(self, task_id: int, state: np.ndarray, max_depth: int,
                 global_beam_width_effective: Optional[int] = None) -> ProductionV6Result:
        """Search from ``state``; every rank calls it with the same arguments (collective when world_size > 1).

        ``global_beam_width_effective`` must equal the beam the dispatcher was built with (the engine's buffers are
        sized for it); the reference passes its alignment-rounded beam here."""
        beam = self.beam_width if global_beam_width_effective is None else int(global_beam_width_effective)
        if beam != self.beam_width:
            raise RuntimeError(f"invalid_config: the dispatcher was built for beam {self.beam_width}, got {beam}")
        if int(max_depth) > int(self.cfg["max_depth"]):
            raise RuntimeError(f"invalid_config: max_depth {max_depth} exceeds the history rows ({self.cfg['max_depth']})")
        eng, pz = self.engine, self.puzzle
        state = np.ascontiguousarray(state, dtype=np.uint8)[: pz.state_len]
        owner = eng.owner_of(state)
        eng.reset_search(bytes(state), active_on_this_rank=(owner == self.rank))
        st = eng.status()
        depth_rows: List[Dict[str, Any]] = []
        status = "max_depth_reached"
        bits = 0
        threshold_initialized, current_threshold = False, UINT32_MAX
        while not st["found"] and st["depth"] < int(max_depth):
            start = time.time()
            frontier_local = int(st["current_size"])
            frontier_global = self._global(frontier_local)
            if frontier_global == 0:
                status = "unsolved"
                break
            eng.step()
            st = eng.status()
            bits |= st["status_bits"]
            unique = int(st["counters"][3])
            if unique >= beam:  # the rule of threshold_update (beam_types.hpp:125-134): set once enough survivors
                new_thr = int(st["threshold_q"]) if st["threshold_valid"] else UINT32_MAX
                current_threshold = min(current_threshold, new_thr) if threshold_initialized else new_thr
                threshold_initialized = True
            next_local = int(st["current_size"])
            depth_rows.append(self._depth_row(
                task_id, st["depth"] - 1, frontier_local, threshold_initialized, current_threshold,
                clean_count_total=int(st["counters"][0]), global_keep_count=self._global(next_local),
                solved_count=int(bool(st["found"])), stop_flag=int(bool(st["found"])), start=start,
                expanded_parent_count=frontier_local, generated=int(st["counters"][2]),
                after_threshold=int(st["counters"][1]), unique=int(st["counters"][0]), next_size=next_local))
            if not st["found"] and depth_rows[-1]["global_keep_count"] == 0:
                status = "unsolved"
                break
        result = ProductionV6Result(task_id=int(task_id), status=status, path="", depth_rows=depth_rows,
                                    path_failure_reason="no_solved_state", status_bits=bits)
        if st["found"]:
            result.status = "solved"
            result.solved_depth = int(st["found_depth"])
            moves = reconstruct_path(eng)  # collective walk-back over the device's back-pointers when world_size > 1
            result.raw_solved_record_exists = bool(st["local_found"]) or st["found_depth"] == 0
            if st["local_found"]:
                result.solved_rank = self.rank
                result.solved_parent_idx = int(st["found_local_index"])
                result.solved_move = int(st["found_action"])
            if moves is None:
                result.path_failure_reason = "parent_chain_broken"
            elif not moves:
                result.path_replay_valid, result.path_failure_reason = True, ""  # the start state was already solved
            else:
                for m in moves:
                    result.path = append_move_to_path(result.path, self.action_names[int(m)])
                ok, _, why = replay_path_to_central(pz, self.action_names, state, result.path)
                result.path_replay_valid, result.path_failure_reason = ok, why
        return result

    def _depth_row(self, task_id: int, depth: int, frontier_size: int, threshold_initialized: bool,
                   current_threshold: int, *, clean_count_total: int, global_keep_count: int, solved_count: int,
                   stop_flag: int, start: float, expanded_parent_count: int, generated: int, after_threshold: int,
                   unique: int, next_size: int) -> Dict[str, Any]:
        """Keys of the reference's per-depth JSONL row (production_v6_dispatcher.py:870-916); the stream-3/4 counters
        map to this engine's stages: candidates passed to the dedup table, unique table entries, rows kept."""
        return {
            "task_id": int(task_id), "depth": int(depth), "frontier_size": int(frontier_size),
            "current_frontier_size_before": int(frontier_size), "expanded_parent_count": int(expanded_parent_count),
            "stream1_scored_parent_count": int(expanded_parent_count),
            "stream2_generated_candidate_count": int(generated),
            "stream3_after_threshold_count": int(after_threshold), "stream3_unique_count": int(unique),
            "stream4_input_count": int(after_threshold), "stream4_clean_count": int(unique),
            "next_frontier_size_after": int(next_size), "threshold_initialized": bool(threshold_initialized),
            "current_threshold": int(current_threshold), "clean_count_total": int(clean_count_total),
            "dirty_count_total": 0, "global_keep_count": int(global_keep_count), "solved_count": int(solved_count),
            "stop_flag": int(stop_flag), "elapsed_sec": float(time.time() - start),
            "gpu_memory_allocated": int(torch.cuda.memory_allocated(self.device)),
            "gpu_memory_reserved": int(torch.cuda.memory_reserved(self.device)),
        }
