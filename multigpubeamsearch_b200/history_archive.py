"""Host-side archive of the search history, with optional on-disk checkpoints and resume.

Counterpart of the reference's cpu_history_archive.CPUHistoryArchive (cpu_history_archive.py:45-360): long searches
(depth 300, beam 2^22) cannot keep every depth's back-pointers on the GPU, and must survive a restart.  After every
depth step the archive copies that depth's back-pointer layer (one packed uint32 per frontier row: parent, source
rank, move) from the device, so the engine needs only a small ring of history rows (``history_rows`` in the config).
With ``checkpoint=True`` it also writes, from a background thread, the layer and the current frontier of every rank
to ``root/sample_<id>/`` and then a manifest (atomic rename) that names the last depth whose files are complete on
every rank; ``try_resume`` validates the manifest against the running configuration, reloads the layers and uploads
the frontier, and the search continues from that depth.

The archive talks to the engine through five members only - ``cfg``, ``status()``, ``frontier()``,
``history_layer(depth, count)``, ``load_frontier(rows, depth)`` - so the same code runs over the CUDA engine and over
the CPU model of it used in the tests.
"""

from __future__ import annotations

import hashlib
import json
import os
from concurrent.futures import Future, ThreadPoolExecutor
from pathlib import Path
from typing import Any, Dict, List, Optional

import numpy as np

from .records import unpack_payload

MANIFEST = "manifest.json"


def _atomic_write_json(path: Path, payload: Dict[str, Any]) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    tmp.write_text(json.dumps(payload, indent=2), encoding="utf-8")
    os.replace(tmp, path)


def _atomic_save(path: Path, array: np.ndarray) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    with open(tmp, "wb") as fh:
        np.save(fh, array)
    os.replace(tmp, path)


class CPUHistoryArchive:
    def __init__(self, engine, root: str, sample_id: Any = 0, checkpoint: bool = False, barrier=None,
                 keep_frontiers: int = 2):
        self.engine = engine
        self.rank = int(engine.cfg["rank"])
        self.world = int(engine.cfg["world_size"])
        self.checkpoint = bool(checkpoint)
        self.root = Path(root) / f"sample_{sample_id}"
        self.layers: List[np.ndarray] = []   # layers[d][i] = packed back-pointer of row i of the depth d+1 frontier
        self.depth = 0
        self.keep_frontiers = max(1, int(keep_frontiers))
        self._barrier = barrier or (lambda: None)
        self._pool: Optional[ThreadPoolExecutor] = ThreadPoolExecutor(max_workers=1) if self.checkpoint else None
        self._pending: Optional[Future] = None
        self._pending_depth: Optional[int] = None
        self.config_hash = self._make_config_hash()

    # -- identity of a run: a checkpoint is only valid for the configuration that wrote it ------------------------
    def _make_config_hash(self) -> str:
        keys = ("state_len", "state_size_bytes", "fanout", "world_size", "global_beam_width", "beta", "gamma",
                "select_mode", "hash_bits", "inference_backend")
        c = self.engine.cfg
        text = json.dumps({k: str(c.get(k)) for k in keys}, sort_keys=True)
        return hashlib.sha256(text.encode()).hexdigest()[:16]

    # -- files -----------------------------------------------------------------------------------------------------
    def _layer_path(self, depth: int, rank: int) -> Path:
        return self.root / f"layer_{depth:05d}_rank{rank}.npy"

    def _frontier_path(self, depth: int, rank: int) -> Path:
        return self.root / f"frontier_{depth:05d}_rank{rank}.npy"

    # -- life cycle ------------------------------------------------------------------------------------------------
    def start_new(self) -> None:
        """Call after reset_search: records depth 0 (and checkpoints the start frontier)."""
        self.finish_pending()
        self.layers = []
        self.depth = 0
        if self.checkpoint:
            self._write_files(0, None, np.ascontiguousarray(self.engine.frontier()))
            self._barrier()
            self._write_manifest(0)

    def after_step(self, depth: int, current_size: int) -> None:
        """Call after the step that produced the depth ``depth`` frontier of ``current_size`` local rows."""
        if depth <= 0:
            return
        if depth != self.depth + 1:
            raise ValueError(f"archive is at depth {self.depth}, cannot record depth {depth}")
        self.finish_pending()
        layer = np.ascontiguousarray(self.engine.history_layer(depth - 1, int(current_size)), dtype=np.uint32)
        self.layers.append(layer)
        self.depth = depth
        if self.checkpoint:
            frontier = np.ascontiguousarray(self.engine.frontier())
            self._pending = self._pool.submit(self._write_files, depth, layer, frontier)
            self._pending_depth = depth

    def finish_pending(self) -> None:
        """Wait for the background write, then (all ranks) publish its depth in the manifest."""
        if self._pending is not None:
            self._pending.result()
            depth = self._pending_depth
            self._pending, self._pending_depth = None, None
            self._barrier()
            self._write_manifest(depth)

    def finish(self) -> None:
        self.finish_pending()
        if self._pool is not None:
            self._pool.shutdown(wait=True)
            self._pool = None

    def _write_files(self, depth: int, layer: Optional[np.ndarray], frontier: np.ndarray) -> None:
        if layer is not None:
            _atomic_save(self._layer_path(depth - 1, self.rank), layer)
        _atomic_save(self._frontier_path(depth, self.rank), frontier)
        old = depth - self.keep_frontiers
        if old >= 0:
            try:
                self._frontier_path(old, self.rank).unlink()
            except FileNotFoundError:
                pass

    def _write_manifest(self, depth: int) -> None:
        if self.rank != 0:
            return
        _atomic_write_json(self.root / MANIFEST, {
            "depth": int(depth), "world_size": self.world, "config_hash": self.config_hash,
            "global_beam_width": int(self.engine.cfg["global_beam_width"]), "complete": True,
        })

    # -- resume ----------------------------------------------------------------------------------------------------
    def try_resume(self) -> Optional[int]:
        """Load the last complete checkpoint into the archive and the engine; returns its depth, or None if there is
        none.  Raises ValueError when the checkpoint belongs to another configuration."""
        path = self.root / MANIFEST
        if not path.exists():
            return None
        m = json.loads(path.read_text(encoding="utf-8"))
        if not m.get("complete", False):
            raise ValueError("checkpoint manifest is not complete")
        if int(m.get("world_size", -1)) != self.world:
            raise ValueError("checkpoint world size mismatch")
        if int(m.get("global_beam_width", -1)) != int(self.engine.cfg["global_beam_width"]):
            raise ValueError("checkpoint global_beam_width mismatch")
        if str(m.get("config_hash", "")) != self.config_hash:
            raise ValueError("checkpoint config_hash mismatch")
        depth = int(m["depth"])
        self.layers = [np.load(self._layer_path(d, self.rank)).astype(np.uint32) for d in range(depth)]
        frontier = np.load(self._frontier_path(depth, self.rank))
        self.engine.load_frontier(frontier, depth=depth)
        self.depth = depth
        self._barrier()
        return depth

    # -- queries ---------------------------------------------------------------------------------------------------
    def history_entry(self, depth: int, local_index: int) -> Dict[str, int]:
        """Back-pointer of row ``local_index`` of the depth ``depth``+1 frontier (history_entry,
        cpu_history_archive.py:152-162)."""
        if depth < 0 or depth >= len(self.layers) or local_index < 0 or local_index >= self.layers[depth].shape[0]:
            return {"valid": 0, "parent_idx": -1, "parent_rank": -1, "action": -1}
        p, r, m = unpack_payload(int(self.layers[depth][local_index]))
        return {"valid": 1, "parent_idx": int(p), "parent_rank": int(r), "action": int(m)}

    def path_to(self, depth: int, local_index: int, rank: Optional[int] = None, exchange=None) -> List[int]:
        """Moves from the start state to row ``local_index`` (on ``rank``) of the depth ``depth`` frontier.

        World 1: a walk over the local layers.  World > 1: collective; ``exchange(value_or_None, src)`` must return
        on every rank the value passed by rank ``src`` (one broadcast per hop, as the reference's driver does,
        scripts/fullbeamnice_current_solver_2gpu.py:97-114)."""
        moves: List[int] = []
        idx, owner = int(local_index), self.rank if rank is None else int(rank)
        for d in range(depth - 1, -1, -1):
            mine = None
            if owner == self.rank:
                mine = int(self.layers[d][idx])
            payload = mine if self.world == 1 else exchange(mine, owner)
            p, r, m = unpack_payload(int(payload))
            moves.append(int(m))
            idx, owner = int(p), int(r)
        return moves[::-1]
