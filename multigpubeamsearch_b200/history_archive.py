"""Host-side archive of the search history, with optional on-disk checkpoints and resume.

Counterpart of the reference's cpu_history_archive.CPUHistoryArchive (cpu_history_archive.py:45-360): long searches
(depth 300, beam 2^22) cannot keep every depth's back-pointers on the GPU, and must survive a restart.  After every
depth step the archive copies that depth's back-pointer layer (one packed uint32 per frontier row: parent, source
rank, move) from the device, so the engine needs only a small ring of history rows (``history_rows`` in the config).
With ``checkpoint=True`` it also writes, from a background thread, the layer and the current frontier of every rank
to ``root/sample_<id>/`` and then a manifest (atomic rename) that names the last depth whose files are complete on
every rank; ``try_resume`` validates the manifest against the running configuration, reloads the layers and uploads
the frontier, and the search continues from that depth.

On-disk layout = the reference's (cpu_history_archive.py:243-318), so checkpoints can be exchanged with it:
  frontier_depthNNNN_rankNNNN.bin    raw rows of state_size_bytes bytes     + .json {"depth", "rank", "count"}
  transition_depthNNNN_rankNNNN.parent_idx.bin (int32), .parent_rank.bin (uint8), .action.bin (uint8),
                                .valid.bin (uint8)                          + .json {"depth", "rank", "count"}
  manifest.json  {sample_id, depth, rank_count, world_size, n_local, global_beam_width, max_depth, config_hash,
                  complete_layer_depth, complete}; config_hash = sha256 of the reference's payload
                  (cpu_history_archive.py:199-211).

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

from .records import pack_payload, unpack_payload

MANIFEST = "manifest.json"


def _atomic_write_json(path: Path, payload: Dict[str, Any]) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    tmp.write_text(json.dumps(payload, indent=2), encoding="utf-8")
    os.replace(tmp, path)


def _atomic_tofile(path: Path, array: np.ndarray) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    np.ascontiguousarray(array).tofile(tmp)
    os.replace(tmp, path)


class CPUHistoryArchive:
    def __init__(self, engine, root: str, sample_id: Any = 0, checkpoint: bool = False, barrier=None,
                 keep_frontiers: int = 2):
        self.engine = engine
        self.rank = int(engine.cfg["rank"])
        self.world = int(engine.cfg["world_size"])
        self.checkpoint = bool(checkpoint)
        self.sample_id = str(sample_id)
        self.root = Path(root) / f"sample_{sample_id}"
        cfg = engine.cfg
        self.state_len = int(cfg["state_len"])
        self.state_size = int(cfg.get("state_size_bytes", self.state_len))
        beam = int(cfg["global_beam_width"])
        sizes = engine.sizes() if hasattr(engine, "sizes") else {}
        self.n_local = int(sizes.get("n_local", (beam + self.world - 1) // self.world))
        self.max_depth = int(cfg.get("max_depth", 0))
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
        """The reference's payload and serialisation (cpu_history_archive.py:199-211)."""
        c = self.engine.cfg
        payload = {
            "backend": "cpu",
            "beta": float(c.get("beta", 0.0)),
            "fanout": int(c["fanout"]),
            "global_beam_width": int(c["global_beam_width"]),
            "hash_load_factor": float(c.get("hash_load_factor", 0.0)),
            "n_local": int(self.n_local),
            "state_size_bytes": int(self.state_size),
            "world_size": int(self.world),
        }
        raw = json.dumps(payload, sort_keys=True, separators=(",", ":")).encode("utf-8")
        return hashlib.sha256(raw).hexdigest()

    # -- files -----------------------------------------------------------------------------------------------------
    def _frontier_path(self, depth: int, rank: int) -> Path:
        return self.root / f"frontier_depth{depth:04d}_rank{rank:04d}.bin"

    def _frontier_meta_path(self, depth: int, rank: int) -> Path:
        return self.root / f"frontier_depth{depth:04d}_rank{rank:04d}.json"

    def _transition_prefix(self, depth: int, rank: int) -> str:
        return str(self.root / f"transition_depth{depth:04d}_rank{rank:04d}")

    def _write_frontier(self, depth: int, rows: np.ndarray) -> None:
        """Rows padded with zeros to state_size_bytes, as the reference's frontier files hold them."""
        n = int(rows.shape[0])
        padded = np.zeros((n, self.state_size), dtype=np.uint8)
        padded[:, : self.state_len] = rows[:, : self.state_len]
        _atomic_tofile(self._frontier_path(depth, self.rank), padded)
        _atomic_write_json(self._frontier_meta_path(depth, self.rank), {"depth": depth, "rank": self.rank, "count": n})

    def _read_frontier(self, depth: int, rank: int) -> np.ndarray:
        meta = json.loads(self._frontier_meta_path(depth, rank).read_text(encoding="utf-8"))
        count = int(meta["count"])
        arr = np.fromfile(self._frontier_path(depth, rank), dtype=np.uint8, count=count * self.state_size)
        return arr.reshape(count, self.state_size)[:, : self.state_len].copy()

    def _write_transition(self, depth: int, layer: np.ndarray) -> None:
        """One layer as the reference's four arrays (cpu_history_archive.py:290-303)."""
        p, r, m = unpack_payload(layer)
        prefix = self._transition_prefix(depth, self.rank)
        n = int(layer.shape[0])
        for suffix, arr in (("parent_idx", np.asarray(p, dtype=np.int32)), ("parent_rank", np.asarray(r, dtype=np.uint8)),
                            ("action", np.asarray(m, dtype=np.uint8)), ("valid", np.ones((n,), dtype=np.uint8))):
            _atomic_tofile(Path(prefix + f".{suffix}.bin"), arr)
        _atomic_write_json(Path(prefix + ".json"), {"depth": depth, "rank": self.rank, "count": n})

    def _read_transition(self, depth: int, rank: int) -> np.ndarray:
        prefix = self._transition_prefix(depth, rank)
        n = int(json.loads(Path(prefix + ".json").read_text(encoding="utf-8"))["count"])
        p = np.fromfile(Path(prefix + ".parent_idx.bin"), dtype=np.int32, count=n).astype(np.uint32)
        r = np.fromfile(Path(prefix + ".parent_rank.bin"), dtype=np.uint8, count=n).astype(np.uint32)
        m = np.fromfile(Path(prefix + ".action.bin"), dtype=np.uint8, count=n).astype(np.uint32)
        v = np.fromfile(Path(prefix + ".valid.bin"), dtype=np.uint8, count=n)
        if not v.all():
            raise ValueError(f"transition layer {depth} of rank {rank} holds invalid rows")
        return pack_payload(p, r, m)

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
        """Wait for the background write, then (all ranks) publish its depth in the manifest, and only after the
        manifest names the new depth drop the frontier files it no longer needs: a crash at any point leaves a
        manifest whose files exist on every rank."""
        if self._pending is not None:
            self._pending.result()
            depth = self._pending_depth
            self._pending, self._pending_depth = None, None
            self._barrier()
            self._write_manifest(depth)
            self._barrier()
            old = depth - self.keep_frontiers
            if old >= 0:
                for path in (self._frontier_path(old, self.rank), self._frontier_meta_path(old, self.rank)):
                    try:
                        path.unlink()
                    except FileNotFoundError:
                        pass

    def finish(self) -> None:
        self.finish_pending()
        if self._pool is not None:
            self._pool.shutdown(wait=True)
            self._pool = None

    def _write_files(self, depth: int, layer: Optional[np.ndarray], frontier: np.ndarray) -> None:
        if layer is not None:
            self._write_transition(depth - 1, layer)
        self._write_frontier(depth, frontier)

    def _write_manifest(self, depth: int) -> None:
        """Keys of the reference's manifest (cpu_history_archive.py:305-318)."""
        if self.rank != 0:
            return
        _atomic_write_json(self.root / MANIFEST, {
            "sample_id": self.sample_id,
            "depth": int(depth),
            "rank_count": self.world,
            "world_size": self.world,
            "n_local": self.n_local,
            "global_beam_width": int(self.engine.cfg["global_beam_width"]),
            "max_depth": self.max_depth,
            "config_hash": self.config_hash,
            "complete_layer_depth": int(depth),
            "complete": True,
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
        if int(m.get("rank_count", m.get("world_size", -1))) != self.world:
            raise ValueError("checkpoint world size mismatch")
        if int(m.get("n_local", -1)) != self.n_local:
            raise ValueError("checkpoint n_local mismatch")
        if int(m.get("global_beam_width", -1)) != int(self.engine.cfg["global_beam_width"]):
            raise ValueError("checkpoint global_beam_width mismatch")
        if str(m.get("config_hash", "")) != self.config_hash:
            raise ValueError("checkpoint config_hash mismatch")
        depth = int(m["depth"])
        self.layers = [self._read_transition(d, self.rank) for d in range(depth)]
        frontier = self._read_frontier(depth, self.rank)
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
