"""Python control plane of the B200 beam-search engine.

Mirror of the reference's beam_engine.py: the same entry points (make_default_config, build_extension,
init_distributed_if_needed, allocate_buffers, create_nccl_id, configure_engine, run_one_search) and the same
``BeamEngine(cfg, buffers, backend)`` object with the method names of the reference's pybind class
(beam_engine.cpp:2114-2148).  Python owns all device memory as torch tensors; the engine underneath is
libmgbs_b200.so, reached through its C ABI (include/mgbs.h).  There is no CPU fallback.

Differences that a caller of the reference will notice:
  * state length, fan-out and value range are run-time config keys (state_len, fanout, num_values) instead of
    the compile-time 120 / 24;
  * scores are "lower is better" integer keys (the v6 orientation, beam_types.hpp:22-27);
  * selection keeps exactly GLOBAL_BEAM_WIDTH states, ties broken on (score, hash, fingerprint); the reference's
    two threshold rules are available as select_mode "v6_inclusive" and "legacy_strict".
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Any, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from . import _lib
from . import build as _build
from .puzzles import Puzzle

HISTORY_NONE = 0xFFFFFFFF


def _flag_enabled(name: str, default: str = "0") -> bool:
    return os.environ.get(name, default).strip().lower() not in {"", "0", "false", "no", "off"}


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def make_default_config() -> Dict[str, Any]:
    """Config dict from the environment; reference keys and env names (beam_engine.py:68-109) plus the shape keys."""
    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    state_len = int(os.environ.get("STATE_LEN", "54"))
    return {
        "world_size": world_size,
        "rank": rank,
        "global_beam_width": int(os.environ.get("GLOBAL_BEAM_WIDTH", str(1 << 16))),
        "fanout": int(os.environ.get("FANOUT", "12")),
        "state_len": state_len,
        "state_size_bytes": _round_up(state_len, 16),
        "num_values": int(os.environ.get("NUM_VALUES", "6")),
        "b_micro": int(os.environ.get("B_MICRO", "32768")),
        "probe_limit": int(os.environ.get("PROBE_LIMIT", "64")),
        "bucket_cap_per_peer": int(os.environ.get("BUCKET_CAP_PER_PEER", "0")),
        "gamma": float(os.environ.get("GAMMA", "1.05")),
        "beta": float(os.environ.get("BETA", "1.15")),
        "hash_load_factor": float(os.environ.get("HASH_LOAD_FACTOR", "0.55")),
        "inference_backend": os.environ.get("INFERENCE_BACKEND", "central_hamming"),
        "max_depth": int(os.environ.get("MAX_DEPTH", "4")),
        "select_mode": os.environ.get("SELECT_MODE", "exact_k"),
        "band_rounds": int(os.environ.get("BAND_ROUNDS", "6")),
        "band_levels": int(os.environ.get("BAND_LEVELS", "3")),
        "hash_bits": int(os.environ.get("ORDER_KEY_HASH_BITS", "24")),
        "materialize_children": _flag_enabled("MATERIALIZE_CHILDREN"),
        "use_cuda_graphs": _flag_enabled("USE_CUDA_GRAPHS", "1"),
        "score_offset": float(os.environ.get("NN_SCORE_BIAS", "0.0")),
        # world > 1: "peer" = candidates stored straight into the owner's buckets over NVLink peer mappings and
        # histograms reduced in-kernel; "nccl" = grouped send/recv + all-reduce (the reference's scheme)
        "exchange": os.environ.get("MGBS_EXCHANGE", "peer"),
        # where the survivors of a depth live: "owner" = on the rank that owns their hash (no extra traffic; uniform
        # hashes keep the ranks within a fraction of a percent of each other), "balanced" = the reference's final
        # placement (production_v6_dispatcher.py:584-588): rows are moved after every depth so that every rank holds
        # exactly its share
        "placement": os.environ.get("MGBS_PLACEMENT", "owner"),
        # Knobs of the reference's tile pipeline (beam_engine.py:44-58, 68-109).  They are accepted so that a
        # reference configuration loads unchanged; this engine has no expand tiles, score ring or net ring (one
        # depth is one fixed-shape launch sequence), so they do not change what runs:
        "k_expand_tile": int(os.environ.get("K_EXPAND_TILE", "0")),
        "score_ring_depth": int(os.environ.get("SCORE_RING_DEPTH", "2")),
        "net_ring_depth": int(os.environ.get("NET_RING_DEPTH", "2")),
        "inference_parallelism": int(os.environ.get("INFERENCE_PARALLELISM", "1")),
        "histogram_period_micro": int(os.environ.get("HISTOGRAM_PERIOD_MICRO", "4")),
        # bounded waits of the cross-rank kernels give up after this many polls (about a second by default)
        "peer_poll_limit": int(os.environ.get("MGBS_PEER_POLL_LIMIT", str(1 << 22))),
    }


def config_for_puzzle(puzzle: Puzzle, **overrides: Any) -> Dict[str, Any]:
    cfg = make_default_config()
    cfg.update({
        "state_len": puzzle.state_len,
        "state_size_bytes": _round_up(puzzle.state_len, 16),
        "fanout": puzzle.fanout,
        "num_values": puzzle.num_values,
    })
    cfg.update(overrides)
    return cfg


class _Ext:
    """What build_extension returns: the reference's module surface (BeamEngine, derive_sizes, get_nccl_unique_id)."""

    def __init__(self, lib: C.CDLL):
        self.lib = lib
        self.BeamEngine = BeamEngine

    def derive_sizes(self, cfg: Dict[str, Any]) -> Dict[str, int]:
        """Derived sizes (ext.derive_sizes, beam_engine.cpp:1692-1748)."""
        out = (C.c_int64 * 6)()
        _lib.check(self.lib.mgbs_derive_sizes(int(cfg["global_beam_width"]), int(cfg["world_size"]),
                                              float(cfg["gamma"]), float(cfg["beta"]),
                                              float(cfg["hash_load_factor"]), int(cfg["band_rounds"]),
                                              int(cfg["band_levels"]), out), "derive_sizes")
        n_local, k_keep, k_work, hash_capacity, pool_target, hist_words = (int(x) for x in out)
        world = int(cfg["world_size"])
        fanout = int(cfg["fanout"])
        cand_cap = k_work * fanout
        bucket = int(cfg.get("bucket_cap_per_peer", 0))
        if world > 1 and bucket <= 0:
            # every rank sends about cand/world records to each peer; 25 % head-room plus a constant
            bucket = int(cand_cap / world * 1.25) + 1024
        return {
            "n_local": n_local, "k_keep": k_keep, "k_work": k_work, "hash_capacity": hash_capacity,
            "pool_target": pool_target, "hist_words": hist_words, "cand_cap": cand_cap,
            "bucket_cap_per_peer": bucket if world > 1 else 0,
            "hash_slot_bytes": 32, "candidate_record_bytes": 24 + int(cfg["state_size_bytes"]),
            "history_records": int(cfg["max_depth"]) * k_work,
            "ctrl_bytes": C.sizeof(_lib.MgbsCtrl),
        }

    def get_nccl_unique_id(self) -> bytes:
        buf = (C.c_uint8 * 128)()
        _lib.check(self.lib.mgbs_nccl_unique_id(_build.nccl_library_path().encode(), C.addressof(buf)),
                   "get_nccl_unique_id")
        return bytes(buf)


def build_extension(verbose: bool = False) -> _Ext:
    """Build (if needed) and load the native library; raises when it cannot (beam_engine.py:112-157)."""
    if _build.needs_build():
        _build.build(verbose=verbose)
    return _Ext(_lib.load())


def init_distributed_if_needed(cfg: Dict[str, Any]) -> None:
    """beam_engine.py:160-168."""
    if not torch.cuda.is_available():
        raise RuntimeError("a CUDA device is required")
    local_rank = int(os.environ.get("LOCAL_RANK", str(cfg["rank"] % torch.cuda.device_count())))
    torch.cuda.set_device(local_rank)
    if cfg["world_size"] > 1 and not dist.is_initialized():
        dist.init_process_group(backend="nccl", rank=cfg["rank"], world_size=cfg["world_size"],
                                device_id=torch.device("cuda", local_rank))


def allocate_buffers(ext: _Ext, cfg: Dict[str, Any]) -> Dict[str, torch.Tensor]:
    """Every device buffer of one engine, zeroed (allocate_buffers, beam_engine.py:171-234)."""
    sizes = ext.derive_sizes(cfg)
    device = torch.device("cuda", torch.cuda.current_device())
    k_work = sizes["k_work"]
    stride = int(cfg["state_size_bytes"])
    cand_cap = sizes["cand_cap"]
    world = int(cfg["world_size"])
    need_children = bool(cfg.get("materialize_children")) or world > 1 or \
        str(cfg.get("inference_backend", "")).lower() not in {"dummy", "central_hamming", "uniform"}

    def z(shape, dtype):
        return torch.zeros(shape, dtype=dtype, device=device)

    peer_mode = world > 1 and str(cfg.get("exchange", "peer")) == "peer"
    buffers = {} if peer_mode else {  # peer mode: the frontiers are views into the symmetric region (below)
        "beam_current": z((k_work, stride), torch.uint8),
        "beam_next": z((k_work, stride), torch.uint8),
    }
    buffers.update({
        "action_table": z((int(cfg["fanout"]), int(cfg["state_len"])), torch.uint8),
        "central_state": z((int(cfg["state_len"]),), torch.uint8),
        "cand_hash": z((cand_cap,), torch.int64),
        "cand_fingerprint": z((cand_cap,), torch.int64),
        "cand_score": z((cand_cap,), torch.int32),
        "cand_payload": z((cand_cap,), torch.int32),
        "hash_table": z((sizes["hash_capacity"] * 32,), torch.uint8),
        "hist": z((sizes["hist_words"],), torch.int32),
        "tie_buf": z((world * _lib.TIE_SEG_WORDS,), torch.int64),
        # back-pointer rows, written round-robin by depth: max_depth rows keep a whole search on the device,
        # "history_rows" = 1 or 2 is enough when a CPUHistoryArchive copies every layer after its step
        "history_payload": z((max(1, int(cfg.get("history_rows") or cfg["max_depth"])), k_work), torch.int32),
        "score_current": z((k_work,), torch.int32),
        "score_next": z((k_work,), torch.int32),
        "ctrl": z((C.sizeof(_lib.MgbsCtrl),), torch.uint8),
        "io_stage": z((k_work * int(cfg["state_len"]),), torch.uint8),
    })
    if need_children:
        buffers["next_state_pool"] = z((cand_cap, stride), torch.uint8)
    if peer_mode:
        tmp = _lib.MgbsConfig()
        tmp.world_size, tmp.state_stride, tmp.bucket_cap = world, stride, sizes["bucket_cap_per_peer"]
        tmp.band_rounds, tmp.band_levels = int(cfg["band_rounds"]), int(cfg["band_levels"])
        tmp.hash_bits = int(cfg.get("hash_bits", 24)) if str(cfg.get("select_mode", "exact_k")) == "exact_k" else 0
        tmp.frontier_cap = k_work
        nbytes, ntick = C.c_int64(0), C.c_int64(0)
        _lib.check(ext.lib.mgbs_sym_bytes(C.byref(tmp), C.byref(nbytes), C.byref(ntick)), "mgbs_sym_bytes")
        offs = (C.c_int64 * 2)()
        _lib.check(ext.lib.mgbs_sym_frontier_offsets(C.byref(tmp), offs), "mgbs_sym_frontier_offsets")
        # its own allocation (not a slice of a bigger one): the whole storage is what gets mapped into the peers
        buffers["sym"] = z((int(nbytes.value),), torch.uint8)
        # the frontier buffers live inside the region: peers read parent rows from them
        for name, off in (("beam_current", int(offs[0])), ("beam_next", int(offs[1]))):
            buffers[name] = buffers["sym"][off:off + k_work * stride].view(k_work, stride)
        buffers["tickets"] = z((int(ntick.value),), torch.int32)
        buffers["send_counts"] = z((world,), torch.int32)
    elif world > 1:
        cap = sizes["bucket_cap_per_peer"]
        for side in ("send", "recv"):
            buffers[f"{side}_hash"] = z((world * cap,), torch.int64)
            buffers[f"{side}_fingerprint"] = z((world * cap,), torch.int64)
            buffers[f"{side}_score"] = z((world * cap,), torch.int32)
            buffers[f"{side}_payload"] = z((world * cap,), torch.int32)
            buffers[f"{side}_states"] = z((world * cap, stride), torch.uint8)
            buffers[f"{side}_counts"] = z((world,), torch.int32)
    return buffers


class BeamEngine:
    """The reference's BeamEngine surface (beam_engine.cpp:2114-2148) over the C ABI."""

    def __init__(self, cfg: Dict[str, Any], buffers: Dict[str, torch.Tensor], backend: str = "dummy"):
        self.lib = _lib.load()
        self.cfg = dict(cfg)
        self.buffers = buffers
        backend = (backend or "dummy").strip().lower()
        if backend not in {"dummy", "central_hamming", "uniform", "mlp"}:
            # the reference throws for backends it cannot build (beam_engine.cpp:700-703)
            raise RuntimeError(f"unknown inference backend: {backend}")
        self.backend = backend
        self._sizes = _Ext(self.lib).derive_sizes(cfg)
        # the engine owns its stream (the reference owns stream_infer_/ingest_/net_, beam_engine.cpp:705-709); stream
        # capture is not allowed on the legacy default stream
        self._stream = torch.cuda.Stream()
        self._use_graph = bool(cfg.get("use_cuda_graphs", True))
        self._graph_used = False
        self._scorer = None
        self._uniform: Optional[int] = None
        self._events = None
        self._timing: Dict[str, float] = {}
        self._limits = [-1, -1]
        self._debug = (False, False, 1)
        self._light_solved_scan = False
        c = _lib.MgbsConfig()
        c.state_len = int(cfg["state_len"])
        c.state_stride = int(cfg["state_size_bytes"])
        c.fanout = int(cfg["fanout"])
        c.world_size = int(cfg["world_size"])
        c.rank = int(cfg["rank"])
        mode = str(cfg.get("select_mode", "exact_k"))
        if mode not in _lib.SELECT_MODES:
            raise RuntimeError(f"unknown select_mode {mode!r}")
        c.select_mode = _lib.SELECT_MODES[mode]
        c.hash_bits = int(cfg.get("hash_bits", 24)) if mode == "exact_k" else 0
        c.score_mode = {"dummy": _lib.SCORE_HAMMING, "central_hamming": _lib.SCORE_HAMMING,
                        "uniform": _lib.SCORE_UNIFORM, "mlp": _lib.SCORE_EXTERNAL}[backend]
        c.band_levels = int(cfg["band_levels"])
        c.band_rounds = int(cfg["band_rounds"])
        c.probe_limit = int(cfg["probe_limit"])
        c.uniform_score = 0
        c.global_beam_width = int(cfg["global_beam_width"])
        c.frontier_cap = self._sizes["k_work"]
        c.pool_target = self._sizes["pool_target"]
        c.hash_capacity = self._sizes["hash_capacity"]
        c.cand_cap = self._sizes["cand_cap"]
        c.bucket_cap = self._sizes["bucket_cap_per_peer"]
        c.history_depths = int(buffers["history_payload"].shape[0])
        b = buffers

        def p(name):
            t = b.get(name)
            if t is None:
                return None
            if not t.is_cuda or not t.is_contiguous():
                raise RuntimeError(f"buffer {name} must be a contiguous CUDA tensor")  # check_cuda_*_tensor
            return t.data_ptr()

        c.frontier[0], c.frontier[1] = p("beam_current"), p("beam_next")
        c.gens, c.solved = p("action_table"), p("central_state")
        c.children = p("next_state_pool")
        c.cand_hash, c.cand_fp = p("cand_hash"), p("cand_fingerprint")
        c.cand_score, c.cand_payload = p("cand_score"), p("cand_payload")
        c.table, c.hist, c.tie_buf = p("hash_table"), p("hist"), p("tie_buf")
        c.history = p("history_payload")
        c.frontier_score[0], c.frontier_score[1] = p("score_current"), p("score_next")
        c.ctrl = p("ctrl")
        c.io_stage = p("io_stage")
        hash_mode = str(cfg.get("hash_mode", "fnv")).lower()
        if hash_mode not in {"fnv", "zobrist128"}:
            raise RuntimeError(f"unknown hash_mode {hash_mode!r}")
        if hash_mode == "zobrist128":
            # the v6 128-bit Zobrist hash (production_v6_dispatcher.py:109-113): table [state_len, num_values, 2] u64
            from .puzzles import zobrist_table
            nv = int(cfg["num_values"])
            tab = zobrist_table(int(cfg["state_len"]), nv)
            self._zobrist_host = tab
            buffers["zobrist"] = torch.from_numpy(tab.view(np.int64)).to(buffers["ctrl"].device)
            c.hash_mode, c.zobrist_values, c.zobrist = 1, nv, buffers["zobrist"].data_ptr()
        for side in ("send", "recv"):
            setattr(c, f"{side}_hash", p(f"{side}_hash"))
            setattr(c, f"{side}_fp", p(f"{side}_fingerprint"))
            setattr(c, f"{side}_score", p(f"{side}_score"))
            setattr(c, f"{side}_payload", p(f"{side}_payload"))
            setattr(c, f"{side}_states", p(f"{side}_states"))
            setattr(c, f"{side}_counts", p(f"{side}_counts"))
        self._peer = int(cfg["world_size"]) > 1 and str(cfg.get("exchange", "peer")) == "peer"
        if str(cfg.get("exchange", "peer")) not in ("peer", "nccl"):
            raise RuntimeError("exchange must be 'peer' or 'nccl'")
        c.exchange_mode = 1 if self._peer else 0
        if self._peer:
            c.sym = p("sym")
            c.sym_bytes = int(b["sym"].numel())
            c.tickets = p("tickets")
        c.peer_poll_limit = int(cfg.get("peer_poll_limit", 0) or 0)
        if str(cfg.get("placement", "owner")) not in ("owner", "balanced"):
            raise RuntimeError("placement must be 'owner' or 'balanced'")
        self._balanced = str(cfg.get("placement", "owner")) == "balanced" and int(cfg["world_size"]) > 1
        pipeline = str(cfg.get("select_pipeline", "persistent"))
        if pipeline not in ("persistent", "staged"):
            raise RuntimeError("select_pipeline must be 'persistent' or 'staged'")
        c.staged_select = int(pipeline == "staged")
        # pinned host summary of the control block, written by the last kernel of every depth: the depth loop
        # reads it instead of copying the control block and synchronising after every depth
        if bool(cfg.get("host_mirror", True)):
            self._mirror = torch.zeros((C.sizeof(_lib.MgbsMirror),), dtype=torch.uint8).pin_memory()
            c.host_mirror = self._mirror.data_ptr()
        if c.score_mode == _lib.SCORE_EXTERNAL and not c.children:
            raise RuntimeError("a neural backend needs the next_state_pool buffer (materialised children)")
        self._c = c
        handle = C.c_void_p()
        _lib.check(self.lib.mgbs_engine_create(C.byref(c), C.byref(handle)), "BeamEngine")
        self._h = handle
        self._ctrl = _lib.MgbsCtrl()
        self._central: Optional[np.ndarray] = None

    def close(self) -> None:
        """Destroy the native engine (unmaps the peers' regions).  With exchange mode "peer" every rank should call
        this, then synchronise with the other ranks, before the buffers are freed: a region must not be released
        while another rank still has it mapped."""
        h = getattr(self, "_h", None)
        if h:
            try:
                torch.cuda.synchronize()
            except Exception:  # interpreter shutdown: torch may already be torn down
                pass
            self.lib.mgbs_engine_destroy(h)
            self._h = None

    def __del__(self):
        self.close()

    # -- set-up ---------------------------------------------------------------------------------
    def _sp(self):
        # work queued by torch on the caller's stream (table uploads, scorer weights) happens-before engine work
        self._stream.wait_stream(torch.cuda.current_stream())
        return C.c_void_p(self._stream.cuda_stream)

    def init_nccl(self, unique_id: bytes) -> None:
        if len(unique_id) != 128:
            raise RuntimeError("NCCL unique id must be 128 bytes")
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        _lib.check(self.lib.mgbs_engine_init_nccl(self._h, _build.nccl_library_path().encode(), C.addressof(buf)),
                   "init_nccl")

    def map_peers(self) -> None:
        """Exchange IPC handles of the symmetric regions over torch.distributed and map every peer's region.

        Collective: every rank of the world calls it once, after construction (exchange mode "peer" only)."""
        if not self._peer:
            return
        sym = self.buffers["sym"]
        hbuf = (C.c_uint8 * 64)()
        off = C.c_int64(0)
        _lib.check(self.lib.mgbs_ipc_export(C.c_void_p(sym.data_ptr()), C.addressof(hbuf), C.byref(off)), "mgbs_ipc_export")
        handle, offset = bytes(hbuf), int(off.value)
        world = int(self.cfg["world_size"])
        gathered = [None] * world
        dist.all_gather_object(gathered, (handle, offset))
        handles = b"".join(h for h, _ in gathered)
        if any(len(h) != 64 for h, _ in gathered):
            raise RuntimeError("unexpected CUDA IPC handle size")
        offs = (C.c_int64 * world)(*[o for _, o in gathered])
        buf = (C.c_uint8 * (64 * world)).from_buffer_copy(handles)
        _lib.check(self.lib.mgbs_engine_set_peers(self._h, C.addressof(buf), offs), "map_peers")
        dist.barrier()

    def set_action_permutation_table(self, table: bytes) -> None:
        """fanout x state_len bytes, row-major gather tables (beam_engine.cpp:979-985)."""
        n, g = int(self.cfg["state_len"]), int(self.cfg["fanout"])
        if len(table) != n * g:
            raise RuntimeError(f"action table must be {g}x{n} bytes, got {len(table)}")
        arr = np.frombuffer(table, dtype=np.uint8).reshape(g, n)
        if arr.max(initial=0) >= n:
            raise RuntimeError("action table entry out of range")
        self.buffers["action_table"].copy_(torch.from_numpy(arr.copy()))

    def set_central_state(self, state: bytes) -> None:
        n = int(self.cfg["state_len"])
        if len(state) != n:
            raise RuntimeError(f"central state must be {n} bytes, got {len(state)}")
        self._central = np.frombuffer(state, dtype=np.uint8).copy()
        self.buffers["central_state"].copy_(torch.from_numpy(self._central))

    def owner_of(self, state: np.ndarray) -> int:
        """Rank that owns ``state`` (where reset_search must be active): hash mod world, or the Zobrist owner rule."""
        world = int(self.cfg["world_size"])
        s = np.ascontiguousarray(state, dtype=np.uint8)
        if getattr(self, "_zobrist_host", None) is not None:
            lo = hi = 0
            for pos in range(int(self.cfg["state_len"])):
                lo ^= int(self._zobrist_host[pos, int(s[pos]), 0])
                hi ^= int(self._zobrist_host[pos, int(s[pos]), 1])
            lo = lo + 4 if lo <= 2 else lo
            hi = 4 if hi == 0 else hi
            return int((hi ^ ((lo * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF)) % world)
        return int(self.lib.mgbs_hash64_host(s.ctypes.data_as(C.c_void_p), int(self.cfg["state_len"])) % world)

    def set_scorer(self, scorer) -> None:
        """Attach a device scorer object (see scorers.MLPValueScorer): it supplies a C callback and its handle."""
        self._scorer = scorer
        fn, user = scorer.c_callback()
        if getattr(scorer, "scores_parents", False):
            # action values: one forward pass per frontier row gives the scores of all its children
            _lib.check(self.lib.mgbs_engine_set_parent_scorer(self._h, fn, user), "set_scorer")
        else:
            _lib.check(self.lib.mgbs_engine_set_parent_scorer(self._h, None, None), "set_scorer")
            _lib.check(self.lib.mgbs_engine_set_scorer(self._h, fn, user), "set_scorer")

    def begin_uniform_score(self, score: int) -> None:
        """Prepass fill: every child gets the same score (beam_engine.cpp:893-915)."""
        if self._uniform is not None:
            raise RuntimeError("uniform score phase already active")
        self._uniform = int(score)
        _lib.check(self.lib.mgbs_engine_set_score_mode(self._h, _lib.SCORE_UNIFORM, int(score)), "begin_uniform_score")

    def set_uniform_score(self, score: int) -> None:
        if self._uniform is None:
            raise RuntimeError("uniform score phase is not active")
        self._uniform = int(score)
        _lib.check(self.lib.mgbs_engine_set_score_mode(self._h, _lib.SCORE_UNIFORM, int(score)), "set_uniform_score")

    def end_uniform_score(self) -> None:
        if self._uniform is None:
            raise RuntimeError("uniform score phase is not active")
        self._uniform = None
        _lib.check(self.lib.mgbs_engine_set_score_mode(self._h, self._c.score_mode, 0), "end_uniform_score")

    def enable_cuda_graphs(self, on: bool) -> None:
        self._use_graph = bool(on)

    def cuda_graph_captured(self) -> bool:
        return self._graph_used

    def enable_step_timers(self, on: bool) -> None:
        """Per-stage CUDA-event timers; enabling them drops the captured graphs and steps run eagerly
        (beam_engine.cpp:1035-1038)."""
        self._events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) if on else None
        _lib.check(self.lib.mgbs_engine_profile(self._h, int(bool(on))), "enable_step_timers")
        self._profile = bool(on)

    def step_timing(self) -> Dict[str, float]:
        """Milliseconds of the last step: total and per stage (step_timing, beam_engine.cpp:1040-1062)."""
        out = dict(self._timing)
        if getattr(self, "_profile", False):
            ms = (C.c_float * 5)()
            _lib.check(self.lib.mgbs_engine_profile_read(self._h, ms), "step_timing")
            out.update({"expand_ms": ms[0], "scorer_ms": ms[1], "exchange_ms": ms[2], "bands_ms": ms[3],
                        "final_ms": ms[4]})
            tr = (C.c_float * 96)()
            n = self.lib.mgbs_engine_trace_read(self._h, tr, 96)
            out["trace_ms"] = [round(float(tr[i]), 4) for i in range(n)]
        return out

    # -- reference methods around the scorer and the prepass -------------------------------------
    def warmup_inference(self, repeats: int = 2) -> None:
        """Run the attached scorer ``repeats`` times on the current frontier's capacity worth of rows
        (warmup_inference, beam_engine.cpp:917-929); no effect on the search state."""
        if self._scorer is None:
            return
        for _ in range(max(1, int(repeats))):
            self.benchmark_inference(min(int(self.cfg.get("b_micro", 32768)), self._sizes["k_work"]), 1, 0)

    def benchmark_inference(self, micro_size: int, repeats: int = 50, warmup: int = 10) -> List[float]:
        """Milliseconds of ``repeats`` scorer passes over ``micro_size`` rows (benchmark_inference,
        beam_engine.cpp:931-977): the value scorers score that many child rows, the action-value scorer that many
        parent rows.  Rows are whatever the buffers hold; timing does not depend on their content."""
        if self._scorer is None:
            raise RuntimeError("benchmark_inference needs a scorer (set_scorer)")
        parents = bool(getattr(self._scorer, "scores_parents", False))
        pool = self.buffers["beam_current"] if parents else self.buffers["next_state_pool"]
        micro = max(1, min(int(micro_size), int(pool.shape[0]), int(self.cfg.get("b_micro", micro_size) or micro_size)))
        rows = pool[:micro]
        out: List[float] = []
        with torch.cuda.stream(self._stream):
            self._stream.wait_stream(torch.cuda.current_stream())
            for i in range(max(0, int(warmup)) + max(1, int(repeats))):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self._stream)
                self._scorer.score(rows)
                e1.record(self._stream)
                e1.synchronize()
                if i >= max(0, int(warmup)):
                    out.append(float(e0.elapsed_time(e1)))
        return out

    def load_torchscript_ensemble(self, module_paths: List[str]) -> None:
        """The reference runs TorchScript modules as a scorer backend (beam_engine.cpp:479-554).  This engine's
        scorers are its own tensor-core kernels over plain weight arrays: export the weights and attach a scorer
        object with set_scorer (scorers.MLPValueScorer, MLPActionValueScorer, TransformerValueScorer)."""
        raise RuntimeError("load_torchscript_ensemble: TorchScript modules are not executed by this engine; "
                           "attach a scorers.* object with set_scorer")

    def load_fullbeamnice_static(self, weights: Dict[str, Any]) -> None:
        """Attach the reference's static Q-network (load_fullbeamnice_static, beam_engine.cpp:887-891) from its
        weight dictionary (keys embed_w_t ... out_bias, action_perm; scripts/static_fullbeamnice_inference.py:59-185).
        See scorers.fullbeamnice_scorer_from_static_weights."""
        from . import scorers
        sc = scorers.fullbeamnice_scorer_from_static_weights(
            weights, int(self.cfg["state_len"]), int(self.cfg["state_size_bytes"]), int(self.cfg["fanout"]),
            max_parents=int(self._sizes["n_local"]), score_offset=float(self.cfg.get("score_offset", 0.0)))
        self.set_scorer(sc)

    def enable_debug(self, verbose: bool = False, print_counters: bool = False, log_period: int = 0) -> None:
        """Debug printing knobs (enable_debug, beam_engine.cpp:1092-1102): with print_counters the status
        dictionary is printed after every ``log_period``-th step."""
        self._debug = (bool(verbose), bool(print_counters), max(1, int(log_period or 1)))

    def set_prepass_light_solved_scan(self, enable: bool) -> None:
        """The reference can skip its separate solved-state scan during the prepass
        (set_prepass_light_solved_scan, beam_engine.cpp:1141-1145).  Here the goal test is part of the expansion
        kernel and costs nothing extra, so the flag is recorded and changes nothing."""
        self._light_solved_scan = bool(enable)

    def set_active_limit(self, active_limit: int) -> None:
        """Process at most ``active_limit`` rows of the current frontier (set_active_limit,
        beam_engine.cpp:1064-1070); drops the captured graphs."""
        self._limits[0] = max(1, min(int(active_limit), self._sizes["k_work"]))
        self._apply_limits()

    def set_next_limit(self, next_limit: int) -> None:
        """Cap the next frontier at ``next_limit`` rows and the dedup table at next_limit / load + 1024 slots
        (set_next_limit, beam_engine.cpp:1072-1083); drops the captured graphs."""
        self._limits[1] = max(1, min(int(next_limit), self._sizes["k_work"]))
        self._apply_limits()

    def clear_logical_limits(self) -> None:
        """beam_engine.cpp:1085-1090."""
        self._limits = [-1, -1]
        self._apply_limits()

    def _apply_limits(self) -> None:
        _lib.check(self.lib.mgbs_engine_set_logical_limits(self._h, int(self._limits[0]), int(self._limits[1])),
                   "set logical limits")

    def step_prepass_fast(self, score: int = 0) -> None:
        """One eager depth with a constant score (step_prepass_fast, beam_engine.cpp:1136-1140)."""
        self.begin_uniform_score(score)
        try:
            self.step_current(1)
        finally:
            self.end_uniform_score()

    # -- search ---------------------------------------------------------------------------------
    def reset_search(self, state: bytes, active_on_this_rank: bool = True) -> None:
        n = int(self.cfg["state_len"])
        if len(state) != n:
            raise RuntimeError(f"state must be {n} bytes, got {len(state)}")
        solved = self._central is not None and bytes(self._central) == bytes(state)
        buf = (C.c_uint8 * n).from_buffer_copy(state)
        # every rank is given the start state, so every rank agrees on "found at depth 0"
        _lib.check(self.lib.mgbs_engine_reset(self._h, C.addressof(buf), int(bool(active_on_this_rank)),
                                              int(solved), self._sp()), "reset_search")
        self._read_ctrl()

    def clear_runtime_state(self) -> None:
        zero = bytes(int(self.cfg["state_len"]))
        _lib.check(self.lib.mgbs_engine_reset(self._h, zero, 0, 0, self._sp()), "clear_runtime_state")
        self._read_ctrl()

    def load_frontier(self, rows: np.ndarray, depth: int = 0) -> None:
        """Make ``rows`` ([K, state_len] uint8) the current frontier at ``depth`` (test and benchmark entry)."""
        rows = np.ascontiguousarray(rows, dtype=np.uint8)
        if rows.ndim != 2 or rows.shape[1] != int(self.cfg["state_len"]):
            raise RuntimeError("frontier rows must be [K, state_len] uint8")
        _lib.check(self.lib.mgbs_engine_load_frontier(self._h, rows.ctypes.data_as(C.c_void_p), rows.shape[0],
                                                      depth & 1, int(depth), self._sp()), "load_frontier")
        self._read_ctrl()

    def _read_ctrl(self) -> _lib.MgbsCtrl:
        _lib.check(self.lib.mgbs_engine_read_ctrl(self._h, C.byref(self._ctrl), self._sp()), "status")
        return self._ctrl

    def step(self, histogram_period_micro: int = 8) -> None:
        """One depth step (BeamEngine::step, beam_engine.cpp:1104-1116); asynchronous on the engine's stream."""
        parity = self._ctrl.depth & 1
        if self._events:
            self._events[0].record(self._stream)
        if self._use_graph and not getattr(self, "_profile", False):
            _lib.check(self.lib.mgbs_engine_step_graph(self._h, parity, self._sp()), "step")
            self._graph_used = True
        else:
            _lib.check(self.lib.mgbs_engine_enqueue_depth(self._h, parity, 0, self._sp()), "step")
        if self._events:
            self._events[1].record(self._stream)
            self._events[1].synchronize()
            self._timing = {"total_cuda_event_ms": self._events[0].elapsed_time(self._events[1])}
        self._ctrl.depth += 1  # host shadow; status() refreshes it from the device

    def rebalance_frontier(self) -> List[int]:
        """Even out the current frontier across the ranks and return the rows each rank holds afterwards.

        The reference's final placement (production_v6_dispatcher.py:584-588): with the survivors numbered g = 0..K-1
        in rank-major order, row g goes to rank min(g * W // K, W - 1) at local index g - ceil(K * rank / W); its
        kernels (beam_kernels_final.cu:18-55) ship requests and rows in two all-to-alls with host regrouping between
        them.  Here the rows, their scores and their back-pointers (the history entries of the depth that made
        them, so that paths still reconstruct) move in three ``all_to_all_single`` calls; the order is kept, so a
        rank's rows are one contiguous run of the global order.  Collective and synchronous: every rank calls it
        between steps.  Off the hot path by design: hash-owner placement already keeps the ranks within a fraction
        of a percent of each other."""
        world, rank = int(self.cfg["world_size"]), int(self.cfg["rank"])
        c = self._read_ctrl()
        parity = c.depth & 1
        n = int(c.frontier_count[parity])
        if world == 1:
            return [n]
        dev = self.buffers["ctrl"].device
        torch.cuda.synchronize(dev)
        counts_t = torch.zeros((world,), dtype=torch.int64, device=dev)
        mine = torch.tensor([n], dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(counts_t, mine)
        counts = [int(x) for x in counts_t.tolist()]
        send, recv, shares = balanced_exchange_plan(counts, rank)
        new_n = sum(recv)
        if new_n > int(self._sizes["k_work"]):
            raise RuntimeError("rebalance_frontier: the balanced share exceeds the frontier capacity")
        rows = self._frontier_tensor(parity)
        scores = self.buffers["score_current" if parity == 0 else "score_next"]
        hist = self.buffers["history_payload"]
        layer = hist[(c.depth - 1) % hist.shape[0]] if c.depth >= 1 else None
        moved = []
        for t in (rows, scores) + ((layer,) if layer is not None else ()):
            out = torch.empty((new_n,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev)
            dist.all_to_all_single(out, t[:n].contiguous(), output_split_sizes=recv, input_split_sizes=send)
            moved.append((t, out))
        for t, out in moved:
            t[:new_n].copy_(out)
        off = _lib.MgbsCtrl.frontier_count.offset + 4 * parity
        self.buffers["ctrl"][off:off + 4].copy_(torch.tensor([new_n], dtype=torch.int32, device=dev).view(torch.uint8))
        torch.cuda.synchronize(dev)
        dist.barrier()  # nobody steps (and reads a peer's frontier) before every rank holds its new rows
        self._read_ctrl()
        return shares

    def step_current(self, histogram_period_micro: int = 8) -> None:
        """Eager step without the graph (beam_engine.cpp:1118-1134)."""
        parity = self._ctrl.depth & 1
        _lib.check(self.lib.mgbs_engine_enqueue_depth(self._h, parity, 0, self._sp()), "step_current")
        self._ctrl.depth += 1

    def search(self, max_depth: int, histogram_period_micro: int = 8) -> Dict[str, Any]:
        """Depth loop until found / max_depth / empty frontier (beam_engine.cpp:1147-1171)."""
        rows = int(self.buffers["history_payload"].shape[0])
        if self._balanced:
            # balanced placement moves rows between depths with host-side collectives: a depth loop on the host
            rc = 0
            while True:
                st = self.status()
                if st["found"] or st["depth"] >= int(max_depth) or (st["status_bits"] & (64 | 128)):
                    break
                self.step()
                if sum(self.rebalance_frontier()) == 0:
                    break
            if self.status()["status_bits"] & (64 | 128):
                rc = -6
        else:
            rc = self.lib.mgbs_engine_search(self._h, int(max_depth), int(self._use_graph), C.byref(self._ctrl), self._sp())
        self._graph_used = self._graph_used or self._use_graph
        if rc == -6:
            # every rank's loop has returned (each wait is bounded and a rank that gives up tells the others): the
            # ranks no longer agree on their frontiers, so the search cannot go on; status() names the bit
            raise RuntimeError("search: a cross-rank wait gave up (peer timeout); status bit peer_timeout is set")
        _lib.check(rc, "search")
        st = self.status()
        # capacity problems are counted, not raised (the reference counts COUNTER_HASH_OVERFLOW / BUCKET_OVERFLOW and
        # its driver asserts on them, scripts/solve_testcsv_2gpu.py:414-415): say so next to the answer
        truncated = [n for n in st["status_names"] if n not in ("peer_timeout", "grid_timeout")]
        if truncated:
            import warnings
            warnings.warn(f"beam search ran with a truncated beam: {', '.join(truncated)}", RuntimeWarning)
        return {"found": bool(st["found"]), "depth": int(st["found_depth"] if st["found"] else st["depth"]),
                "status": st, "beam_truncated": bool(truncated), "status_names": st["status_names"],
                "history_rows": rows}

    def status(self) -> Dict[str, Any]:
        """Keys of the reference's status() (beam_engine.cpp:1173-1198) plus this engine's own counters."""
        c = self._read_ctrl()
        parity = c.depth & 1
        from .records import unpack_payload
        fp, fr, fm = unpack_payload(c.found_payload)
        bits = int(c.status)
        return {
            "current_size": int(c.frontier_count[parity]),
            "compacted_size": int(c.next_count),
            "found": int(c.found),
            "local_found": int(c.found and c.found_payload != 0xFFFFFFFF),
            "found_local_index": int(fp) if c.found_payload != 0xFFFFFFFF else -1,
            "found_action": int(fm) if c.found_payload != 0xFFFFFFFF else -1,
            "found_depth": int(c.found_depth),
            "cuda_graph_captured": self._graph_used,
            "threshold_valid": int(c.threshold_key != 0xFFFFFFFFFFFFFFFF),
            "threshold_q": int(c.threshold_key >> self._c.hash_bits) if c.threshold_key != 0xFFFFFFFFFFFFFFFF else 0,
            "threshold_key": int(c.threshold_key),
            "depth": int(c.depth),
            "counters": [int(c.table_count), int(c.inserted_total), int(c.cand_count), int(c.unique_total),
                         int(c.hash_overflow), int(c.rounds_used), int(c.bands_done), bits],
            "status_bits": bits,
            "status_names": [n for b, n in _lib.STATUS_NAMES.items() if bits & b],
            "total_candidates": int(c.total_candidates),
        }

    def sizes(self) -> Dict[str, int]:
        return dict(self._sizes)

    # -- results --------------------------------------------------------------------------------
    def _frontier_tensor(self, parity: int) -> torch.Tensor:
        return self.buffers["beam_current" if parity == 0 else "beam_next"]

    def frontier(self) -> np.ndarray:
        """Current frontier rows [K, state_len] (host copy)."""
        c = self._read_ctrl()
        parity = c.depth & 1
        k = int(c.frontier_count[parity])
        n = int(self.cfg["state_len"])
        return self._frontier_tensor(parity)[:k, :n].cpu().numpy()

    def frontier_into(self, out: np.ndarray) -> int:
        """Copy the current frontier into ``out`` ([capacity, state_len] uint8, C-contiguous; pinned memory is
        fastest) and return the number of rows written."""
        if out.dtype != np.uint8 or out.ndim != 2 or out.shape[1] != int(self.cfg["state_len"]) or not out.flags["C_CONTIGUOUS"]:
            raise RuntimeError("out must be a C-contiguous [capacity, state_len] uint8 array")
        n = C.c_int64(0)
        _lib.check(self.lib.mgbs_engine_read_frontier(self._h, self._ctrl.depth & 1, out.ctypes.data_as(C.c_void_p),
                                                      out.shape[0], C.byref(n), self._sp()), "frontier_into")
        return int(n.value)

    def frontier_scores(self) -> np.ndarray:
        c = self._read_ctrl()
        parity = c.depth & 1
        k = int(c.frontier_count[parity])
        t = self.buffers["score_current" if parity == 0 else "score_next"]
        return t[:k].cpu().numpy().astype(np.uint32)

    def frontier_payloads(self) -> np.ndarray:
        """Back-pointers (parent, rank, move packed) of the current frontier rows; depth must be >= 1."""
        c = self._read_ctrl()
        k = int(c.frontier_count[c.depth & 1])
        h = self.buffers["history_payload"]
        return h[(c.depth - 1) % h.shape[0], :k].cpu().numpy().astype(np.uint32)

    def history_layer(self, depth: int, count: int) -> np.ndarray:
        """Packed back-pointers of the first ``count`` rows of the depth ``depth``+1 frontier (valid until the ring of
        history rows wraps past it)."""
        h = self.buffers["history_payload"]
        return h[depth % h.shape[0], :count].cpu().numpy().astype(np.uint32)

    def current_state_bytes(self, i: int) -> bytes:
        c = self._read_ctrl()
        parity = c.depth & 1
        if i < 0 or i >= int(c.frontier_count[parity]):
            raise RuntimeError("frontier index out of range")
        return bytes(self._frontier_tensor(parity)[i, : int(self.cfg["state_len"])].cpu().numpy())

    def history_entry(self, depth: int, local_index: int) -> Dict[str, int]:
        """Back-pointer of row ``local_index`` of the depth ``depth``+1 frontier (beam_engine.cpp:1200-1219)."""
        from .records import unpack_payload
        h = self.buffers["history_payload"]
        # the device keeps the last h.shape[0] layers as a ring (row = depth mod rows): older layers were overwritten
        newest = int(self._ctrl.depth) - 1
        if depth < 0 or depth > newest or depth <= newest - h.shape[0] or local_index < 0 or local_index >= h.shape[1]:
            return {"valid": 0, "parent_idx": -1, "parent_rank": -1, "action": -1}
        payload = int(h[depth % h.shape[0], local_index].item()) & 0xFFFFFFFF
        p, r, m = unpack_payload(payload)
        return {"valid": 1, "parent_idx": int(p), "parent_rank": int(r), "action": int(m)}

    def reconstruct_path(self) -> Optional[List[int]]:
        """Moves from the start state to the solved state after a successful single-GPU search."""
        from .records import unpack_payload
        c = self._read_ctrl()
        if not c.found:
            return None
        if c.found_depth == 0:
            return []
        if c.found_payload == 0xFFFFFFFF or int(self.cfg["world_size"]) > 1:
            return None
        p, _, m = unpack_payload(c.found_payload)
        moves = [int(m)]
        idx = int(p)
        hist = self.buffers["history_payload"]
        if c.found_depth - 1 > hist.shape[0]:
            raise RuntimeError(f"the device keeps {hist.shape[0]} history layers but the path has {c.found_depth - 1}: "
                               "walk back through CPUHistoryArchive.path_to, or size history_rows / max_depth to the search")
        for d in range(c.found_depth - 2, -1, -1):
            pp, _, mm = unpack_payload(int(hist[d % hist.shape[0], idx].item()) & 0xFFFFFFFF)
            moves.append(int(mm))
            idx = int(pp)
        return moves[::-1]


def balanced_exchange_plan(counts: List[int], rank: int):
    """Who sends how many rows to whom when a frontier held as ``counts[q]`` rows on rank q (numbered g = 0..K-1 in
    rank-major order) is rebalanced so that row g lives on rank min(g * W // K, W - 1), i.e. rank q holds the run
    ceil(K q / W) .. ceil(K (q + 1) / W) (production_v6_dispatcher.py:584-588).  Returns for ``rank``: rows it sends
    to each rank, rows it receives from each rank (both in rank order, which is also global order), and every rank's
    share afterwards."""
    world = len(counts)
    total = sum(counts)
    base = [sum(counts[:q]) for q in range(world + 1)]
    lo = [-(-total * q // world) for q in range(world + 1)]  # ceil(K q / W): first global index of rank q

    def overlap(a0, a1, b0, b1):
        return max(0, min(a1, b1) - max(a0, b0))

    send = [overlap(base[rank], base[rank + 1], lo[q], lo[q + 1]) for q in range(world)]
    recv = [overlap(base[q], base[q + 1], lo[rank], lo[rank + 1]) for q in range(world)]
    return send, recv, [lo[q + 1] - lo[q] for q in range(world)]


def create_nccl_id(ext: _Ext, cfg: Dict[str, Any]) -> bytes:
    """Rank 0 creates the id, every rank receives it over torch.distributed (beam_engine.py:512-519)."""
    if cfg["world_size"] <= 1:
        return bytes(128)
    obj = [ext.get_nccl_unique_id() if cfg["rank"] == 0 else None]
    dist.broadcast_object_list(obj, src=0)
    return obj[0]


def configure_engine(puzzle: Puzzle, cfg: Optional[Dict[str, Any]] = None, scorer=None, **overrides: Any):
    """Build, allocate, construct and wire one engine for a puzzle (configure_engine, beam_engine.py:2553-2603)."""
    cfg = dict(cfg) if cfg is not None else config_for_puzzle(puzzle, **overrides)
    ext = build_extension(verbose=False)
    init_distributed_if_needed(cfg)
    if scorer is not None:
        cfg["inference_backend"] = "mlp"
    buffers = allocate_buffers(ext, cfg)
    engine = ext.BeamEngine(cfg, buffers, cfg["inference_backend"])
    engine.set_action_permutation_table(puzzle.action_table_bytes())
    engine.set_central_state(bytes(puzzle.solved))
    if scorer is not None:
        engine.set_scorer(scorer)
    if cfg["world_size"] > 1:
        engine.init_nccl(create_nccl_id(ext, cfg))
        engine.map_peers()
    engine.enable_cuda_graphs(bool(cfg.get("use_cuda_graphs", True)))
    return ext, cfg, buffers, engine


def make_shallow_scramble(puzzle: Puzzle, actions) -> np.ndarray:
    """The solved state with ``actions`` (move indices) applied in order (make_shallow_scramble,
    beam_engine.py:2627-2631)."""
    state = puzzle.solved.copy()
    for a in actions:
        state = state[puzzle.generators[int(a)].astype(np.int64)]
    return state.astype(np.uint8)


def run_one_search(engine: BeamEngine, state: np.ndarray, max_depth: int) -> Dict[str, Any]:
    """Reset on the owner rank and search (run_one_search, beam_engine.py)."""
    state = np.ascontiguousarray(state, dtype=np.uint8)
    world, rank = int(engine.cfg["world_size"]), int(engine.cfg["rank"])
    n = int(engine.cfg["state_len"])
    owner = engine.owner_of(state)
    engine.reset_search(bytes(state), active_on_this_rank=(owner == rank))
    return engine.search(max_depth)
