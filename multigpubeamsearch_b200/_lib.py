"""ctypes binding of libmgbs_b200.so (the C ABI declared in include/mgbs.h).

There is no fallback: if the library is missing or a symbol cannot be resolved, loading raises.  The structures
below mirror MgbsRadix / MgbsCtrl / MgbsConfig field for field; their sizes are checked against the library.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import build as _build

RADIX_BINS = 2048
HIST_STRIDE = 2096
MAX_LEVELS = 6
MAX_ROUNDS = 8
TIE_CAP = 256
TIE_SEG_WORDS = 1 + 3 * TIE_CAP
MAX_WORLD = 16
MAX_FANOUT = 32
MAX_STATE_LEN = 128

SELECT_MODES = {"exact_k": 0, "v6_inclusive": 1, "legacy_strict": 2}
SCORE_EXTERNAL, SCORE_HAMMING, SCORE_UNIFORM = 0, 1, 2

ST_HASH_OVERFLOW = 1
ST_BAND_STALL = 2
ST_TIE_OVERFLOW = 4
ST_FRONTIER_OVERFLOW = 8
ST_BUCKET_OVERFLOW = 16
ST_ROUNDS_EXHAUSTED = 32
ST_PEER_TIMEOUT = 64
ST_GRID_TIMEOUT = 128
STATUS_NAMES = {
    ST_HASH_OVERFLOW: "hash_overflow", ST_BAND_STALL: "band_stall", ST_TIE_OVERFLOW: "tie_overflow",
    ST_FRONTIER_OVERFLOW: "frontier_overflow", ST_BUCKET_OVERFLOW: "bucket_overflow",
    ST_ROUNDS_EXHAUSTED: "rounds_exhausted", ST_PEER_TIMEOUT: "peer_timeout", ST_GRID_TIMEOUT: "grid_timeout",
}


class MgbsRadix(C.Structure):
    _fields_ = [
        ("prefix", C.c_uint64), ("remaining", C.c_uint64), ("bits_done", C.c_uint32), ("done", C.c_uint32),
        ("flag", C.c_uint32), ("pad", C.c_uint32), ("result", C.c_uint64), ("tie_key", C.c_uint64),
        ("tie_need", C.c_uint64), ("kept_below", C.c_uint64),
    ]


class MgbsCtrl(C.Structure):
    _fields_ = [
        ("depth", C.c_int32), ("frontier_count", C.c_int32 * 2), ("found", C.c_int32),
        ("found_payload", C.c_uint32), ("found_depth", C.c_int32), ("status", C.c_uint32),
        ("table_count", C.c_uint32), ("next_count", C.c_uint32), ("tie_count", C.c_uint32),
        ("cand_count", C.c_uint32), ("unique_total", C.c_uint32), ("inserted_total", C.c_uint32),
        ("hash_overflow", C.c_uint32), ("rounds_used", C.c_uint32), ("bands_done", C.c_uint32),
        ("epoch", C.c_uint32), ("active_rows", C.c_int32),
        ("band_lo", C.c_uint64 * (MAX_ROUNDS + 1)), ("threshold_key", C.c_uint64),
        ("rho_num", C.c_uint64), ("rho_den", C.c_uint64), ("total_candidates", C.c_uint64),
        ("halt", C.c_uint32), ("exhausted", C.c_uint32), ("grid_bar", C.c_uint32), ("win_lo", C.c_uint32),
        ("launch_seq", C.c_uint64),
        ("band", (MgbsRadix * (MAX_LEVELS + 1)) * MAX_ROUNDS), ("fin", MgbsRadix * (MAX_LEVELS + 1)),
    ]


_P = C.c_void_p


class MgbsConfig(C.Structure):
    _fields_ = [
        ("state_len", C.c_int32), ("state_stride", C.c_int32), ("fanout", C.c_int32), ("world_size", C.c_int32),
        ("rank", C.c_int32), ("select_mode", C.c_int32), ("score_mode", C.c_int32), ("hash_bits", C.c_int32),
        ("band_levels", C.c_int32), ("band_rounds", C.c_int32), ("probe_limit", C.c_int32),
        ("uniform_score", C.c_int32),
        ("global_beam_width", C.c_int64), ("frontier_cap", C.c_int64), ("pool_target", C.c_int64),
        ("hash_capacity", C.c_int64), ("cand_cap", C.c_int64), ("bucket_cap", C.c_int64),
        ("history_depths", C.c_int64),
        ("frontier", _P * 2), ("gens", _P), ("solved", _P), ("children", _P),
        ("cand_hash", _P), ("cand_fp", _P), ("cand_score", _P), ("cand_payload", _P),
        ("table", _P), ("hist", _P), ("tie_buf", _P), ("history", _P),
        ("frontier_hash", _P * 2), ("frontier_score", _P * 2), ("ctrl", _P),
        ("send_hash", _P), ("send_fp", _P), ("send_score", _P), ("send_payload", _P), ("send_states", _P),
        ("recv_hash", _P), ("recv_fp", _P), ("recv_score", _P), ("recv_payload", _P), ("recv_states", _P),
        ("send_counts", _P), ("recv_counts", _P),
        ("exchange_mode", C.c_int32), ("pad1", C.c_int32), ("sym", _P), ("sym_bytes", C.c_int64), ("tickets", _P),
        ("io_stage", _P), ("hash_mode", C.c_int32), ("zobrist_values", C.c_int32), ("zobrist", _P),
        ("host_mirror", _P), ("peer_poll_limit", C.c_int64), ("staged_select", C.c_int32), ("pad2", C.c_int32),
    ]


class MgbsMirror(C.Structure):
    _fields_ = [
        ("depth", C.c_int32), ("found", C.c_int32), ("found_depth", C.c_int32), ("frontier_next", C.c_int32),
        ("found_payload", C.c_uint32), ("status", C.c_uint32), ("unique_total", C.c_uint32), ("epoch", C.c_uint32),
        ("total_candidates", C.c_uint64), ("seq", C.c_uint64),
    ]


# name -> (restype, argtypes); every symbol include/mgbs.h declares
_I32, _I64, _U8P = C.c_int32, C.c_int64, C.POINTER(C.c_uint8)
SIGNATURES = {
    "mgbs_version": (C.c_int, []),
    "mgbs_sizeof_ctrl": (C.c_int, []),
    "mgbs_sizeof_config": (C.c_int, []),
    "mgbs_derive_sizes": (C.c_int, [_I64, _I32, C.c_double, C.c_double, C.c_double, _I32, _I32, C.POINTER(_I64)]),
    "mgbs_engine_create": (C.c_int, [C.POINTER(MgbsConfig), C.POINTER(_P)]),
    "mgbs_engine_destroy": (C.c_int, [_P]),
    "mgbs_nccl_unique_id": (C.c_int, [C.c_char_p, _P]),
    "mgbs_engine_init_nccl": (C.c_int, [_P, C.c_char_p, _P]),
    "mgbs_engine_set_parent_scorer": (C.c_int, [_P, _P, _P]),
    "mgbs_sym_bytes": (C.c_int, [C.POINTER(MgbsConfig), C.POINTER(_I64), C.POINTER(_I64)]),
    "mgbs_sym_frontier_offsets": (C.c_int, [C.POINTER(MgbsConfig), C.POINTER(_I64)]),
    "mgbs_engine_set_peers": (C.c_int, [_P, _P, C.POINTER(_I64)]),
    "mgbs_engine_set_peer_pointers": (C.c_int, [_P, C.POINTER(_P)]),
    "mgbs_engine_set_logical_limits": (C.c_int, [_P, _I64, _I64]),
    "mgbs_ipc_export": (C.c_int, [_P, _P, C.POINTER(_I64)]),
    "mgbs_engine_set_scorer": (C.c_int, [_P, _P, _P]),
    "mgbs_engine_set_score_mode": (C.c_int, [_P, _I32, _I32]),
    "mgbs_engine_reset": (C.c_int, [_P, _P, _I32, _I32, _P]),
    "mgbs_engine_load_frontier": (C.c_int, [_P, _P, _I64, _I32, _I32, _P]),
    "mgbs_engine_read_frontier": (C.c_int, [_P, _I32, _P, _I64, C.POINTER(_I64), _P]),
    "mgbs_engine_enqueue_depth": (C.c_int, [_P, _I32, _I32, _P]),
    "mgbs_engine_step_graph": (C.c_int, [_P, _I32, _P]),
    "mgbs_engine_profile": (C.c_int, [_P, _I32]),
    "mgbs_engine_profile_read": (C.c_int, [_P, C.POINTER(C.c_float)]),
    "mgbs_engine_trace_read": (C.c_int, [_P, C.POINTER(C.c_float), _I32]),
    "mgbs_engine_read_ctrl": (C.c_int, [_P, C.POINTER(MgbsCtrl), _P]),
    "mgbs_engine_search": (C.c_int, [_P, _I32, _I32, C.POINTER(MgbsCtrl), _P]),
    "mgbs_launch_expand": (C.c_int, [_P, _P, _I64, _P, _P, _I32, _I32, _I32, _I32, _I32, _I32, _P, _P, _P, _P, _P, _P, _P]),
    "mgbs_hash64_host": (C.c_uint64, [_P, _I32]),
    "mgbs_fingerprint64_host": (C.c_uint64, [_P, _I32]),
}

_lib = None


def library_path() -> Path:
    return _build.LIB


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load the shared library (building it in-tree first if asked and needed); raise if that is impossible."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if build_if_missing and _build.needs_build():
        _build.build()
    if not path.exists():
        raise RuntimeError(f"{path} is missing: run `python -m multigpubeamsearch_b200.build` (there is no CPU fallback)")
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is absent
        fn.restype = res
        fn.argtypes = args
    if lib.mgbs_sizeof_ctrl() != C.sizeof(MgbsCtrl) or lib.mgbs_sizeof_config() != C.sizeof(MgbsConfig):
        raise RuntimeError("structure layout mismatch between _lib.py and libmgbs_b200.so")
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    """C++ errors become RuntimeError, as CUDA_CHECK / NCCL_CHECK do in the reference (beam_engine.cpp:34-46)."""
    if rc == 0:
        return
    names = {-1: "bad argument", -2: "unsupported shape", -3: "NCCL error", -4: "bad engine state",
             -5: "request too large", -6: "a cross-rank wait gave up (peer timeout)"}
    if rc < 0:
        raise RuntimeError(f"{what}: {names.get(rc, rc)}")
    raise RuntimeError(f"{what}: CUDA error {rc}")
