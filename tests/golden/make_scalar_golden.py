"""Generate tests/golden/scalar_reference.json from the reference's own scalar functions.

Run in a container that has the reference checkout:

    make -C oracle REF=/path/to/reference
    python tests/golden/make_scalar_golden.py

The Makefile compiles the reference's per-state device functions (hash_state_120, fingerprint_state_120, tie16,
make_best_key, apply_move_table, hamming_to_central, is_central_state, apply_move_state128, is_goal_state128,
hash_state128_zobrist, owner_from_hash128, candidate_better) and the host helpers of its beam_types.hpp as host
C++ into oracle/_ref/libref_scalar.so; this script calls them on seeded inputs and records the outputs.  The
tests regenerate the inputs from the recorded seeds, so only seeds and outputs are stored.
"""

import ctypes as C
import json
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
U64 = np.uint64


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def legacy_tables(seed: int):
    """Seeded stand-ins for the two uploaded tables of the legacy kernels: 24 random permutations of 120
    positions and a central state with values 0..119."""
    rng = np.random.default_rng(seed)
    table = np.stack([rng.permutation(120) for _ in range(24)]).astype(np.uint8)
    central = rng.integers(0, 120, size=120, dtype=np.uint8)
    return table, central


def v6_tables(seed: int, moves: int = 24):
    """Seeded State128 generators ([moves, 128], a permutation of the first 120 positions, padding positions map to
    themselves), a central state and a Zobrist table [128, 128, 2] of {lo, hi}."""
    rng = np.random.default_rng(seed)
    gens = np.tile(np.arange(128, dtype=np.uint8), (moves, 1))
    for m in range(moves):
        gens[m, :120] = rng.permutation(120).astype(np.uint8)
    central = np.zeros(128, dtype=np.uint8)
    central[:120] = rng.integers(0, 120, size=120, dtype=np.uint8)
    zob = rng.integers(0, np.iinfo(np.uint64).max, size=(128, 128, 2), dtype=np.uint64)
    return gens, central, zob


def main() -> None:
    so = ROOT / "oracle" / "_ref" / "libref_scalar.so"
    if not so.exists():
        raise SystemExit(f"{so} missing: run `make -C oracle REF=/path/to/reference` first")
    lib = C.CDLL(str(so))
    lib.ref_mix64.restype = C.c_uint64
    lib.ref_mix64.argtypes = [C.c_uint64]
    lib.ref_hash_state_120.restype = C.c_uint64
    lib.ref_hash_state_120.argtypes = [C.c_void_p]
    lib.ref_fingerprint_state_120.restype = C.c_uint64
    lib.ref_fingerprint_state_120.argtypes = [C.c_void_p]
    lib.ref_tie16.restype = C.c_uint32
    lib.ref_tie16.argtypes = [C.c_uint64]
    lib.ref_make_best_key.restype = C.c_uint32
    lib.ref_make_best_key.argtypes = [C.c_uint32, C.c_uint64]
    lib.ref_set_action_table.argtypes = [C.c_void_p, C.c_int]
    lib.ref_set_central_state.argtypes = [C.c_void_p, C.c_int]
    lib.ref_apply_move_table.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
    lib.ref_hamming_to_central.argtypes = [C.c_void_p]
    lib.ref_is_central_state.argtypes = [C.c_void_p]
    lib.ref_apply_move_state128.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    lib.ref_is_goal_state128.argtypes = [C.c_void_p, C.c_void_p]
    lib.ref_hash_state128_zobrist.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ref_owner_from_hash128.restype = C.c_uint32
    lib.ref_owner_from_hash128.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32]
    lib.ref_candidate_better.argtypes = [C.c_uint32, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint32]
    lib.ref_q_to_score_key.restype = C.c_uint32
    lib.ref_q_to_score_key.argtypes = [C.c_float]
    lib.ref_pack_route.restype = C.c_uint32
    lib.ref_pack_route.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
    lib.ref_threshold_update.restype = C.c_uint32
    lib.ref_threshold_update.argtypes = [C.c_uint32, C.POINTER(C.c_int), C.c_uint64, C.c_uint64, C.c_uint32]

    assert lib.ref_state_len() == 120 and lib.ref_fanout() == 24
    out = {"state_size": 120, "fanout": 24}

    # --- mix64, hash, fingerprint, tie16, best key on seeded random states ------------------------------
    mix_in = [0, 1, 2, 0xFFFFFFFFFFFFFFFF, 0x9E3779B97F4A7C15, 0x0123456789ABCDEF]
    out["mix64"] = [{"x": x, "y": int(lib.ref_mix64(x))} for x in mix_in]
    cases = []
    states = [("arange", 0, np.arange(120, dtype=np.uint8)), ("zeros", 0, np.zeros(120, dtype=np.uint8))]
    for seed in range(1, 49):
        rng = np.random.default_rng(910000 + seed)
        hi = (6, 120, 256)[seed % 3]
        states.append((f"uniform{hi}", 910000 + seed, rng.integers(0, hi, size=120, dtype=np.uint8)))
    for kind, seed, s in states:
        s = np.ascontiguousarray(s)
        fp = int(lib.ref_fingerprint_state_120(_ptr(s)))
        score_q = (seed * 2654435761) & 0xFFFF
        cases.append({"kind": kind, "seed": seed, "hash64": int(lib.ref_hash_state_120(_ptr(s))),
                      "fingerprint64": fp, "tie16": int(lib.ref_tie16(fp)), "score_q": score_q,
                      "best_key": int(lib.ref_make_best_key(score_q, fp))})
    out["state_cases"] = cases

    # --- legacy expansion + Hamming + goal test on a seeded table -------------------------------------------
    table_seed = 920001
    table, central = legacy_tables(table_seed)
    lib.ref_set_action_table(_ptr(table), 1)
    lib.ref_set_central_state(_ptr(central), 1)
    exp = []
    for j in range(6):
        rng = np.random.default_rng(920100 + j)
        parent = rng.integers(0, 120, size=120, dtype=np.uint8) if j else central.copy()
        children = np.zeros((24, 120), dtype=np.uint8)
        ham = []
        for a in range(24):
            lib.ref_apply_move_table(_ptr(parent), a, _ptr(children[a]))
            ham.append(int(lib.ref_hamming_to_central(_ptr(children[a]))))
        exp.append({
            "parent_seed": 920100 + j if j else None,  # None: the central state itself
            "child_hash64": [int(lib.ref_hash_state_120(_ptr(np.ascontiguousarray(children[a])))) for a in range(24)],
            "child_fingerprint64": [int(lib.ref_fingerprint_state_120(_ptr(np.ascontiguousarray(children[a]))))
                                    for a in range(24)],
            "child_hamming": ham,
            "child_bytes_move0": children[0].tolist(),
            "parent_is_central": int(lib.ref_is_central_state(_ptr(parent))),
            "parent_hamming": int(lib.ref_hamming_to_central(_ptr(parent))),
        })
    out["legacy_expand"] = {"table_seed": table_seed, "cases": exp}

    # --- v6: State128 expansion, goal test, Zobrist hash, owner rule ----------------------------------------
    v6_seed = 930001
    gens, central128, zob = v6_tables(v6_seed)
    zob_c = np.ascontiguousarray(zob)
    v6 = []
    for j in range(4):
        rng = np.random.default_rng(930100 + j)
        parent = np.zeros(128, dtype=np.uint8)
        parent[:120] = rng.integers(0, 120, size=120, dtype=np.uint8) if j else central128[:120]
        lo_hi, owners, goal = [], [], []
        child = np.zeros(128, dtype=np.uint8)
        first_child = None
        for m in range(24):
            lib.ref_apply_move_state128(_ptr(parent), _ptr(gens), m, _ptr(child))
            if m == 0:
                first_child = child.copy()
            h = np.zeros(2, dtype=np.uint64)
            lib.ref_hash_state128_zobrist(_ptr(child), _ptr(zob_c), _ptr(h))
            lo_hi.append([int(h[0]), int(h[1])])
            owners.append([int(lib.ref_owner_from_hash128(int(h[1]), int(h[0]), w)) for w in (1, 2, 3, 8)])
            goal.append(int(lib.ref_is_goal_state128(_ptr(child), _ptr(central128))))
        v6.append({"parent_seed": 930100 + j if j else None, "child_lo_hi": lo_hi, "owner_w1_2_3_8": owners,
                   "child_is_goal": goal, "child_bytes_move0": first_child.tolist(),
                   "parent_is_goal": int(lib.ref_is_goal_state128(_ptr(parent), _ptr(central128)))})
    out["v6_expand"] = {"seed": v6_seed, "cases": v6}

    # --- duplicate winner order (candidate_better) on seeded pairs with forced ties --------------------------
    rng = np.random.default_rng(940001)
    pairs = []
    for j in range(64):
        sa, sb = int(rng.integers(0, 4)), int(rng.integers(0, 4))
        pa, pb = int(rng.integers(0, 3)), int(rng.integers(0, 3))
        ra = int(lib.ref_pack_route(int(rng.integers(0, 3)), int(rng.integers(0, 2)), int(rng.integers(0, 3))))
        rb = int(lib.ref_pack_route(int(rng.integers(0, 3)), int(rng.integers(0, 2)), int(rng.integers(0, 3))))
        pairs.append({"a": [sa, pa, ra], "b": [sb, pb, rb],
                      "a_better": int(lib.ref_candidate_better(sa, pa, ra, sb, pb, rb))})
    out["candidate_better"] = pairs
    out["pack_route"] = [{"args": [r, o, m], "packed": int(lib.ref_pack_route(r, o, m))}
                         for r, o, m in ((0, 0, 0), (1, 0, 5), (7, 3, 23), (15, 1, 31))]

    # --- score key and monotone threshold -------------------------------------------------------------------
    qs = [-5.0, 0.0, 0.001, 0.0019, 0.00196, 1.0, 17.3333, 149.998, 299.999, 300.0, 301.0, 1e9]
    out["q_to_score_key"] = [{"q": q, "key": int(lib.ref_q_to_score_key(q))} for q in qs]
    seq = []
    cur, init = 0xFFFFFFFF, C.c_int(0)
    for total, new in ((10, 500), (99, 400), (100, 300), (150, 350), (120, 200), (50, 100), (100, 250)):
        cur = int(lib.ref_threshold_update(cur, C.byref(init), total, 100, new))
        seq.append({"total": total, "beam": 100, "new": new, "threshold": cur, "initialised": int(init.value)})
    out["threshold_update"] = seq

    dst = Path(__file__).resolve().parent / "scalar_reference.json"
    dst.write_text(json.dumps(out, separators=(",", ":")))
    print(f"wrote {dst}: {len(cases)} state cases, {len(exp)} legacy expansions, {len(v6)} v6 expansions")


if __name__ == "__main__":
    main()
