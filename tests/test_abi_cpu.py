"""CPU checks of the C ABI: the library loads, exports every symbol the header declares, and its host-only helpers
(size derivation, structure sizes, host hash) agree with the oracle and the reference's formulas.  No compute calls."""

import ctypes as C
import re
from pathlib import Path

import numpy as np

from oracle import beam_oracle as bo
from multigpubeamsearch_b200 import _lib, scorers, beam_engine as be

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "mgbs.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mgbs_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_structure_sizes_match_ctypes_mirrors():
    lib = _lib.load()
    assert lib.mgbs_sizeof_ctrl() == C.sizeof(_lib.MgbsCtrl)
    assert lib.mgbs_sizeof_config() == C.sizeof(_lib.MgbsConfig)
    lib.mgbs_sizeof_mlp_config.restype = C.c_int
    lib.mgbs_sizeof_tf_config.restype = C.c_int
    assert lib.mgbs_sizeof_mlp_config() == C.sizeof(scorers.MgbsMlpConfig)
    assert lib.mgbs_sizeof_tf_config() == C.sizeof(scorers.MgbsTfConfig)


def test_derive_sizes_follow_reference_formulas():
    # EngineConfig::derive (beam_engine.cpp:244-252): n_local = ceil(B/W), k_keep = round(gamma n_local),
    # k_work = round(beta k_keep), hash_capacity = max(1024, round(k_work / load))
    ext = be._Ext(_lib.load())
    cfg = be.make_default_config()
    cfg.update(global_beam_width=65536, world_size=2, gamma=1.05, beta=1.2, hash_load_factor=0.45, fanout=12,
               state_size_bytes=64, max_depth=10, band_rounds=3, band_levels=3)
    s = ext.derive_sizes(cfg)
    assert s["n_local"] == 32768 and s["k_keep"] == 34406 and s["k_work"] == 41287
    assert s["hash_capacity"] == round(41287 / 0.45)
    assert s["cand_cap"] == 41287 * 12 and s["bucket_cap_per_peer"] > s["cand_cap"] // 2
    cfg.update(global_beam_width=100, world_size=1)
    assert ext.derive_sizes(cfg)["hash_capacity"] == 1024
    lib = _lib.load()
    out = (C.c_int64 * 6)()
    assert lib.mgbs_derive_sizes(0, 1, 1.05, 1.2, 0.45, 3, 3, out) == -1        # bad beam
    assert lib.mgbs_derive_sizes(100, 1, 1.05, 1.2, 1.5, 3, 3, out) == -1      # bad load factor
    assert lib.mgbs_derive_sizes(100, 99, 1.05, 1.2, 0.45, 3, 3, out) == -1    # too many ranks


def test_host_hash_matches_oracle():
    lib = _lib.load()
    rng = np.random.default_rng(3)
    for n in (16, 54, 96, 120):
        s = np.ascontiguousarray(rng.integers(0, 8, size=(5, n), dtype=np.uint8))
        want_h, want_f = bo.hash64(s), bo.fingerprint64(s)
        for i in range(5):
            row = np.ascontiguousarray(s[i])
            assert lib.mgbs_hash64_host(row.ctypes.data_as(C.c_void_p), n) == int(want_h[i])
            assert lib.mgbs_fingerprint64_host(row.ctypes.data_as(C.c_void_p), n) == int(want_f[i])


def test_host_hash_matches_reference_device_functions():
    """The library's host helpers against vectors produced by the reference's own hash_state_120 /
    fingerprint_state_120 (beam_kernels.cu:38-59) compiled as host C++ (tests/golden/make_scalar_golden.py)."""
    import json
    lib = _lib.load()
    data = json.loads((ROOT / "tests" / "golden" / "scalar_reference.json").read_text())
    for c in data["state_cases"]:
        if c["kind"] == "arange":
            s = np.arange(120, dtype=np.uint8)
        elif c["kind"] == "zeros":
            s = np.zeros(120, dtype=np.uint8)
        else:
            s = np.random.default_rng(c["seed"]).integers(0, int(c["kind"][7:]), size=120, dtype=np.uint8)
        s = np.ascontiguousarray(s)
        assert lib.mgbs_hash64_host(s.ctypes.data_as(C.c_void_p), 120) == c["hash64"]
        assert lib.mgbs_fingerprint64_host(s.ctypes.data_as(C.c_void_p), 120) == c["fingerprint64"]


def test_engine_create_rejects_bad_configs_without_a_gpu():
    lib = _lib.load()
    c = _lib.MgbsConfig()
    h = C.c_void_p()
    assert lib.mgbs_engine_create(C.byref(c), C.byref(h)) == -1  # empty config
    c.state_len, c.state_stride, c.fanout, c.world_size = 54, 48, 12, 1
    assert lib.mgbs_engine_create(C.byref(c), C.byref(h)) == -1  # stride smaller than the state
    nb, nt = C.c_int64(0), C.c_int64(0)
    c.state_stride, c.world_size, c.bucket_cap, c.band_rounds, c.band_levels, c.hash_bits = 64, 4, 1000, 3, 3, 44
    c.frontier_cap = 500
    assert lib.mgbs_sym_bytes(C.byref(c), C.byref(nb), C.byref(nt)) == 0
    # two parities of (hash, fp, score, payload) record buckets + two frontier buffers + counts, flags, histogram slots
    assert nb.value > 2 * 4 * 1000 * (8 + 8 + 4 + 4) + 2 * 500 * 64 and nt.value == 3 * 3 + 6 + 1
    offs = (C.c_int64 * 2)()
    assert lib.mgbs_sym_frontier_offsets(C.byref(c), offs) == 0
    assert offs[0] % 256 == 0 and offs[1] - offs[0] >= 500 * 64 and offs[1] + 500 * 64 <= nb.value


def test_python_surface_has_the_reference_names():
    """Every method the reference binds on BeamEngine (beam_engine.cpp:2114-2148), its module-level functions
    (beam_engine.py) and the names of its scorers.py / production_v6_dispatcher.py exist here."""
    from multigpubeamsearch_b200 import beam_engine as be
    from multigpubeamsearch_b200 import production_v6_dispatcher as pd
    from multigpubeamsearch_b200 import scorers
    methods = ["init_nccl", "load_torchscript_ensemble", "load_fullbeamnice_static", "begin_uniform_score",
               "set_uniform_score", "end_uniform_score", "warmup_inference", "benchmark_inference",
               "set_action_permutation_table", "set_central_state", "reset_search", "clear_runtime_state",
               "enable_cuda_graphs", "cuda_graph_captured", "enable_step_timers", "step_timing", "set_active_limit",
               "set_next_limit", "clear_logical_limits", "enable_debug", "step", "step_current", "step_prepass_fast",
               "set_prepass_light_solved_scan", "search", "status", "history_entry", "current_state_bytes", "sizes"]
    missing = [m for m in methods if not callable(getattr(be.BeamEngine, m, None))]
    assert not missing, missing
    for name in ("build_extension", "configure_engine", "allocate_buffers", "make_default_config", "init_distributed_if_needed",
                 "create_nccl_id", "make_shallow_scramble", "run_one_search"):
        assert callable(getattr(be, name, None)), name
    for name in ("MLPActionScorer", "QuantizedActionScorer", "make_default_mlp_scorer"):
        assert callable(getattr(scorers, name, None)), name
    assert callable(pd.ProductionV6Dispatcher.run_task)
    fields = set(pd.ProductionV6Result.__dataclass_fields__)
    assert {"task_id", "status", "path", "depth_rows", "solved_depth", "solved_rank", "solved_parent_idx",
            "solved_move", "raw_solved_record_exists", "path_replay_valid", "path_failure_reason"} <= fields
    for key in ("k_expand_tile", "score_ring_depth", "net_ring_depth", "inference_parallelism",
                "histogram_period_micro", "beta", "hash_load_factor", "probe_limit", "global_beam_width"):
        assert key in be.make_default_config(), key


def test_balanced_exchange_plan_matches_the_reference_placement():
    """Host arithmetic of the balanced placement against the oracle's balance_targets
    (production_v6_dispatcher.py:584-588) on ragged, empty and tiny frontiers."""
    from multigpubeamsearch_b200 import beam_engine as be
    from oracle import beam_oracle as bo
    rng = np.random.default_rng(4)
    cases = [[5, 0, 9, 2], [0, 0, 0], [1], [0, 7], [3, 3, 3, 3, 3, 3, 3, 4]]
    cases += [rng.integers(0, 50, size=int(w)).tolist() for w in rng.integers(1, 9, size=40)]
    for counts in cases:
        world, total = len(counts), sum(counts)
        t_rank, t_local = bo.balance_targets(total, world)
        owner_before = np.repeat(np.arange(world), counts)  # rank holding global row g before
        plans = [be.balanced_exchange_plan(counts, r) for r in range(world)]
        want_shares = [int((t_rank == q).sum()) for q in range(world)]
        for r, (send, recv, shares) in enumerate(plans):
            assert shares == want_shares
            assert sum(send) == counts[r] and sum(recv) == want_shares[r]
            for q in range(world):
                # rows that sit on r and belong on q, counted straight from the reference formula
                assert send[q] == int(((owner_before == r) & (t_rank == q)).sum()), (counts, r, q)
                assert recv[q] == plans[q][0][r]
        # local index after the move = position in the receiver's run
        for g in range(total):
            q = int(t_rank[g])
            first = -(-total * q // world)
            assert int(t_local[g]) == g - first
