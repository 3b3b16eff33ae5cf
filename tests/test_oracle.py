"""CPU checks that pin the oracle to the reference's own known answers."""

import json
from pathlib import Path

import numpy as np
import pytest

from oracle import beam_oracle as bo
from multigpubeamsearch_b200 import puzzles

GOLDEN = Path(__file__).resolve().parent / "golden"


def _golden_state(case):
    if case["kind"] == "arange":
        return np.arange(120, dtype=np.uint8)
    hi = int(case["kind"][len("uniform"):])
    return np.random.default_rng(case["seed"]).integers(0, hi, size=120, dtype=np.uint8)


def test_hash64_matches_reference_cpu_helper():
    data = json.loads((GOLDEN / "hash64_reference.json").read_text())
    assert data["state_size"] == 120
    states = np.stack([_golden_state(c) for c in data["cases"]])
    h = bo.hash64(states)
    assert [int(x) for x in h] == [c["hash64"] for c in data["cases"]]
    # the reference documents this value for the identity arrangement
    assert int(h[0]) == 0x64F5E55CD40D3123
    for w in (2, 3, 8):
        assert bo.owner_rank(h, w).tolist() == [c[f"owner_w{w}"] for c in data["cases"]]


def _scalar_golden():
    """Vectors produced by the reference's own scalar functions compiled as host C++ (oracle/Makefile,
    tests/golden/make_scalar_golden.py) and the seeded input generators of that script."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_scalar_golden", GOLDEN / "make_scalar_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return json.loads((GOLDEN / "scalar_reference.json").read_text()), mod


def _scalar_state(case):
    if case["kind"] == "arange":
        return np.arange(120, dtype=np.uint8)
    if case["kind"] == "zeros":
        return np.zeros(120, dtype=np.uint8)
    hi = int(case["kind"][len("uniform"):])
    return np.random.default_rng(case["seed"]).integers(0, hi, size=120, dtype=np.uint8)


def test_fingerprint_hash_and_best_key_match_reference_device_functions():
    """hash_state_120, fingerprint_state_120, tie16, make_best_key, mix64 (beam_kernels.cu:29-67)."""
    data, _ = _scalar_golden()
    assert data["state_size"] == 120 and data["fanout"] == 24
    for c in data["mix64"]:
        assert int(bo.mix64(np.array([c["x"]], dtype=np.uint64))[0]) == c["y"]
    cases = data["state_cases"]
    states = np.stack([_scalar_state(c) for c in cases])
    assert [int(x) for x in bo.hash64(states)] == [c["hash64"] for c in cases]
    fp = bo.fingerprint64(states)
    assert [int(x) for x in fp] == [c["fingerprint64"] for c in cases]
    assert [int(x) for x in bo.tie16(fp)] == [c["tie16"] for c in cases]
    score_q = np.array([c["score_q"] for c in cases], dtype=np.uint32)
    assert [int(x) for x in bo.make_best_key(score_q, fp)] == [c["best_key"] for c in cases]


def test_expansion_and_hamming_match_reference_device_functions():
    """apply_move_table, hamming_to_central, is_central_state (beam_kernels.cu:69-103) on a seeded table."""
    data, mod = _scalar_golden()
    table, central = mod.legacy_tables(data["legacy_expand"]["table_seed"])
    for c in data["legacy_expand"]["cases"]:
        parent = central.copy() if c["parent_seed"] is None else \
            np.random.default_rng(c["parent_seed"]).integers(0, 120, size=120, dtype=np.uint8)
        children = bo.expand(parent[None, :], table)
        assert children[0].tolist() == c["child_bytes_move0"]
        assert [int(x) for x in bo.hash64(children)] == c["child_hash64"]
        assert [int(x) for x in bo.fingerprint64(children)] == c["child_fingerprint64"]
        assert bo.hamming(children, central).tolist() == c["child_hamming"]
        assert int(bo.hamming(parent[None, :], central)[0]) == c["parent_hamming"]
        assert int(np.array_equal(parent, central)) == c["parent_is_central"]
        # the legacy u16 score of kernel_dummy_inference follows from the Hamming distance (beam_kernels.cu:133-143)
        assert bo.legacy_hamming_q(np.array(c["child_hamming"])).tolist() == \
            [65535 if h == 0 else max(65535 - 512 * h, 1) for h in c["child_hamming"]]


def test_v6_expansion_zobrist_and_owner_match_reference_device_functions():
    """apply_move_state128, is_goal_state128, hash_state128_zobrist (beam_kernels_stream2.cu:8-38),
    owner_from_hash128 (beam_kernels_stream3.cu:29-35)."""
    data, mod = _scalar_golden()
    gens, central, zob = mod.v6_tables(data["v6_expand"]["seed"])
    for c in data["v6_expand"]["cases"]:
        parent = np.zeros(128, dtype=np.uint8)
        parent[:120] = central[:120] if c["parent_seed"] is None else \
            np.random.default_rng(c["parent_seed"]).integers(0, 120, size=120, dtype=np.uint8)
        children = bo.expand(parent[None, :], gens)
        assert children[0].tolist() == c["child_bytes_move0"]
        lo, hi = bo.hash128_zobrist(children, zob)
        assert [[int(a), int(b)] for a, b in zip(lo, hi)] == c["child_lo_hi"]
        for k, w in enumerate((1, 2, 3, 8)):
            assert bo.owner_from_hash128(hi, lo, w).tolist() == [o[k] for o in c["owner_w1_2_3_8"]]
        assert [(int(np.array_equal(ch, central))) for ch in children] == c["child_is_goal"]
        assert int(np.array_equal(parent, central)) == c["parent_is_goal"]


def test_duplicate_winner_order_matches_reference_candidate_better():
    """candidate_better (beam_kernels_stream4.cu:25-33): (score, parent, route) lexicographic; the packed
    back-pointer of this build orders (parent, rank, move) the same way for equal owners."""
    data, _ = _scalar_golden()
    for c in data["pack_route"]:
        r, o, m = c["args"]
        assert (r << 16) | (o << 8) | m == c["packed"]
    for c in data["candidate_better"]:
        a, b = tuple(c["a"]), tuple(c["b"])
        assert int(a < b) == c["a_better"]
        # dedup_by_key keeps the minimum sort value: the winner of a two-element group is the better candidate
        won = bo.dedup_by_key(["k", "k"], [a, b])["k"]
        assert won == (a if c["a_better"] or a == b else b)


def test_score_key_and_monotone_threshold_match_reference_host_helpers():
    """q_to_score_key_host, threshold_update (beam_types.hpp:103-106, 125-134)."""
    data, _ = _scalar_golden()
    for c in data["q_to_score_key"]:
        assert int(bo.q_to_score_key(np.array([c["q"]], dtype=np.float32))[0]) == c["key"]
    cur, init = bo.UINT32_MAX, False
    for c in data["threshold_update"]:
        cur, init = bo.v6_threshold_update(cur, init, c["total"], c["beam"], c["new"])
        assert cur == c["threshold"] and int(init) == c["initialised"]


def test_hash64_scalar_definition():
    # independent scalar restatement with Python ints
    rng = np.random.default_rng(5)
    for n in (16, 54, 96, 120):
        s = rng.integers(0, 8, size=(7, n), dtype=np.uint8)
        for row, got_h, got_f in zip(s, bo.hash64(s), bo.fingerprint64(s)):
            h = bo.FNV_OFFSET
            f = bo.GOLDEN
            for v in row.tolist():
                h = ((h ^ v) * bo.FNV_PRIME) & bo.MASK64
                f ^= (v + bo.GOLDEN + (f << 6) + (f >> 2)) & bo.MASK64
                f &= bo.MASK64

            def mix(x):
                x ^= x >> 33
                x = (x * 0xFF51AFD7ED558CCD) & bo.MASK64
                x ^= x >> 33
                x = (x * 0xC4CEB9FE1A85EC53) & bo.MASK64
                x ^= x >> 33
                return x

            h = mix(h)
            if h in (0, 1, 2):
                h += 4
            f = mix(f ^ bo.FP_XOR)
            if f == 0:
                f = 4
            assert int(got_h) == h and int(got_f) == f


def test_dedup_known_answers_stream3():
    # tests/stream3_dedup_smoke.py:73-147: duplicates resolve to the min (score, payload)
    a, b, c = (0x101, 0xAAA), (0x202, 0xBBB), (0x303, 0xCCC)
    keys = [a, a, b, b, c]
    vals = [(50, 0), (40, 1), (40, 2), (40, 3), (10, 24)]
    best = bo.dedup_by_key(keys, vals)
    assert best == {a: (40, 1), b: (40, 2), c: (10, 24)}


def test_dedup_known_answers_stream4():
    # tests/stream4_shard_smoke.py:45-105: score beats parent beats route; threshold 100 drops score 200
    a, b, c, d = (0x101, 0xAAA), (0x202, 0xBBB), (0x303, 0xCCC), (0x404, 0xDDD)
    metas = [(a, 10, 80, 0x010101), (b, 20, 90, 0x020202), (a, 9, 70, 0x030303),
             (b, 19, 90, 0x040404), (c, 30, 200, 0x050505), (d, 40, 10, 0x060606)]
    kept = [(k, (score, parent, route)) for k, parent, score, route in metas if score <= 100]
    best = bo.dedup_by_key([k for k, _ in kept], [v for _, v in kept])
    assert best[a] == (70, 9, 0x030303)
    assert best[b] == (90, 19, 0x040404)
    assert best[d] == (10, 40, 0x060606)
    assert c not in best and len(best) == 3


def test_threshold_rules():
    # beam_engine.py:1662-1759: six survivors [10,20,40 | 30,50,60], beam 6 -> T = 60
    assert bo.v6_histogram_threshold([10, 20, 40, 30, 50, 60], 6) == 60
    assert bo.v6_histogram_threshold([10, 20, 40, 30, 50, 60], 3) == 30
    assert bo.v6_histogram_threshold([], 3) == bo.UINT32_MAX
    assert bo.v6_histogram_threshold([1, 2], 3) == bo.UINT32_MAX
    # beam_types.hpp:125-134: unset until enough survivors, then monotone
    assert bo.v6_threshold_update(bo.UINT32_MAX, False, 5, 6, 77) == (bo.UINT32_MAX, False)
    assert bo.v6_threshold_update(bo.UINT32_MAX, False, 6, 6, 60) == (60, True)
    assert bo.v6_threshold_update(60, True, 9, 6, 80) == (60, True)
    assert bo.v6_threshold_update(60, True, 9, 6, 40) == (40, True)
    assert bo.v6_threshold_update(60, True, 2, 6, 10) == (60, True)
    # beam_kernels.cu:657-680
    assert bo.legacy_threshold([5, 5, 7, 9], 2) == (True, 7)
    assert bo.legacy_threshold([5, 5, 7, 9], 5) == (False, 0)
    # tests/test_architecture_v6_static.py:69-114 score constants
    assert bo.SCORE_BIN_COUNT == 76801
    assert int(bo.q_to_score_key(np.float32(300.0))) == 76800
    assert int(bo.q_to_score_key(np.float32(1e9))) == 76800
    assert int(bo.q_to_score_key(np.float32(-3.0))) == 0


def test_balance_targets():
    # production_v6_dispatcher.py:584-588
    rank, local = bo.balance_targets(10, 4)
    assert rank.tolist() == [0, 0, 0, 1, 1, 2, 2, 2, 3, 3]
    assert local.tolist() == [0, 1, 2, 0, 1, 0, 1, 2, 0, 1]


def test_legacy_hamming_q():
    # beam_kernels.cu:133-143
    assert bo.legacy_hamming_q([0, 1, 2, 127, 200]).tolist() == [65535, 65023, 64511, 511, 1]


def test_select_mode_nesting():
    pz = puzzles.puzzle54()
    f = np.stack([pz.scramble(j, 12) for j in range(40)])
    c = bo.expand(f, pz.generators)
    k = bo.hamming(c, pz.solved)
    payload = np.arange(c.shape[0], dtype=np.uint32)
    u = bo.dedup_exact(c, k, payload)
    for beam in (1, 17, 100, 10 ** 6):
        legacy = set(bo.select(u, beam, "legacy_strict").tolist())
        exact = set(bo.select(u, beam, "exact_k").tolist())
        incl = set(bo.select(u, beam, "v6_inclusive").tolist())
        assert len(exact) == min(beam, u.score.size)
        assert legacy <= exact <= incl


def test_expand_inverse_pairs_and_identity_generators():
    pz = puzzles.puzzle54()
    g = pz.fanout // 2
    s = pz.scramble(3, 20)[None, :]
    c = bo.expand(s, pz.generators)
    for m in range(g):
        back = bo.expand(c[m:m + 1], pz.generators)[m + g]
        assert np.array_equal(back, s[0])  # data_loader.validate_inverse_pairs
    # tests/dispatcher_skeleton_smoke.py:11-46: identity generators collapse 2 parents x 24 moves to 2 unique
    ident = np.tile(np.arange(20, dtype=np.uint8), (24, 1))
    f = np.stack([np.arange(20, dtype=np.uint8), np.arange(20, dtype=np.uint8)[::-1].copy()])
    ch = bo.expand(f, ident)
    u = bo.dedup_exact(ch, np.zeros(48, np.uint32), np.arange(48, dtype=np.uint32))
    assert ch.shape[0] == 48 and u.score.size == 2
    assert sorted(u.payload.tolist()) == [0, 24]


def test_search_known_shallow_scrambles():
    # scripts/kaggle_correctness_check.py:154-179: scrambles of length 0/1/2 are found at depth 0/1/2
    pz = puzzles.puzzle54()
    sc = bo.hamming_scorer(pz.solved)
    g = pz.generators.astype(np.int64)
    s0 = pz.solved
    s1 = s0[g[0]]
    s2 = s1[g[1]]
    for start, depth in ((s0, 0), (s1, 1), (s2, 2)):
        r = bo.search(start, pz.generators, pz.solved, sc, beam=64, max_depth=4)
        assert r.found and r.depth == depth
        assert np.array_equal(bo.replay(start, pz.generators, r.path), pz.solved)


@pytest.mark.parametrize("world", [1, 2, 3])
def test_search_lrx_world_invariance(world):
    pz = puzzles.lrx(8)
    sc = bo.hamming_scorer(pz.solved)
    start = pz.scramble(1, 14)
    base = bo.search(start, pz.generators, pz.solved, sc, beam=64, max_depth=30, keep_frontiers=True)
    r = bo.search(start, pz.generators, pz.solved, sc, beam=64, max_depth=30, world=world, keep_frontiers=True)
    assert (r.found, r.depth, r.frontier_sizes) == (base.found, base.depth, base.frontier_sizes)
    for a, b in zip(base.frontiers, r.frontiers):
        assert np.array_equal(a, b)
    if r.found:
        assert np.array_equal(bo.replay(start, pz.generators, r.path), pz.solved)


def test_action_value_network_reduces_to_the_value_network_for_one_move():
    """mlp_action_values with an output layer of width 1 is mlp_forward; wider outputs are independent columns."""
    rng = np.random.default_rng(4)
    states = rng.integers(0, 6, size=(37, 20)).astype(np.uint8)
    w = {"w1": rng.standard_normal((64, 120)).astype(np.float32) * 0.1, "b1": rng.standard_normal(64).astype(np.float32) * 0.1,
         "w2": rng.standard_normal((32, 64)).astype(np.float32) * 0.1, "b2": rng.standard_normal(32).astype(np.float32) * 0.1}
    w3 = rng.standard_normal((5, 32)).astype(np.float32) * 0.1
    b3 = rng.standard_normal(5).astype(np.float32) * 0.1
    q = bo.mlp_action_values(states, [dict(w, w3=w3, b3=b3)], 6)
    assert q.shape == (37, 5)
    for m in range(5):
        v = bo.mlp_forward(states, [dict(w, w3=w3[m], b3=b3[m])], 6)
        assert np.allclose(q[:, m], v, atol=1e-6)


def test_zobrist_hash_is_the_xor_of_table_entries_and_owner_rule():
    """hash128_zobrist against a scalar restatement of the reference's CPU mirror (tests/stream2_reference_smoke.py:41-48)
    and owner_from_hash128 against the Python rule (production_v6_dispatcher.py:116-119)."""
    table = bo.zobrist_table(54, 6)
    assert table.shape == (54, 6, 2) and table.dtype == np.uint64
    # the table is the corner of the (128, 128, 2) production table drawn from default_rng(0xC0DEC0DE)
    full = np.random.default_rng(0xC0DEC0DE).integers(0, np.iinfo(np.uint64).max, size=(128, 128, 2), dtype=np.uint64)
    assert np.array_equal(table, full[:54, :6])
    rng = np.random.default_rng(12)
    states = rng.integers(0, 6, size=(40, 54)).astype(np.uint8)
    lo, hi = bo.hash128_zobrist(states, table)
    for i in (0, 17, 39):
        l = h = 0
        for p in range(54):
            l ^= int(table[p, states[i, p], 0])
            h ^= int(table[p, states[i, p], 1])
        assert (int(lo[i]), int(hi[i])) == (l, h)
        for w in (2, 3, 8):
            assert int(bo.owner_from_hash128(hi[i:i + 1], lo[i:i + 1], w)[0]) == \
                (h ^ ((l * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF)) % w
    # a different hash only reorders equal scores: the kept set has the same size and the same score multiset
    pz = puzzles.puzzle54()
    frontier = np.unique(np.stack([pz.scramble(j, 12) for j in range(60)]), axis=0)
    a = bo.depth_step([frontier], pz.generators, pz.solved, bo.hamming_scorer(pz.solved), 200)
    b = bo.depth_step([frontier], pz.generators, pz.solved, bo.hamming_scorer(pz.solved), 200,
                      hasher=lambda c: bo.hash128_zobrist(c, table))
    assert a.states.shape == b.states.shape and np.array_equal(np.sort(a.score), np.sort(b.score))


def _residual_q_golden():
    """Outputs of the reference's static_forward_q / static_forward_scores / _fold_bn_linear on seeded inputs
    (tests/golden/make_residual_q_golden.py) and that script's seeded generators."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_residual_q_golden", GOLDEN / "make_residual_q_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return json.loads((GOLDEN / "residual_q_reference.json").read_text()), mod


def test_residual_q_network_matches_reference_static_forward():
    data, mod = _residual_q_golden()
    assert len(data["forward"]) == 3
    for c in data["forward"]:
        w = mod.residual_q_weights(c["seed"], c["state_size"], c["num_classes"], c["hidden1"], c["hidden2"], c["outputs"])
        states = mod.residual_q_states(c["seed"] + 50, c["rows"], c["state_len"], c["value_range"])
        q = bo.residual_q_forward(states, w)
        want = np.asarray(c["q"], dtype=np.float32)
        assert q.shape == want.shape
        assert np.max(np.abs(q - want)) <= 2e-5 * max(1.0, float(np.max(np.abs(want))))  # float32 summation order
        sc = bo.residual_q_scores_u16(want, w["action_perm"], w["score_scale"], w["score_bias"])
        assert sc.tolist() == c["scores_i16"]  # the quantiser itself, on the reference's own q, is exact
        assert np.max(np.abs(bo.residual_q_scores_u16(q, w["action_perm"]).astype(np.int64)
                             - np.asarray(c["scores_i16"], dtype=np.int64))) <= 1  # the reference's own bound


def test_batch_norm_folding_matches_reference():
    data, mod = _residual_q_golden()
    for c in data["fold_bn"]:
        case = mod.bn_case(c["seed"], c["outs"], c["ins"])
        fw, fb = bo.fold_bn_linear(case["weight"], case["bias"], case["bn_weight"], case["bn_bias"],
                                   case["running_mean"], case["running_var"])
        assert np.allclose(fw, np.asarray(c["weight"], dtype=np.float32), rtol=1e-6, atol=1e-7)
        assert np.allclose(fb, np.asarray(c["bias"], dtype=np.float32), rtol=1e-6, atol=1e-6)


def test_action_scorer_and_quantiser_match_reference_modules():
    """MLPActionScorer / QuantizedActionScorer of the reference's scorers.py on seeded weights."""
    data, mod = _residual_q_golden()
    assert len(data["action_scorer"]) == 2
    for c in data["action_scorer"]:
        layers = mod.action_scorer_weights(c["seed"], 120, tuple(c["hidden"]), 24)
        states = mod.residual_q_states(c["seed"] + 50, c["rows"], 120, 120)
        y = bo.action_scorer_forward(states, layers)
        want = np.asarray(c["y"], dtype=np.float32)
        assert np.max(np.abs(y - want)) <= 1e-5
        for mode in ("sigmoid_u16", "float_u16"):
            bits = np.asarray(c[mode], dtype=np.int64) & 0xFFFF  # int16 bit pattern -> unsigned score
            got = bo.quantized_action_scores(want, mode).astype(np.int64)
            assert np.max(np.abs(got - bits)) <= (1 if mode == "sigmoid_u16" else 0)  # last bit of exp()
