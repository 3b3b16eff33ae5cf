"""GPU parity tests: the CUDA step, called through the C ABI, against the numpy oracle (bit-exact)."""

import ctypes as C

import numpy as np
import pytest
import torch

from oracle import beam_oracle as bo
from multigpubeamsearch_b200 import beam_engine as be
from multigpubeamsearch_b200 import puzzles, _lib

pytestmark = pytest.mark.gpu


def make_engine(pz, **kw):
    kw.setdefault("global_beam_width", 1024)
    kw.setdefault("max_depth", 64)
    kw.setdefault("beta", 1.2)
    kw.setdefault("hash_load_factor", 0.45)
    kw.setdefault("probe_limit", 256)
    kw.setdefault("band_rounds", 8)
    ext, cfg, buffers, engine = be.configure_engine(pz, **kw)
    return engine


def random_frontier(pz, count, seed, walk=25):
    rng = np.random.default_rng(seed)
    g = pz.generators.astype(np.int64)
    rows = np.tile(pz.solved, (count, 1))
    for _ in range(walk):
        mv = rng.integers(0, pz.fanout, size=count)
        rows = np.take_along_axis(rows, g[mv], axis=1)
    return np.unique(rows, axis=0)


@pytest.mark.parametrize("n,fanout", [(16, 3), (54, 12), (96, 18), (120, 24), (33, 7)])
def test_expand_kernel_bit_exact(n, fanout):
    lib = _lib.load()
    rng = np.random.default_rng(n * 100 + fanout)
    stride = (n + 15) // 16 * 16
    if stride // 4 not in (4, 8, 16, 24, 32):
        stride = 64
    P = 777
    frontier = rng.integers(0, 8, size=(P, n), dtype=np.uint8)
    gens = np.stack([rng.permutation(n) for _ in range(fanout)]).astype(np.uint8)
    solved = frontier[5][gens[2].astype(np.int64)].copy()  # make one child equal to "solved"
    dev = torch.device("cuda", 0)
    f_pad = np.zeros((P, stride), np.uint8)
    f_pad[:, :n] = frontier
    t_f = torch.from_numpy(f_pad).to(dev)
    t_g = torch.from_numpy(gens).to(dev)
    t_s = torch.from_numpy(solved).to(dev)
    Cn = P * fanout
    t_children = torch.zeros((Cn, stride), dtype=torch.uint8, device=dev)
    t_h = torch.zeros(Cn, dtype=torch.int64, device=dev)
    t_fp = torch.zeros(Cn, dtype=torch.int64, device=dev)
    t_k = torch.zeros(Cn, dtype=torch.int32, device=dev)
    t_p = torch.zeros(Cn, dtype=torch.int32, device=dev)
    ctrl = torch.zeros(C.sizeof(_lib.MgbsCtrl), dtype=torch.uint8, device=dev)
    host = _lib.MgbsCtrl()
    host.found_payload = 0xFFFFFFFF
    ctrl.copy_(torch.frombuffer(bytearray(bytes(host)), dtype=torch.uint8))
    rc = lib.mgbs_launch_expand(t_f.data_ptr(), None, P, t_g.data_ptr(), t_s.data_ptr(), n, stride, fanout, 3,
                                _lib.SCORE_HAMMING, 0, t_children.data_ptr(), t_h.data_ptr(), t_fp.data_ptr(),
                                t_k.data_ptr(), t_p.data_ptr(), ctrl.data_ptr(),
                                C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    want_c = bo.expand(frontier, gens)
    assert np.array_equal(t_children.cpu().numpy()[:, :n], want_c)
    assert not t_children.cpu().numpy()[:, n:].any()
    assert np.array_equal(t_h.cpu().numpy().view(np.uint64), bo.hash64(want_c))
    assert np.array_equal(t_fp.cpu().numpy().view(np.uint64), bo.fingerprint64(want_c))
    assert np.array_equal(t_k.cpu().numpy().view(np.uint32), bo.hamming(want_c, solved))
    pidx = np.repeat(np.arange(P, dtype=np.uint32), fanout)
    mv = np.tile(np.arange(fanout, dtype=np.uint32), P)
    assert np.array_equal(t_p.cpu().numpy().view(np.uint32), bo.pack_payload(pidx, np.full_like(pidx, 3), mv))
    got = _lib.MgbsCtrl.from_buffer_copy(bytes(ctrl.cpu().numpy()))
    goal = (want_c == solved[None, :]).all(axis=1)
    assert got.found_payload == int(bo.pack_payload(pidx, np.full_like(pidx, 3), mv)[goal].min())
    # host helpers use the same arithmetic
    row = np.ascontiguousarray(want_c[17])
    assert lib.mgbs_hash64_host(row.ctypes.data_as(C.c_void_p), n) == int(bo.hash64(row)[0])
    assert lib.mgbs_fingerprint64_host(row.ctypes.data_as(C.c_void_p), n) == int(bo.fingerprint64(row)[0])


def test_expand_kernel_matches_reference_device_functions():
    """The expansion kernel at the reference's native shape (120 bytes, 24 moves) against vectors produced by
    the reference's own apply_move_table / hash_state_120 / fingerprint_state_120 / hamming_to_central
    (beam_kernels.cu:38-94) compiled as host C++ - no oracle in between."""
    import importlib.util
    import json
    from pathlib import Path
    golden = Path(__file__).resolve().parent / "golden"
    spec = importlib.util.spec_from_file_location("make_scalar_golden", golden / "make_scalar_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    data = json.loads((golden / "scalar_reference.json").read_text())["legacy_expand"]
    table, central = mod.legacy_tables(data["table_seed"])
    parents = np.stack([central if c["parent_seed"] is None else
                        np.random.default_rng(c["parent_seed"]).integers(0, 120, size=120, dtype=np.uint8)
                        for c in data["cases"]])
    lib = _lib.load()
    n, stride, fanout, P = 120, 128, 24, parents.shape[0]
    dev = torch.device("cuda", 0)
    f_pad = np.zeros((P, stride), np.uint8)
    f_pad[:, :n] = parents
    t_f, t_g, t_s = (torch.from_numpy(x).to(dev) for x in (f_pad, table, central))
    Cn = P * fanout
    t_children = torch.zeros((Cn, stride), dtype=torch.uint8, device=dev)
    t_h = torch.zeros(Cn, dtype=torch.int64, device=dev)
    t_fp = torch.zeros(Cn, dtype=torch.int64, device=dev)
    t_k = torch.zeros(Cn, dtype=torch.int32, device=dev)
    t_p = torch.zeros(Cn, dtype=torch.int32, device=dev)
    rc = lib.mgbs_launch_expand(t_f.data_ptr(), None, P, t_g.data_ptr(), t_s.data_ptr(), n, stride, fanout, 0,
                                _lib.SCORE_HAMMING, 0, t_children.data_ptr(), t_h.data_ptr(), t_fp.data_ptr(),
                                t_k.data_ptr(), t_p.data_ptr(), None,
                                C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    h = t_h.cpu().numpy().view(np.uint64).reshape(P, fanout)
    fp = t_fp.cpu().numpy().view(np.uint64).reshape(P, fanout)
    ham = t_k.cpu().numpy().reshape(P, fanout)
    rows = t_children.cpu().numpy().reshape(P, fanout, stride)
    for i, c in enumerate(data["cases"]):
        assert [int(x) for x in h[i]] == c["child_hash64"]
        assert [int(x) for x in fp[i]] == c["child_fingerprint64"]
        assert ham[i].tolist() == c["child_hamming"]
        assert rows[i, 0, :n].tolist() == c["child_bytes_move0"]


def check_step(engine, pz, frontier, beam, mode="exact_k", graph=False):
    engine.load_frontier(frontier, depth=0)
    engine.enable_cuda_graphs(graph)
    engine.step()
    st = engine.status()
    want = bo.depth_step([frontier], pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam, mode)
    assert st["status_bits"] == 0, st["status_names"]
    got_rows = engine.frontier()
    assert got_rows.shape[0] == want.states.shape[0]
    assert np.array_equal(bo.sorted_rows(got_rows), bo.sorted_rows(want.states))
    # back-pointers: same winner (parent, rank, move) for every surviving state
    got_pay = engine.frontier_payloads()
    got_map = {bytes(r): int(p) for r, p in zip(got_rows, got_pay)}
    want_map = {bytes(r): int(p) for r, p in zip(want.states, want.payload)}
    assert got_map == want_map
    got_scores = engine.frontier_scores()
    assert {bytes(r): int(k) for r, k in zip(got_rows, got_scores)} == \
        {bytes(r): int(k) for r, k in zip(want.states, want.score)}
    assert st["counters"][2] == want.candidates
    assert bool(st["found"]) == want.found_child
    return st, want


@pytest.mark.parametrize("pipeline", ["persistent", "staged"])
@pytest.mark.parametrize("name,count,beam", [("lrx16", 300, 256), ("rand54", 500, 1024), ("rand96", 400, 2048),
                                             ("rand54", 40, 100000), ("rand54", 1, 16)])
def test_single_step_matches_oracle(name, count, beam, pipeline):
    pz = puzzles.by_name(name)
    engine = make_engine(pz, global_beam_width=beam, select_pipeline=pipeline)
    frontier = random_frontier(pz, count, seed=count + beam)[: engine.sizes()["k_work"]]
    for graph in (False, True):
        st, want = check_step(engine, pz, frontier, beam, graph=graph)
    assert st["counters"][3] >= min(beam, want.unique) or st["counters"][3] == want.unique


@pytest.mark.parametrize("mode", ["v6_inclusive", "legacy_strict"])
def test_threshold_modes_match_oracle(mode):
    pz = puzzles.puzzle54()
    # score-only order: a whole score level must fit the pool, so give the pool room (beta) and keep beams small
    engine = make_engine(pz, global_beam_width=300, select_mode=mode, beta=8.0)
    frontier = random_frontier(pz, 120, seed=9)
    check_step(engine, pz, frontier, 300, mode=mode)


def test_tie_resolution_path():
    # few hash bits in the order key -> many candidates share the cut key; the result must still be exact
    pz = puzzles.puzzle54()
    for hb in (1, 3, 6):
        engine = make_engine(pz, global_beam_width=64, hash_bits=hb, beta=4.0)
        frontier = random_frontier(pz, 30, seed=hb)
        check_step(engine, pz, frontier, 64)


def test_empty_frontier_and_status_reset():
    pz = puzzles.puzzle54()
    engine = make_engine(pz, global_beam_width=64)
    engine.load_frontier(np.zeros((0, pz.state_len), np.uint8))
    engine.step()
    st = engine.status()
    assert st["current_size"] == 0 and st["status_bits"] == 0 and not st["found"]


def test_probe_limit_overflow_is_reported_not_trapped():
    pz = puzzles.puzzle54()
    engine = make_engine(pz, global_beam_width=4096, probe_limit=1, hash_load_factor=0.9, beta=1.0, gamma=1.0)
    frontier = random_frontier(pz, 2000, seed=4)
    engine.load_frontier(frontier)
    engine.step()
    st = engine.status()
    assert st["status_bits"] & _lib.ST_HASH_OVERFLOW
    assert st["counters"][4] > 0
    # the engine is still usable
    engine2 = make_engine(pz, global_beam_width=512)
    check_step(engine2, pz, frontier[:200], 512)


@pytest.mark.parametrize("scramble", [0, 1, 2, 3])
def test_full_search_lrx16_matches_oracle(scramble):
    # the reference's CPU-runnable case: S_16 under L, R, X; beam 1024; depth 40; Hamming scorer
    pz = puzzles.lrx(16)
    start = pz.scramble(scramble, 30)
    want = bo.search(start, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam=1024, max_depth=40,
                     keep_frontiers=True)
    engine = make_engine(pz, global_beam_width=1024, max_depth=40)
    engine.reset_search(bytes(start))
    depth = 0
    while True:
        rows = engine.frontier()
        assert np.array_equal(bo.sorted_rows(rows), want.frontiers[depth]), f"depth {depth}"
        st = engine.status()
        if st["found"] or depth == 40 or rows.shape[0] == 0:
            break
        engine.step()
        depth += 1
        st = engine.status()
        assert st["status_bits"] == 0, st["status_names"]
        if st["found"]:
            break
    st = engine.status()
    assert bool(st["found"]) == want.found
    if want.found:
        assert st["found_depth"] == want.depth
        path = engine.reconstruct_path()
        assert len(path) == want.depth
        assert np.array_equal(bo.replay(start, pz.generators, path), pz.solved)
    # the same search through the engine's own depth loop (graph replay)
    engine.enable_cuda_graphs(True)
    res = be.run_one_search(engine, start, 40)
    assert res["found"] == want.found and res["depth"] == want.depth
    assert engine.cuda_graph_captured()


def test_all_64_lrx16_scrambles_through_the_depth_loop():
    """The reference's CPU-runnable configuration in full: S_16 under L, R, X, 64 seeded scrambles of 30 moves,
    beam 1024, depth 40, Hamming scorer.  The engine's own depth loop (graph replay, the host one depth ahead of the
    device summaries) must stop at the oracle's depth with a path that replays to the solved state, or, when the
    oracle does not solve within 40, end on the oracle's frontier."""
    pz = puzzles.lrx(16)
    engine = make_engine(pz, global_beam_width=1024, max_depth=40)
    engine.enable_cuda_graphs(True)
    solved = 0
    for j in range(64):
        start = pz.scramble(j, 30)
        want = bo.search(start, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam=1024, max_depth=40,
                         keep_frontiers=True)
        res = be.run_one_search(engine, start, 40)
        assert res["status"]["status_bits"] == 0, (j, res["status_names"])
        assert (res["found"], res["depth"]) == (want.found, want.depth), (j, res["found"], res["depth"], want.depth)
        if want.found:
            solved += 1
            path = engine.reconstruct_path()
            assert len(path) == want.depth and np.array_equal(bo.replay(start, pz.generators, path), pz.solved), j
        else:
            assert np.array_equal(bo.sorted_rows(engine.frontier()), want.frontiers[-1]), j
    assert solved > 0


def test_saturated_step_at_benchmark_scale_matches_oracle():
    """One depth at the benchmark's exact knobs: 54-byte states, 12 moves, global beam 65 536 with a saturated
    frontier (65 536 rows, 786 432 candidates), BETA 1.2, GAMMA 1.05, load 0.45, probe limit 256, three band rounds of
    three levels - where the band sizing from the duplicate ratio, the 17 % insertion and the 183 k-slot table
    actually operate.  Hamming scores make the oracle's expectation exact; eager launch and graph replay."""
    pz = puzzles.puzzle54()
    beam = 65536
    engine = make_engine(pz, global_beam_width=beam, max_depth=24, beta=1.2, gamma=1.05, hash_load_factor=0.45,
                         probe_limit=256, band_rounds=3, band_levels=3)
    # saturate the frontier with the engine's own search, as the benchmark does
    be.run_one_search(engine, pz.scramble(0, 40), 8)
    frontier = engine.frontier()
    assert frontier.shape[0] == beam
    for graph in (False, True):
        st, want = check_step(engine, pz, frontier, beam, graph=graph)
        assert want.candidates == beam * pz.fanout and st["counters"][3] >= beam
    # and two more depths in sequence from there: duplicates concentrate as the search goes on
    engine.load_frontier(frontier, depth=0)
    rows = frontier
    for _ in range(2):
        want = bo.depth_step([rows], pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam)
        engine.step()
        assert engine.status()["status_bits"] == 0
        rows = engine.frontier()
        assert np.array_equal(bo.sorted_rows(rows), bo.sorted_rows(want.states))


def test_logical_limits_clamp_the_step():
    """set_active_limit / set_next_limit / clear_logical_limits (beam_engine.cpp:1064-1090)."""
    pz = puzzles.puzzle54()
    engine = make_engine(pz, global_beam_width=2048)
    frontier = random_frontier(pz, 400, seed=21)
    # active limit: only the first rows of the frontier are expanded
    engine.set_active_limit(100)
    engine.load_frontier(frontier)
    engine.step()
    st = engine.status()
    want = bo.depth_step([frontier[:100]], pz.generators, pz.solved, bo.hamming_scorer(pz.solved), 2048)
    assert st["counters"][2] == 100 * pz.fanout and st["status_bits"] == 0
    assert np.array_equal(bo.sorted_rows(engine.frontier()), bo.sorted_rows(want.states))
    # next limit below what the step would keep: the pool, the table and the next frontier shrink with it, the
    # frontier stays within the limit and the truncation is reported
    engine.clear_logical_limits()
    engine.set_next_limit(300)
    engine.load_frontier(frontier)
    engine.step()
    st = engine.status()
    assert 0 < st["current_size"] <= 300
    assert st["status_bits"] & (_lib.ST_FRONTIER_OVERFLOW | _lib.ST_BAND_STALL | _lib.ST_ROUNDS_EXHAUSTED)
    # and the rows it kept are the best ones: a prefix of the full step's (score, hash) order
    full = bo.depth_step([frontier], pz.generators, pz.solved, bo.hamming_scorer(pz.solved), 2048)
    kept = {bytes(r) for r in engine.frontier()}
    assert kept <= {bytes(r) for r in full.states}
    # cleared: the full step again
    engine.clear_logical_limits()
    check_step(engine, pz, frontier, 2048)
    # the prepass helper: one eager depth with a constant score
    engine.load_frontier(frontier[:50])
    engine.step_prepass_fast(3)
    want = bo.depth_step([frontier[:50]], pz.generators, pz.solved, lambda c: np.full(c.shape[0], 3, np.uint32), 2048)
    assert np.array_equal(bo.sorted_rows(engine.frontier()), bo.sorted_rows(want.states))


def test_depth_loop_halts_on_the_device_and_mirror_matches_control_block():
    """The depth loop runs one depth ahead of the summaries it reads; the depth that was already enqueued when the
    solved state turned up must not change anything (it halts on the device)."""
    pz = puzzles.puzzle54()
    engine = make_engine(pz, global_beam_width=2048, max_depth=16)
    start = be.make_shallow_scramble(pz, [3, 7, 2, 10, 0])  # no move undoes its predecessor
    assert not np.array_equal(start, pz.solved)
    for graph in (True, False):
        engine.enable_cuda_graphs(graph)
        res = be.run_one_search(engine, start, 12)
        want = bo.search(start, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam=2048, max_depth=12)
        assert res["found"] and res["depth"] == want.depth
        st = engine.status()
        assert st["depth"] == want.depth and st["status_bits"] == 0  # no extra depth was taken after the find
        mirror = _lib.MgbsMirror.from_buffer_copy(bytes(engine._mirror.numpy()))
        assert mirror.found == 1 and mirror.found_depth == want.depth and mirror.depth == st["depth"]
        path = engine.reconstruct_path()
        assert np.array_equal(bo.replay(start, pz.generators, path), pz.solved)
    # a search that runs out of depth stops exactly at max_depth
    far = pz.scramble(5, 40)
    res = be.run_one_search(engine, far, 7)
    assert not res["found"] and res["depth"] == 7 and engine.status()["depth"] == 7


def test_history_ring_smaller_than_the_search():
    """Two device history rows: entries older than the ring are reported invalid and the walk-back refuses."""
    pz = puzzles.puzzle54()
    engine = make_engine(pz, global_beam_width=512, max_depth=16, history_rows=2)
    start = be.make_shallow_scramble(pz, [2, 5, 8, 11, 0])
    res = be.run_one_search(engine, start, 10)
    assert res["found"] and res["depth"] >= 4
    d = res["depth"]
    assert engine.history_entry(d - 1, 0)["valid"] in (0, 1)  # the finding depth wrote no layer: found before select
    assert engine.history_entry(0, 0)["valid"] == 0            # overwritten long ago
    with pytest.raises(RuntimeError, match="history"):
        engine.reconstruct_path()


def test_bounded_peer_wait_gives_up_and_reports():
    """A two-rank engine in peer mode whose peer never answers: rank 1's region is a zeroed buffer on the same GPU
    that nothing writes.  With a short poll limit every cross-rank wait runs out, the step ends by itself with the
    peer_timeout bit, the depth loop returns an error instead of stepping on, and the GPU stays usable."""
    pz = puzzles.puzzle54()
    cfg = be.config_for_puzzle(pz, world_size=2, rank=0, global_beam_width=1024, max_depth=8, beta=1.2, gamma=1.25,
                               hash_load_factor=0.45, probe_limit=256, band_rounds=3, exchange="peer",
                               peer_poll_limit=2000)
    ext = be.build_extension()
    buffers = be.allocate_buffers(ext, cfg)
    engine = ext.BeamEngine(cfg, buffers, "central_hamming")
    engine.set_action_permutation_table(pz.action_table_bytes())
    engine.set_central_state(bytes(pz.solved))
    dead_peer = torch.zeros_like(buffers["sym"])
    bases = (C.c_void_p * 2)(buffers["sym"].data_ptr(), dead_peer.data_ptr())
    _lib.check(engine.lib.mgbs_engine_set_peer_pointers(engine._h, bases), "set_peer_pointers")
    start = pz.scramble(2, 20)
    engine.reset_search(bytes(start), active_on_this_rank=True)
    with pytest.raises(RuntimeError, match="peer timeout"):
        engine.search(6)
    st = engine.status()
    assert st["status_bits"] & _lib.ST_PEER_TIMEOUT and "peer_timeout" in st["status_names"]
    assert st["depth"] <= 1  # the loop did not step on after the failed wait
    # a later launch on the broken engine halts at once and changes nothing
    engine.step()
    assert engine.status()["depth"] == st["depth"]
    engine.close()
    # the context is intact: an ordinary engine on the same GPU works
    check_step(make_engine(pz, global_beam_width=512), pz, random_frontier(pz, 100, seed=8), 512)


def test_known_shallow_scrambles_rand54():
    # scrambles of length 0, 1, 2 are found at depth 0, 1, 2 (scripts/kaggle_correctness_check.py:154-179)
    pz = puzzles.puzzle54()
    g = pz.generators.astype(np.int64)
    engine = make_engine(pz, global_beam_width=4096, max_depth=8)
    s = pz.solved.copy()
    for depth, mv in enumerate([None, 0, 1]):
        if mv is not None:
            s = s[g[mv]]
        res = be.run_one_search(engine, s, 6)
        assert res["found"] and res["depth"] == depth
        path = engine.reconstruct_path()
        assert np.array_equal(bo.replay(s, pz.generators, path), pz.solved)


def test_uniform_prepass_fill():
    # uniform score: every child ties, the cut is by hash alone; still exact and deterministic
    pz = puzzles.puzzle54()
    engine = make_engine(pz, global_beam_width=500)
    frontier = random_frontier(pz, 100, seed=77)
    engine.begin_uniform_score(7)
    engine.load_frontier(frontier)
    engine.step()
    rows = engine.frontier()
    want = bo.depth_step([frontier], pz.generators, pz.solved, lambda c: np.full(c.shape[0], 7, np.uint32), 500)
    assert np.array_equal(bo.sorted_rows(rows), bo.sorted_rows(want.states))
    engine.end_uniform_score()
    check_step(engine, pz, frontier, 500)


def test_rejects_bad_arguments():
    pz = puzzles.puzzle54()
    engine = make_engine(pz, global_beam_width=64)
    with pytest.raises(RuntimeError):
        engine.set_action_permutation_table(b"\x00" * 5)
    with pytest.raises(RuntimeError):
        engine.set_central_state(b"\x00" * 5)
    with pytest.raises(RuntimeError):
        engine.reset_search(b"\x00" * 3)
    with pytest.raises(RuntimeError):
        be.BeamEngine(engine.cfg, engine.buffers, "no_such_backend")


def test_frontier_into_pinned_buffer():
    pz = puzzles.puzzle54()
    engine = make_engine(pz, global_beam_width=300)
    frontier = random_frontier(pz, 80, seed=12)
    engine.load_frontier(frontier)
    engine.step()
    want = engine.frontier()
    out = torch.empty((engine.sizes()["k_work"], pz.state_len), dtype=torch.uint8).pin_memory()
    n = engine.frontier_into(out.numpy())
    assert n == want.shape[0] and np.array_equal(out.numpy()[:n], want)
    small = np.zeros((10, pz.state_len), np.uint8)
    assert engine.frontier_into(small) == 10 and np.array_equal(small, want[:10])


def test_maximum_shape_state128_fanout32():
    # largest supported shape: 128-byte states, 32 generators
    rng = np.random.default_rng(77)
    n, g = 128, 32
    base = [rng.permutation(n) for _ in range(g // 2)]
    gens = np.stack(base + [np.argsort(b) for b in base]).astype(np.uint8)
    solved = (np.arange(n) // 16).astype(np.uint8)
    pz = puzzles.Puzzle("max128", n, 8, gens, solved, scramble_seed=9000)
    engine = make_engine(pz, global_beam_width=3000)
    frontier = np.unique(np.stack([pz.scramble(j, 9) for j in range(200)]), axis=0)
    for graph in (False, True):
        check_step(engine, pz, frontier, 3000, graph=graph)


def test_solver_loop_with_prepass_matches_oracle(tmp_path):
    # the per-sample driver: uniform-fill prepass, scored steps, depth log, path validation
    from multigpubeamsearch_b200 import solver
    pz = puzzles.lrx(16)
    engine = make_engine(pz, global_beam_width=1024, max_depth=40)
    starts = [pz.scramble(j, 30) for j in range(8, 14)]
    log = tmp_path / "run.jsonl"
    summary = solver.solve_many(engine, pz, starts, 40, log_path=str(log))
    assert summary["status_bits"] == 0 and summary["invalid_paths"] == 0
    for s, r in zip(starts, summary["results"]):
        want = bo.search(s, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam=1024, max_depth=40)
        assert (r["found"], r["depth"]) == (want.found, want.depth)
        assert r["depths_prepass"] >= 5  # 3^d * 3 <= 1024 for the first depths
        if want.found:
            assert r["valid"] and len(r["path"]) == want.depth
    rows = [__import__("json").loads(x) for x in log.read_text().splitlines()]
    assert sum(1 for x in rows if x["tag"] == "SAMPLE_RESULT") == len(starts)
    assert any(x["tag"] == "DEPTH_TUNING" and x["prepass"] for x in rows)
    # same answers without the prepass
    r2 = solver.solve_one(engine, pz, starts[0], 40, prepass=False)
    assert (r2["found"], r2["depth"]) == (summary["results"][0]["found"], summary["results"][0]["depth"])


def test_history_archive_with_one_device_row_and_resume(tmp_path):
    """The device keeps a ring of ONE history row; the host archive collects every layer, checkpoints it, and a
    second engine resumes from the files and finishes the search with the same answer and a valid path."""
    from multigpubeamsearch_b200 import solver
    from multigpubeamsearch_b200.history_archive import CPUHistoryArchive
    pz = puzzles.lrx(16)
    start = pz.scramble(9, 30)
    want = bo.search(start, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam=1024, max_depth=40)
    assert want.found and want.depth > 6
    # whole search through the archive
    engine = make_engine(pz, global_beam_width=1024, max_depth=40, history_rows=1)
    assert engine.buffers["history_payload"].shape[0] == 1
    arch = CPUHistoryArchive(engine, str(tmp_path / "full"), sample_id=1, checkpoint=True)
    r = solver.solve_one(engine, pz, start, 40, prepass=False, archive=arch)
    arch.finish()
    assert r["found"] and r["depth"] == want.depth and r["valid"] and len(r["path"]) == want.depth
    # stop after 5 depths, resume in a fresh engine
    e1 = make_engine(pz, global_beam_width=1024, max_depth=40, history_rows=1)
    a1 = CPUHistoryArchive(e1, str(tmp_path / "cut"), sample_id=1, checkpoint=True)
    e1.reset_search(bytes(start))
    a1.start_new()
    for _ in range(5):
        e1.step()
        st = e1.status()
        a1.after_step(st["depth"], st["current_size"])
    a1.finish()
    e2 = make_engine(pz, global_beam_width=1024, max_depth=40, history_rows=1)
    a2 = CPUHistoryArchive(e2, str(tmp_path / "cut"), sample_id=1, checkpoint=True)
    assert a2.try_resume() == 5
    st = e2.status()
    assert st["depth"] == 5
    while not st["found"] and st["depth"] < 40:
        e2.step()
        st = e2.status()
        a2.after_step(st["depth"], st["current_size"])
    a2.finish()
    assert st["found"] and st["found_depth"] == want.depth and st["status_bits"] == 0
    path = solver.reconstruct_path_from_archive(e2, a2)
    assert len(path) == want.depth and np.array_equal(solver.replay(start, pz.generators, path), pz.solved)


@pytest.mark.parametrize("name,count,beam", [("rand54", 500, 1024), ("rand96", 300, 700), ("lrx16", 200, 64)])
def test_zobrist_hash_mode_matches_oracle(name, count, beam):
    """The v6 128-bit Zobrist hash instead of FNV + fingerprint: candidate hashes are the oracle's (lo, hi) pairs and
    a step keeps exactly the oracle's survivors under the (score, lo, hi) order."""
    pz = puzzles.by_name(name)
    engine = make_engine(pz, global_beam_width=beam, hash_mode="zobrist128")
    table = bo.zobrist_table(pz.state_len, pz.num_values)
    frontier = random_frontier(pz, count, seed=count + 3)[: engine.sizes()["k_work"]]
    hasher = lambda c: bo.hash128_zobrist(c, table)
    for graph in (False, True):
        engine.load_frontier(frontier, depth=0)
        engine.enable_cuda_graphs(graph)
        engine.step()
        st = engine.status()
        assert st["status_bits"] == 0, st["status_names"]
        ncand = frontier.shape[0] * pz.fanout
        lo, hi = hasher(bo.expand(frontier, pz.generators))
        assert np.array_equal(engine.buffers["cand_hash"][:ncand].cpu().numpy().view(np.uint64), lo)
        assert np.array_equal(engine.buffers["cand_fingerprint"][:ncand].cpu().numpy().view(np.uint64), hi)
        want = bo.depth_step([frontier], pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam, hasher=hasher)
        got = engine.frontier()
        assert np.array_equal(bo.sorted_rows(got), bo.sorted_rows(want.states))
        assert {bytes(r): int(p) for r, p in zip(got, engine.frontier_payloads())} == \
            {bytes(r): int(p) for r, p in zip(want.states, want.payload)}
    # the start state's owner under the Zobrist rule, as the host computes it
    lo0, hi0 = hasher(frontier[:1])
    for w in (2, 3, 8):
        engine.cfg["world_size"] = w
        assert engine.owner_of(frontier[0]) == int(bo.owner_from_hash128(hi0, lo0, w)[0])
    engine.cfg["world_size"] = 1


@pytest.mark.parametrize("select_mode,hash_mode", [("v6_inclusive", "zobrist128"), ("exact_k", "fnv")])
def test_production_v6_dispatcher_runs_tasks(select_mode, hash_mode):
    """ProductionV6Dispatcher.run_task (production_v6_dispatcher.py:708-868): one object, several start states; the
    result carries the reference's fields, a path that replays to the solved state, and one row per depth with the
    reference's keys.  The start state itself and a state one move away are the reference's own known answers
    (scripts/kaggle_correctness_check.py:154-179: depths 0, 1, 2)."""
    from multigpubeamsearch_b200.production_v6_dispatcher import ProductionV6Dispatcher, replay_path_to_central
    pz = puzzles.puzzle54()
    disp = ProductionV6Dispatcher(0, 1, torch.device("cuda", 0), beam_width=2048, b_micro=8192, puzzle=pz,
                                  max_depth=16, select_mode=select_mode, hash_mode=hash_mode)
    try:
        for task, moves in enumerate(([], [4], [4, 9], [2, 5, 8, 11, 0])):
            start = be.make_shallow_scramble(pz, moves)
            want = bo.search(start, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam=2048, max_depth=12)
            res = disp.run_task(task, start, 12, 2048)
            assert res.task_id == task and res.status == "solved", (moves, res)
            # inclusive ties on the coarse Hamming scale can exceed the frontier rows (capacity bits, reported);
            # no timeout bit in any mode, and no bit at all with exact top-K
            assert res.status_bits & (64 | 128) == 0 and (select_mode != "exact_k" or res.status_bits == 0), res
            assert res.solved_depth <= len(moves)
            if select_mode == "exact_k":
                assert res.solved_depth == want.depth
            assert res.path_replay_valid and res.path_failure_reason == ""
            names = res.path.split(".") if res.path else []
            assert len(names) == res.solved_depth
            if names:
                assert replay_path_to_central(pz, disp.action_names, start, res.path) == (True, len(names), "")
            assert len(res.depth_rows) == res.solved_depth
            for d, row in enumerate(res.depth_rows):
                assert row["task_id"] == task and row["depth"] == d
                for key in ("frontier_size", "expanded_parent_count", "stream2_generated_candidate_count",
                            "stream3_after_threshold_count", "stream3_unique_count", "stream4_clean_count",
                            "next_frontier_size_after", "threshold_initialized", "current_threshold",
                            "global_keep_count", "solved_count", "stop_flag", "elapsed_sec"):
                    assert key in row, key
                assert row["stream2_generated_candidate_count"] == row["frontier_size"] * pz.fanout
            if res.depth_rows:
                assert res.depth_rows[-1]["stop_flag"] == 1
        far = pz.scramble(7, 40)
        res = disp.run_task(99, far, 3, 2048)  # cannot be solved in three depths
        assert res.status == "max_depth_reached" and res.path == "" and res.path_failure_reason == "no_solved_state"
        assert len(res.depth_rows) == 3 and res.depth_rows[-1]["next_frontier_size_after"] > 0
        with pytest.raises(RuntimeError, match="invalid_config"):
            disp.run_task(100, far, 3, 4096)
    finally:
        disp.close()


def test_solve_rate_on_the_benchmark_puzzle_matches_oracle():
    """"Solve rate unchanged" on the benchmark's own state space (54 positions, 12 moves): 24 seeded scrambles of 7 to
    12 moves, Hamming scorer, beam 4096, depth limit 14.  The depth loop must report found / not found and the depth
    exactly as the oracle does for every scramble (bit-exact selection makes this an equality, not a rate), and every
    found path must replay to the solved state."""
    pz = puzzles.puzzle54()
    engine = make_engine(pz, global_beam_width=4096, max_depth=16)
    engine.enable_cuda_graphs(True)
    outcomes = []
    for j in range(24):
        start = pz.scramble(2000 + j, 7 + j % 6)
        want = bo.search(start, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam=4096, max_depth=14)
        res = be.run_one_search(engine, start, 14)
        assert res["status"]["status_bits"] == 0, (j, res["status_names"])
        assert (bool(res["found"]), res["depth"]) == (bool(want.found), want.depth), (j, res["found"], res["depth"], want.depth)
        if want.found:
            path = engine.reconstruct_path()
            assert np.array_equal(bo.replay(start, pz.generators, path), pz.solved), j
        outcomes.append(bool(want.found))
    assert any(outcomes)
    print("solve rate", sum(outcomes), "of", len(outcomes))
