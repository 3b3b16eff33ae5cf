"""Worker of the multi-GPU parity test: launched by torch.distributed.run, one process per GPU."""

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from multigpubeamsearch_b200 import beam_engine as be  # noqa: E402
from multigpubeamsearch_b200 import puzzles, scorers  # noqa: E402
from oracle import beam_oracle as bo  # noqa: E402


def gather_rows(rows):
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, rows)
    return out


def run_case(name, beam, scramble_len, depths, backend, graph, exchange="peer", hash_mode="fnv"):
    world, rank = dist.get_world_size(), dist.get_rank()
    pz = puzzles.by_name(name)
    cfg = be.config_for_puzzle(pz, world_size=world, rank=rank, global_beam_width=beam, max_depth=depths + 2,
                               beta=1.2, gamma=1.25, hash_load_factor=0.45, probe_limit=256, band_rounds=8,
                               inference_backend=backend, use_cuda_graphs=graph, exchange=exchange, hash_mode=hash_mode)
    table = bo.zobrist_table(pz.state_len, pz.num_values) if hash_mode == "zobrist128" else None
    hasher = (lambda c: bo.hash128_zobrist(c, table)) if table is not None else None

    def owners(rows):
        if table is not None:
            lo, hi = bo.hash128_zobrist(rows, table)
            return bo.owner_from_hash128(hi, lo, world)
        return bo.owner_rank(bo.hash64(rows), world)

    sc = None
    weights = None
    if backend == "mlp":
        ext = be.build_extension()
        sizes = ext.derive_sizes(cfg)
        weights = puzzles.mlp_weights(pz.state_len * pz.num_values, 1024)
        sc = scorers.MLPValueScorer(weights, pz.state_len, cfg["state_size_bytes"], pz.num_values,
                                    max_rows=sizes["cand_cap"])
    if backend == "qmlp":
        # action values on the parent rows (the expansion then writes no child rows in peer mode)
        cfg["inference_backend"] = "mlp"
        ext = be.build_extension()
        sizes = ext.derive_sizes(cfg)
        weights = puzzles.q_mlp_weights(pz.state_len * pz.num_values, pz.fanout, 1024, 512)
        sc = scorers.MLPActionValueScorer(weights, pz.state_len, cfg["state_size_bytes"], pz.num_values, pz.fanout,
                                          max_parents=sizes["k_work"])
    _, cfg, buffers, engine = be.configure_engine(pz, cfg=cfg, scorer=sc)
    start = pz.scramble(3, scramble_len)
    n = pz.state_len
    owner = int(owners(start[None, :])[0])
    assert engine.owner_of(start) == owner
    engine.reset_search(bytes(start), active_on_this_rank=(owner == rank))
    fronts = [start[None, :] if r == owner else start[:0][None, :].reshape(0, n) for r in range(world)]
    for depth in range(depths):
        # oracle step on the same per-rank frontiers (so that back-pointers are comparable)
        if backend == "mlp":
            # device scores of this rank's candidates are known only after the step; use the float32 network's keys
            # for the expected set only when they agree with the device (checked below through the survivor scores)
            pass
        engine.step()
        st = engine.status()
        assert st["status_bits"] == 0, (depth, st["status_names"])
        rows = engine.frontier()
        pay = engine.frontier_payloads()
        sco = engine.frontier_scores()
        all_rows = gather_rows((rows, pay, sco))
        # every row lives on its hash owner
        if rows.shape[0]:
            assert (owners(rows) == rank).all()
        if backend in ("mlp", "qmlp"):
            # expected set from the device's own scores: gather (child bytes -> key) of all candidates of all ranks
            ncand = fronts[rank].shape[0] * pz.fanout
            dev_scores = buffers["cand_score"][:ncand].cpu().numpy().astype(np.uint32)
            sc_all = [None] * world
            dist.all_gather_object(sc_all, dev_scores)
            want = bo.depth_step(fronts, pz.generators, pz.solved, None, beam, score_override=sc_all, hasher=hasher)
        else:
            want = bo.depth_step(fronts, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam, hasher=hasher)
        got = np.concatenate([r for r, _, _ in all_rows]) if any(r.shape[0] for r, _, _ in all_rows) else rows[:0]
        assert got.shape[0] == want.states.shape[0], (depth, got.shape, want.states.shape)
        assert np.array_equal(bo.sorted_rows(got), bo.sorted_rows(want.states)), f"depth {depth}"
        got_pay = np.concatenate([p for _, p, _ in all_rows])
        got_map = {bytes(r): int(p) for r, p in zip(got, got_pay)}
        want_map = {bytes(r): int(p) for r, p in zip(want.states, want.payload)}
        assert got_map == want_map, f"back-pointers differ at depth {depth}"
        assert bool(st["found"]) == want.found_child
        fronts = [r for r, _, _ in all_rows]
        if st["found"]:
            break
    if rank == 0:
        print(f"CASE_OK {name} beam={beam} backend={backend} graph={graph} exchange={exchange} hash={hash_mode} depths={depth + 1} "
              f"frontier={sum(f.shape[0] for f in fronts)}", flush=True)
    engine.close()
    dist.barrier()
    del engine, buffers


def run_scale_case(beam, exchange, pipeline="persistent"):
    """The sharded benchmark configuration: 54-byte states, 12 moves, global beam `beam` (262 144 = the reference
    configuration's beam) over all ranks, benchmark knobs.  The frontier is saturated by the engine's own depth loop
    (unchecked), then ONE depth is compared with the oracle: survivors, back-pointers, scores, owner placement."""
    world, rank = dist.get_world_size(), dist.get_rank()
    pz = puzzles.puzzle54()
    cfg = be.config_for_puzzle(pz, world_size=world, rank=rank, global_beam_width=beam, max_depth=16, beta=1.2,
                               gamma=1.05, hash_load_factor=0.45, probe_limit=256, band_rounds=3, band_levels=3,
                               inference_backend="central_hamming", use_cuda_graphs=True, exchange=exchange,
                               select_pipeline=pipeline)
    _, cfg, buffers, engine = be.configure_engine(pz, cfg=cfg)
    res = be.run_one_search(engine, pz.scramble(0, 40), 8)
    assert not res["found"] and res["status"]["status_bits"] == 0, res["status_names"]
    fronts = gather_rows(engine.frontier())
    assert sum(f.shape[0] for f in fronts) == beam, [f.shape for f in fronts]
    engine.step()
    st = engine.status()
    assert st["status_bits"] == 0, st["status_names"]
    rows, pay, sco = engine.frontier(), engine.frontier_payloads(), engine.frontier_scores()
    if rows.shape[0]:
        assert (bo.owner_rank(bo.hash64(rows), world) == rank).all()
    parts = gather_rows((rows, pay, sco))
    if rank == 0:
        want = bo.depth_step(fronts, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam)
        got = np.concatenate([r for r, _, _ in parts])
        assert got.shape[0] == want.states.shape[0] == beam, (got.shape, want.states.shape)
        assert np.array_equal(bo.sorted_rows(got), bo.sorted_rows(want.states))
        got_pay = np.concatenate([p for _, p, _ in parts])
        got_sco = np.concatenate([k for _, _, k in parts])
        assert {bytes(r): (int(p), int(k)) for r, p, k in zip(got, got_pay, got_sco)} == \
            {bytes(r): (int(p), int(k)) for r, p, k in zip(want.states, want.payload, want.score)}
        print(f"SCALE_OK beam={beam} world={world} exchange={exchange} pipeline={pipeline} candidates={want.candidates} "
              f"unique={want.unique}", flush=True)
    engine.close()
    dist.barrier()
    del engine, buffers


def run_balance_case():
    """Balanced placement (the reference's final balance, production_v6_dispatcher.py:584-588): after a step the
    survivors sit on their hash owners, unevenly; rebalance_frontier must leave rank q with exactly the rows
    ceil(K q / W) .. ceil(K (q + 1) / W) of the rank-major order (the oracle's balance_targets), rows, scores and
    back-pointers moved together; and a search under placement="balanced" must give the oracle's answer with a path
    that replays."""
    world, rank = dist.get_world_size(), dist.get_rank()
    pz = puzzles.puzzle54()
    beam = 3000 + 7 * world
    _, cfg, buffers, engine = be.configure_engine(pz, world_size=world, rank=rank, global_beam_width=beam, max_depth=16,
                                                  beta=1.2, gamma=1.25, hash_load_factor=0.45, probe_limit=256,
                                                  placement="balanced")
    start = pz.scramble(3, 30)
    owner = engine.owner_of(start)
    engine.reset_search(bytes(start), active_on_this_rank=(owner == rank))
    for _ in range(5):
        engine.step()  # plain steps: survivors stay on their owners

    def snapshot():
        mine = (engine.frontier(), engine.frontier_scores(), engine.frontier_payloads())
        parts = gather_rows(mine)
        return parts

    before = snapshot()
    shares = engine.rebalance_frontier()
    after = snapshot()
    total = sum(p[0].shape[0] for p in before)
    t_rank, t_local = bo.balance_targets(total, world)
    want_counts = [int((t_rank == q).sum()) for q in range(world)]
    assert shares == want_counts and [p[0].shape[0] for p in after] == want_counts, (shares, want_counts)
    for k in range(3):  # rows, scores, back-pointers: the global rank-major sequence is unchanged
        a = np.concatenate([p[k] for p in before], axis=0)
        b = np.concatenate([p[k] for p in after], axis=0)
        assert np.array_equal(a, b), k
    assert len({p[0].shape[0] for p in before}) > 1 or world == 1  # the case was uneven to begin with
    # the step after a rebalance still matches the oracle (parents are fetched from their new places)
    fronts = [p[0] for p in after]
    engine.step()
    got = gather_rows(engine.frontier())
    want = bo.depth_step(fronts, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam)
    assert np.array_equal(bo.sorted_rows(np.concatenate(got, axis=0)), bo.sorted_rows(want.states))
    # whole searches with the rows rebalanced after every depth
    for j in (1, 21, 22):
        s = pz.scramble(j, 6)
        res = be.run_one_search(engine, s, 10)
        w = bo.search(s, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam=beam, max_depth=10)
        assert (bool(res["found"]), res["depth"]) == (bool(w.found), w.depth), (j, res["found"], res["depth"], w.found, w.depth)
        if w.found:
            from multigpubeamsearch_b200.solver import reconstruct_path
            path = reconstruct_path(engine)  # collective walk-back over the ranks' history entries
            assert path is not None and len(path) == w.depth, (j, path)
            assert np.array_equal(bo.replay(s, pz.generators, path), pz.solved), j
    if rank == 0:
        print(f"BALANCE_OK world={world} rows before {[p[0].shape[0] for p in before]} after {want_counts}", flush=True)
    engine.close()
    dist.barrier()


def run_late_rank_case():
    """Failure detection without any GPU fault: the last rank is late on the HOST (it sleeps before it starts its
    depth loop) and the poll limit is short, so the other ranks' waits run out.  Every rank must come back from
    search() with an error and the peer_timeout bit: the early ranks because their waits gave up, the late rank
    because the others told it so (its own waits find their flags already there).  Nothing hangs, no collective is
    left unmatched (peer mode has no NCCL call inside the step)."""
    import time
    world, rank = dist.get_world_size(), dist.get_rank()
    pz = puzzles.puzzle54()
    cfg = be.config_for_puzzle(pz, world_size=world, rank=rank, global_beam_width=2048, max_depth=12, beta=1.2,
                               gamma=1.25, hash_load_factor=0.45, probe_limit=256, band_rounds=3, exchange="peer",
                               peer_poll_limit=100000)
    _, cfg, buffers, engine = be.configure_engine(pz, cfg=cfg)
    start = pz.scramble(1, 30)
    engine.reset_search(bytes(start), active_on_this_rank=(engine.owner_of(start) == rank))
    dist.barrier()
    if rank == world - 1:
        time.sleep(4.0)
    t0 = time.perf_counter()
    failed = False
    try:
        engine.search(10)
    except RuntimeError as exc:
        failed = "peer timeout" in str(exc)
    took = time.perf_counter() - t0
    st = engine.status()
    ok = failed and bool(st["status_bits"] & 64) and took < 30.0
    flags = [None] * world
    dist.all_gather_object(flags, (ok, round(took, 2), st["depth"]))
    assert all(f[0] for f in flags), flags
    if rank == 0:
        print(f"LATE_RANK_OK world={world} per-rank (ok, seconds, depth) = {flags}", flush=True)
    engine.close()
    dist.barrier()
    del engine, buffers


def main():
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if os.environ.get("MGBS_TEST_SCALE", "1") != "0":
        run_scale_case(262144, "peer")
        run_scale_case(262144, "nccl")
    for exchange in ("peer", "nccl"):
        run_case("lrx16", 1024, 30, 12, "central_hamming", False, exchange)
        run_case("rand54", 4096, 12, 6, "central_hamming", True, exchange)
        run_case("rand54", 2048, 30, 5, "mlp", True, exchange)
        run_case("rand54", 4096, 12, 5, "central_hamming", True, exchange, hash_mode="zobrist128")
        run_case("rand54", 2048, 30, 5, "qmlp", True, exchange)
    # the engine's own depth loop: all ranks stop at the same depth with the same answer
    pz = puzzles.puzzle54()
    world, rank = dist.get_world_size(), dist.get_rank()
    _, cfg, buffers, engine = be.configure_engine(pz, world_size=world, rank=rank, global_beam_width=4096, max_depth=16,
                                                  beta=1.2, gamma=1.25, hash_load_factor=0.45, probe_limit=256)
    start = pz.scramble(1, 5)
    res = be.run_one_search(engine, start, 12)
    want = bo.search(start, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam=4096, max_depth=12)
    assert res["found"] == want.found and res["depth"] == want.depth, (res["found"], res["depth"], want.found, want.depth)
    # the solver loop (prepass + cross-rank path walk-back): every found path must replay to the solved state
    from multigpubeamsearch_b200 import solver
    starts = [pz.scramble(j, 6) for j in range(20, 24)]
    summary = solver.solve_many(engine, pz, starts, 10)
    for s, r in zip(starts, summary["results"]):
        w = bo.search(s, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam=4096, max_depth=10)
        assert (r["found"], r["depth"]) == (w.found, w.depth), (r, w.found, w.depth)
        assert (not w.found) or (r["valid"] and len(r["path"]) == w.depth), r
    assert summary["status_bits"] == 0
    if rank == 0:
        print(f"SEARCH_OK found={res['found']} depth={res['depth']} solved={summary['solved']}", flush=True)
    engine.close()
    dist.barrier()
    del engine, buffers
    run_balance_case()
    run_late_rank_case()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
