"""world_size-2 (and 3) gloo test on CPU of the sharded selection protocol.

Each CPU rank expands its own frontier rows, routes the candidates by hash owner through an all-to-all of Python
objects, runs the band-round / radix top-K protocol with all-reduced histograms, and the union of the ranks'
survivors must equal the single-rank oracle's beam, for Hamming scores (massive ties) and for few-hash-bit keys
(cross-rank tie records).
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import beam_oracle as bo
from oracle import sharded_model as sm
from multigpubeamsearch_b200 import puzzles


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, beam, hash_bits, out_q, band_routed=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pz = puzzles.puzzle54()
        # every rank derives the same global frontier, then keeps the rows it owns
        rows = np.unique(np.stack([pz.scramble(j, 14) for j in range(160)]), axis=0)
        own = bo.owner_rank(bo.hash64(rows), world)
        mine = rows[own == rank]
        children = bo.expand(mine, pz.generators)
        pidx = np.repeat(np.arange(mine.shape[0], dtype=np.uint32), pz.fanout)
        mv = np.tile(np.arange(pz.fanout, dtype=np.uint32), mine.shape[0])
        cand = sm.Candidates(children, bo.hash64(children), bo.fingerprint64(children),
                             bo.hamming(children, pz.solved), bo.pack_payload(pidx, np.full_like(pidx, rank), mv))
        def exchange(buckets):
            """bucket r goes to rank r; returns the buckets sent here"""
            gathered = [None] * world
            dist.all_gather_object(gathered, buckets)
            return [gathered[src][rank] for src in range(world)]

        if not band_routed:
            recv = exchange(sm.route(cand, world))
            local = sm.Candidates(*(np.concatenate([getattr(b, f) for b in recv])
                                    for f in ("states", "h", "fp", "score", "payload")))
            assert (bo.owner_rank(local.h, world) == rank).all()

        def allreduce_sum(a):
            t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.int64))
            dist.all_reduce(t)
            return t.numpy()

        def allgather(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out

        n_local = (beam + world - 1) // world
        pool_target = int(1.2 * n_local + 0.5)
        hash_capacity = max(1024, int(1.2 * 1.25 * n_local / 0.45 + 0.5))
        if band_routed:
            local, keep, stats = sm.sharded_select(cand, beam, world, pool_target, hash_capacity, allreduce_sum,
                                                   allgather, hash_bits=hash_bits, band_exchange=exchange)
            assert (bo.owner_rank(local.h, world) == rank).all()
            stats["received"] = int(local.h.shape[0])
            stats["generated"] = int(cand.h.shape[0])
        else:
            keep, stats = sm.sharded_select(local, beam, world, pool_target, hash_capacity, allreduce_sum, allgather,
                                            hash_bits=hash_bits)
        survivors = allgather((local.states[keep], local.payload[keep]))
        if rank == 0:
            fronts = [rows[own == r] for r in range(world)]
            want = bo.depth_step(fronts, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam)
            got = np.concatenate([s for s, _ in survivors])
            got_pay = np.concatenate([p for _, p in survivors])
            ok = got.shape[0] == want.states.shape[0] and \
                np.array_equal(bo.sorted_rows(got), bo.sorted_rows(want.states)) and \
                {bytes(r): int(p) for r, p in zip(got, got_pay)} == {bytes(r): int(p) for r, p in zip(want.states, want.payload)}
            out_q.put((ok, stats, int(got.shape[0])))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,beam,hash_bits", [(2, 300, 44), (2, 64, 2), (3, 500, 44), (2, 100000, 44)])
def test_sharded_selection_equals_single_rank_oracle(world, beam, hash_bits):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, beam, hash_bits, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    ok, stats, count = q.get(timeout=10)
    assert ok, (stats, count)
    assert stats["stalls"] == 0


@pytest.mark.parametrize("world,beam,hash_bits", [(2, 300, 24), (2, 64, 2), (3, 500, 44)])
def test_band_routed_selection_equals_single_rank_oracle(world, beam, hash_bits):
    """The peer-exchange order of operations: histograms where the candidates were generated, then only the band
    travels.  Same survivors as the single-rank oracle, and fewer records cross than were generated."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, beam, hash_bits, q, True)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    ok, stats, count = q.get(timeout=10)
    assert ok, (stats, count)
    assert stats["stalls"] == 0
    assert stats["received"] < stats["generated"]
