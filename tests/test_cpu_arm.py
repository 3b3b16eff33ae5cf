"""The benchmark's CPU arm (oracle/torch_cpu_step.py, the PyTorch-CPU restatement timed by `bench.py --impl reference`
and by the `cpu_baseline` leg) must do the same work as the numpy oracle: same surviving set, same keys."""

import numpy as np
import torch

from oracle import beam_oracle as bo
from oracle import torch_cpu_step as tcs
from multigpubeamsearch_b200 import puzzles


def _frontier(pz, count, seed, walk=25):
    rng = np.random.default_rng(seed)
    g = pz.generators.astype(np.int64)
    rows = np.tile(pz.solved, (count, 1))
    for _ in range(walk):
        rows = np.take_along_axis(rows, g[rng.integers(0, pz.fanout, size=count)], axis=1)
    return np.unique(rows, axis=0)


def test_torch_hashes_equal_oracle_hashes():
    rng = np.random.default_rng(11)
    for n in (16, 54, 120):
        s = rng.integers(0, 120 if n == 120 else 6, size=(64, n), dtype=np.uint8)
        t = torch.from_numpy(s)
        assert np.array_equal(tcs.hash64(t).numpy().view(np.uint64), bo.hash64(s))
        assert np.array_equal(tcs.fingerprint64(t).numpy().view(np.uint64), bo.fingerprint64(s))


def test_cpu_arm_hamming_step_equals_oracle_step():
    for name, count, beam in (("lrx16", 200, 128), ("rand54", 400, 1024), ("rand54", 50, 100000)):
        pz = puzzles.by_name(name)
        f = _frontier(pz, count, seed=count)
        nxt, keys = tcs.depth_step(torch.from_numpy(f), torch.from_numpy(pz.generators.astype(np.int64)),
                                   torch.from_numpy(pz.solved), beam, pz.num_values, models=None)
        want = bo.depth_step([f], pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam)
        # same rows in the same (score, hash, fingerprint) order, same keys
        assert np.array_equal(nxt.numpy(), want.states)
        assert np.array_equal(keys.numpy().astype(np.uint32), want.score)


def test_cpu_arm_mlp_step_equals_oracle_step_on_its_own_keys():
    pz = puzzles.puzzle54()
    w = puzzles.mlp_weights(pz.state_len * pz.num_values, 1024)
    f = _frontier(pz, 300, seed=3)
    model = tcs.TorchMLP(w)
    beam = 512
    nxt, keys = tcs.depth_step(torch.from_numpy(f), torch.from_numpy(pz.generators.astype(np.int64)),
                               torch.from_numpy(pz.solved), beam, pz.num_values, [model], -150.0)
    children = bo.expand(f, pz.generators)
    # float32 network: torch and numpy agree to rounding, so the keys differ by at most one unit
    q_np = bo.mlp_forward(children, [w], pz.num_values)
    with torch.no_grad():
        x = torch.nn.functional.one_hot(torch.from_numpy(children).to(torch.int64), pz.num_values).flatten(1).float()
        q_t = model(x).numpy()
    assert np.abs(q_t - q_np).max() < 1e-5
    k_t = bo.q_to_score_key(q_t, -150.0)
    assert np.abs(k_t.astype(np.int64) - bo.q_to_score_key(q_np, -150.0).astype(np.int64)).max() <= 1
    # selection given the arm's own keys is the oracle's selection
    want = bo.depth_step([f], pz.generators, pz.solved, None, beam, score_override=[k_t])
    assert np.array_equal(bo.sorted_rows(nxt.numpy()), bo.sorted_rows(want.states))
    assert sorted(keys.numpy().tolist()) == sorted(want.score.tolist())
