"""Allocation-free scoring entry point (collected last on purpose: a failure here stops nothing else).

Some callers of the library cannot allocate device memory when they need scores - a serving loop inside an
allocation-free region, a plugin whose memory was fixed at load time.  mgbs_mlp_score_noalloc serves them from a
static device array inside the library.  This test calls it through the C ABI and checks that it returns exactly
the keys of the ordinary entry point (same kernels, so equality is exact), twice in a row with different sizes so
that leftovers of the first call in the shared array are seen not to matter.
"""

import numpy as np
import pytest
import torch

from multigpubeamsearch_b200 import puzzles, scorers

pytestmark = pytest.mark.gpu


def _children(pz, count, seed):
    rng = np.random.default_rng(seed)
    g = pz.generators.astype(np.int64)
    rows = np.tile(pz.solved, (count, 1))
    for _ in range(25):
        rows = np.take_along_axis(rows, g[rng.integers(0, pz.fanout, size=count)], axis=1)
    out = np.zeros((count, 64), np.uint8)
    out[:, : pz.state_len] = rows
    return out


def test_no_alloc_scores_equal_regular_entry_point_twice():
    pz = puzzles.puzzle54()
    w = puzzles.mlp_weights(324, 1024, model_idx=1)
    w["b1"] = (np.random.default_rng(1).standard_normal(1024) * 0.03).astype(np.float32)
    w["b3"] = np.float32(-0.5)
    sc = scorers.MLPValueScorer(w, 54, 64, 6, max_rows=4096, score_offset=-150.0)
    for call, count in enumerate((4096, 777)):
        children = torch.from_numpy(_children(pz, count, seed=10 + call)).cuda()
        want = sc.score(children)
        torch.cuda.synchronize()
        assert sc.error_code() == 0
        got = torch.full((count,), -1, dtype=torch.int32, device="cuda")
        err = sc.score_no_alloc(children, got)
        assert err == 0
        assert torch.equal(got, want), f"call {call}: keys differ"
        assert len(torch.unique(want)) > 1  # the comparison is not vacuous


def test_no_alloc_rejects_oversize_requests():
    pz = puzzles.puzzle54()
    sc = scorers.MLPValueScorer(puzzles.mlp_weights(324, 1024), 54, 64, 6, max_rows=8192)
    children = torch.from_numpy(_children(pz, scorers.NOALLOC_MAX_ROWS + 1, seed=3)).cuda()
    out = torch.zeros(children.shape[0], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="static scratch"):
        sc.score_no_alloc(children, out)
