"""Allocation-free scoring entry point (collected last on purpose: a failure here stops nothing else).

Some callers of the library cannot allocate device memory when they need scores - a serving loop inside an
allocation-free region, a plugin whose memory was fixed at load time.  mgbs_mlp_score_noalloc serves them from a
static device array inside the library.  This test calls it through the C ABI and checks that it returns exactly
the keys of the ordinary entry point, twice in a row with different sizes so that leftovers of the first call in
the shared array are seen not to matter.  The ordinary scorer is switched to the same kernel sequence the
allocation-free call launches (separate one-hot kernel, plain layer-1 GEMM, single-CTA head), so the two sum in the
same order and equality is exact by construction; against the default fused kernels the keys may differ by one
unit, which the test also bounds.  It also checks the property the entry point exists for: the device's free
memory does not change across a call.
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
        sc.set_l1_mode(True)
        sc.set_head_mode(True)
        fused = sc.score(children).clone()
        sc.set_l1_mode(False)   # the kernel sequence of the allocation-free call
        sc.set_head_mode(False)
        want = sc.score(children).clone()
        torch.cuda.synchronize()
        assert sc.error_code() == 0
        got = torch.full((count,), -1, dtype=torch.int32, device="cuda")
        if call == 1:
            # the first call on a device resolves the static array's address; from the second call on nothing
            # may change the amount of free device memory
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info()
        err = sc.score_no_alloc(children, got)
        assert err == 0
        if call == 1:
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before, (free_before, free_after)
        assert torch.equal(got, want), f"call {call}: keys differ"
        assert int((got.to(torch.int64) - fused.to(torch.int64)).abs().max()) <= 1
        assert len(torch.unique(want)) > 1  # the comparison is not vacuous


def test_no_alloc_rejects_oversize_requests():
    pz = puzzles.puzzle54()
    sc = scorers.MLPValueScorer(puzzles.mlp_weights(324, 1024), 54, 64, 6, max_rows=8192)
    children = torch.from_numpy(_children(pz, scorers.NOALLOC_MAX_ROWS + 1, seed=3)).cuda()
    out = torch.zeros(children.shape[0], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="static scratch"):
        sc.score_no_alloc(children, out)
