"""GPU tests of the tcgen05 MLP scorer against a float32 evaluation (tolerance stated in each test)."""

import numpy as np
import pytest
import torch

from oracle import beam_oracle as bo
from multigpubeamsearch_b200 import beam_engine as be
from multigpubeamsearch_b200 import puzzles, scorers

pytestmark = pytest.mark.gpu


def children_of(pz, count, seed):
    rng = np.random.default_rng(seed)
    g = pz.generators.astype(np.int64)
    rows = np.tile(pz.solved, (count, 1))
    for _ in range(30):
        mv = rng.integers(0, pz.fanout, size=count)
        rows = np.take_along_axis(rows, g[mv], axis=1)
    return rows


def padded(rows, stride):
    out = np.zeros((rows.shape[0], stride), np.uint8)
    out[:, : rows.shape[1]] = rows
    return out


@pytest.mark.parametrize("name,count,models", [("rand54", 1000, 1), ("rand54", 40000, 1), ("rand96", 5000, 3),
                                               ("rand54", 1, 1), ("rand54", 129, 2)])
def test_mlp_scorer_matches_fp32(name, count, models):
    pz = puzzles.by_name(name)
    stride = (pz.state_len + 15) // 16 * 16
    ws = [puzzles.mlp_weights(pz.state_len * pz.num_values, 1024, model_idx=i) for i in range(models)]
    # non-zero biases so that every epilogue term is exercised
    rng = np.random.default_rng(3)
    for w in ws:
        w["b1"] = (rng.standard_normal(1024) * 0.05).astype(np.float32)
        w["b2"] = (rng.standard_normal(1024) * 0.05).astype(np.float32)
        w["b3"] = np.float32(0.25)
    sc = scorers.MLPValueScorer(ws, pz.state_len, stride, pz.num_values, max_rows=count, score_offset=-150.0)
    rows = children_of(pz, count, seed=count)
    keys = sc.score(torch.from_numpy(padded(rows, stride)).cuda())
    torch.cuda.synchronize()
    assert sc.error_code() == 0
    q_ref = bo.mlp_forward(rows, ws, pz.num_values)  # float32, mean over members
    q_dev = (sc.last_q(count).cpu().numpy() + sum(float(w["b3"]) for w in ws)) / models
    # bf16 operands (8 mantissa bits), fp32 accumulation: observed error ~1e-3 on outputs of magnitude ~0.3
    assert np.abs(q_dev - q_ref).max() <= 5e-3
    key_ref = bo.q_to_score_key(q_ref, -150.0)
    assert np.abs(keys.cpu().numpy().astype(np.int64) - key_ref.astype(np.int64)).max() <= 2
    # keys are exactly the quantisation of the device's own q
    assert np.array_equal(keys.cpu().numpy().astype(np.uint32), bo.q_to_score_key(q_dev.astype(np.float32), -150.0))


def test_scorer_rows_are_batch_invariant():
    # the same state gets the same key wherever it sits in the batch (needed for dedup: equal states, equal scores)
    pz = puzzles.puzzle54()
    w = puzzles.mlp_weights(324, 1024)
    sc = scorers.MLPValueScorer(w, 54, 64, 6, max_rows=3000)
    rows = children_of(pz, 3000, seed=1)
    a = sc.score(torch.from_numpy(padded(rows, 64)).cuda()).cpu().numpy()
    perm = np.random.default_rng(0).permutation(3000)
    b = sc.score(torch.from_numpy(padded(rows[perm], 64)).cuda()).cpu().numpy()
    assert np.array_equal(a[perm], b)


def test_engine_with_mlp_scorer_matches_oracle_on_device_scores():
    # selection logic is exact given the scores the device produced: feed them to the oracle
    pz = puzzles.puzzle54()
    beam = 2048
    w = puzzles.mlp_weights(324, 1024)
    cfg = be.config_for_puzzle(pz, global_beam_width=beam, max_depth=8, beta=1.2, hash_load_factor=0.45,
                               probe_limit=256, band_rounds=8, inference_backend="mlp")
    ext = be.build_extension()
    be.init_distributed_if_needed(cfg)
    sizes = ext.derive_sizes(cfg)
    sc = scorers.MLPValueScorer(w, 54, 64, 6, max_rows=sizes["cand_cap"])
    _, cfg, buffers, engine = be.configure_engine(pz, cfg=cfg, scorer=sc)
    frontier = np.unique(children_of(pz, 1500, seed=5), axis=0)
    engine.load_frontier(frontier)
    engine.enable_cuda_graphs(False)
    engine.step()
    st = engine.status()
    assert st["status_bits"] == 0 and sc.error_code() == 0
    ncand = frontier.shape[0] * pz.fanout
    dev_scores = buffers["cand_score"][:ncand].cpu().numpy().astype(np.uint32)
    want = bo.depth_step([frontier], pz.generators, pz.solved, None, beam, score_override=[dev_scores])
    got = engine.frontier()
    assert np.array_equal(bo.sorted_rows(got), bo.sorted_rows(want.states))
    # and the device scores are within 2 key units of the float32 network
    q_ref = bo.mlp_forward(bo.expand(frontier, pz.generators), [w], 6)
    assert np.abs(dev_scores.astype(np.int64) - bo.q_to_score_key(q_ref, -150.0).astype(np.int64)).max() <= 2
    # graph replay gives the same frontier
    engine.load_frontier(frontier)
    engine.enable_cuda_graphs(True)
    engine.step()
    assert np.array_equal(bo.sorted_rows(engine.frontier()), bo.sorted_rows(want.states))


def test_fused_layer1_equals_unfused_path():
    # the in-shared-memory one-hot operand and the TMA-store epilogue change no bit of the result
    pz = puzzles.puzzle96()
    ws = [puzzles.mlp_weights(96 * 8, 1024, model_idx=i) for i in range(2)]
    ws[0]["b1"] = (np.random.default_rng(8).standard_normal(1024) * 0.05).astype(np.float32)
    sc = scorers.MLPValueScorer(ws, 96, 96, 8, max_rows=20000)
    rows = children_of(pz, 20000 - 37, seed=2)
    dev = torch.from_numpy(padded(rows, 96)).cuda()
    sc.set_l1_mode(True)
    a = sc.score(dev).clone()
    h1_a = sc.h1[: rows.shape[0]].clone()
    sc.set_l1_mode(False)
    b = sc.score(dev).clone()
    torch.cuda.synchronize()
    assert sc.error_code() == 0
    assert torch.equal(h1_a, sc.h1[: rows.shape[0]])
    assert torch.equal(a, b)


@pytest.mark.parametrize("dtype,count", [("bf16", 1000), ("bf16", 257), ("fp8", 513), ("bf16", 70000)])
def test_head_on_cta_pairs_equals_single_cta_path(dtype, count):
    """Layer 2 + head on CTA pairs (default) against the one-CTA-per-tile kernel: the same products summed in the
    same order inside every output row, so the raw head outputs agree to float32 rounding of the row sums."""
    pz = puzzles.puzzle54()
    ws = [puzzles.mlp_weights(324, 1024, model_idx=i) for i in range(2)]
    rng = np.random.default_rng(5)
    for w in ws:
        w["b1"] = (rng.standard_normal(1024) * 0.05).astype(np.float32)
        w["b2"] = (rng.standard_normal(1024) * 0.05).astype(np.float32)
    sc = scorers.MLPValueScorer(ws, 54, 64, 6, max_rows=count, score_offset=-150.0, dtype=dtype)
    dev = torch.from_numpy(padded(children_of(pz, count, seed=9), 64)).cuda()
    sc.set_head_mode(True)
    k_pair = sc.score(dev).cpu().numpy()
    q_pair = sc.last_q(count).cpu().numpy().copy()
    sc.set_head_mode(False)
    k_single = sc.score(dev).cpu().numpy()
    q_single = sc.last_q(count).cpu().numpy().copy()
    assert sc.error_code() == 0
    assert np.abs(q_pair - q_single).max() <= 1e-5, np.abs(q_pair - q_single).max()
    assert np.abs(k_pair.astype(np.int64) - k_single.astype(np.int64)).max() <= 1


@pytest.mark.parametrize("name,count,models", [("rand54", 20000, 1), ("rand96", 5000, 2), ("rand54", 77, 1)])
def test_fp8_scorer_within_tolerance(name, count, models):
    # FP8 E4M3 operands with per-channel weight scales: max-abs error of the network output <= 2e-2 (stated bound)
    pz = puzzles.by_name(name)
    stride = (pz.state_len + 15) // 16 * 16
    ws = [puzzles.mlp_weights(pz.state_len * pz.num_values, 1024, model_idx=10 + i) for i in range(models)]
    rng = np.random.default_rng(4)
    for w in ws:
        w["b1"] = (rng.standard_normal(1024) * 0.05).astype(np.float32)
        w["b2"] = (rng.standard_normal(1024) * 0.05).astype(np.float32)
        w["b3"] = np.float32(0.1)
    sc = scorers.MLPValueScorer(ws, pz.state_len, stride, pz.num_values, max_rows=count, dtype="fp8")
    rows = children_of(pz, count, seed=count + 1)
    dev = torch.from_numpy(padded(rows, stride)).cuda()
    keys = sc.score(dev)
    torch.cuda.synchronize()
    assert sc.error_code() == 0
    q_ref = bo.mlp_forward(rows, ws, pz.num_values)
    q_dev = (sc.last_q(count).cpu().numpy() + sum(float(w["b3"]) for w in ws)) / models
    err = np.abs(q_dev - q_ref).max()
    assert err <= 2e-2, err
    assert np.abs(q_dev - q_ref).mean() <= 5e-3
    # keys are the quantisation of the device's own q (the host recomputation may round a .5 boundary differently)
    rekey = bo.q_to_score_key(q_dev.astype(np.float32), -150.0).astype(np.int64)
    assert np.abs(keys.cpu().numpy().astype(np.int64) - rekey).max() <= 1
    # same rows in another order give the same keys
    perm = np.random.default_rng(1).permutation(count)
    keys2 = sc.score(dev[torch.from_numpy(perm).cuda()].contiguous())
    assert np.array_equal(keys.cpu().numpy()[perm], keys2.cpu().numpy())


def _dequantize_nvfp4_activations(sc, count):
    """Host view of the scorer's packed 4-bit activations: E2M1 codes x E4M3 block factors x tensor scale, read
    back from the device buffers in the tile layout the tensor core consumes."""
    vals = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], np.float32)
    hidden = sc.hidden
    packed = sc.h1q[:count].cpu().numpy()
    codes = np.empty((count, hidden), np.uint8)
    codes[:, 0::2] = packed & 15
    codes[:, 1::2] = packed >> 4
    deq = np.where(codes & 8, -1.0, 1.0).astype(np.float32) * vals[codes & 7]
    sf = sc.sf_h1.view(torch.float8_e4m3fn).to(torch.float32).cpu().numpy().reshape(-1, hidden // 256, 4, 32, 4, 4)
    tscale = np.float32(sc.act_bound / (6.0 * 448.0))
    out = np.zeros((count, hidden), np.float32)
    for r in range(count):  # factors of row r: tile r // 128, lane (r % 128) % 32, column (r % 128) // 32
        mt, rr = divmod(r, 128)
        r1, r0 = divmod(rr, 32)
        out[r] = deq[r] * np.repeat(sf[mt, :, :, r0, r1, :].reshape(-1), 16) * tscale
    return out


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("name,count,wscale", [("rand54", 20000, 1.0), ("rand96", 5000, 1.0), ("rand54", 77, 1.0),
                                               ("rand54", 3000, 6.0)])
def test_nvfp4_scorer_within_tolerance(name, count, wscale, fused):
    """Second layer on the block-scaled 4-bit tensor-core path (E2M1 elements, E4M3 factor per 16, float32 tensor
    scale; first layer e4m3).  Three checks: (1) the stated bound, max-abs error of the network output <= 5e-2
    against the float32 network; (2) the tensor-core GEMM itself is exact: the device output equals a float32
    evaluation on the host of the device's own packed activations and the host-packed weights to 1e-5 - any mistake
    in the operand or scale-factor layouts would show here, while (1) alone would not notice (the random-init
    network's outputs are only a few hundredths wide); (3) the activation quantiser agrees with the oracle's NVFP4
    model except where the two float32 sums fall on different sides of a rounding boundary.  One case scales the
    weights up so that outputs are of order one."""
    pz = puzzles.by_name(name)
    stride = (pz.state_len + 15) // 16 * 16
    w = puzzles.mlp_weights(pz.state_len * pz.num_values, 1024, model_idx=20)
    rng = np.random.default_rng(5)
    w["w1"] = (w["w1"] * wscale).astype(np.float32)
    w["w2"] = (w["w2"] * wscale).astype(np.float32)
    w["b1"] = (rng.standard_normal(1024) * 0.05).astype(np.float32)
    w["b2"] = (rng.standard_normal(1024) * 0.05).astype(np.float32)
    w["b3"] = np.float32(0.1)
    sc = scorers.MLPValueScorer([w], pz.state_len, stride, pz.num_values, max_rows=count, dtype="nvfp4")
    sc.set_l1_mode(fused)
    rows = children_of(pz, count, seed=count + 2)
    dev = torch.from_numpy(padded(rows, stride)).cuda()
    keys = sc.score(dev)
    torch.cuda.synchronize()
    assert sc.error_code() == 0
    q_dev = sc.last_q(count).cpu().numpy() + float(w["b3"])
    q_ref = bo.mlp_forward(rows, [w], pz.num_values)
    # (2) exact GEMM on the device's own operands
    n_chk = min(count, 2000)
    h1q_dev = _dequantize_nvfp4_activations(sc, n_chk)
    w2q = bo.quantize_nvfp4(w["w2"], bo.nvfp4_tensor_scale(float(np.abs(w["w2"]).max())))
    q_host = np.maximum(h1q_dev @ w2q.T + w["b2"][None, :], 0.0) @ w["w3"] + float(w["b3"])
    assert np.abs(q_dev[:n_chk] - q_host).max() <= 1e-5 * max(1.0, wscale ** 2), np.abs(q_dev[:n_chk] - q_host).max()
    # (3) activation quantiser against the oracle's model
    x = bo.one_hot(rows[:n_chk], pz.num_values)
    w1q, s1 = bo._e4m3_rows(w["w1"])
    h1 = np.maximum(x @ (w1q * s1[:, None]).T + w["b1"][None, :], 0.0).astype(np.float32)
    h1q_model = bo.quantize_nvfp4(h1 if fused else bo._e4m3_tensor(h1, sc.act_bound), bo.nvfp4_tensor_scale(sc.act_bound))
    differs = np.abs(h1q_dev - h1q_model) > 1e-6
    # two-pass form: e4m3 values over an e4m3 factor often sit exactly on an E2M1 midpoint (2.5, 1.25, ...), where the
    # device's x * (1 / step) and the model's x / step round to different neighbours; the fused form has no such ties
    assert differs.mean() < (1e-4 if fused else 0.03), differs.mean()
    assert np.abs(h1q_dev - h1q_model).max() <= 0.26 * float(h1.max()), np.abs(h1q_dev - h1q_model).max()
    q_model = bo.mlp_forward_nvfp4_model(rows, [w], pz.num_values, sc.act_bound, via_e4m3=not fused)
    assert np.abs(q_dev - q_model).max() <= 2e-2 * max(1.0, wscale ** 2)
    # (1) the stated bound
    if wscale == 1.0:
        assert np.abs(q_dev - q_ref).max() <= 5e-2, np.abs(q_dev - q_ref).max()
    else:
        spread = float(q_ref.max() - q_ref.min())
        assert spread > 0.3 and np.corrcoef(q_dev, q_ref)[0, 1] > 0.97, (spread, np.corrcoef(q_dev, q_ref)[0, 1])
    rekey = bo.q_to_score_key(q_dev.astype(np.float32), -150.0).astype(np.int64)
    assert np.abs(keys.cpu().numpy().astype(np.int64) - rekey).max() <= 1
    perm = np.random.default_rng(1).permutation(count)
    keys2 = sc.score(dev[torch.from_numpy(perm).cuda()].contiguous())
    assert np.array_equal(keys.cpu().numpy()[perm], keys2.cpu().numpy())


def test_nvfp4_head_variants_agree():
    """The two forms of the block-scaled head (256-column tiles with one accumulator, 128-column tiles with two) read
    the same quantised operands: their outputs differ only by float32 summation order in the epilogue."""
    pz = puzzles.by_name("rand54")
    count = 30000 + 55
    w = puzzles.mlp_weights(pz.state_len * pz.num_values, 1024)
    sc = scorers.MLPValueScorer(w, pz.state_len, 64, pz.num_values, max_rows=count, dtype="nvfp4")
    dev = torch.from_numpy(padded(children_of(pz, count, seed=31), 64)).cuda()
    qs = []
    for wide in (True, False):
        sc.set_head_mode(wide)
        sc.score(dev)
        torch.cuda.synchronize()
        assert sc.error_code() == 0, wide
        qs.append(sc.last_q(count).cpu().numpy().copy())
    sc.set_head_mode(True)
    scale = float(np.abs(qs[1]).max())
    assert np.abs(qs[0] - qs[1]).max() <= 1e-5 * max(scale, 1.0), (np.abs(qs[0] - qs[1]).max(), scale)


def test_nvfp4_ensemble_within_tolerance():
    """Three members (the large-frontier configuration's scorer): the members' head outputs add up in one buffer."""
    pz = puzzles.puzzle96()
    ws = [puzzles.mlp_weights(pz.state_len * pz.num_values, 1024, model_idx=30 + i) for i in range(3)]
    sc = scorers.MLPValueScorer(ws, pz.state_len, 96, pz.num_values, max_rows=4000, dtype="nvfp4")
    rows = children_of(pz, 4000, seed=9)
    sc.score(torch.from_numpy(padded(rows, 96)).cuda())
    torch.cuda.synchronize()
    assert sc.error_code() == 0
    q_dev = (sc.last_q(4000).cpu().numpy() + sum(float(w["b3"]) for w in ws)) / 3
    assert np.abs(q_dev - bo.mlp_forward(rows, ws, pz.num_values)).max() <= 5e-2


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
def test_layer1_kernel_variants_agree(dtype):
    """Four or eight epilogue warps, single CTAs or CTA pairs: the same activations and keys, bit for bit."""
    pz = puzzles.by_name("rand54")
    count = 20000 + 77  # a ragged last tile, and an odd number of tiles for the pairs
    w = puzzles.mlp_weights(pz.state_len * pz.num_values, 1024)
    w["b1"] = (np.random.default_rng(3).standard_normal(1024) * 0.05).astype(np.float32)
    sc = scorers.MLPValueScorer(w, pz.state_len, 64, pz.num_values, max_rows=count, dtype=dtype)
    dev = torch.from_numpy(padded(children_of(pz, count, seed=21), 64)).cuda()
    base = None
    for ew in (4, 8):
        for pair in (0, 1):
            sc.set_l1_variant(ew, pair)
            sc.h1.zero_()
            keys = sc.score(dev)
            torch.cuda.synchronize()
            assert sc.error_code() == 0, (ew, pair)
            got = (sc.h1[:count].view(torch.uint8).clone(), keys.clone())
            if base is None:
                base = got
            else:
                assert torch.equal(got[0], base[0]) and torch.equal(got[1], base[1]), (ew, pair)
    sc.set_l1_variant(0, -1)


def _q_weights(pz, models, h1=1024, h2=512):
    ws = [puzzles.q_mlp_weights(pz.state_len * pz.num_values, pz.fanout, h1, h2, model_idx=i) for i in range(models)]
    rng = np.random.default_rng(17)
    for w in ws:  # non-zero biases so that every epilogue term is exercised
        w["b1"] = (rng.standard_normal(h1) * 0.05).astype(np.float32)
        w["b2"] = (rng.standard_normal(h2) * 0.05).astype(np.float32)
        w["b3"] = (rng.standard_normal(pz.fanout) * 0.1).astype(np.float32)
    return ws


@pytest.mark.parametrize("name,count,models,h2", [("rand54", 1000, 1, 512), ("rand96", 4097, 2, 256), ("rand54", 1, 1, 1024)])
def test_action_value_scorer_matches_fp32(name, count, models, h2):
    """One forward pass per parent, one value per move (the reference's scorer contract) against float32."""
    pz = puzzles.by_name(name)
    stride = (pz.state_len + 15) // 16 * 16
    ws = _q_weights(pz, models, 1024, h2)
    sc = scorers.MLPActionValueScorer(ws, pz.state_len, stride, pz.num_values, pz.fanout, max_parents=count)
    rows = children_of(pz, count, seed=count + 5)
    keys = sc.score(torch.from_numpy(padded(rows, stride)).cuda())
    torch.cuda.synchronize()
    assert sc.error_code() == 0
    q_ref = bo.mlp_action_values(rows, ws, pz.num_values)  # [P, G], mean over members
    q_dev = sc.last_q(count).cpu().numpy() / models
    assert q_dev.shape == q_ref.shape
    # bf16 operands and bf16 activations between layers, fp32 accumulation
    assert np.abs(q_dev - q_ref).max() <= 5e-3, np.abs(q_dev - q_ref).max()
    assert np.array_equal(keys.cpu().numpy().astype(np.uint32),
                          bo.q_to_score_key(q_dev.reshape(-1).astype(np.float32), -150.0))


def _golden_generators():
    import importlib.util
    from pathlib import Path
    path = Path(__file__).resolve().parent / "golden" / "make_residual_q_golden.py"
    spec = importlib.util.spec_from_file_location("make_residual_q_golden", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("size,classes,state_len,h1,h2,outs,rows,embed_sum", [
    (54, 6, 54, 512, 256, 12, 3000, False),     # one-hot contraction for the first layer
    (54, 6, 54, 512, 256, 12, 3000, True),      # the same network through the embedding sum
    (128, 128, 120, 512, 256, 24, 1500, None),  # the reference's own layout: 120-byte states in 128 x 128 storage
    (54, 6, 54, 256, 512, 12, 1, True),
])
def test_residual_action_value_network_matches_fp32(size, classes, state_len, h1, h2, outs, rows, embed_sum):
    """The reference's static network (embedding sum, hidden layer, two residual blocks, one value per move) from its
    weight dictionary, against the float32 restatement of static_forward_q that the golden vectors pin."""
    mod = _golden_generators()
    w = mod.residual_q_weights(9700 + h1 + h2, size, classes, h1, h2, outs)
    states = mod.residual_q_states(9800 + rows, rows, state_len, min(classes, 120))
    stride = (state_len + 15) // 16 * 16
    sc = scorers.fullbeamnice_scorer_from_static_weights(w, state_len, stride, outs, max_parents=rows,
                                                         embed_sum=embed_sum)
    assert sc.num_res_blocks == 2 and sc.embed_sum == (embed_sum if embed_sum is not None else True)
    keys = sc.score(torch.from_numpy(padded(states, stride)).cuda())
    torch.cuda.synchronize()
    assert sc.error_code() == 0
    q_ref = bo.residual_q_forward(states, w)[:, w["action_perm"]]  # column m = move m of the engine
    q_dev = sc.last_q(rows).cpu().numpy()
    assert q_dev.shape == q_ref.shape
    # bf16 operands and bf16 activations across six layers, float32 accumulation: 2e-2 of the output range
    span = float(q_ref.max() - q_ref.min()) if rows > 1 else float(np.abs(q_ref).max())
    assert np.abs(q_dev - q_ref).max() <= 2e-2 * max(span, 1.0), (np.abs(q_dev - q_ref).max(), span)
    assert np.array_equal(keys.cpu().numpy().astype(np.uint32), bo.q_to_score_key(q_dev.reshape(-1), 0.0))


def test_embedding_sum_equals_one_hot_contraction():
    """Both forms of the first layer on the same bf16 table: the sums differ only in float32 summation order."""
    mod = _golden_generators()
    w = mod.residual_q_weights(9901, 54, 6, 512, 256, 12)
    states = mod.residual_q_states(9902, 2000, 54, 6)
    dev = torch.from_numpy(padded(states, 64)).cuda()
    qs = []
    for form in (False, True):
        sc = scorers.fullbeamnice_scorer_from_static_weights(w, 54, 64, 12, max_parents=2000, embed_sum=form)
        sc.score(dev)
        torch.cuda.synchronize()
        assert sc.error_code() == 0
        qs.append(sc.last_q(2000).cpu().numpy().copy())
    assert np.abs(qs[0] - qs[1]).max() <= 5e-2  # one bf16 rounding step of a first-layer activation, propagated


@pytest.mark.parametrize("mode", ["q", "sigmoid_u16", "float_u16"])
def test_reference_action_scorer_module_on_the_device(mode):
    """MLPActionScorer (dense layer on scaled bytes, GELU, two hidden layers) through the embedding-sum kernel, and the
    16-bit quantiser modes as keys 65535 - score."""
    mod = _golden_generators()
    n, V, fanout, rows = 120, 120, 24, 2500
    layers = mod.action_scorer_weights(9931, n, (512, 256), fanout)
    if mode == "float_u16":  # spread the outputs over a useful range of the 16-bit scale
        layers[-1] = (layers[-1][0] * 2000.0, layers[-1][1] * 2000.0 + 30000.0)
    base = scorers.MLPActionScorer(n, (512, 256), fanout)
    with torch.no_grad():
        for lin, (wm, bv) in zip((*base.linears, base.out), layers):
            lin.weight.copy_(torch.from_numpy(wm))
            lin.bias.copy_(torch.from_numpy(bv))
    module = base if mode == "q" else scorers.QuantizedActionScorer(base, mode)
    sc = scorers.action_scorer_to_device(module, n, 128, V, max_parents=rows)
    states = mod.residual_q_states(9932, rows, n, V)
    keys = sc.score(torch.from_numpy(padded(states, 128)).cuda()).cpu().numpy().astype(np.uint32)
    torch.cuda.synchronize()
    assert sc.error_code() == 0
    y_ref = bo.action_scorer_forward(states, layers)
    y_dev = sc.last_q(rows).cpu().numpy()
    span = float(y_ref.max() - y_ref.min())
    assert np.abs(y_dev - y_ref).max() <= 2e-2 * max(span, 1.0), (np.abs(y_dev - y_ref).max(), span)
    if mode == "q":
        assert np.array_equal(keys, bo.q_to_score_key(y_dev.reshape(-1), 0.0))
    else:  # exact on the device's own outputs up to the last bit of exp / rounding at .5
        want = 65535 - bo.quantized_action_scores(y_dev.reshape(-1), mode).astype(np.int64)
        assert np.abs(keys.astype(np.int64) - want).max() <= 1


def test_engine_loads_the_static_network_and_steps():
    """BeamEngine.load_fullbeamnice_static (beam_engine.cpp:887-891): the dictionary becomes the parent scorer; the
    step then selects exactly on the keys the device computed."""
    mod = _golden_generators()
    pz = puzzles.puzzle54()
    w = mod.residual_q_weights(9911, 54, 6, 512, 256, pz.fanout)
    cfg = be.config_for_puzzle(pz, global_beam_width=500, max_depth=4, beta=1.2, hash_load_factor=0.45,
                               probe_limit=256, band_rounds=8, inference_backend="mlp", score_offset=0.0)
    _, cfg, buffers, engine = be.configure_engine(pz, cfg=cfg)
    engine.load_fullbeamnice_static(w)
    frontier = np.unique(children_of(pz, 300, seed=8), axis=0)
    engine.load_frontier(frontier)
    engine.step()
    st = engine.status()
    assert st["status_bits"] == 0
    ncand = frontier.shape[0] * pz.fanout
    dev_scores = buffers["cand_score"][:ncand].cpu().numpy().astype(np.uint32)
    q_ref = bo.residual_q_forward(frontier, w)[:, w["action_perm"]].reshape(-1)
    assert np.abs(dev_scores.astype(np.int64) - bo.q_to_score_key(q_ref, 0.0).astype(np.int64)).max() <= 16  # 0.06 in q
    want = bo.depth_step([frontier], pz.generators, pz.solved, None, 500, score_override=[dev_scores])
    assert np.array_equal(bo.sorted_rows(engine.frontier()), bo.sorted_rows(want.states))


def test_engine_with_action_value_scorer_matches_oracle_on_device_scores():
    """Engine step with the parent scorer: candidate p*G + m takes q[p, m]; selection is exact given those keys."""
    pz = puzzles.puzzle54()
    beam = 700
    ws = _q_weights(pz, 2)
    cfg = be.config_for_puzzle(pz, global_beam_width=beam, max_depth=6, beta=1.2, hash_load_factor=0.45,
                               probe_limit=256, band_rounds=8, inference_backend="mlp")
    ext = be.build_extension()
    be.init_distributed_if_needed(cfg)
    sizes = ext.derive_sizes(cfg)
    sc = scorers.MLPActionValueScorer(ws, 54, cfg["state_size_bytes"], 6, pz.fanout, max_parents=sizes["k_work"])
    _, cfg, buffers, engine = be.configure_engine(pz, cfg=cfg, scorer=sc)
    frontier = np.unique(children_of(pz, 400, seed=3), axis=0)
    for graph in (False, True):
        engine.load_frontier(frontier)
        engine.enable_cuda_graphs(graph)
        engine.step()
        st = engine.status()
        assert st["status_bits"] == 0 and sc.error_code() == 0
        ncand = frontier.shape[0] * pz.fanout
        dev_scores = buffers["cand_score"][:ncand].cpu().numpy().astype(np.uint32)
        q_ref = bo.mlp_action_values(frontier, ws, 6).reshape(-1)
        assert np.abs(dev_scores.astype(np.int64) - bo.q_to_score_key(q_ref, -150.0).astype(np.int64)).max() <= 2
        want = bo.depth_step([frontier], pz.generators, pz.solved, None, beam, score_override=[dev_scores])
        assert np.array_equal(bo.sorted_rows(engine.frontier()), bo.sorted_rows(want.states))
