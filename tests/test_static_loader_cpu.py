"""Host-side loader of the reference's static action-value network: batch-norm folding and table re-layout
(load_static_weights, scripts/static_fullbeamnice_inference.py:74-143), checked against an unfolded evaluation."""

import numpy as np

from oracle import beam_oracle as bo
from multigpubeamsearch_b200 import scorers


def _bn(rng, n, prefix, sd):
    sd[f"{prefix}.weight"] = (rng.random(n) + 0.5).astype(np.float32)
    sd[f"{prefix}.bias"] = (rng.standard_normal(n) * 0.2).astype(np.float32)
    sd[f"{prefix}.running_mean"] = (rng.standard_normal(n) * 0.3).astype(np.float32)
    sd[f"{prefix}.running_var"] = (rng.random(n) + 0.2).astype(np.float32)


def _state_dict(seed, n, classes, h1, h2, outs, blocks):
    rng = np.random.default_rng(seed)
    sd = {"input_layer.weight": (rng.standard_normal((h1, n * classes)) * 0.2).astype(np.float32),
          "input_layer.bias": (rng.standard_normal(h1) * 0.1).astype(np.float32),
          "hidden_layer.weight": (rng.standard_normal((h2, h1)) * 0.2).astype(np.float32),
          "hidden_layer.bias": (rng.standard_normal(h2) * 0.1).astype(np.float32),
          "output_layer.weight": (rng.standard_normal((outs, h2)) * 0.2).astype(np.float32),
          "output_layer.bias": (rng.standard_normal(outs) * 0.1).astype(np.float32)}
    _bn(rng, h1, "bn1", sd)
    _bn(rng, h2, "bn2", sd)
    for b in range(blocks):
        for fc, bn in (("fc1", "bn1"), ("fc2", "bn2")):
            sd[f"residual_blocks.{b}.{fc}.weight"] = (rng.standard_normal((h2, h2)) * 0.2).astype(np.float32)
            sd[f"residual_blocks.{b}.{fc}.bias"] = (rng.standard_normal(h2) * 0.1).astype(np.float32)
            _bn(rng, h2, f"residual_blocks.{b}.{bn}", sd)
    return sd


def _unfolded(states, sd, classes, blocks, eps=1e-5):
    def bn(x, p):
        return (x - sd[f"{p}.running_mean"]) / np.sqrt(sd[f"{p}.running_var"] + eps) * sd[f"{p}.weight"] + sd[f"{p}.bias"]

    x = bo.one_hot(states, classes).astype(np.float64)
    x = np.maximum(bn(x @ sd["input_layer.weight"].T + sd["input_layer.bias"], "bn1"), 0)
    x = np.maximum(bn(x @ sd["hidden_layer.weight"].T + sd["hidden_layer.bias"], "bn2"), 0)
    for b in range(blocks):
        p = f"residual_blocks.{b}"
        r = x
        x = np.maximum(bn(x @ sd[f"{p}.fc1.weight"].T + sd[f"{p}.fc1.bias"], f"{p}.bn1"), 0)
        x = np.maximum(bn(x @ sd[f"{p}.fc2.weight"].T + sd[f"{p}.fc2.bias"], f"{p}.bn2") + r, 0)
    return x @ sd["output_layer.weight"].T + sd["output_layer.bias"]


def test_folded_static_weights_reproduce_the_network_with_batch_norm():
    n, classes, h1, h2, outs, blocks = 10, 7, 24, 16, 5, 2
    sd = _state_dict(31, n, classes, h1, h2, outs, blocks)
    states = np.random.default_rng(32).integers(0, classes, size=(40, n), dtype=np.uint8)
    want = _unfolded(states, sd, classes, blocks)
    # same layout, and the reference's padded layout (more positions, more rows per position)
    for size, pad in ((n, classes), (16, 8)):
        w = scorers.static_weights_from_state_dict(sd, blocks, n, classes, state_size=size, class_pad=pad)
        assert w["embed_w_t"].shape == (size * pad, h1) and w["state_size"] == size and w["num_classes"] == pad
        got = bo.residual_q_forward(states, w)
        assert np.allclose(got, want, rtol=1e-4, atol=1e-4)
    # input_layer.weight stored [in, out] is accepted as well (the reference transposes on shape, :95-97)
    sd_t = dict(sd)
    sd_t["input_layer.weight"] = np.ascontiguousarray(sd["input_layer.weight"].T)
    w = scorers.static_weights_from_state_dict(sd_t, blocks, n, classes)
    assert np.allclose(bo.residual_q_forward(states, w), want, rtol=1e-4, atol=1e-4)


def test_fold_bn_linear_equals_the_oracle():
    rng = np.random.default_rng(5)
    args = [rng.standard_normal((6, 4)).astype(np.float32), rng.standard_normal(6).astype(np.float32),
            (rng.random(6) + 0.5).astype(np.float32), rng.standard_normal(6).astype(np.float32),
            rng.standard_normal(6).astype(np.float32), (rng.random(6) + 0.1).astype(np.float32)]
    for a, b in zip(scorers.fold_bn_linear(*args), bo.fold_bn_linear(*args)):
        assert np.array_equal(a, b)


def test_action_scorer_modules_keep_the_reference_contract():
    """scorers.MLPActionScorer / QuantizedActionScorer / make_default_mlp_scorer (the names of the reference's
    scorers.py): same constructor defaults, uint8 [B, 120] in, [B, 24] out, int16 bit patterns from the quantiser;
    numerics against the float32 restatement that the golden vectors pin."""
    import torch
    m = scorers.make_default_mlp_scorer()
    assert isinstance(m, scorers.QuantizedActionScorer) and isinstance(m.base, scorers.MLPActionScorer)
    assert [l.in_features for l in m.base.linears] == [120, 1024] and m.base.out.out_features == 24
    base = scorers.MLPActionScorer(120, (32, 16), 24)
    states = np.random.default_rng(3).integers(0, 120, size=(9, 120), dtype=np.uint8)
    layers = [(l.weight.detach().numpy(), l.bias.detach().numpy()) for l in (*base.linears, base.out)]
    with torch.no_grad():
        y = base(torch.from_numpy(states)).numpy()
        for mode in ("sigmoid_u16", "float_u16"):
            q = scorers.QuantizedActionScorer(base, mode)(torch.from_numpy(states))
            assert q.dtype == torch.int16 and q.shape == (9, 24)
            bits = q.numpy().astype(np.int64) & 0xFFFF
            assert np.max(np.abs(bits - bo.quantized_action_scores(y, mode).astype(np.int64))) <= 1
    assert np.max(np.abs(y - bo.action_scorer_forward(states, layers))) <= 1e-5
    try:
        scorers.QuantizedActionScorer(base, "other")
        raise AssertionError("an unknown score_mode must be refused")
    except RuntimeError as e:
        assert "unsupported score_mode" in str(e)


def test_nvfp4_weight_rounding_equals_the_oracle_model():
    """scorers.nvfp4_round_weights (what the transformer's NVFP4-weight mode feeds its GEMMs) against the oracle's
    NVFP4 model of the same matrix, bit for bit."""
    rng = np.random.default_rng(12)
    for shape, scale in (((64, 256), 0.02), ((24, 1024), 1.0), ((8, 16), 5.0)):
        w = (rng.standard_normal(shape) * scale).astype(np.float32)
        w[0, :16] = 0.0  # an all-zero block keeps factor 0
        got = scorers.nvfp4_round_weights(w)
        want = bo.quantize_nvfp4(w, bo.nvfp4_tensor_scale(float(np.abs(w).max())))
        assert np.array_equal(got, want)
        assert np.abs(got - w).max() <= 0.26 * np.abs(w).max()  # E2M1 steps are at most a quarter of the block maximum
