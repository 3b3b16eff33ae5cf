"""Generate tests/golden/residual_q_reference.json from the reference's own Python functions.

Run in a container that has the reference checkout (it is imported, never copied):

    python tests/golden/make_residual_q_golden.py /path/to/reference

Calls the reference's ``static_forward_q``, ``static_forward_scores`` and ``_fold_bn_linear``
(scripts/static_fullbeamnice_inference.py) and its ``MLPActionScorer`` / ``QuantizedActionScorer`` (scorers.py) on
seeded random weights and states and records the outputs.  The
tests rebuild weights and states from the recorded seeds with ``residual_q_weights`` / ``residual_q_states`` below, so
only seeds, shapes and outputs are stored.
"""

import json
import sys
from pathlib import Path

import numpy as np


def residual_q_weights(seed: int, state_size: int, num_classes: int, hidden1: int, hidden2: int, outputs: int,
                       blocks: int = 2):
    """Seeded float32 weights with the key names and [in, out] layout of the reference's static dictionary."""
    rng = np.random.default_rng(seed)

    def mat(rows, cols, scale):
        return (rng.standard_normal((rows, cols)) * scale).astype(np.float32)

    w = {
        "embed_w_t": mat(state_size * num_classes, hidden1, 0.3 / np.sqrt(state_size)),
        "embed_bias": (rng.standard_normal(hidden1) * 0.1).astype(np.float32),
        "hidden_w_t": mat(hidden1, hidden2, 1.4 / np.sqrt(hidden1)),
        "hidden_bias": (rng.standard_normal(hidden2) * 0.1).astype(np.float32),
    }
    for b in range(blocks):
        for fc in ("fc1", "fc2"):
            w[f"res{b}_{fc}_w_t"] = mat(hidden2, hidden2, 1.0 / np.sqrt(hidden2))
            w[f"res{b}_{fc}_bias"] = (rng.standard_normal(hidden2) * 0.1).astype(np.float32)
    w["out_w_t"] = mat(hidden2, outputs, 2.0 / np.sqrt(hidden2))
    w["out_bias"] = (rng.standard_normal(outputs) * 0.5 + 4.0).astype(np.float32)
    w["action_perm"] = rng.permutation(outputs).astype(np.int64)
    w["state_size"], w["num_classes"] = int(state_size), int(num_classes)
    w["score_scale"], w["score_bias"] = 1024.0, 65535.0
    return w


def residual_q_states(seed: int, rows: int, state_len: int, num_values: int) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, num_values, size=(rows, state_len), dtype=np.uint8)


def action_scorer_weights(seed: int, input_dim: int, hidden: tuple, fanout: int):
    """Seeded float32 [out, in] matrices and biases of the reference's MLPActionScorer (Linear, GELU, ..., Linear)."""
    rng = np.random.default_rng(seed)
    sizes = [input_dim, *hidden, fanout]
    return [((rng.standard_normal((b, a)) * (1.5 / np.sqrt(a))).astype(np.float32),
             (rng.standard_normal(b) * 0.2).astype(np.float32)) for a, b in zip(sizes[:-1], sizes[1:])]


def bn_case(seed: int, outs: int, ins: int):
    rng = np.random.default_rng(seed)
    return {
        "weight": rng.standard_normal((outs, ins)).astype(np.float32),
        "bias": rng.standard_normal(outs).astype(np.float32),
        "bn_weight": (rng.random(outs) + 0.5).astype(np.float32),
        "bn_bias": rng.standard_normal(outs).astype(np.float32),
        "running_mean": rng.standard_normal(outs).astype(np.float32),
        "running_var": (rng.random(outs) + 0.1).astype(np.float32),
    }


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_residual_q_golden.py /path/to/reference")
    ref = Path(sys.argv[1])
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(ref))
    sys.path.insert(0, str(ref / "scripts"))
    import torch
    import static_fullbeamnice_inference as sfi

    out = {"forward": [], "fold_bn": []}
    # (seed, state_size, num_classes, hidden1, hidden2, outputs, rows, state_len of the rows fed in)
    for seed, size, classes, h1, h2, outs, rows, n in ((9501, 128, 128, 64, 32, 24, 12, 120),
                                                        (9502, 128, 128, 64, 32, 24, 12, 128),
                                                        (9503, 54, 6, 256, 256, 12, 16, 54)):
        w = residual_q_weights(seed, size, classes, h1, h2, outs)
        fields = {k: (torch.from_numpy(v) if isinstance(v, np.ndarray) else v) for k, v in w.items()}
        sw = sfi.StaticFullBeamNiceWeights(**fields)
        # the reference pads rows of its own STATE_LEN to its storage length; other widths must come in full
        if n == sfi.STATE_LEN:
            assert size == sfi.STATE_STORAGE_LEN
        else:
            assert n == size
        states = residual_q_states(seed + 50, rows, n, min(classes, 120))
        with torch.no_grad():
            q = sfi.static_forward_q(torch.from_numpy(states), sw)
            sc = sfi.static_forward_scores(torch.from_numpy(states), sw)
        out["forward"].append({"seed": seed, "state_size": size, "num_classes": classes, "hidden1": h1, "hidden2": h2,
                               "outputs": outs, "rows": rows, "state_len": n, "value_range": min(classes, 120),
                               "q": [[float(x) for x in r] for r in q.numpy()],
                               "scores_i16": sc.numpy().astype(int).tolist()})
    for seed, outs, ins in ((9601, 8, 5), (9602, 16, 16)):
        c = bn_case(seed, outs, ins)
        fw, fb = sfi._fold_bn_linear(*(torch.from_numpy(c[k]) for k in
                                       ("weight", "bias", "bn_weight", "bn_bias", "running_mean", "running_var")))
        out["fold_bn"].append({"seed": seed, "outs": outs, "ins": ins,
                               "weight": [[float(x) for x in r] for r in fw.numpy()],
                               "bias": [float(x) for x in fb.numpy()]})
    import scorers as ref_scorers  # the reference's scorers.py
    out["action_scorer"] = []
    for seed, hidden, rows in ((9701, (32, 16), 10), (9702, (48, 24), 6)):
        layers = action_scorer_weights(seed, 120, hidden, 24)
        base = ref_scorers.MLPActionScorer(120, hidden, 24)
        sd = {}
        for i, (wm, bv) in enumerate(layers):
            sd[f"net.{2 * i}.weight"], sd[f"net.{2 * i}.bias"] = torch.from_numpy(wm), torch.from_numpy(bv)
        base.load_state_dict(sd, strict=True)
        states = residual_q_states(seed + 50, rows, 120, 120)
        with torch.no_grad():
            y = base(torch.from_numpy(states))
            sig = ref_scorers.QuantizedActionScorer(base, "sigmoid_u16")(torch.from_numpy(states))
            flt = ref_scorers.QuantizedActionScorer(base, "float_u16")(torch.from_numpy(states))
        out["action_scorer"].append({"seed": seed, "hidden": list(hidden), "rows": rows,
                                     "y": [[float(x) for x in r] for r in y.numpy()],
                                     "sigmoid_u16": sig.numpy().astype(int).tolist(),
                                     "float_u16": flt.numpy().astype(int).tolist()})
    dst = Path(__file__).resolve().parent / "residual_q_reference.json"
    dst.write_text(json.dumps(out, separators=(",", ":")))
    print(f"wrote {dst} ({dst.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
