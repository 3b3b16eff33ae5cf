"""Small, self-ending workload for profiler captures of the scorer kernels.

    python -m multigpubeamsearch_b200.profile_case [--rows R] [--repeat N]

Scores R random child states N times with the MLP 324 -> 1024 -> 1024 -> 1 (default), its e4m3 variant, or the
two-encoder transformer ensemble in bf16 or e4m3.  The default R = 151 552 is 8 row tiles per SM on 148 SMs; the
MLP's first-layer activations are then 310 MB, larger than L2.  A few hundred MB on the device.
"""

from __future__ import annotations

import argparse

import numpy as np
import torch

from . import puzzles, scorers


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=151552)
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--scorer", default="mlp", choices=["mlp", "mlp_fp8", "transformer", "transformer_fp8"])
    ap.add_argument("--micro-batch", type=int, default=32768)
    ap.add_argument("--head", default="pair", choices=["pair", "single"],
                    help="MLP layer 2 + head on CTA pairs (default) or single CTAs")
    args = ap.parse_args()
    pz = puzzles.puzzle54()
    rng = np.random.default_rng(0)
    g = pz.generators.astype(np.int64)
    rows = np.tile(pz.solved, (args.rows, 1))
    for _ in range(20):
        rows = np.take_along_axis(rows, g[rng.integers(0, pz.fanout, size=args.rows)], axis=1)
    padded = np.zeros((args.rows, 64), np.uint8)
    padded[:, :54] = rows
    children = torch.from_numpy(padded).cuda()
    if args.scorer.startswith("transformer"):
        sc = scorers.TransformerValueScorer([puzzles.transformer_weights(54, 6, model_idx=i) for i in range(2)], 54, 64, 6,
                                            max_rows=args.rows, micro_batch=args.micro_batch,
                                            dtype="fp8" if args.scorer.endswith("fp8") else "bf16")
    else:
        sc = scorers.MLPValueScorer(puzzles.mlp_weights(324, 1024), 54, 64, 6, max_rows=args.rows,
                                    dtype="fp8" if args.scorer == "mlp_fp8" else "bf16")
        sc.set_head_mode(args.head == "pair")
    times = []
    for _ in range(args.repeat):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        keys = sc.score(children)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = min(times)
    print("keys", int(keys.min()), int(keys.max()), "err", sc.error_code(), "ms", [round(t, 3) for t in times],
          "TFLOP/s", round(sc.flops_per_state() * args.rows / (ms * 1e-3) / 1e12, 1))


if __name__ == "__main__":
    main()
