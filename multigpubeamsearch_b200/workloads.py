"""Timed runs of the other benchmark configurations (the default one lives in bench.py).

    python -m multigpubeamsearch_b200.workloads --name c4|c5|c2q [--steps K] [--beam-per-gpu B] [--dtype bf16|fp8]
    python -m torch.distributed.run --nproc-per-node N -m multigpubeamsearch_b200.workloads --name c5

c4: state length 54, 12 generators, transformer ensemble (2 encoders x 4 layers, d 256, 8 heads, FFN 1024, bf16),
    scoring micro-batch 32 768, global beam 65 536 over all ranks.
c2q: the benchmark's puzzle and beam (65 536 per rank) with an action-value MLP 324 -> 1024 -> 1024 -> 12 evaluated once
    per parent row (the reference's own scorer contract) instead of a value MLP evaluated on every child.
c5: state length 96, 18 generators, ensemble of 3 MLPs 768 -> 1024 -> 1024 -> 1 (bf16 here; the block-scaled 4-bit
    format is not built), global beam 2^22 on 8 ranks = 524 288 per rank, BETA 1.2, load 0.45, probe limit 256,
    depth loop through CUDA graphs.
Prints one JSON line from rank 0: candidates per second over K saturated depth steps (CUDA events, max over ranks).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

from . import beam_engine as be
from . import puzzles, scorers


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--name", choices=["c4", "c5", "c2q"], required=True)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--beam-per-gpu", type=int, default=0)
    ap.add_argument("--prep", type=int, default=10)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"], help="GEMM operand type of the scorer")
    ap.add_argument("--hash-mode", default="fnv", choices=["fnv", "zobrist128"])
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if args.name == "c4":
        pz = puzzles.puzzle54()
        per_gpu = args.beam_per_gpu or max(65536 // world, 1)
        scramble_len = 40
    elif args.name == "c2q":
        pz = puzzles.puzzle54()
        per_gpu = args.beam_per_gpu or 65536
        scramble_len = 40
    else:
        pz = puzzles.puzzle96()
        per_gpu = args.beam_per_gpu or 524288
        scramble_len = 60
    beam = per_gpu * world
    depths = args.prep + args.warmup + args.steps + 4
    cfg = be.config_for_puzzle(pz, world_size=world, rank=rank, global_beam_width=beam, max_depth=depths, beta=1.2,
                               gamma=1.05, hash_load_factor=0.45, probe_limit=256, band_rounds=3, band_levels=3,
                               inference_backend="mlp", use_cuda_graphs=True, hash_mode=args.hash_mode)
    ext = be.build_extension()
    be.init_distributed_if_needed(cfg)
    sizes = ext.derive_sizes(cfg)
    if args.name == "c4":
        sc = scorers.TransformerValueScorer([puzzles.transformer_weights(54, 6, model_idx=i) for i in range(2)],
                                            pz.state_len, cfg["state_size_bytes"], pz.num_values,
                                            max_rows=sizes["cand_cap"], micro_batch=32768, dtype=args.dtype)
        scorer_name = f"transformer 2x(4 layers, d256, 8 heads, ffn 1024) {args.dtype}"
    elif args.name == "c2q":
        sc = scorers.MLPActionValueScorer(puzzles.q_mlp_weights(pz.state_len * pz.num_values, pz.fanout, 1024, 1024),
                                          pz.state_len, cfg["state_size_bytes"], pz.num_values, pz.fanout,
                                          max_parents=sizes["k_work"])
        scorer_name = "action-value MLP 324-1024-1024-12 bf16 on parent rows"
    else:
        sc = scorers.MLPValueScorer([puzzles.mlp_weights(pz.state_len * pz.num_values, 1024, model_idx=i) for i in range(3)],
                                    pz.state_len, cfg["state_size_bytes"], pz.num_values, max_rows=sizes["cand_cap"],
                                    dtype=args.dtype)
        scorer_name = f"3 x MLP 768-1024-1024-1 {args.dtype}"
    _, cfg, buffers, engine = be.configure_engine(pz, cfg=cfg, scorer=sc)
    dev = torch.device("cuda", local_rank)
    stream = engine._stream

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    be.run_one_search(engine, pz.scramble(0, scramble_len), args.prep)
    size_t = torch.tensor([engine.status()["current_size"]], device=dev, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(size_t)

    def timed(n):
        evs = []
        for _ in range(n):
            with torch.cuda.stream(stream):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                engine.step()
                e1.record(stream)
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]

    timed(args.warmup)
    c0 = engine.status()["total_candidates"]
    barrier()
    ms = timed(args.steps)
    barrier()
    st = engine.status()
    t = torch.tensor([sum(ms), float(st["total_candidates"] - c0), float(st["status_bits"]), float(sc.error_code())],
                     device=dev, dtype=torch.float64)
    tmax = t.clone()
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    if rank == 0:
        total_ms = float(tmax[0].item())
        cands = float(t[1].item())
        print(json.dumps({
            "workload": args.name, "puzzle": pz.name, "scorer": scorer_name, "n_gpus": world, "global_beam": beam,
            "frontier_after_prep": int(size_t.item()), "steps": args.steps,
            "value": cands / (total_ms * 1e-3), "unit": "states/s", "ms_per_step": total_ms / args.steps,
            "p50_ms_per_step": statistics.median(ms), "candidates_per_step": cands / args.steps,
            "scorer_tflops": sc.flops_per_state() * cands / (total_ms * 1e-3) / 1e12,
            "status_bits": int(t[2].item()), "scorer_err": int(t[3].item()),
            "unique_per_step": st["counters"][3], "band_rounds_used": st["counters"][5],
        }))
    engine.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
