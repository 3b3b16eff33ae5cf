"""Benchmark of the per-depth beam-search step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one depth of the search at a saturated frontier: expand every frontier state by every generator,
hash, score with the value MLP, dedup, select the global beam, write the next frontier.  Workload at N = 1: state
length 54, values 0..5, 12 generators (6 products of five 4-cycles and their inverses), global beam 65 536,
scorer 324 -> 1024 -> 1024 -> 1 in bf16 (fp32 accumulation), HASH_LOAD_FACTOR 0.45, PROBE_LIMIT 256.  With N > 1
ranks the beam is 65 536 x N (weak scaling; N = 4 is the 262 144 beam of the sharded configuration), the frontier
is sharded by hash owner and every depth has one NCCL candidate exchange.  Inputs are synthetic and seeded.

Prints ONE JSON line.  ``value`` = candidates expanded+scored per second over the whole job with the frontier
resident in HBM (CUDA events around each step, max over ranks, L2 flushed between steps).  ``e2e`` = the same
metric through the host-facing calls load_frontier -> step -> frontier with pinned host buffers inside the timed
region.  ``--impl reference`` times the PyTorch-CPU restatement of the step on the host cores instead.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "expanded+scored states/sec"
UNIT = "states/s"
BEAM_PER_GPU = 65536
SCORE_OFFSET = -150.0
PREP_DEPTHS = 8  # untimed depths that grow the frontier from one state to the full beam
CPU_SAMPLE_PARENTS = 4096
GEMM2_DRAM_BYTES_PER_ROW = 2107.0


def workload_name(n_gpus: int) -> str:
    return (f"rand54 n=54 V=6 G=12, global beam {BEAM_PER_GPU * n_gpus}, MLP 324-1024-1024-1 bf16, "
            f"one depth step at a saturated frontier")


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_indices):
        """One nvidia-smi process for all listed GPUs (an empty list = no sampling: with several ranks only rank 0
        samples, for every GPU of the job - eight pollers at once were seen to stall the GPUs for milliseconds)."""
        self.proc = None
        self.gpu_indices = list(gpu_indices)

    def start(self):
        if not self.gpu_indices:
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms",
                 "100" if len(self.gpu_indices) == 1 else "200",
                 "-i", ",".join(str(i) for i in self.gpu_indices)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons, per_gpu = [], [], set(), {}
        for line in out.strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                per_gpu.setdefault(parts[0], []).append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons),
                "per_gpu_sm_mhz": {k: statistics.median(v) for k, v in sorted(per_gpu.items())}}


def cpu_baseline_step_rate(threads: int, steps: int = 3, parents: int = CPU_SAMPLE_PARENTS):
    """Candidates per second of the PyTorch-CPU step on a bounded sample (a frontier of `parents` states)."""
    from multigpubeamsearch_b200 import puzzles
    from oracle import torch_cpu_step as tcs

    torch.set_num_threads(threads)
    pz = puzzles.puzzle54()
    gens = torch.from_numpy(pz.generators.astype(np.int64))
    solved = torch.from_numpy(pz.solved)
    model = tcs.TorchMLP(puzzles.mlp_weights(pz.state_len * pz.num_values, 1024))
    rng = np.random.default_rng(123)
    rows = np.tile(pz.solved, (parents * 2, 1))
    g = pz.generators.astype(np.int64)
    for _ in range(30):
        rows = np.take_along_axis(rows, g[rng.integers(0, pz.fanout, size=rows.shape[0])], axis=1)
    frontier = torch.from_numpy(np.unique(rows, axis=0)[:parents])
    times = []
    cands = 0
    for i in range(steps + 1):
        t0 = time.perf_counter()
        nxt, _ = tcs.depth_step(frontier, gens, solved, parents, pz.num_values, [model], SCORE_OFFSET)
        dt = time.perf_counter() - t0
        if i > 0:  # first pass warms the allocator and thread pool
            times.append(dt)
            cands += frontier.shape[0] * pz.fanout
        frontier = nxt
    return cands / sum(times), sum(times) / len(times), f"{steps} depth steps on a {parents}-state frontier ({parents * pz.fanout} candidates each), float32 torch CPU"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    steps = max(1, min(args.steps, 5))
    value, sec_per_step, sample = cpu_baseline_step_rate(threads, steps=steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": 1, "ms_per_step": sec_per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.gpus), "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_ours(args):
    import torch.distributed as dist

    from multigpubeamsearch_b200 import beam_engine as be
    from multigpubeamsearch_b200 import puzzles, scorers

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    pz = puzzles.puzzle54()
    beam = BEAM_PER_GPU * world
    K, W = args.steps, max(args.warmup, 3)
    depths = PREP_DEPTHS + 2 * (W + K) + 8  # history rows: later depths than this are simply not recorded
    cfg = be.config_for_puzzle(pz, world_size=world, rank=rank, global_beam_width=beam, max_depth=depths, beta=1.2,
                               gamma=1.05, hash_load_factor=0.45, probe_limit=256, band_rounds=3, band_levels=3,
                               inference_backend="mlp", use_cuda_graphs=True)
    ext = be.build_extension()
    be.init_distributed_if_needed(cfg)
    sizes = ext.derive_sizes(cfg)
    sc = scorers.MLPValueScorer(puzzles.mlp_weights(pz.state_len * pz.num_values, 1024), pz.state_len,
                                cfg["state_size_bytes"], pz.num_values, max_rows=sizes["cand_cap"],
                                score_offset=SCORE_OFFSET, dtype=args.dtype)
    _, cfg, buffers, engine = be.configure_engine(pz, cfg=cfg, scorer=sc)
    dev = torch.device("cuda", local_rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    stream = engine._stream

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # grow the frontier to the full beam (untimed)
    start = pz.scramble(0, 40)
    be.run_one_search(engine, start, PREP_DEPTHS)
    st = engine.status()
    size_t = torch.tensor([st["current_size"]], device=dev, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(size_t)
    if int(size_t.item()) < beam:
        raise SystemExit(f"frontier not saturated after {PREP_DEPTHS} depths: {int(size_t.item())} < {beam}")

    def timed_steps(n):
        evs = []
        for _ in range(n):
            with torch.cuda.stream(stream):
                flush.zero_()  # evict L2 between steps (not timed)
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                engine.step()
                e1.record(stream)
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]

    sampler = ClockSampler([local_rank] if world == 1 else (list(range(world)) if rank == 0 else []))
    sampler.start()  # nvidia-smi needs a moment to start: it samples the warm-up, the timed steps and the passes after
    timed_steps(W)  # warm-up (captures the graphs)
    cand_before = engine.status()["total_candidates"]
    barrier()
    t_wall0 = time.perf_counter()
    ms = timed_steps(K)
    barrier()
    wall = time.perf_counter() - t_wall0
    st = engine.status()
    cands_local = st["total_candidates"] - cand_before
    status_bits = st["status_bits"]
    t = torch.tensor([sum(ms), float(cands_local), float(status_bits), float(sc.error_code())], device=dev,
                     dtype=torch.float64)
    tmax = t.clone()
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    total_ms = float(tmax[0].item())
    total_cands = float(t[1].item())
    rank_means = [sum(ms) / len(ms)]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, sum(ms) / len(ms))
        rank_means = [float(x) for x in gathered]
    value = total_cands / (total_ms * 1e-3)

    # ---- per-kernel timing for the roofline (eager steps with events between kernels), same frontier regime ----
    engine.enable_step_timers(True)
    sc.profile(True)
    prof = {"gemm2_ms": [], "gemm1_ms": [], "onehot_ms": [], "key_ms": [], "expand_ms": [], "scorer_ms": [],
            "exchange_ms": [], "bands_ms": [], "final_ms": [], "total_cuda_event_ms": []}
    prof_rows = []
    for _ in range(K):
        with torch.cuda.stream(stream):
            flush.zero_()
        rows_before = engine.status()["current_size"]
        engine.step()
        tm = engine.step_timing()
        tm.update(sc.profile_read())
        for k in prof:
            prof[k].append(tm[k])
        last_trace = tm.get("trace_ms")
        prof_rows.append(rows_before * pz.fanout)
    sc.profile(False)
    engine.enable_step_timers(False)
    peaks = measured_peaks()
    gemm2_ms = statistics.mean(prof["gemm2_ms"])
    rows_per_launch = statistics.mean(prof_rows)
    flops_per_row_l2 = 2 * (1024 * 1024 + 1024)  # layer 2 + scalar head
    achieved_tflops = rows_per_launch * flops_per_row_l2 / (gemm2_ms * 1e-3) / 1e12
    # DRAM bytes of the layer-2 GEMM per scored row, from one ncu capture of a 151 552-row case
    # (dram__bytes_read.sum + dram__bytes_write.sum = 319.36 MB); traffic grows with the row count
    traffic = GEMM2_DRAM_BYTES_PER_ROW * rows_per_launch
    roofline = {"bound": "tensor", "kernel": "k_mlp_head_pair<0> (layer 2 GEMM + scalar head on CTA pairs)", "achieved": achieved_tflops,
                "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": achieved_tflops / peaks["bf16_tflops_sustained"], "peak_source": peaks["source"] + " (sustained bf16)",
                "traffic": traffic,
                "stage_ms": {k: statistics.mean(v) for k, v in prof.items()},
                "last_step_trace_ms": last_trace}

    # ---- end to end: host frontier in pinned memory -> device -> one step -> host frontier ----
    n = pz.state_len
    rows_dev = engine.frontier()  # numpy [K_local, n]
    pinned_in = torch.empty((rows_dev.shape[0], n), dtype=torch.uint8).pin_memory()
    pinned_in.numpy()[:] = rows_dev
    depth0 = engine.status()["depth"]
    pinned_out = torch.empty((sizes["k_work"], n), dtype=torch.uint8).pin_memory()
    e2e_steps = max(3, min(K, 10))
    # untimed: the stage timers above ran eager steps and dropped the captured graphs; capture them again first
    for i in range(2):
        engine.load_frontier(pinned_in.numpy(), depth=(depth0 + i) % 2)
        engine.step()
        engine.frontier_into(pinned_out.numpy())
    barrier()
    t0 = time.perf_counter()
    e2e_cands = 0
    d2h = 0
    for i in range(e2e_steps):
        engine.load_frontier(pinned_in.numpy(), depth=depth0 % 2)  # host rows -> device (syncs)
        engine.step()
        got = engine.frontier_into(pinned_out.numpy())              # device rows -> host (syncs)
        e2e_cands += pinned_in.shape[0] * pz.fanout
        d2h = got * n + 4 + 4208
    barrier()
    e2e_wall = time.perf_counter() - t0
    e2e_t = torch.tensor([e2e_wall], device=dev, dtype=torch.float64)
    e2e_c = torch.tensor([float(e2e_cands)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
        dist.all_reduce(e2e_c, op=dist.ReduceOp.SUM)
    e2e_value = float(e2e_c.item()) / float(e2e_t.item())
    clocks = sampler.stop()

    # ---- the same steps with the scorer in FP8 (E4M3 operands, per-channel scales): short extra pass ----
    fp8 = None
    if args.dtype == "bf16" and not args.no_fp8:
        engine.close()
        barrier()
        del engine, buffers, sc
        torch.cuda.empty_cache()
        sc8 = scorers.MLPValueScorer(puzzles.mlp_weights(pz.state_len * pz.num_values, 1024), pz.state_len,
                                     cfg["state_size_bytes"], pz.num_values, max_rows=sizes["cand_cap"],
                                     score_offset=SCORE_OFFSET, dtype="fp8")
        cfg8 = dict(cfg)
        _, cfg8, buffers, engine = be.configure_engine(pz, cfg=cfg8, scorer=sc8)
        stream = engine._stream
        be.run_one_search(engine, start, PREP_DEPTHS)
        timed_steps(W)
        c0 = engine.status()["total_candidates"]
        barrier()
        k8 = max(3, min(K, 20))
        ms8 = timed_steps(k8)
        barrier()
        st8 = engine.status()
        t8 = torch.tensor([sum(ms8), float(st8["total_candidates"] - c0), float(st8["status_bits"]),
                           float(sc8.error_code())], device=dev, dtype=torch.float64)
        t8max = t8.clone()
        if world > 1:
            dist.all_reduce(t8max, op=dist.ReduceOp.MAX)
            dist.all_reduce(t8, op=dist.ReduceOp.SUM)
        fp8 = {"value": float(t8[1].item()) / (float(t8max[0].item()) * 1e-3), "unit": UNIT,
               "ms_per_step": float(t8max[0].item()) / k8, "steps": k8, "status_bits": int(t8[2].item()),
               "scorer_err": int(t8[3].item()), "dtype": "fp8 e4m3 operands, fp32 accumulation"}

    if rank == 0:
        cpu_val, _, cpu_sample = (None, None, None)
        cpu_obj = None
        if world == 1:
            threads = os.cpu_count() or 1
            cpu_val, _, cpu_sample = cpu_baseline_step_rate(threads, steps=3)
            cpu_obj = {"value": cpu_val, "unit": UNIT, "cores": threads, "kind": "port", "sample": cpu_sample}
        # kernels of ours inside one timed step: depth_begin, expand, layer 1, layer 2 + head, key, per band round
        # (levels histograms + insert, + the band route when world > 1), final-cut levels, emit, finish
        key_bits = 20 + int(cfg.get("hash_bits", 24))
        final_levels = (key_bits + 10) // 11
        band_levels = min(int(cfg["band_levels"]), final_levels)
        launches_per_step = 1 + 1 + 3 + cfg["band_rounds"] * (band_levels + 1 + (1 if world > 1 else 0)) + final_levels + 2
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": total_ms / K, "p50_ms_per_step": statistics.median(ms),
            "p90_ms_per_step": sorted(ms)[min(len(ms) - 1, int(0.9 * len(ms)))], "max_ms_per_step": max(ms),
            "rank_ms_per_step": rank_means,
            "slow_steps": sum(1 for x in ms if x > 1.5 * statistics.median(ms)), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": workload_name(world), "global_beam": beam, "beam_per_gpu": BEAM_PER_GPU,
                       "candidates_per_step": total_cands / K, "l2": "256 MB buffer written between timed steps",
                       "parallelism": f"hash-owner dp{world}", "cuda_graph": True,
                       "unique_per_step": st["counters"][3], "band_rounds_used": st["counters"][5],
                       "table_inserts_per_step_rank0": st["counters"][1]},
            "roofline": roofline,
            "cpu_baseline": cpu_obj,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(pinned_in.numel()),
                    "d2h_bytes_per_step": int(d2h), "steps": e2e_steps},
            "fp8": fp8,
            "gpu_launches": launches_per_step * K,
            "clocks": clocks,
            "status_bits": int(t[2].item()), "scorer_err": int(t[3].item()),
            "wall_s_timed_region": wall,
        }
        print(json.dumps(line))
    engine.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"], help="scorer operand type of the headline run")
    ap.add_argument("--no-fp8", action="store_true", help="skip the short extra FP8 pass")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
