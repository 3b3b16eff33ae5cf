"""Benchmark of the per-depth beam-search step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--case c2|c4|c5|c2q|scorer]

One "step" is one depth of the search at a saturated frontier: expand every frontier state by every generator,
hash, score with the value MLP, dedup, select the global beam, write the next frontier.  Default workload (case
c2) at N = 1: state length 54, values 0..5, 12 generators (6 products of five 4-cycles and their inverses), global
beam 65 536, scorer 324 -> 1024 -> 1024 -> 1 in bf16 (fp32 accumulation), HASH_LOAD_FACTOR 0.45, PROBE_LIMIT 256.
With N > 1 ranks the headline beam is 65 536 x N (weak scaling; N = 4 is the 262 144 beam of the sharded reference
configuration), the frontier is sharded by hash owner and every depth has one candidate exchange; the line then also
carries ``c3``: the same step at the fixed global beam 262 144 on these N ranks.  Inputs are synthetic and seeded.

Prints ONE JSON line.  ``value`` = candidates expanded+scored per second over the whole job with the frontier
resident in HBM (CUDA events around each step, max over ranks, L2 flushed between steps), after an untimed pre-roll
of at least a second of steps so that every N is measured at its sustained clocks.  ``e2e`` = the same metric
through the host-facing calls load_frontier -> step -> frontier with pinned host buffers inside the timed region.
``parity_check`` = an untimed Hamming-scored depth of the same N-rank engine compared with the CPU oracle.
``fp8`` / ``nvfp4`` = short extra passes of the same steps with the scorer in E4M3 and in NVFP4.
``--impl reference`` times the PyTorch-CPU restatement of the step on the host cores on the same frontier size.

Other cases (one JSON line each, no contract keys): c4 transformer ensemble, c5 large frontier with three MLPs,
c2q action-value MLP on parent rows, scorer = a small self-ending scorer-only workload for profiler captures.
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
C3_BEAM = 262144
SCORE_OFFSET = -150.0
PREP_DEPTHS = 8        # untimed depths that grow the frontier from one state to the full beam
PREROLL_SECONDS = 1.0  # untimed steps before the timed region (sustained clocks at every N)
GEMM2_DRAM_BYTES_PER_ROW = 2107.0  # layer-2 GEMM, dram read+write per scored row from an ncu capture of 151 552 rows
RECORD_BYTES = 24      # hash64 + fingerprint64 + score32 + back-pointer32


def workload_name(n_gpus: int, beam: int) -> str:
    return (f"rand54 n=54 V=6 G=12, global beam {beam} on {n_gpus} GPU(s), MLP 324-1024-1024-1, "
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
        sm, mx, power, reasons, per_gpu = [], [], [], set(), {}
        for line in out.strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
                per_gpu.setdefault(parts[0], []).append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons),
                "per_gpu_sm_mhz": {k: statistics.median(v) for k, v in sorted(per_gpu.items())}}


# ----------------------------------------------------------------------------------------------------------------
# CPU arm: the PyTorch-CPU restatement of the same step (oracle/torch_cpu_step.py), timed on the host cores
# ----------------------------------------------------------------------------------------------------------------

def cpu_saturated_frontier(pz, parents: int):
    rng = np.random.default_rng(123)
    rows = np.tile(pz.solved, (parents * 2, 1))
    g = pz.generators.astype(np.int64)
    for _ in range(30):
        rows = np.take_along_axis(rows, g[rng.integers(0, pz.fanout, size=rows.shape[0])], axis=1)
    return np.unique(rows, axis=0)[:parents]


def cpu_baseline_step_rate(threads: int, steps: int, parents: int = BEAM_PER_GPU):
    """Candidates per second of the PyTorch-CPU step on a frontier of `parents` states (the GPU arm's per-GPU
    frontier), one untimed pass first."""
    from multigpubeamsearch_b200 import puzzles
    from oracle import torch_cpu_step as tcs

    torch.set_num_threads(threads)
    pz = puzzles.puzzle54()
    gens = torch.from_numpy(pz.generators.astype(np.int64))
    solved = torch.from_numpy(pz.solved)
    model = tcs.TorchMLP(puzzles.mlp_weights(pz.state_len * pz.num_values, 1024))
    frontier = torch.from_numpy(cpu_saturated_frontier(pz, parents))
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
    sample = (f"{steps} depth steps on a {parents}-state frontier ({parents * pz.fanout} candidates each, the GPU arm's "
              f"per-GPU step), float32 torch CPU, {threads} threads")
    return cands / sum(times), sum(times) / len(times), sample


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    steps = max(1, min(args.steps, 4))
    value, sec_per_step, sample = cpu_baseline_step_rate(threads, steps=steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": 1, "ms_per_step": sec_per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.gpus, BEAM_PER_GPU * args.gpus), "sample": sample,
                   "note": "the reference has no CPU path of its own (every entry point needs CUDA tensors): this is "
                           "the PyTorch-CPU restatement of the step, one host, all cores, one GPU's share of the "
                           "frontier per step; it does not scale with --gpus"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------------------------

class Job:
    """One engine with its scorer on this rank, plus the helpers every pass of the benchmark uses."""

    def __init__(self, pz, world, rank, local_rank, beam, depths, scorer_dtype="bf16", backend="mlp", **cfg_extra):
        from multigpubeamsearch_b200 import beam_engine as be
        from multigpubeamsearch_b200 import puzzles, scorers
        self.be, self.pz, self.world, self.rank = be, pz, world, rank
        self.dev = torch.device("cuda", local_rank)
        cfg = be.config_for_puzzle(pz, world_size=world, rank=rank, global_beam_width=beam, max_depth=depths,
                                   history_rows=min(depths, 64), beta=1.2, gamma=1.05, hash_load_factor=0.45,
                                   probe_limit=256, band_rounds=3, band_levels=3, inference_backend=backend,
                                   use_cuda_graphs=True, **cfg_extra)
        ext = be.build_extension()
        be.init_distributed_if_needed(cfg)
        self.sizes = ext.derive_sizes(cfg)
        self.scorer = None
        if backend == "mlp":
            self.scorer = scorers.MLPValueScorer(puzzles.mlp_weights(pz.state_len * pz.num_values, 1024), pz.state_len,
                                                 cfg["state_size_bytes"], pz.num_values, max_rows=self.sizes["cand_cap"],
                                                 score_offset=SCORE_OFFSET, dtype=scorer_dtype)
        _, self.cfg, self.buffers, self.engine = be.configure_engine(pz, cfg=cfg, scorer=self.scorer)
        self.stream = self.engine._stream
        self.beam = beam

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def allreduce(self, values, op="sum"):
        t = torch.tensor(values, device=self.dev, dtype=torch.float64)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
        return [float(x) for x in t.tolist()]

    def saturate(self, start):
        self.be.run_one_search(self.engine, start, PREP_DEPTHS)
        size = self.allreduce([self.engine.status()["current_size"]])[0]
        if int(size) < self.beam:
            raise SystemExit(f"frontier not saturated after {PREP_DEPTHS} depths: {int(size)} < {self.beam}")

    def timed_steps(self, n, flush):
        evs = []
        for _ in range(n):
            with torch.cuda.stream(self.stream):
                if flush is not None:
                    flush.zero_()  # evict L2 between steps (not timed)
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record(self.stream)
                self.engine.step()
                e1.record(self.stream)
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]

    def preroll(self, seconds):
        """Untimed steps for at least `seconds` of device time on every rank (the same count on all ranks)."""
        done, spent = 0, 0.0
        while spent < seconds * 1e3 and done < 4000:
            ms = self.timed_steps(50, None)
            spent += self.allreduce([sum(ms)], "max")[0]
            done += 50
        return done, spent / 1e3

    def measure(self, steps, flush):
        """(total ms = max over ranks of the per-rank sums, candidates over all ranks, per-step ms of this rank)."""
        c0 = self.engine.status()["total_candidates"]
        self.barrier()
        t0 = time.perf_counter()
        ms = self.timed_steps(steps, flush)
        self.barrier()
        wall = time.perf_counter() - t0
        st = self.engine.status()
        err = self.scorer.error_code() if self.scorer is not None else 0
        total_ms = self.allreduce([sum(ms)], "max")[0]
        cands, bits, errs = self.allreduce([st["total_candidates"] - c0, st["status_bits"], err])
        return {"total_ms": total_ms, "cands": cands, "ms": ms, "status_bits": int(bits), "scorer_err": int(errs),
                "wall": wall, "status": st}

    def close(self):
        self.engine.close()
        self.barrier()


def parity_check(pz, world, rank, local_rank):
    """Untimed: one Hamming-scored depth of the N-rank engine at the benchmark's knobs against the CPU oracle
    (oracle/beam_oracle.py, used as the checker only).  Global beam = min(65 536 x N, 262 144)."""
    import torch.distributed as dist
    from oracle import beam_oracle as bo
    beam = min(BEAM_PER_GPU * world, C3_BEAM)
    job = Job(pz, world, rank, local_rank, beam, 16, backend="central_hamming")
    try:
        job.saturate(pz.scramble(0, 40))
        eng = job.engine
        mine = eng.frontier()
        fronts = [mine]
        if world > 1:
            fronts = [None] * world
            dist.all_gather_object(fronts, mine)
        eng.step()
        st = eng.status()
        got = (eng.frontier(), eng.frontier_payloads(), eng.frontier_scores())
        parts = [got]
        if world > 1:
            parts = [None] * world
            dist.all_gather_object(parts, got)
        bits = int(job.allreduce([st["status_bits"]])[0])
        out = None
        if rank == 0:
            want = bo.depth_step(fronts, pz.generators, pz.solved, bo.hamming_scorer(pz.solved), beam)
            rows = np.concatenate([p[0] for p in parts])
            pay = np.concatenate([p[1] for p in parts])
            sco = np.concatenate([p[2] for p in parts])
            same_set = rows.shape[0] == want.states.shape[0] and \
                np.array_equal(bo.sorted_rows(rows), bo.sorted_rows(want.states))
            same_meta = same_set and {bytes(r): (int(p), int(k)) for r, p, k in zip(rows, pay, sco)} == \
                {bytes(r): (int(p), int(k)) for r, p, k in zip(want.states, want.payload, want.score)}
            owners_ok = all((bo.owner_rank(bo.hash64(p[0]), world) == r).all() for r, p in enumerate(parts) if p[0].shape[0])
            out = {"ranks": world, "ok": bool(same_set and same_meta and owners_ok and bits == 0),
                   "survivors": int(rows.shape[0]), "global_beam": beam, "candidates": int(want.candidates),
                   "unique": int(want.unique), "status_bits": bits, "scorer": "hamming",
                   "checked": "survivor set, back-pointers, scores, owner placement vs oracle.depth_step"}
        return out
    finally:
        job.close()


def run_ours(args):
    import torch.distributed as dist

    from multigpubeamsearch_b200 import puzzles, scorers

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    pz = puzzles.puzzle54()
    beam = BEAM_PER_GPU * world
    K, W = args.steps, max(args.warmup, 3)
    start = pz.scramble(0, 40)
    dev = torch.device("cuda", local_rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    peaks = measured_peaks()
    n = pz.state_len

    job = Job(pz, world, rank, local_rank, beam, 64, scorer_dtype=args.dtype)
    engine, sc, sizes, cfg = job.engine, job.scorer, job.sizes, job.cfg
    job.saturate(start)
    sampler = ClockSampler([local_rank] if world == 1 else (list(range(world)) if rank == 0 else []))
    sampler.start()  # samples the pre-roll, the warm-up, the timed steps and the passes after
    pre_steps, pre_s = job.preroll(args.preroll_s) if args.preroll_s > 0 else (0, 0.0)
    job.timed_steps(W, flush)  # warm-up with the flush in place
    res = job.measure(K, flush)
    clocks_main = sampler.stop()
    ms = res["ms"]
    total_ms, total_cands, st = res["total_ms"], res["cands"], res["status"]
    rank_means = [sum(ms) / len(ms)]
    rank_rows = [int(st["current_size"])]  # frontier rows each rank holds (hash-owner placement: how even it is)
    if world > 1:
        rows_all = [None] * world
        dist.all_gather_object(rows_all, rank_rows[0])
        rank_rows = [int(x) for x in rows_all]
        gathered = [None] * world
        dist.all_gather_object(gathered, sum(ms) / len(ms))
        rank_means = [float(x) for x in gathered]
    value = total_cands / (total_ms * 1e-3)

    # ---- per-kernel timing for the rooflines (eager steps with events between kernels), same frontier regime ----
    engine.enable_step_timers(True)
    sc.profile(True)
    keys = ("gemm2_ms", "gemm1_ms", "onehot_ms", "key_ms", "expand_ms", "scorer_ms", "exchange_ms", "bands_ms",
            "final_ms", "total_cuda_event_ms")
    prof = {k: [] for k in keys}
    prof_rows, prof_parents, prof_unique, prof_kept, last_trace = [], [], [], [], None
    for _ in range(min(K, 30)):
        with torch.cuda.stream(job.stream):
            flush.zero_()
        rows_before = engine.status()["current_size"]
        engine.step()
        tm = engine.step_timing()
        tm.update(sc.profile_read())
        for k in keys:
            prof[k].append(tm[k])
        last_trace = tm.get("trace_ms")
        s2 = engine.status()
        prof_parents.append(rows_before)
        prof_rows.append(rows_before * pz.fanout)
        prof_unique.append(s2["counters"][0])
        prof_kept.append(s2["current_size"])
    sc.profile(False)
    engine.enable_step_timers(False)
    stage = {k: statistics.mean(v) for k, v in prof.items()}
    stage["select_ms"] = stage["bands_ms"] + stage["final_ms"]
    rows_per_launch = statistics.mean(prof_rows)
    # dominant kernel: layer 2 GEMM + scalar head
    gemm2_ms = stage["gemm2_ms"]
    flops_per_row_l2 = 2 * (1024 * 1024 + 1024)
    achieved_tflops = rows_per_launch * flops_per_row_l2 / (gemm2_ms * 1e-3) / 1e12
    # which measured peak the fraction is taken against: the burst figure when the sampled clocks sat at the maximum
    # with no power cap, the sustained figure otherwise (the timed region follows >= 1 s of steps)
    sm, smx = clocks_main.get("sm_mhz"), clocks_main.get("sm_max_mhz")
    at_max = bool(sm and smx and sm >= 0.97 * smx and "sw_power_cap" not in clocks_main.get("reasons", []))
    peak_used = peaks["bf16_tflops"] if at_max else peaks["bf16_tflops_sustained"]
    # HBM stages: algorithmic bytes per depth on this rank (record m = 24 B, row n = 54 B) over CUDA-event time
    P = statistics.mean(prof_parents)
    Cn = rows_per_launch
    U = statistics.mean(prof_unique)
    Kk = statistics.mean(prof_kept)
    H = sizes["hash_capacity"]
    m = RECORD_BYTES
    bytes_expand = P * n + Cn * m + Cn * n + H * 16          # parents read, records + child rows written, table reset
    bytes_select = Cn * m + Cn * 32 + U * 4 + U * m + Kk * m + Kk * (m + n) + Kk * n  # dedup + select + materialise
    hbm = peaks["hbm_gbs"]

    def hbm_stage(nbytes, ms_):
        gbs = nbytes / (ms_ * 1e-3) / 1e9 if ms_ > 0 else 0.0
        return {"algorithmic_bytes": nbytes, "ms": ms_, "gbs": gbs, "frac": gbs / hbm}

    roofline = {
        "bound": "tensor", "kernel": "k_mlp_head_pair<0> (layer 2 GEMM + scalar head on CTA pairs)",
        "achieved": achieved_tflops, "peak": peak_used, "unit": "TFLOP/s", "frac": achieved_tflops / peak_used,
        "peak_source": f"{peaks['source']} ({'burst' if at_max else 'sustained'} bf16: clocks "
                       f"{'at max, no power cap' if at_max else 'below max or power-capped'} during the timed region)",
        "peak_burst": peaks["bf16_tflops"], "peak_sustained": peaks["bf16_tflops_sustained"],
        "frac_of_burst": achieved_tflops / peaks["bf16_tflops"],
        "frac_of_sustained": achieved_tflops / peaks["bf16_tflops_sustained"],
        "traffic": GEMM2_DRAM_BYTES_PER_ROW * rows_per_launch,
        "layer1": {"kernel": "k_mlp_l1 (one-hot operand built in shared memory, 324 -> 1024)", "ms": stage["gemm1_ms"],
                   "achieved": rows_per_launch * 2 * 324 * 1024 / (stage["gemm1_ms"] * 1e-3) / 1e12, "unit": "TFLOP/s"},
        "stages": {
            "hbm_peak_gbs": hbm, "peak_source": peaks["source"],
            "expand": hbm_stage(bytes_expand, stage["expand_ms"]),
            "select": hbm_stage(bytes_select, stage["select_ms"]),
            "non_scorer_total": hbm_stage(bytes_expand + bytes_select, stage["expand_ms"] + stage["select_ms"] + stage["exchange_ms"]),
            "note": "expand = depth open + table/histogram clears + expansion kernel (bound by the two serial 64-bit "
                    "hash chains per candidate, not by bytes); select = band rounds, final cut, emit, finish in one "
                    "persistent kernel; bytes = per-depth algorithmic count E + D + S + M of the scope table",
        },
        "stage_ms": stage, "last_step_trace_ms": last_trace,
    }

    # ---- end to end: host frontier in pinned memory -> device -> one step -> host frontier ----
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
    job.barrier()
    t0 = time.perf_counter()
    e2e_cands, d2h = 0, 0
    for i in range(e2e_steps):
        engine.load_frontier(pinned_in.numpy(), depth=depth0 % 2)  # host rows -> device (syncs)
        engine.step()
        got = engine.frontier_into(pinned_out.numpy())              # device rows -> host (syncs)
        e2e_cands += pinned_in.shape[0] * pz.fanout
        d2h = got * n + 4 + 4312
    job.barrier()
    e2e_wall = time.perf_counter() - t0
    e2e_value = job.allreduce([e2e_cands])[0] / job.allreduce([e2e_wall], "max")[0]
    h2d = int(pinned_in.numel())
    job.close()
    del engine, sc, job
    torch.cuda.empty_cache()

    # ---- the same steps with the scorer in FP8 (E4M3 operands, per-channel scales) and NVFP4: short extra passes ----
    def quantised_pass(dtype, label, kernels):
        jq = Job(pz, world, rank, local_rank, beam, 64, scorer_dtype=dtype)
        jq.saturate(start)
        jq.timed_steps(W, flush)
        kq = max(3, min(K, 20))
        rq = jq.measure(kq, flush)
        jq.scorer.profile(True)
        jq.engine.enable_step_timers(True)
        g1, g2 = [], []
        for _ in range(5):
            jq.engine.step()
            jq.engine.step_timing()
            tq = jq.scorer.profile_read()
            g1.append(tq["gemm1_ms"])
            g2.append(tq["gemm2_ms"])
        jq.scorer.profile(False)
        jq.engine.enable_step_timers(False)
        out = {"value": rq["cands"] / (rq["total_ms"] * 1e-3), "unit": UNIT, "ms_per_step": rq["total_ms"] / kq,
               "steps": kq, "status_bits": rq["status_bits"], "scorer_err": rq["scorer_err"], "dtype": label,
               "kernel_ms": {kernels[0]: statistics.mean(g1), kernels[1]: statistics.mean(g2)}}
        jq.close()
        del jq
        torch.cuda.empty_cache()
        return out

    fp8 = nvfp4 = None
    if args.dtype == "bf16" and not args.no_fp8:
        fp8 = quantised_pass("fp8", "fp8 e4m3 operands, fp32 accumulation", ("k_mlp_l1<1,8,0>", "k_mlp_head_pair<1>"))
        nvfp4 = quantised_pass("nvfp4", "layer 1 e4m3 operands with NVFP4 output; layer 2 NVFP4 (E2M1, E4M3 block-16 factors)",
                               ("k_mlp_l1<1,8,0,1>", "k_mlp_head_nvfp4_wide"))

    # ---- N > 1: the sharded reference configuration itself (global beam 262 144 on these N ranks) ----
    c3 = None
    if world > 1 and not args.no_c3:
        if beam == C3_BEAM:
            c3 = {"value": value, "unit": UNIT, "ms_per_step": total_ms / K, "global_beam": C3_BEAM,
                  "note": "identical to the headline run at this N"}
        else:
            j3 = Job(pz, world, rank, local_rank, C3_BEAM, 64, scorer_dtype=args.dtype)
            j3.saturate(start)
            j3.preroll(0.5)
            j3.timed_steps(W, flush)
            k3 = max(3, min(K, 30))
            r3 = j3.measure(k3, flush)
            c3 = {"value": r3["cands"] / (r3["total_ms"] * 1e-3), "unit": UNIT, "ms_per_step": r3["total_ms"] / k3,
                  "steps": k3, "global_beam": C3_BEAM, "beam_per_gpu": C3_BEAM // world,
                  "status_bits": r3["status_bits"], "scorer_err": r3["scorer_err"]}
            j3.close()
            del j3
            torch.cuda.empty_cache()

    # ---- untimed parity check of the N-rank engine against the oracle ----
    parity = None if args.no_parity else parity_check(pz, world, rank, local_rank)

    if rank == 0:
        cpu_obj = None
        if world == 1 and not args.no_cpu:
            threads = os.cpu_count() or 1
            cpu_val, _, cpu_sample = cpu_baseline_step_rate(threads, steps=2)
            cpu_obj = {"value": cpu_val, "unit": UNIT, "cores": threads, "kind": "port", "sample": cpu_sample}
        # kernels of ours inside one timed step: depth open, expansion, layer 1, layer 2 + head, score key, selection
        launches_per_step = 6
        sm_mhz = clocks_main.get("sm_mhz")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": total_ms / K, "p50_ms_per_step": statistics.median(ms),
            "p90_ms_per_step": sorted(ms)[min(len(ms) - 1, int(0.9 * len(ms)))], "max_ms_per_step": max(ms),
            "rank_ms_per_step": rank_means, "frontier_rows_per_rank": rank_rows,
            "ms_x_sm_mhz": (total_ms / K) * sm_mhz if sm_mhz else None,
            "slow_steps": sum(1 for x in ms if x > 1.5 * statistics.median(ms)), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": workload_name(world, beam), "global_beam": beam, "beam_per_gpu": BEAM_PER_GPU,
                       "candidates_per_step": total_cands / K, "l2": "256 MB buffer written between timed steps",
                       "preroll": f"{pre_steps} untimed steps ({pre_s:.2f} s) before warm-up and the timed region",
                       "parallelism": f"hash-owner dp{world}", "cuda_graph": True,
                       "select_pipeline": cfg.get("select_pipeline", "persistent"),
                       "exchange": cfg.get("exchange", "peer") if world > 1 else None,
                       "unique_per_step": st["counters"][3], "band_rounds_used": st["counters"][5],
                       "table_inserts_per_step_rank0": st["counters"][1]},
            "roofline": roofline,
            "cpu_baseline": cpu_obj,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(d2h),
                    "steps": e2e_steps},
            "parity_check": parity,
            "fp8": fp8,
            "nvfp4": nvfp4,
            "c3": c3,
            "gpu_launches": launches_per_step * K,
            "clocks": clocks_main,
            "status_bits": res["status_bits"], "scorer_err": res["scorer_err"],
            "wall_s_timed_region": res["wall"],
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------------------------
# Other configurations and the profiler workload
# ----------------------------------------------------------------------------------------------------------------

def run_case(args):
    """c4 / c5 / c2q: K saturated depth steps of another configuration; one JSON line from rank 0."""
    import torch.distributed as dist

    from multigpubeamsearch_b200 import beam_engine as be
    from multigpubeamsearch_b200 import puzzles, scorers

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if args.case == "c5":
        pz, per_gpu, scramble_len = puzzles.puzzle96(), args.beam_per_gpu or 524288, 60
    else:
        pz, scramble_len = puzzles.puzzle54(), 40
        per_gpu = args.beam_per_gpu or (max(65536 // world, 1) if args.case == "c4" else 65536)
    beam = per_gpu * world
    prep = 10
    depths = prep + max(args.warmup, 3) + args.steps + 8
    cfg = be.config_for_puzzle(pz, world_size=world, rank=rank, global_beam_width=beam, max_depth=depths,
                               history_rows=min(depths, 64), beta=1.2, gamma=1.05, hash_load_factor=0.45,
                               probe_limit=256, band_rounds=3, band_levels=3, inference_backend="mlp",
                               use_cuda_graphs=True, hash_mode=args.hash_mode)
    ext = be.build_extension()
    be.init_distributed_if_needed(cfg)
    sizes = ext.derive_sizes(cfg)
    k1 = pz.state_len * pz.num_values
    if args.case == "c4":
        sc = scorers.TransformerValueScorer([puzzles.transformer_weights(54, 6, model_idx=i) for i in range(2)],
                                            pz.state_len, cfg["state_size_bytes"], pz.num_values,
                                            max_rows=sizes["cand_cap"], micro_batch=32768,
                                            dtype="nvfp4_weights" if args.dtype == "nvfp4" else args.dtype)
        scorer_name = f"transformer 2x(4 layers, d256, 8 heads, ffn 1024) {args.dtype}" + (
            " weights on bf16 GEMMs" if args.dtype == "nvfp4" else "")
    elif args.case == "c2q":
        sc = scorers.MLPActionValueScorer(puzzles.q_mlp_weights(k1, pz.fanout, 1024, 1024), pz.state_len,
                                          cfg["state_size_bytes"], pz.num_values, pz.fanout, max_parents=sizes["k_work"])
        scorer_name = "action-value MLP 324-1024-1024-12 bf16 on parent rows"
    else:
        sc = scorers.MLPValueScorer([puzzles.mlp_weights(k1, 1024, model_idx=i) for i in range(3)], pz.state_len,
                                    cfg["state_size_bytes"], pz.num_values, max_rows=sizes["cand_cap"], dtype=args.dtype)
        scorer_name = f"3 x MLP 768-1024-1024-1 {args.dtype}"
    _, cfg, buffers, engine = be.configure_engine(pz, cfg=cfg, scorer=sc)
    dev = torch.device("cuda", local_rank)
    stream = engine._stream

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler([local_rank] if world == 1 else (list(range(world)) if rank == 0 else []))
    sampler.start()
    be.run_one_search(engine, pz.scramble(0, scramble_len), prep)
    size_t = torch.tensor([engine.status()["current_size"]], device=dev, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(size_t)

    def timed(count):
        evs = []
        for _ in range(count):
            with torch.cuda.stream(stream):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                engine.step()
                e1.record(stream)
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]

    timed(max(args.warmup, 3))
    c0 = engine.status()["total_candidates"]
    barrier()
    ms = timed(args.steps)
    barrier()
    clocks = sampler.stop()
    st = engine.status()
    # per-stage times of the same steps, eager with CUDA events between the launches (every rank steps; rank 0 reports)
    engine.enable_step_timers(True)
    acc, n_prof = {}, 3
    for _ in range(n_prof):
        engine.step()
        for k, v in engine.step_timing().items():
            if k.endswith("_ms") and isinstance(v, float):
                acc[k] = acc.get(k, 0.0) + v / n_prof
    engine.enable_step_timers(False)
    acc["select_ms"] = acc.get("bands_ms", 0.0) + acc.get("final_ms", 0.0)
    t = torch.tensor([sum(ms), float(st["total_candidates"] - c0), float(st["status_bits"]), float(sc.error_code())],
                     device=dev, dtype=torch.float64)
    tmax = t.clone()
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    if rank == 0:
        total_ms, cands = float(tmax[0].item()), float(t[1].item())
        print(json.dumps({
            "case": args.case, "puzzle": pz.name, "scorer": scorer_name, "n_gpus": world, "global_beam": beam,
            "frontier_after_prep": int(size_t.item()), "steps": args.steps, "metric": METRIC,
            "value": cands / (total_ms * 1e-3), "unit": UNIT, "ms_per_step": total_ms / args.steps,
            "p50_ms_per_step": statistics.median(ms), "candidates_per_step": cands / args.steps,
            "scorer_tflops": sc.flops_per_state() * cands / (total_ms * 1e-3) / 1e12,
            "status_bits": int(t[2].item()), "scorer_err": int(t[3].item()),
            "unique_per_step": st["counters"][3], "band_rounds_used": st["counters"][5], "clocks": clocks,
            "stage_ms": {k: round(v, 4) for k, v in acc.items()},
            "hash_capacity_slots": sizes["hash_capacity"], "table_mb": round(sizes["hash_capacity"] * 32 / 1e6, 1),
        }))
    engine.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_scorer_case(args):
    """Small, self-ending scorer-only workload for profiler captures: scores --rows random child states --repeat
    times with the MLP 324 -> 1024 -> 1024 -> 1 (bf16 / fp8 / nvfp4) or the two-encoder transformer ensemble.  The
    default 151 552 rows are 8 row tiles per SM on 148 SMs; the MLP's first-layer activations are then 310 MB, larger
    than L2; a few hundred MB on the device."""
    from multigpubeamsearch_b200 import puzzles, scorers

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
        dtype = {"mlp": "bf16", "mlp_fp8": "fp8", "mlp_nvfp4": "nvfp4"}[args.scorer]
        sc = scorers.MLPValueScorer(puzzles.mlp_weights(324, 1024), 54, 64, 6, max_rows=args.rows, dtype=dtype)
        if dtype != "nvfp4":
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
    print(json.dumps({"case": "scorer", "scorer": args.scorer, "rows": args.rows, "keys_min": int(keys.min()),
                      "keys_max": int(keys.max()), "err": sc.error_code(), "ms": [round(t, 3) for t in times],
                      "tflops": round(sc.flops_per_state() * args.rows / (ms * 1e-3) / 1e12, 1)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default="c2", choices=["c2", "c4", "c5", "c2q", "scorer"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8", "nvfp4"], help="scorer operand type of the headline run")
    ap.add_argument("--no-fp8", action="store_true", help="skip the short extra FP8 and NVFP4 passes")
    ap.add_argument("--no-c3", action="store_true", help="N > 1: skip the extra pass at global beam 262 144")
    ap.add_argument("--no-parity", action="store_true", help="skip the untimed oracle check")
    ap.add_argument("--no-cpu", action="store_true", help="N = 1: skip the CPU baseline leg")
    ap.add_argument("--preroll-s", type=float, default=PREROLL_SECONDS,
                    help="seconds of untimed steps before the warm-up (0 for a short run under a profiler)")
    ap.add_argument("--beam-per-gpu", type=int, default=0, help="cases c4/c5/c2q")
    ap.add_argument("--hash-mode", default="fnv", choices=["fnv", "zobrist128"], help="cases c4/c5/c2q")
    ap.add_argument("--rows", type=int, default=151552, help="case scorer")
    ap.add_argument("--repeat", type=int, default=3, help="case scorer")
    ap.add_argument("--scorer", default="mlp", choices=["mlp", "mlp_fp8", "mlp_nvfp4", "transformer", "transformer_fp8"])
    ap.add_argument("--micro-batch", type=int, default=32768, help="case scorer, transformer")
    ap.add_argument("--head", default="pair", choices=["pair", "single"], help="case scorer, MLP layer 2 + head")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.case == "c2":
        run_ours(args)
    elif args.case == "scorer":
        run_scorer_case(args)
    else:
        run_case(args)


if __name__ == "__main__":
    main()
