#!/usr/bin/env python
"""Benchmark of the generation-step hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (the headline metric): PSO + Ackley, 1,000,000 particles x 1,000 dimensions, fp32,
one generation per step, random draws from the in-kernel Philox stream. For N > 1 the same swarm is
row-sharded over the ranks (strong scaling) and launched with torch.distributed.run.

One JSON line is printed by rank 0. `value` is the device-timed throughput with the state resident
in HBM; `e2e` is the same metric through StdWorkflow.step() with the step's host inputs (the three
hyper-parameters) copied from pinned memory and the best fitness read back every step.
`--impl reference` times the CPU restatement of the reference's eager torch path (oracle/) on the
host cores instead.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Bytes per particle-dimension the fused step must move: read pop, velocity, personal best
# (12 B), write pop, velocity (8 B). The conditional personal-best write and the per-row
# vectors are left out, which makes `achieved` conservative.
PSO_BYTES_PER_ELEM = 20.0

# DRAM traffic per particle-dimension of pso_move_eval_kernel from the ncu capture summarised in
# profiles/pso_move_eval_kernel_ackley_65536x1000.md: (589.6 MB read + 665.7 MB written) over the
# 65,536,000 particle-dimensions of the captured launch. Traffic grows in proportion to the number of
# particle-dimensions (every element is read and written once), so it is scaled to the launch size.
PSO_NCU_TRAFFIC_BYTES_PER_ELEM = 19.15

WORKLOADS = {
    # name: (fitness, pop, dim, lb, ub, w, phi_p, phi_g)
    "pso_ackley_1e6x1000": ("ackley", 1_000_000, 1000, -32.768, 32.768, 0.6, 2.5, 0.8),
    "pso_rastrigin_1e6x1000": ("rastrigin", 1_000_000, 1000, -5.12, 5.12, 0.7, 1.5, 1.5),
    "pso_ackley_1e4x500": ("ackley", 10_000, 500, -32.768, 32.768, 0.6, 2.5, 0.8),
    "pso_ackley_small": ("ackley", 65_536, 1000, -32.768, 32.768, 0.6, 2.5, 0.8),
    "pso_ackley_4e6x128": ("ackley", 4_000_000, 128, -32.768, 32.768, 0.6, 2.5, 0.8),  # short rows: one chunk per lane
    "pso_ackley_2e6x256": ("ackley", 2_000_000, 256, -32.768, 32.768, 0.6, 2.5, 0.8),
}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle samples taken while the timed region runs."""

    FIELDS = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=f, stderr=subprocess.DEVNULL,
            )
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def sample_count(self) -> int:
        """Samples of this GPU written so far."""
        if self.path is None or not os.path.exists(self.path):
            return 0
        n = 0
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            n += len(parts) >= 9 and parts[0].isdigit() and int(parts[0]) == self.gpu_index
        return n

    def summary(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.path is None or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9 or not parts[0].isdigit() or int(parts[0]) != self.gpu_index:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            # under load = the upper half of the samples (the sampler also sees idle gaps)
            out["sm_mhz"] = statistics.median(sorted(sm)[len(sm) // 2:])
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v for v in vis.split(",") if v.strip()]
        if local < len(ids) and ids[local].strip().isdigit():
            return int(ids[local])
    return local


# ---------------------------------------------------------------------------------------------
# CPU baseline: the oracle's restatement of the reference's eager torch path, on the host cores.
# ---------------------------------------------------------------------------------------------
def cpu_pso_gens_per_s(workload: str, budget_s: float, steps: int, warmup: int):
    """Times oracle.pso.step on a row sample of the workload and scales to the full swarm
    (the step is linear in the number of particles). Returns (gens/s full-size, sample text, ms/step list)."""
    from oracle import pso as opso

    fit_name, P, d, lb, ub, w, pp, pg = WORKLOADS[workload]
    torch.set_num_threads(os.cpu_count() or 1)
    fitness = opso.FITNESS[fit_name]
    # calibrate on a small sample, then size the timed sample to the budget
    probe_rows = min(P, 5_000)
    s = opso.init_step(opso.make_state(probe_rows, d, lb, ub, w, pp, pg, seed=0), fitness)
    rg, rp = opso.draws(probe_rows, d, 1)
    opso.step(s, rg, rp, fitness)
    t0 = time.perf_counter()
    opso.step(s, rg, rp, fitness)
    per_row = (time.perf_counter() - t0) / probe_rows
    rows = int(budget_s / max(per_row * (steps + warmup), 1e-12))
    rows = max(min(rows, P, 200_000), min(P, 2_000))
    s = opso.init_step(opso.make_state(rows, d, lb, ub, w, pp, pg, seed=0), fitness)
    times = []
    for g in range(warmup + steps):
        t0 = time.perf_counter()
        rg = torch.rand(rows, d)  # the reference draws both inside the step (pso.py:96-97)
        rp = torch.rand(rows, d)
        s = opso.step(s, rg, rp, fitness)
        dt = time.perf_counter() - t0
        if g >= warmup:
            times.append(dt)
    per_gen_full = statistics.mean(times) * (P / rows)
    sample = f"{rows} of {P} particles x {d} dims, {steps} generations after {warmup} warm-up, scaled linearly"
    return 1.0 / per_gen_full, sample, [t * 1e3 for t in times]


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    workload = args.workload
    value, sample, ms = cpu_pso_gens_per_s(workload, budget_s=90.0, steps=args.steps, warmup=args.warmup)
    fit_name, P, d, *_ = WORKLOADS[workload]
    line = {
        "impl": "reference",
        "metric": "pso_generations_per_s",
        "value": value,
        "unit": "gens/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": 1e3 / value,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload, "fitness": fit_name, "pop_size": P, "dim": d},
        "cpu_baseline": {"value": value, "unit": "gens/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "gens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: evox_b200 has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from evox_b200 import _cabi
    from evox_b200.algorithms import PSO
    from evox_b200.problems.numerical import Ackley, Rastrigin
    from evox_b200.workflows import StdWorkflow

    fit_name, P, d, lb, ub, w, pp, pg = WORKLOADS[args.workload]
    torch.manual_seed(0)
    algo = PSO(P, torch.full((d,), lb), torch.full((d,), ub), w, pp, pg, device=dev, shard=world > 1, seed=2026)
    # the benchmark configurations start with velocities in +-0.2 * range
    algo.velocity.mul_(0.2)
    problem = Ackley() if fit_name == "ackley" else Rastrigin()
    wf = StdWorkflow(algo, problem, device=dev)
    assert wf._fused_plan() is not None
    wf.init_step()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    # the sampler runs from the warm-up to the last timed loop (all of it is under load): the
    # timed region alone can be shorter than one nvidia-smi sampling period
    clocks = ClockSampler(physical_gpu_index(local))
    clocks.__enter__()
    # The timed region carries a CUDA-event pair around every launch of the dominant kernel
    # (pso_move_eval_kernel; the algorithm then issues its launches one C call at a time instead of
    # through the single fused call — same kernels, same stream, same order), so the roofline below
    # and `value` come from the same generations and the same clocks.
    a = wf.algorithm
    a._kernel_events = []
    for _ in range(max(args.warmup, 3)):
        wf.step()
    a._kernel_events = []
    total_ms = timed(wf.step, args.steps)
    kernel_ms = sum(e0.elapsed_time(e1) for e0, e1 in a._kernel_events) / len(a._kernel_events)
    a._kernel_events = None
    if world > 1:
        t = torch.tensor([kernel_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        kernel_ms = t.item()
    launches_per_step = 2 if world == 1 else 3
    ms_per_step = total_ms / args.steps
    value = 1e3 / ms_per_step

    # -- end to end: host inputs in, result out, every step ---------------------------------
    hyper_host = torch.tensor([w, pp, pg], dtype=torch.float32).pin_memory()
    hyper_dev = torch.empty(3, dtype=torch.float32, device=dev)
    best_host = torch.empty((), dtype=torch.float32).pin_memory()

    def e2e_step():
        hyper_dev.copy_(hyper_host, non_blocking=True)
        a.w.data.copy_(hyper_dev[0])
        a.phi_p.data.copy_(hyper_dev[1])
        a.phi_g.data.copy_(hyper_dev[2])
        wf.step()
        best_host.copy_(a.global_best_fit, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    e2e_ms = timed(e2e_step, args.steps) / args.steps

    n_local = a.local_size
    # nvidia-smi needs a few hundred milliseconds before its first sample: short runs (many GPUs, few steps)
    # keep stepping, untimed, until the clock record of the load has a few samples (every rank runs the same
    # number of extra generations: the count is agreed on rank 0's record)
    for _ in range(20):
        enough = torch.tensor([1 if clocks.sample_count() >= 4 else 0], device=dev)
        if world > 1:
            dist.broadcast(enough, src=0)
        if int(enough.item()):
            break
        for _ in range(max(args.steps // 2, 10)):
            wf.step()
        barrier()
    clocks.__exit__(None, None, None)
    clock_summary = clocks.summary()
    peak, peak_kind = measured_peaks()
    alg_bytes = PSO_BYTES_PER_ELEM * n_local * d
    achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
    traffic = None if PSO_NCU_TRAFFIC_BYTES_PER_ELEM is None else PSO_NCU_TRAFFIC_BYTES_PER_ELEM * n_local * d

    if rank == 0:
        line = {
            "metric": "pso_generations_per_s",
            "value": value,
            "unit": "gens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "f32",
            "data": "synthetic",
            "config": {
                "workload": args.workload, "fitness": fit_name, "pop_size": P, "dim": d,
                "rows_per_gpu": n_local, "random_draws": "in-kernel Philox4x32-10",
                "l2": "state per GPU (%.1f GB) is larger than L2, no flush needed" % (12.0 * n_local * d / 1e9)
                if 12.0 * n_local * d > 4 * 126e6 else "state fits in L2: numbers are L2-resident",
                "sharding": "rows over ranks, one best-particle allgather per generation" if world > 1 else "single GPU",
            },
            "e2e": {
                "value": 1e3 / e2e_ms, "unit": "gens/s", "h2d_bytes_per_step": 12, "d2h_bytes_per_step": 4,
                "note": "StdWorkflow.step(); swarm state is device-resident by design, host inputs are the hyper-parameters",
            },
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {
                "bound": "hbm", "kernel": "pso_move_eval_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": peak_kind, "traffic": traffic,
                "bytes_per_launch": alg_bytes, "ms_per_launch": kernel_ms,
            },
            "clocks": clock_summary,
        }
        if world == 1 and not args.no_cpu_baseline:
            v, sample, _ = cpu_pso_gens_per_s(args.workload, budget_s=15.0, steps=3, warmup=1)
            line["cpu_baseline"] = {"value": v, "unit": "gens/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_nds(args):
    """Secondary workload: non-dominated rank / full environmental selection on DTLZ2-shaped
    objectives (benchmark configuration 1 at 2N = 20,000 and the metric's 2N = 100,000)."""
    from evox_b200.operators.selection import nd_environmental_selection, non_dominate_rank
    from oracle import nds as onds

    dev = torch.device("cuda", 0)
    n = {"nds_rank_2e4": 20_000, "nds_rank_1e5": 100_000}[args.workload]
    gen = torch.Generator().manual_seed(0)
    x = torch.rand(n, 12, generator=gen)
    f = onds.dtlz2_objectives(x, 3)
    xd, fd = x.to(dev), f.to(dev)

    def timed(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    rank_ms = timed(lambda: non_dominate_rank(fd), args.steps)
    sel_ms = timed(lambda: nd_environmental_selection(xd, fd, n // 2), args.steps)
    rank = non_dominate_rank(fd, check=True)
    line = {
        "metric": "nds_rank_ms", "value": rank_ms, "unit": "ms", "n_gpus": 1, "steps": args.steps, "warmup": 3,
        "ms_per_step": rank_ms, "higher_is_better": False, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "n": n, "m": 3, "fronts": int(rank.max()) + 1},
        "selection_ms": sel_ms,
        "pairs_per_s": n * n / (rank_ms * 1e-3),
    }
    if not args.no_cpu_baseline and n <= 20_000:
        t0 = time.perf_counter()
        onds.non_dominate_rank(f)
        line["cpu_baseline"] = {"value": (time.perf_counter() - t0) * 1e3, "unit": "ms", "cores": torch.get_num_threads(),
                                "kind": "port", "sample": "whole workload, one run"}
    print(json.dumps(line), flush=True)


def run_rvea(args):
    """Secondary workload: RVEA selection at benchmark configuration 2 (50,000 x 10 objectives, 275 vectors)
    and at 5,000,000 rows, where the pass is long enough for its HBM rate to show."""
    from evox_b200.operators.selection import ref_vec_guided
    from oracle import rvea as orvea

    dev = torch.device("cuda", 0)
    n = {"rvea_config2": 50_000, "rvea_5e6": 5_000_000}[args.workload]
    x, f, v, theta = orvea.config2_inputs(n=n)
    xd, fd, vd, td = x.to(dev), f.to(dev), v.to(dev), theta.to(dev)
    for _ in range(3):
        ref_vec_guided(xd, fd, vd, td)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        ref_vec_guided(xd, fd, vd, td)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    m, nv, dx = f.shape[1], v.shape[0], x.shape[1]
    alg_bytes = n * m * 4 * 2 + nv * (dx + m) * 4  # objectives are read twice: ideal point, then association
    peak, kind = measured_peaks()
    line = {
        "metric": "rvea_selection_ms", "value": ms, "unit": "ms", "n_gpus": 1, "steps": args.steps, "warmup": 3,
        "ms_per_step": ms, "higher_is_better": False, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "n": n, "m": m, "nv": nv},
        "roofline": {"bound": "hbm", "kernel": "rvea_assign_kernel + rvea_ideal_kernel", "achieved": alg_bytes / (ms * 1e-3) / 1e9,
                     "peak": peak, "unit": "GB/s", "frac": alg_bytes / (ms * 1e-3) / 1e9 / peak, "peak_kind": kind, "traffic": None},
        "pairs_per_s": n * nv / (ms * 1e-3),
    }
    if not args.no_cpu_baseline and n <= 50_000:
        t0 = time.perf_counter()
        orvea.ref_vec_guided(x, f, v, theta)
        line["cpu_baseline"] = {"value": (time.perf_counter() - t0) * 1e3, "unit": "ms", "cores": torch.get_num_threads(),
                                "kind": "port", "sample": "whole workload, one run"}
    print(json.dumps(line), flush=True)


def run_cso(args):
    """Secondary workloads: the PSO variants on Ackley at 1,000,000 x 1,000 (the headline swarm size),
    in-kernel Philox, fused evaluation; one step = StdWorkflow.step()."""
    from evox_b200.algorithms import CLPSO, CSO, DE, SLPSOGS
    from evox_b200.problems.numerical import Ackley
    from evox_b200.workflows import StdWorkflow

    dev = torch.device("cuda", 0)
    kind, size = args.workload.split("_ackley_")
    n, d = {"1e6x1000": (1_000_000, 1000), "small": (65_536, 1000)}[size]
    lb, ub = torch.full((d,), -32.768), torch.full((d,), 32.768)
    torch.manual_seed(0)
    if kind == "cso":
        algo = CSO(n, lb, ub, phi=0.1, device=dev, seed=1, store_velocity=True)
        # per student-dimension: velocity, teacher and student rows read, student row and velocity written
        alg_bytes, kernel = (n // 2) * d * 20.0, "cso_update_kernel (incl. randperm and the mean's finish)"
    elif kind == "clpso":
        algo = CLPSO(n, lb, ub, device=dev, seed=1)
        # position, velocity, exemplar row read; position, velocity written (+ 8 B per improved particle-dimension)
        alg_bytes, kernel = n * d * 20.0, "clpso_move_eval_kernel (incl. personal-best update and exemplar bookkeeping)"
    elif kind == "de":
        algo = DE(n, lb, ub, device=dev, seed=1)
        # own row and three other rows read, trial written (+ 8 B per accepted individual-dimension)
        alg_bytes, kernel = n * d * 20.0, "de_trial_kernel + de_select_kernel (incl. the index draws)"
    else:
        algo = SLPSOGS(n, lb, ub, device=dev, seed=1)
        alg_bytes, kernel = n * d * 20.0, "slpso_update_kernel (incl. the fitness sort and the mean's finish)"
    if hasattr(algo, "velocity"):
        algo.velocity.mul_(0.2)
    wf = StdWorkflow(algo, Ackley(), device=dev)
    wf.init_step()
    for _ in range(max(args.warmup, 3)):
        wf.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clocks:
        e0.record()
        for _ in range(args.steps):
            wf.step()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    peak, peak_kind = measured_peaks()
    line = {
        "metric": f"{kind}_generations_per_s", "value": 1e3 / ms, "unit": "gens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "pop_size": n, "dim": d, "l2": "state larger than L2"},
        "roofline": {"bound": "hbm", "kernel": kernel, "achieved": alg_bytes / (ms * 1e-3) / 1e9,
                     "peak": peak, "unit": "GB/s", "frac": alg_bytes / (ms * 1e-3) / 1e9 / peak, "peak_kind": peak_kind, "traffic": None},
        "clocks": clocks.summary(),
    }
    print(json.dumps(line), flush=True)


def run_lora_es(args):
    """Secondary workload: benchmark configuration 3 — VirtualLoRAES over a 3 x (4096 -> 4096) bf16 MLP,
    1,024 individuals with their own 64 x 4096 batch, rank-8 factors, sigma 0.02, lr 0.01, centred
    ranks, SGD. One step = seeds -> forward (tensor cores) -> fitness -> gradient -> centre update,
    through StdWorkflow.step()."""
    from torch import nn

    from evox_b200.algorithms import VirtualLoRAES
    from evox_b200.problems import VirtualLoRAProblem
    from evox_b200.transforms import CenteredRank
    from evox_b200.workflows import StdWorkflow

    dev = torch.device("cuda", 0)
    pop, batch, width, layers, rank = args.lora_pop, 64, 4096, 3, 8
    gen = torch.Generator().manual_seed(0)
    mods = []
    for i in range(layers):
        lin = nn.Linear(width, width, bias=False)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(width, width, generator=gen) / width**0.5)
        mods.append(lin)
        if i + 1 < layers:
            mods.append(nn.ReLU())
    model = nn.Sequential(*mods)
    x = torch.randn(pop, batch, width, generator=gen).bfloat16().to(dev)
    target = torch.randn(batch, width, generator=gen).to(dev)
    prob = VirtualLoRAProblem(model, [(x, target)], nn.MSELoss(reduction="none"), rank, device=dev, compute_dtype=torch.bfloat16)
    center = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    algo = VirtualLoRAES(prob.param_shapes, rank, pop, center, 0.01, 0.02, device=dev, gradient_passes=args.gradient_passes)
    wf = StdWorkflow(algo, prob, device=dev, fitness_transform=CenteredRank())

    def timed(fn, reps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    for _ in range(3):
        wf.step()
    with ClockSampler(0) as clocks:
        step_ms = timed(wf.step, args.steps)
        seeds = wf.algorithm.seeds
        fwd_ms = timed(lambda: prob.evaluate((wf.algorithm.center, seeds, 0.02)), args.steps)
    m = pop * batch
    flop_fwd = layers * (2.0 * m * width * width + 2.0 * m * rank * 2 * width)
    flop_grad = layers * 2.0 * width * (pop * rank) * width
    from evox_b200.lora_kernels import lora_layer_bf16

    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    line = {
        "metric": "lora_es_generations_per_s", "value": 1e3 / step_ms, "unit": "gens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": 3, "ms_per_step": step_ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "lora_es_config3", "pop": pop, "batch": batch, "width": width, "layers": layers, "rank": rank,
                   "gradient_passes": args.gradient_passes},
        "forward_ms": fwd_ms,
        "roofline": {"bound": "tensor", "kernel": "lora_gemm_kernel (forward, 3 layers)", "achieved": flop_fwd / (fwd_ms * 1e-3) / 1e12,
                     "peak": peak, "unit": "TFLOP/s", "frac": flop_fwd / (fwd_ms * 1e-3) / 1e12 / peak,
                     "peak_kind": "measured sustained" if peaks else "fallback", "traffic": None},
        "generation_tflops": (flop_fwd + flop_grad) / (step_ms * 1e-3) / 1e12,
        "gemm_error_flag": int(lora_layer_bf16.last_error_flag),
        "clocks": clocks.summary(),
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="pso_ackley_1e6x1000", choices=sorted(WORKLOADS) + ["nds_rank_2e4", "nds_rank_1e5", "lora_es_config3", "rvea_config2", "rvea_5e6", "cso_ackley_1e6x1000", "cso_ackley_small", "clpso_ackley_1e6x1000", "slpso_ackley_1e6x1000", "de_ackley_1e6x1000"])
    ap.add_argument("--lora-pop", type=int, default=1024)
    ap.add_argument("--gradient-passes", type=int, default=3, choices=[1, 3, 6])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.workload.startswith("nds_"):
        run_nds(args)
    elif args.workload == "lora_es_config3":
        run_lora_es(args)
    elif args.workload.split("_")[0] in ("cso", "clpso", "slpso", "de"):
        run_cso(args)
    elif args.workload.startswith("rvea_"):
        run_rvea(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
