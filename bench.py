#!/usr/bin/env python
"""Benchmark of the generation-step hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (the headline metric): PSO + Ackley, 1,000,000 particles x 1,000 dimensions, fp32,
one generation per step, random draws from the in-kernel Philox stream. For N > 1 the same swarm is
row-sharded over the ranks (strong scaling) and launched with torch.distributed.run.

One JSON line is printed by rank 0. `value` is the device-timed throughput with the state resident
in HBM; `e2e` is the same metric through StdWorkflow.step() with the step's host inputs (the three
hyper-parameters) copied from pinned memory and the best fitness read back every step.
On one GPU the line also carries `secondary`: the other paths of the metric (non-dominated rank at
2N = 100,000 and 20,000, RVEA selection, a virtual-LoRA ES generation, the PSO configurations 0 and
4), each timed with CUDA events over its own repeats and with its own clock record, plus the fp32
compare issue-rate microbenchmark the non-dominated sort's roofline is measured against.
On several GPUs the line carries `sharded_equals_single` (small sharded runs compared bit for bit
with single-GPU runs before anything is timed), the Rastrigin configuration, the latency of a
4 KB NCCL allgather and the row-sharded RVEA / virtual-LoRA / non-dominated-sort steps.
`--impl reference` times the reference's own eager torch implementation on the host cores (imported
from oracle/_ref when `oracle/build_ref.py` has installed it there, else its restatement in oracle/).
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

# DRAM traffic per particle-dimension of the update kernel from one ncu capture of a 65,536 x 1,000
# launch: (589.6 MB read + 665.7 MB written) over its 65,536,000 particle-dimensions. Traffic grows in
# proportion to the number of particle-dimensions (every element is read and written once), so it is
# scaled to the launch size; `roofline.traffic_source` says so in the line.
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
OTHER_WORKLOADS = ["nds_rank_2e4", "nds_rank_1e5", "lora_es_config3", "rvea_config2", "rvea_5e6", "cso_ackley_1e6x1000",
                   "cso_ackley_small", "clpso_ackley_1e6x1000", "slpso_ackley_1e6x1000", "de_ackley_1e6x1000",
                   "microbench_compare", "nccl_allgather_4k"]


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


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


def timed_ms(fn, reps: int, warmup: int = 3) -> float:
    """Mean milliseconds of `fn` over `reps` back-to-back calls, CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def pso_config(workload: str, world: int) -> dict:
    """The `config` object of the PSO lines; both arms print exactly this."""
    fit_name, P, d, *_ = WORKLOADS[workload]
    rows = -(-P // world)
    return {
        "workload": workload, "fitness": fit_name, "pop_size": P, "dim": d, "rows_per_gpu": rows,
        "random_draws": "in-kernel Philox4x32-10 (the reference arm: torch.rand, as the reference draws them)",
        "l2": "state per GPU (%.1f GB) is larger than L2, no flush needed" % (12.0 * rows * d / 1e9)
        if 12.0 * rows * d > 4 * 126e6 else "state fits in L2: numbers are L2-resident",
        "sharding": "rows over ranks, every shard's best-particle record exchanged once per generation" if world > 1 else "single GPU",
    }


# ---------------------------------------------------------------------------------------------
# CPU baseline and reference arm: the reference's own eager torch path on the host cores.
# ---------------------------------------------------------------------------------------------
def load_reference():
    """The reference package installed by oracle/build_ref.py, or None."""
    from oracle.build_ref import reference_package

    path = reference_package()
    if path is None:
        return None
    if str(path) not in sys.path:
        sys.path.insert(0, str(path))
    try:
        import evox  # noqa: F401

        return evox
    except Exception:
        return None


def reference_pso_workflow(workload: str, rows: int, device: torch.device):
    """StdWorkflow(PSO, problem) of the reference itself, `rows` particles of the workload's swarm."""
    from evox.algorithms import PSO
    from evox.problems.numerical import Ackley, Rastrigin
    from evox.workflows import StdWorkflow

    fit_name, P, d, lb, ub, w, pp, pg = WORKLOADS[workload]
    torch.manual_seed(0)
    algo = PSO(rows, torch.full((d,), lb, device=device), torch.full((d,), ub, device=device), w, pp, pg, device=device)
    algo.velocity = 0.2 * algo.velocity  # the benchmark configurations start with velocities in +-0.2 * range
    wf = StdWorkflow(algo, Ackley() if fit_name == "ackley" else Rastrigin(), device=device)
    wf.init_step()
    return wf


def host_memory_available() -> float:
    try:
        import psutil

        return float(psutil.virtual_memory().available)
    except Exception:
        return 0.0


def cpu_pso_gens_per_s(workload: str, budget_s: float, steps: int, warmup: int, allow_full: bool):
    """Times one PSO generation of the reference on the host cores: the reference's own code when it is
    installed under oracle/_ref (kind "reference"), else oracle.pso.step (kind "port"). The swarm is the
    workload's own when memory and the time budget allow, otherwise a row sample whose time is scaled to the
    full swarm (the step is linear in the number of particles).
    Returns (gens/s at full size, kind, sample text, un-scaled ms per step, rows)."""
    from oracle import pso as opso

    fit_name, P, d, lb, ub, w, pp, pg = WORKLOADS[workload]
    torch.set_num_threads(os.cpu_count() or 1)
    ref = load_reference()
    kind = "reference" if ref is not None else "port"
    cpu = torch.device("cpu")
    fitness = opso.FITNESS[fit_name]

    def make(rows):
        if ref is not None:
            wf = reference_pso_workflow(workload, rows, cpu)
            return wf.step
        state = {"s": opso.init_step(opso.make_state(rows, d, lb, ub, w, pp, pg, seed=0), fitness)}

        def step():
            rg = torch.rand(rows, d)  # the reference draws both inside the step (pso.py:96-97)
            rp = torch.rand(rows, d)
            state["s"] = opso.step(state["s"], rg, rp, fitness)

        return step

    # calibrate on a small sample, then size the timed swarm to the budget and to the host's memory
    probe_rows = min(P, 20_000)
    step = make(probe_rows)
    step()
    t0 = time.perf_counter()
    step()
    per_row = (time.perf_counter() - t0) / probe_rows
    rows = int(budget_s / max(per_row * (steps + warmup), 1e-12))
    mem_rows = int(host_memory_available() / (16 * 4.0 * d)) if host_memory_available() > 0 else 200_000  # ~16 live (rows, d) arrays
    cap = P if allow_full else min(P, 200_000)
    rows = max(min(rows, cap, max(mem_rows, 2_000)), min(P, 2_000))
    if rows >= 0.9 * P and mem_rows >= P:
        rows = P
    step = make(rows)
    times = []
    for g in range(warmup + steps):
        t0 = time.perf_counter()
        step()
        dt = time.perf_counter() - t0
        if g >= warmup:
            times.append(dt)
    mean_s = statistics.mean(times)
    per_gen_full = mean_s * (P / rows)
    sample = (f"the whole swarm ({P} x {d}), {steps} generations after {warmup} warm-up" if rows == P else
              f"{rows} of {P} particles x {d} dims, {steps} generations after {warmup} warm-up, scaled linearly")
    return 1.0 / per_gen_full, kind, sample, mean_s * 1e3, rows


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    workload = args.workload
    # the whole swarm when 25 generations of it fit in about seven minutes and in the host's memory
    value, kind, sample, ms_sample, rows = cpu_pso_gens_per_s(workload, budget_s=args.reference_budget_s, steps=args.steps,
                                                              warmup=args.warmup, allow_full=True)
    fit_name, P, d, *_ = WORKLOADS[workload]
    line = {
        "impl": "reference",
        "metric": "pso_generations_per_s",
        "value": value,
        "unit": "gens/s",
        "n_gpus": 0,
        "gpus_requested": args.gpus,
        "reference_class": "cpu",
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": 1e3 / value,
        "ms_per_step_as_timed": ms_sample,
        "rows_timed": rows,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": pso_config(workload, world),
        "cpu_baseline": {"value": value, "unit": "gens/s", "cores": torch.get_num_threads(), "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "gens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def reference_on_gpu(workload: str, dev: torch.device, steps: int = 10) -> dict:
    """The reference's own eager torch PSO on the CUDA device (its operators run unchanged there): the
    same-hardware comparison. Timed with CUDA events; the whole swarm when it fits."""
    if load_reference() is None:
        return {"unavailable": "the reference is not installed under oracle/_ref"}
    fit_name, P, d, *_ = WORKLOADS[workload]
    free, _ = torch.cuda.mem_get_info(dev)
    rows = P if free > 20 * 4.0 * P * d else int(free / (24 * 4.0 * d))
    try:
        wf = reference_pso_workflow(workload, rows, dev)
        ms = timed_ms(wf.step, steps, warmup=3)
    except Exception as exc:  # the comparison is optional: say why it is missing
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    finally:
        wf = None
        torch.cuda.empty_cache()
    return {"value": 1e3 / (ms * P / rows), "unit": "gens/s", "ms_per_step_as_timed": ms, "rows_timed": rows,
            "what": "reference StdWorkflow(PSO, problem).step() in eager mode on the same GPU, torch.rand draws"}


# ---------------------------------------------------------------------------------------------
# Secondary measurements (each returns one JSON object)
# ---------------------------------------------------------------------------------------------
def measure_compare_rate(dev: torch.device) -> dict:
    """fp32 set-predicate issue rate of this GPU (see csrc/microbench.cu)."""
    from evox_b200 import _cabi

    threads = _cabi.lib.evox_bench_compare_rate_threads()
    src = torch.rand(1024, device=dev)
    src[1023] = 1e-3
    out = torch.empty(threads, dtype=torch.int32, device=dev)
    iters = 20_000

    def run():
        _cabi.check(_cabi.lib.evox_bench_compare_rate(_cabi.ptr(src), _cabi.ptr(out), iters, _cabi.stream_ptr(dev)))

    with ClockSampler(physical_gpu_index(dev.index or 0)) as clocks:
        ms = min(timed_ms(run, 5, warmup=2) for _ in range(3))
    rate = 64.0 * iters * threads / (ms * 1e-3)
    return {"compares_per_s": rate, "ms_per_launch": ms, "threads": threads, "compares_per_thread": 64 * iters,
            "clocks": clocks.summary(),
            "what": "fp32 <= comparisons AND-combined into predicates, 64 per iteration and thread + 4 select-adds"}


def nds_floor_ms(n: int, m: int, compare_rate: float | None) -> dict:
    """Roofline of the rank: m * n^2 comparisons at the measured issue rate, against writing and reading
    the bit matrix once (n^2 / 8 bytes each) plus the objectives at the measured HBM rate."""
    pk = peaks()
    hbm_ms = (2.0 * n * n / 8 + 4.0 * n * m) / (pk["hbm_gbs"] * 1e9) * 1e3
    alu_ms = None if not compare_rate else (float(m) * n * n) / compare_rate * 1e3
    return {"hbm_floor_ms": hbm_ms, "alu_floor_ms": alu_ms, "floor_ms": max(hbm_ms, alu_ms or 0.0)}


def measure_nds(n: int, reps: int, dev: torch.device, compare_rate: float | None, cpu: bool, selection: bool = True) -> dict:
    """Non-dominated rank and the full environmental selection on DTLZ2-shaped objectives (benchmark
    configuration 1 at 2N = 20,000; the metric's 2N = 100,000)."""
    from evox_b200.operators.selection import nd_environmental_selection, non_dominate_rank
    from oracle import nds as onds

    x = torch.rand(n, 12, generator=torch.Generator().manual_seed(0))
    f = onds.dtlz2_objectives(x, 3)
    xd, fd = x.to(dev), f.to(dev)
    with ClockSampler(physical_gpu_index(dev.index or 0)) as clocks:
        rank_ms = timed_ms(lambda: non_dominate_rank(fd), reps, warmup=3 if n <= 100_000 else 1)
        sel_ms = timed_ms(lambda: nd_environmental_selection(xd, fd, n // 2), reps) if selection else None
    rank = non_dominate_rank(fd, check=True)
    floor = nds_floor_ms(n, 3, compare_rate)
    out = {
        "metric": "nds_rank_ms", "value": rank_ms, "unit": "ms", "repeats": reps, "selection_ms": sel_ms,
        "config": {"n": n, "m": 3, "fronts": int(rank.max()) + 1, "objectives": "DTLZ2 of uniform [0,1]^12, seed 0"},
        "roofline": {"bound": "fp32 compare issue rate (dominance) / hbm (bit matrix)", **floor,
                     "frac": floor["floor_ms"] / rank_ms, "peak_kind": peaks()["kind"],
                     "note": "floor = max(m n^2 comparisons at the measured issue rate, n^2/4 bytes at measured HBM)"},
        "pairs_per_s": n * n / (rank_ms * 1e-3),
        "clocks": clocks.summary(),
    }
    if cpu:
        # the oracle's blocked bit-packed restatement; at 2N = 100,000 only the dominance phase of a row sample
        rows = n if n <= 20_000 else 4096
        t0 = time.perf_counter()
        if rows == n:
            onds.non_dominate_rank(f)
            secs, sample = time.perf_counter() - t0, "whole workload, one run"
        else:
            d = onds.dominate_relation(f[:rows], f)
            d.sum(dim=0)
            secs = (time.perf_counter() - t0) * n / rows
            sample = f"dominance rows {rows} of {n} (the peel is not included), scaled linearly"
        out["cpu_baseline"] = {"value": secs * 1e3, "unit": "ms", "cores": torch.get_num_threads(), "kind": "port", "sample": sample}
    return out


def measure_rvea(n: int, reps: int, dev: torch.device, cpu: bool) -> dict:
    """RVEA selection at benchmark configuration 2 (50,000 x 10 objectives, 275 vectors) or at 5,000,000 rows."""
    from evox_b200.operators.selection import ref_vec_guided
    from oracle import rvea as orvea

    x, f, v, theta = orvea.config2_inputs(n=n)
    xd, fd, vd, td = x.to(dev), f.to(dev), v.to(dev), theta.to(dev)
    with ClockSampler(physical_gpu_index(dev.index or 0)) as clocks:
        ms = timed_ms(lambda: ref_vec_guided(xd, fd, vd, td), reps)
    m, nv, dx = f.shape[1], v.shape[0], x.shape[1]
    alg_bytes = n * m * 4 * 2 + nv * (dx + m) * 4  # objectives are read twice: ideal point, then association
    pk = peaks()
    out = {
        "metric": "rvea_selection_ms", "value": ms, "unit": "ms", "repeats": reps,
        "config": {"n": n, "m": m, "nv": nv, "dx": dx, "theta": float(theta)},
        "roofline": {"bound": "hbm", "achieved": alg_bytes / (ms * 1e-3) / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": alg_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], "peak_kind": pk["kind"],
                     "note": "the pass is bound by n * nv cosine arithmetic, not by its bytes; at 50,000 rows by launch latency"},
        "pairs_per_s": n * nv / (ms * 1e-3),
        "clocks": clocks.summary(),
    }
    if cpu and n <= 50_000:
        t0 = time.perf_counter()
        orvea.ref_vec_guided(x, f, v, theta)
        out["cpu_baseline"] = {"value": (time.perf_counter() - t0) * 1e3, "unit": "ms", "cores": torch.get_num_threads(),
                               "kind": "port", "sample": "whole workload, one run"}
    return out


def lora_es_workflow(dev: torch.device, pop: int, shard: bool, gradient_passes: int = 3):
    """Benchmark configuration 3: VirtualLoRAES over a 3 x (4096 -> 4096) bf16 MLP, `pop` individuals with their
    own 64 x 4096 batch, rank-8 factors, sigma 0.02, lr 0.01, centred ranks, SGD."""
    from torch import nn

    from evox_b200.algorithms import VirtualLoRAES
    from evox_b200.problems import VirtualLoRAProblem
    from evox_b200.transforms import CenteredRank
    from evox_b200.workflows import StdWorkflow

    batch, width, layers, rank = 64, 4096, 3, 8
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
    prob = VirtualLoRAProblem(model, [(x, target)], nn.MSELoss(reduction="none"), rank, device=dev, compute_dtype=torch.bfloat16,
                              shard=shard)
    center = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    algo = VirtualLoRAES(prob.param_shapes, rank, pop, center, 0.01, 0.02, device=dev, gradient_passes=gradient_passes, shard=shard)
    wf = StdWorkflow(algo, prob, device=dev, fitness_transform=CenteredRank())
    return wf, prob, (pop, batch, width, layers, rank)


def measure_lora_es(reps: int, dev: torch.device, pop: int = 1024, gradient_passes: int = 3, shard: bool = False) -> dict:
    """One step = seeds -> forward (tensor cores) -> fitness -> gradient -> centre update, through StdWorkflow.step()."""
    from evox_b200.lora_kernels import lora_layer_bf16

    wf, prob, (pop, batch, width, layers, rank) = lora_es_workflow(dev, pop, shard, gradient_passes)
    with ClockSampler(physical_gpu_index(dev.index or 0)) as clocks:
        step_ms = timed_ms(wf.step, reps)
        seeds = wf.algorithm.seeds
        fwd_ms = timed_ms(lambda: prob.evaluate((wf.algorithm.center, seeds, 0.02)), reps)
    m = pop * batch
    flop_fwd = layers * (2.0 * m * width * width + 2.0 * m * rank * 2 * width)
    flop_grad = layers * 2.0 * width * (pop * rank) * width
    pk = peaks()
    peak = pk["bf16_tflops_sustained"]
    world = torch.distributed.get_world_size() if shard and torch.distributed.is_initialized() else 1
    return {
        "metric": "lora_es_generation_ms", "value": step_ms, "unit": "ms", "repeats": reps, "forward_ms": fwd_ms,
        "config": {"pop": pop, "batch": batch, "width": width, "layers": layers, "rank": rank, "gradient_passes": gradient_passes,
                   "sharded_over": world},
        "roofline": {"bound": "tensor", "flop_per_generation": flop_fwd + flop_grad,
                     "achieved": (flop_fwd + flop_grad) / (step_ms * 1e-3) / 1e12 / world, "peak": peak, "unit": "TFLOP/s per GPU",
                     "frac": (flop_fwd + flop_grad) / (step_ms * 1e-3) / 1e12 / world / peak,
                     "forward_frac": flop_fwd / (fwd_ms * 1e-3) / 1e12 / world / peak,
                     "peak_kind": pk["kind"] + " sustained bf16",
                     "note": "algorithmic flop (one product per gradient block); the kernel runs three fp16 products for fp32 accuracy"},
        "gemm_error_flag": int(lora_layer_bf16.last_error_flag),
        "clocks": clocks.summary(),
    }


def measure_pso_small(workload: str, reps: int, dev: torch.device) -> dict:
    """A PSO configuration other than the headline one, whole generations through StdWorkflow.step()."""
    from evox_b200.algorithms import PSO
    from evox_b200.problems.numerical import Ackley, Rastrigin
    from evox_b200.workflows import StdWorkflow

    fit_name, P, d, lb, ub, w, pp, pg = WORKLOADS[workload]
    algo = PSO(P, torch.full((d,), lb), torch.full((d,), ub), w, pp, pg, device=dev, seed=2026)
    algo.velocity.mul_(0.2)
    wf = StdWorkflow(algo, Ackley() if fit_name == "ackley" else Rastrigin(), device=dev)
    wf.init_step()
    with ClockSampler(physical_gpu_index(dev.index or 0)) as clocks:
        ms = timed_ms(wf.step, reps, warmup=5)
    pk = peaks()
    gbs = PSO_BYTES_PER_ELEM * P * d / (ms * 1e-3) / 1e9
    return {"metric": "pso_generations_per_s", "value": 1e3 / ms, "unit": "gens/s", "ms_per_step": ms, "repeats": reps,
            "config": pso_config(workload, 1), "gpu_launches_per_step": 1,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                         "peak_kind": pk["kind"]},
            "clocks": clocks.summary()}


def measure_allgather_latency(dev: torch.device, reps: int = 200) -> dict:
    """Latency of the one collective of a sharded PSO generation: an NCCL allgather of a 4 KB record per rank."""
    import torch.distributed as dist

    world = dist.get_world_size()
    rec = torch.zeros(1024, dtype=torch.int32, device=dev)
    out = torch.zeros(world * 1024, dtype=torch.int32, device=dev)
    ms = timed_ms(lambda: dist.all_gather_into_tensor(out, rec), reps, warmup=20)
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"us_per_allgather": t.item() * 1e3, "bytes_per_rank": 4096, "ranks": world, "repeats": reps,
            "what": "back-to-back all_gather_into_tensor on one stream, CUDA events, max over ranks"}


def sharded_checks(dev: torch.device, rank: int, world: int) -> dict:
    """Small sharded runs compared bit for bit with single-GPU runs on the same device (tests/multigpu_check.py)."""
    from tests import multigpu_check as mc

    out = {}
    for name, fn in (("pso", mc.check_pso), ("lora_es", mc.check_lora_es), ("rvea", mc.check_rvea), ("nds", getattr(mc, "check_nds", None))):
        if fn is None:
            continue
        ok = torch.ones(1, device=dev)
        try:
            fn(dev, rank, world)
        except AssertionError:
            ok.zero_()
        torch.distributed.all_reduce(ok, op=torch.distributed.ReduceOp.MIN)
        out[name] = bool(ok.item())
    return out


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

    from evox_b200.algorithms import PSO
    from evox_b200.problems.numerical import Ackley, Rastrigin
    from evox_b200.workflows import StdWorkflow

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

    extras = {}
    if world > 1:
        checks = sharded_checks(dev, rank, world)
        extras["sharded_equals_single"] = all(checks.values())
        extras["sharded_checks"] = checks
        extras["nccl_allgather_4k"] = measure_allgather_latency(dev)

    def pso_run(workload, steps, warmup, with_e2e=True, peer_exchange=True):
        fit_name, P, d, lb, ub, w, pp, pg = WORKLOADS[workload]
        torch.manual_seed(0)
        algo = PSO(P, torch.full((d,), lb), torch.full((d,), ub), w, pp, pg, device=dev, shard=world > 1, seed=2026,
                   peer_exchange=peer_exchange)
        algo.velocity.mul_(0.2)  # the benchmark configurations start with velocities in +-0.2 * range
        wf = StdWorkflow(algo, Ackley() if fit_name == "ackley" else Rastrigin(), device=dev)
        assert wf._fused_plan() is not None
        wf.init_step()
        a = wf.algorithm
        # `value`: StdWorkflow.step() — one C call, one kernel launch (plus the allgather on several GPUs) per
        # generation. The same generations carry a CUDA-event pair around the kernel for the roofline.
        for _ in range(warmup):
            wf.step()
        a._kernel_events = []
        total_ms = timed(wf.step, steps)
        kernel_ms = sum(e0.elapsed_time(e1) for e0, e1 in a._kernel_events) / len(a._kernel_events)
        a._kernel_events = None
        if world > 1:
            t = torch.tensor([kernel_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            kernel_ms = t.item()
        res = {"ms_per_step": total_ms / steps, "kernel_ms": kernel_ms, "rows": a.local_size, "P": P, "d": d,
               "exchange": "single GPU" if world == 1 else ("peer stores by the generation kernel" if a._peer else "NCCL allgather")}
        if a.exchange_status() != 0:
            raise RuntimeError("PSO: a wait for another GPU's best-particle record gave up during the timed run")
        if with_e2e:
            # end to end: host inputs in (three pinned scalars), result out, every step
            host = [torch.tensor(v, dtype=torch.float32).pin_memory() for v in (w, pp, pg)]
            params = [a.w.data, a.phi_p.data, a.phi_g.data]
            best_host = torch.empty((), dtype=torch.float32).pin_memory()

            def e2e_step():
                for dst, src in zip(params, host):
                    dst.copy_(src, non_blocking=True)
                wf.step()
                best_host.copy_(a.global_best_fit, non_blocking=True)
                torch.cuda.current_stream().synchronize()

            for _ in range(3):
                e2e_step()
            res["e2e_ms"] = timed(e2e_step, steps) / steps
        return res, wf

    clocks = ClockSampler(physical_gpu_index(local))
    clocks.__enter__()
    warmup = max(args.warmup, 3)
    main, wf = pso_run(args.workload, args.steps, warmup)
    # nvidia-smi needs a few hundred milliseconds before its first sample: short runs (many GPUs, few steps)
    # keep stepping, untimed, until the clock record of the load has a few samples (every rank runs the same
    # number of extra generations: the count is agreed on rank 0's record)
    t_wait = time.perf_counter()
    while True:
        enough = torch.tensor([1 if (clocks.sample_count() >= 4 or time.perf_counter() - t_wait > 5.0) else 0], device=dev)
        if world > 1:
            dist.broadcast(enough, src=0)
        if int(enough.item()):
            break
        for _ in range(100):
            wf.step()
        barrier()
    clocks.__exit__(None, None, None)
    clock_summary = clocks.summary()
    wf = None
    torch.cuda.empty_cache()

    fit_name, P, d, *_ = WORKLOADS[args.workload]
    n_local = main["rows"]
    pk = peaks()
    alg_bytes = PSO_BYTES_PER_ELEM * n_local * d
    achieved = alg_bytes / (main["kernel_ms"] * 1e-3) / 1e9
    # the generation kernel (+ NCCL's allgather kernel when the records do not travel by peer stores)
    launches_per_step = 2 if main["exchange"] == "NCCL allgather" else 1

    if world > 1 and args.workload == "pso_ackley_1e6x1000" and not args.no_secondary:
        # benchmark configuration 4 names Rastrigin (w = 0.7, phi = 1.5 / 1.5) for the sharded swarm
        with ClockSampler(physical_gpu_index(local)) as c4:
            r4, wf4 = pso_run("pso_rastrigin_1e6x1000", args.steps, warmup)
        wf4 = None
        torch.cuda.empty_cache()
        # the headline swarm again with the records exchanged by one NCCL allgather per generation
        rn, wfn = pso_run(args.workload, args.steps, warmup, with_e2e=False, peer_exchange=False)
        wfn = None
        torch.cuda.empty_cache()
        extras["pso_ackley_nccl_exchange"] = {"value": 1e3 / rn["ms_per_step"], "unit": "gens/s", "ms_per_step": rn["ms_per_step"],
                                              "kernel_ms": rn["kernel_ms"], "exchange": rn["exchange"]}
        extras["pso_rastrigin_1e6x1000"] = {
            "value": 1e3 / r4["ms_per_step"], "unit": "gens/s", "ms_per_step": r4["ms_per_step"], "kernel_ms": r4["kernel_ms"],
            "e2e": {"value": 1e3 / r4["e2e_ms"], "unit": "gens/s", "h2d_bytes_per_step": 12, "d2h_bytes_per_step": 4},
            "config": pso_config("pso_rastrigin_1e6x1000", world), "clocks": c4.summary(), "exchange": r4["exchange"],
        }
        sec = {}
        from evox_b200.operators.selection import ref_vec_guided_sharded
        from evox_b200.sharding import shard_bounds
        from oracle import rvea as orvea

        x, f, v, theta = orvea.config2_inputs(n=5_000_000)
        lo, hi = shard_bounds(x.shape[0], world, rank)
        xd, fd, vd, td = x[lo:hi].to(dev), f[lo:hi].to(dev), v.to(dev), theta.to(dev)
        ms = timed(lambda: ref_vec_guided_sharded(xd, fd, vd, td, lo), 20) / 20
        sec["rvea_5e6_sharded"] = {"metric": "rvea_selection_ms", "value": ms, "unit": "ms", "repeats": 20,
                                   "config": {"n": 5_000_000, "m": 10, "nv": int(v.shape[0]), "rows_per_gpu": hi - lo}}
        del x, f, xd, fd
        sec["lora_es_config3_sharded"] = measure_lora_es(10, dev, shard=True)
        t = torch.tensor([sec["lora_es_config3_sharded"]["value"]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec["lora_es_config3_sharded"]["value"] = t.item()
        torch.cuda.empty_cache()
        try:
            from evox_b200.operators.selection import non_dominate_rank_sharded
        except ImportError:
            non_dominate_rank_sharded = None
        if non_dominate_rank_sharded is not None:
            from oracle import nds as onds

            for n in (100_000, 400_000):
                fobj = onds.dtlz2_objectives(torch.rand(n, 12, generator=torch.Generator().manual_seed(0)), 3).to(dev)
                ms = timed(lambda: non_dominate_rank_sharded(fobj), 5) / 5
                sec[f"nds_rank_sharded_{n}"] = {"metric": "nds_rank_ms", "value": ms, "unit": "ms", "repeats": 5,
                                                "config": {"n": n, "m": 3, "dominator_rows_per_gpu": -(-n // world)}}
                del fobj
                torch.cuda.empty_cache()
        extras["secondary"] = sec

    if world == 1 and args.workload == "pso_ackley_1e6x1000" and not args.no_secondary:
        sec = {}
        mb = measure_compare_rate(dev)
        sec["microbench_compare"] = mb
        rate = mb["compares_per_s"]
        cpu = not args.no_cpu_baseline
        sec["nds_rank_1e5"] = measure_nds(100_000, 20, dev, rate, cpu)
        sec["nds_rank_2e4"] = measure_nds(20_000, 50, dev, rate, cpu)
        # the size at which one GPU's bit matrix is 20 GB: the single-GPU side of the split-matrix comparison
        sec["nds_rank_4e5"] = measure_nds(400_000, 3, dev, rate, False, selection=False)
        torch.cuda.empty_cache()
        sec["rvea_config2"] = measure_rvea(50_000, 100, dev, cpu)
        sec["rvea_5e6"] = measure_rvea(5_000_000, 20, dev, False)
        torch.cuda.empty_cache()
        sec["lora_es_config3"] = measure_lora_es(20, dev)
        torch.cuda.empty_cache()
        sec["pso_rastrigin_1e6x1000"] = measure_pso_small("pso_rastrigin_1e6x1000", 20, dev)
        torch.cuda.empty_cache()
        sec["pso_ackley_1e4x500"] = measure_pso_small("pso_ackley_1e4x500", 200, dev)
        extras["secondary"] = sec
        extras["reference_gpu_eager"] = reference_on_gpu(args.workload, dev)

    if rank == 0:
        line = {
            "metric": "pso_generations_per_s",
            "value": 1e3 / main["ms_per_step"],
            "unit": "gens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": warmup,
            "ms_per_step": main["ms_per_step"],
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "f32",
            "data": "synthetic",
            "config": pso_config(args.workload, world),
            "e2e": {
                "value": 1e3 / main["e2e_ms"], "unit": "gens/s", "h2d_bytes_per_step": 12, "d2h_bytes_per_step": 4,
                "note": "StdWorkflow.step(); swarm state is device-resident by design, host inputs are the hyper-parameters",
            },
            "gpu_launches": launches_per_step * args.steps,
            "exchange": main["exchange"],
            "roofline": {
                "bound": "hbm", "kernel": "pso_move_eval_kernel (fused generation)", "achieved": achieved, "peak": pk["hbm_gbs"],
                "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "peak_kind": pk["kind"],
                "traffic": PSO_NCU_TRAFFIC_BYTES_PER_ELEM * n_local * d,
                "traffic_source": "ncu capture of a 65,536 x 1,000 launch, scaled by particle-dimensions",
                "bytes_per_launch": alg_bytes, "ms_per_launch": main["kernel_ms"],
            },
            "clocks": clock_summary,
            **extras,
        }
        if world == 1 and not args.no_cpu_baseline:
            v, kind, sample, _, _ = cpu_pso_gens_per_s(args.workload, budget_s=15.0, steps=3, warmup=1, allow_full=False)
            line["cpu_baseline"] = {"value": v, "unit": "gens/s", "cores": torch.get_num_threads(), "kind": kind, "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_other(args):
    """Stand-alone runs of the secondary workloads (the commands the profiles were captured with)."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    cpu = not args.no_cpu_baseline
    w = args.workload
    if w == "microbench_compare":
        line = measure_compare_rate(dev)
    elif w.startswith("nds_rank_"):
        n = {"nds_rank_2e4": 20_000, "nds_rank_1e5": 100_000}[w]
        rate = None if args.no_secondary else measure_compare_rate(dev)["compares_per_s"]
        line = measure_nds(n, args.steps, dev, rate, cpu)
    elif w.startswith("rvea_"):
        line = measure_rvea({"rvea_config2": 50_000, "rvea_5e6": 5_000_000}[w], args.steps, dev, cpu)
    elif w == "lora_es_config3":
        line = measure_lora_es(args.steps, dev, pop=args.lora_pop, gradient_passes=args.gradient_passes)
    else:
        line = run_variant(args, dev)
    line = {"n_gpus": 1, "steps": args.steps, "warmup": 3, "data": "synthetic", "workload": w, **line}
    print(json.dumps(line), flush=True)


def run_variant(args, dev):
    """The PSO variants on Ackley at 1,000,000 x 1,000 (the headline swarm size), in-kernel Philox, fused
    evaluation; one step = StdWorkflow.step()."""
    from evox_b200.algorithms import CLPSO, CSO, DE, SLPSOGS
    from evox_b200.problems.numerical import Ackley
    from evox_b200.workflows import StdWorkflow

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
    with ClockSampler(0) as clocks:
        ms = timed_ms(wf.step, args.steps, warmup=max(args.warmup, 3))
    pk = peaks()
    return {
        "metric": f"{kind}_generations_per_s", "value": 1e3 / ms, "unit": "gens/s", "ms_per_step": ms, "higher_is_better": True,
        "dtype": "f32", "config": {"workload": args.workload, "pop_size": n, "dim": d, "l2": "state larger than L2"},
        "roofline": {"bound": "hbm", "kernel": kernel, "achieved": alg_bytes / (ms * 1e-3) / 1e9, "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": alg_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], "peak_kind": pk["kind"], "traffic": None},
        "clocks": clocks.summary(),
    }


def run_allgather(args):
    """NCCL allgather latency at 4 KB per rank, under torch.distributed.run."""
    import torch.distributed as dist

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    res = measure_allgather_latency(dev)
    if dist.get_rank() == 0:
        print(json.dumps({"workload": "nccl_allgather_4k", "n_gpus": dist.get_world_size(), **res}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="pso_ackley_1e6x1000", choices=sorted(WORKLOADS) + OTHER_WORKLOADS)
    ap.add_argument("--lora-pop", type=int, default=1024)
    ap.add_argument("--gradient-passes", type=int, default=3, choices=[1, 3, 6])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="only the headline workload (profiling runs)")
    ap.add_argument("--reference-budget-s", type=float, default=420.0,
                    help="time the reference arm may spend on its timed generations; the swarm is sampled to fit")
    args = ap.parse_args()
    if args.workload == "nccl_allgather_4k":
        run_allgather(args)
    elif args.workload in OTHER_WORKLOADS:
        run_other(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
