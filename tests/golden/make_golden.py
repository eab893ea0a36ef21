"""Generate the golden vectors under tests/golden/ by running the REFERENCE implementation.

Run in a container that has the reference checkout:
    python tests/golden/make_golden.py --reference <checkout>/src [--only pso,...]
The reference is imported from that path, run in eager mode on CPU (torch's own CPU kernels),
and its inputs / outputs are saved as small .npz files. The tests never import the reference;
they only read these files. Random draws the reference takes from torch's global generator
(`torch.rand` inside `PSO.step`) are replaced by recorded tensors so that the same draws can
be fed to the oracle and to the CUDA kernels.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _np(t):
    # a copy: some reference algorithms update their state tensors in place afterwards
    return t.detach().cpu().numpy().copy() if isinstance(t, torch.Tensor) else np.asarray(t)


def golden_pso(out: dict):
    """PSO.init_step + 3 teacher-forced steps on Ackley and Rastrigin, dims 12 (vector path)
    and 10 (scalar path); every state tensor before and after each step is stored."""
    from evox.algorithms import PSO
    from evox.problems.numerical import Ackley, Rastrigin
    from evox.workflows import StdWorkflow

    import evox.algorithms.so.pso_variants.pso as pso_mod

    names = ["pop", "velocity", "fit", "local_best_location", "local_best_fit", "global_best_location", "global_best_fit"]
    for prob_name, prob_cls, lo, hi, hyper in (
        ("ackley", Ackley, -32.768, 32.768, (0.6, 2.5, 0.8)),
        ("rastrigin", Rastrigin, -5.12, 5.12, (0.7, 1.5, 1.5)),
    ):
        for dim in (12, 10):
            pop_size = 37
            torch.manual_seed(1234 + dim)
            lb = torch.full((dim,), lo)
            ub = torch.full((dim,), hi)
            algo = PSO(pop_size, lb, ub, *hyper)
            # the benchmark configurations start with velocities in +-0.2 * range
            algo.velocity = 0.2 * algo.velocity
            wf = StdWorkflow(algo, prob_cls())
            tag = f"pso_{prob_name}_d{dim}"
            out[f"{tag}_hyper"] = np.asarray(hyper, dtype=np.float32)
            out[f"{tag}_bounds"] = np.asarray([lo, hi], dtype=np.float32)
            state0 = {k: v.clone() for k, v in wf.algorithm.state_dict().items()}
            for n in names:
                out[f"{tag}_s0_{n}"] = _np(state0[n])
            wf.init_step()
            for n in names:
                out[f"{tag}_s1_{n}"] = _np(wf.algorithm.state_dict()[n])
            gen = torch.Generator().manual_seed(99 + dim)
            for g in range(3):
                rg = torch.rand(pop_size, dim, generator=gen)
                rp = torch.rand(pop_size, dim, generator=gen)
                queue = [rg, rp]
                real_rand = torch.rand

                def fake_rand(*a, **k):
                    return queue.pop(0)

                pso_mod.torch.rand = fake_rand
                try:
                    wf.step()
                finally:
                    pso_mod.torch.rand = real_rand
                assert not queue
                out[f"{tag}_g{g}_rg"] = _np(rg)
                out[f"{tag}_g{g}_rp"] = _np(rp)
                for n in names:
                    out[f"{tag}_s{g + 2}_{n}"] = _np(wf.algorithm.state_dict()[n])


def nds_cases():
    """Inputs of the NSGA-II selection goldens (shared with the tests through the .npz)."""
    g = torch.Generator().manual_seed(7)
    cases = {}
    x = torch.rand(300, 12, generator=g)
    from evox.problems.numerical import DTLZ2

    cases["dtlz2"] = (DTLZ2(d=12, m=3).evaluate(x), 150)
    cases["ties_m2"] = (torch.round(torch.rand(257, 2, generator=g) * 8) / 8, 100)
    f = torch.rand(130, 5, generator=g)
    f[3, 1] = float("nan")
    f[77] = float("nan")
    f[12, 0] = float("inf")
    f[13, 4] = float("-inf")
    cases["nan_m5"] = (f, 64)
    f = torch.rand(64, 3, generator=g)
    f[:, 1] = 0.5
    cases["flat_objective"] = (f, 20)
    cases["single_front"] = (torch.stack([torch.linspace(0, 1, 40), torch.linspace(1, 0, 40)], dim=1), 17)
    cases["tiny"] = (torch.tensor([[1.0, 2.0], [2.0, 1.0], [3.0, 3.0]]), 2)
    return cases


def golden_nds(out: dict):
    """non_dominate_rank, crowding_distance on the last selected front and
    nd_environmental_selection (x = row index, so the selected order is visible)."""
    from evox.operators.selection import crowding_distance, nd_environmental_selection, non_dominate_rank

    for name, (f, topk) in nds_cases().items():
        n = f.shape[0]
        rank = non_dominate_rank(f)
        worst = torch.topk(rank, topk, largest=False)[0][-1]
        mask = rank == worst
        crowd = crowding_distance(f, mask)
        x = torch.arange(n, dtype=torch.float32)[:, None].repeat(1, 2)
        sx, sf, srank, scrowd = nd_environmental_selection(x, f, topk)
        out[f"{name}_f"] = _np(f)
        out[f"{name}_topk"] = np.asarray(topk)
        out[f"{name}_rank"] = _np(rank)
        out[f"{name}_mask"] = _np(mask)
        out[f"{name}_crowd"] = _np(crowd)
        out[f"{name}_sel_index"] = _np(sx[:, 0].to(torch.int64))
        out[f"{name}_sel_f"] = _np(sf)
        out[f"{name}_sel_rank"] = _np(srank)
        out[f"{name}_sel_crowd"] = _np(scrowd)


def golden_rvea(out: dict):
    """ref_vec_guided on (a) the shape of the reference's own unit test (12 x 4, 5 vectors, one
    NaN row), (b) 10 objectives with the 275 two-layer lattice vectors, (c) 3 objectives."""
    from evox.operators.sampling import uniform_sampling
    from evox.operators.selection import ref_vec_guided

    g = torch.Generator().manual_seed(21)
    cases = {}
    f = torch.rand(12, 4, generator=g)
    f[5] = float("nan")
    cases["unit"] = (torch.rand(12, 6, generator=g), f, torch.rand(5, 4, generator=g), torch.tensor(0.5))
    f = torch.rand(600, 10, generator=g) + 0.05 * torch.randn(600, 10, generator=g).abs()
    cases["m10"] = (torch.rand(600, 19, generator=g), f, uniform_sampling(275, 10)[0], torch.tensor(0.25))
    f = torch.rand(400, 3, generator=g)
    f[17, 1] = float("nan")
    cases["m3"] = (torch.rand(400, 5, generator=g), f, uniform_sampling(28, 3)[0], torch.tensor(0.81))
    for name, (x, f, v, theta) in cases.items():
        nx, nf = ref_vec_guided(x, f, v, theta)
        out[f"{name}_x"], out[f"{name}_f"], out[f"{name}_v"], out[f"{name}_theta"] = _np(x), _np(f), _np(v), _np(theta)
        out[f"{name}_next_x"], out[f"{name}_next_f"] = _np(nx), _np(nf)


def golden_es(out: dict):
    """Philox streams, LoRA factors / delta / gradient, one VirtualLoRAES step and one OpenES step."""
    from evox.algorithms import OpenES
    from evox.algorithms.so.es_variants.virtual_lora_es import VirtualLoRAES
    from evox.triton_kernels.kernels.lora_noise import (
        compute_counter_offsets, generate_lora_factors, lora_delta_output, lora_gradient)
    from evox.triton_kernels.kernels.philox import philox_normal, philox_uniform

    g = torch.Generator().manual_seed(5)
    seeds = torch.randint(0, 2**31, (6,), generator=g, dtype=torch.int64)
    seeds[1] = (3 << 32) + 12345  # exercises the high key word
    out["seeds"] = _np(seeds)
    for n, counter in ((10, 0), (7, 5), (64, (1 << 31) - 40), (33, (7 << 32) + 9)):
        out[f"uniform_n{n}_c{counter}"] = _np(philox_uniform(seeds, n, counter))
        out[f"normal_n{n}_c{counter}"] = _np(philox_normal(seeds, n, counter))
    shapes = [(10,), (4, 3), (2, 5)]
    out["offsets_kat"] = np.asarray(compute_counter_offsets(shapes, 2))  # == [0, 12, 28] in the reference's test
    a, b = generate_lora_factors(seeds, (12, 20), 4, 40)
    out["factors_A"], out["factors_B"] = _np(a), _np(b)
    x = torch.randn(6, 5, 20, generator=g)
    out["delta_x"] = _np(x)
    out["delta_out"] = _np(lora_delta_output(x, a, b, 0.1))
    fit = torch.randn(6, generator=g)
    out["grad_fitness"] = _np(fit)
    out["grad_out"] = _np(lora_gradient(fit, a, b, 6, 0.1, (12, 20)))
    noise = generate_lora_factors(seeds, (9,), 4, 3)
    out["bias_noise"] = _np(noise)
    out["grad_bias"] = _np(lora_gradient(fit, noise, None, 6, 0.1, (9,)))

    # VirtualLoRAES.step with the seeds fixed and a quadratic fitness on the perturbed weights
    import evox.algorithms.so.es_variants.virtual_lora_es as vmod

    shapes = [(8, 6), (8,), (3, 8), (3,)]
    dim = sum(int(np.prod(s)) for s in shapes)
    for opt in (None, "adam"):
        center = torch.randn(dim, generator=g) * 0.3
        algo = VirtualLoRAES(shapes, 2, 10, center.clone(), 0.05, 0.1, optimizer=opt)
        step_seeds = torch.randint(0, 2**31, (10,), generator=g, dtype=torch.int64)
        fitness = torch.randn(10, generator=g)
        algo.evaluate = lambda payload, fitness=fitness: fitness
        real = vmod.torch.randint
        vmod.torch.randint = lambda *a, **k: step_seeds
        try:
            algo.step()
        finally:
            vmod.torch.randint = real
        tag = f"vlora_{opt}"
        out[f"{tag}_center0"], out[f"{tag}_seeds"], out[f"{tag}_fitness"] = _np(center), _np(step_seeds), _np(fitness)
        out[f"{tag}_center1"] = _np(algo.center)
        if opt:
            out[f"{tag}_exp_avg"], out[f"{tag}_exp_avg_sq"] = _np(algo.exp_avg), _np(algo.exp_avg_sq)

    # OpenES.step with the normal draws fixed, sphere fitness
    import evox.algorithms.so.es_variants.open_es as omod

    for opt in (None, "adam"):
        center = torch.randn(12, generator=g)
        algo = OpenES(8, center.clone(), 0.05, 0.1, optimizer=opt)
        noise = torch.randn(4, 12, generator=g)
        algo.evaluate = lambda pop: (pop**2).sum(dim=1)
        real = omod.torch.randn
        omod.torch.randn = lambda *a, **k: noise
        try:
            algo.step()
        finally:
            omod.torch.randn = real
        tag = f"openes_{opt}"
        out[f"{tag}_center0"], out[f"{tag}_noise"], out[f"{tag}_center1"] = _np(center), _np(noise), _np(algo.center)


def golden_variation(out: dict):
    """tournament_selection_multifit, simulated_binary and polynomial_mutation with their random
    draws replaced by recorded tensors (queued in the order the reference draws them)."""
    import evox.operators.crossover.sbx as sbx_mod
    import evox.operators.mutation.pm_mutation as pm_mod
    import evox.operators.selection  # noqa: F401  (the package re-exports a function under the module's name)

    ts_mod = sys.modules["evox.operators.selection.tournament_selection"]

    g = torch.Generator().manual_seed(77)

    def with_queue(mod, rands, ints, fn):
        rq, iq = list(rands), list(ints)
        real_rand, real_randint = mod.torch.rand, mod.torch.randint
        mod.torch.rand = lambda *a, **k: rq.pop(0)
        mod.torch.randint = lambda *a, **k: iq.pop(0)
        try:
            res = fn()
        finally:
            mod.torch.rand, mod.torch.randint = real_rand, real_randint
        assert not rq and not iq
        return res

    n, d = 40, 7
    lb, ub = torch.full((d,), -1.0), torch.linspace(1.0, 3.0, d)
    x = lb + (ub - lb) * torch.rand(n, d, generator=g)
    x[3, 2] = 5.0  # outside the box: exercises the clamps inside the mutation
    h = n // 2
    mu, sign = torch.rand(h, d, generator=g), torch.randint(0, 2, (h, d), generator=g)
    r_half, r_pc = torch.rand(h, d, generator=g), torch.rand(h, d, generator=g)
    crossed = with_queue(sbx_mod, [mu, r_half, r_pc], [sign], lambda: sbx_mod.simulated_binary(x))
    site = torch.rand(n, d, generator=g) * 0.5  # pro_m / d = 1/7: make mutation sites common
    pmu = torch.rand(n, d, generator=g)
    mutated = with_queue(pm_mod, [site, pmu], [], lambda: pm_mod.polynomial_mutation(crossed, lb, ub))
    for k, v in dict(x=x, lb=lb, ub=ub, sbx_mu=mu, sbx_sign=sign, sbx_half=r_half, sbx_pc=r_pc, crossed=crossed,
                     pm_site=site, pm_mu=pmu, mutated=mutated).items():
        out[f"var_{k}"] = _np(v)

    rank = torch.randint(0, 4, (n,), generator=g).float()
    dis = torch.rand(n, generator=g)
    dis[::5] = float("inf")
    parents = torch.randint(0, n, (n, 2), generator=g)
    picked = with_queue(ts_mod, [], [parents], lambda: ts_mod.tournament_selection_multifit(n, [-dis, rank]))
    out["ts_rank"], out["ts_dis"], out["ts_parents"], out["ts_selected"] = _np(rank), _np(dis), _np(parents), _np(picked)


def golden_cso(out: dict):
    """CSO.init_step + 3 teacher-forced steps (randperm and the three lambda draws recorded) on Ackley
    and Sphere, dims 12 and 10, 38 particles, phi 0.1; pop / fit / velocity after every step."""
    from evox.algorithms import CSO
    from evox.problems.numerical import Ackley, Sphere
    from evox.workflows import StdWorkflow

    import evox.algorithms.so.pso_variants.cso as cso_mod

    names = ["pop", "fit", "velocity"]
    for prob_name, prob_cls, lo, hi in (("ackley", Ackley, -32.768, 32.768), ("sphere", Sphere, -5.0, 7.0)):
        for dim in (12, 10):
            pop_size, phi = 38, 0.1
            torch.manual_seed(4321 + dim)
            algo = CSO(pop_size, torch.full((dim,), lo), torch.full((dim,), hi), phi=phi)
            wf = StdWorkflow(algo, prob_cls())
            tag = f"cso_{prob_name}_d{dim}"
            out[f"{tag}_phi"] = np.asarray(phi, dtype=np.float32)
            out[f"{tag}_bounds"] = np.asarray([lo, hi], dtype=np.float32)
            for n in names:
                out[f"{tag}_s0_{n}"] = _np(wf.algorithm.state_dict()[n])
            wf.init_step()
            for n in names:
                out[f"{tag}_s1_{n}"] = _np(wf.algorithm.state_dict()[n])
            gen = torch.Generator().manual_seed(77 + dim)
            for g in range(3):
                perm = torch.randperm(pop_size, generator=gen)
                lambdas = torch.rand(3, pop_size // 2, dim, generator=gen)
                real_rand, real_perm = torch.rand, torch.randperm
                cso_mod.torch.rand = lambda *a, **k: lambdas
                cso_mod.torch.randperm = lambda *a, **k: perm
                try:
                    wf.step()
                finally:
                    cso_mod.torch.rand, cso_mod.torch.randperm = real_rand, real_perm
                out[f"{tag}_g{g}_perm"] = _np(perm)
                out[f"{tag}_g{g}_lambdas"] = _np(lambdas)
                for n in names:
                    out[f"{tag}_s{g + 2}_{n}"] = _np(wf.algorithm.state_dict()[n])


def golden_ars(out: dict):
    """ARS.step (es_variants/ars.py:62-98) with the normal draws fixed, a shifted-sphere fitness, SGD and Adam,
    two consecutive steps each (the second exercises the optimiser state)."""
    from evox.algorithms import ARS

    import evox.algorithms.so.es_variants.ars as amod

    g = torch.Generator().manual_seed(2468)
    shift = torch.randn(24, generator=g)
    for opt in (None, "adam"):
        center = torch.randn(24, generator=g)
        algo = ARS(16, center.clone(), elite_ratio=0.5, lr=0.05, sigma=0.1, optimizer=opt)
        algo.evaluate = lambda pop: ((pop - shift) ** 2).sum(dim=1)
        tag = f"ars_{opt}"
        out[f"{tag}_center0"], out[f"{tag}_shift"] = _np(center), _np(shift)
        for k in range(2):
            z = torch.randn(8, 24, generator=g)
            real = amod.torch.randn
            amod.torch.randn = lambda *a, **kw: z
            try:
                algo.step()
            finally:
                amod.torch.randn = real
            out[f"{tag}_z{k}"], out[f"{tag}_center{k + 1}"] = _np(z), _np(algo.center)
        if opt:
            out[f"{tag}_exp_avg"], out[f"{tag}_exp_avg_sq"] = _np(algo.exp_avg), _np(algo.exp_avg_sq)


def golden_clpso(out: dict):
    """CLPSO.init_step + 3 teacher-forced steps (the four draws of clpso.py:92-95 recorded) on Ackley and
    Sphere, dims 12 and 10, 37 particles, learning probability 0.3; all state after every step."""
    from evox.algorithms import CLPSO
    from evox.problems.numerical import Ackley, Sphere
    from evox.workflows import StdWorkflow

    import evox.algorithms.so.pso_variants.clpso as cmod

    names = ["pop", "fit", "velocity", "personal_best_location", "personal_best_fit", "global_best_location", "global_best_fit"]
    for prob_name, prob_cls, lo, hi in (("ackley", Ackley, -32.768, 32.768), ("sphere", Sphere, -5.0, 7.0)):
        for dim in (12, 10):
            pop_size = 37
            torch.manual_seed(999 + dim)
            algo = CLPSO(pop_size, torch.full((dim,), lo), torch.full((dim,), hi), 0.5, 1.5, 0.3)
            algo.velocity = 0.2 * algo.velocity
            wf = StdWorkflow(algo, prob_cls())
            tag = f"clpso_{prob_name}_d{dim}"
            out[f"{tag}_bounds"] = np.asarray([lo, hi], dtype=np.float32)
            for n in names:
                out[f"{tag}_s0_{n}"] = _np(wf.algorithm.state_dict()[n])
            wf.init_step()
            for n in names:
                out[f"{tag}_s1_{n}"] = _np(wf.algorithm.state_dict()[n])
            gen = torch.Generator().manual_seed(55 + dim)
            for g in range(3):
                coeff = torch.rand(pop_size, dim, generator=gen)
                i1 = torch.randint(0, pop_size, (pop_size,), generator=gen)
                i2 = torch.randint(0, pop_size, (pop_size,), generator=gen)
                poss = torch.rand(pop_size, generator=gen)
                rq, iq = [coeff, poss], [i1, i2]
                real_rand, real_randint = torch.rand, torch.randint
                cmod.torch.rand = lambda *a, **k: rq.pop(0)
                cmod.torch.randint = lambda *a, **k: iq.pop(0)
                try:
                    wf.step()
                finally:
                    cmod.torch.rand, cmod.torch.randint = real_rand, real_randint
                assert not rq and not iq
                out[f"{tag}_g{g}_coeff"], out[f"{tag}_g{g}_i1"], out[f"{tag}_g{g}_i2"], out[f"{tag}_g{g}_poss"] = _np(coeff), _np(i1), _np(i2), _np(poss)
                for n in names:
                    out[f"{tag}_s{g + 2}_{n}"] = _np(wf.algorithm.state_dict()[n])


def golden_pes(out: dict):
    """PersistentES.step (es_variants/persistent_es.py:74-112) with the normal draws fixed: four steps with
    T = 3 K (the accumulator resets after the third), sigma decay 0.9, SGD and Adam."""
    from evox.algorithms import PersistentES

    import evox.algorithms.so.es_variants.persistent_es as pmod

    g = torch.Generator().manual_seed(1357)
    shift = torch.randn(20, generator=g)
    for opt in (None, "adam"):
        center = torch.randn(20, generator=g)
        algo = PersistentES(12, center.clone(), optimizer=opt, lr=0.05, sigma=0.1, T=30, K=10, sigma_decay=0.9, sigma_limit=0.075)
        algo.evaluate = lambda pop: ((pop - shift) ** 2).sum(dim=1)
        tag = f"pes_{opt}"
        out[f"{tag}_center0"], out[f"{tag}_shift"] = _np(center), _np(shift)
        for k in range(4):
            z = torch.randn(6, 20, generator=g)
            real = pmod.torch.randn
            pmod.torch.randn = lambda *a, **kw: z
            try:
                algo.step()
            finally:
                pmod.torch.randn = real
            out[f"{tag}_z{k}"], out[f"{tag}_center{k + 1}"] = _np(z), _np(algo.center)
            out[f"{tag}_accum{k + 1}"], out[f"{tag}_sigma{k + 1}"] = _np(algo.pert_accum), _np(algo.sigma)
            out[f"{tag}_counter{k + 1}"] = _np(algo.inner_step_counter)


def golden_slpso(out: dict):
    """SLPSOGS / SLPSOUS: init_step + 3 teacher-forced steps (the demonstrator draw and r1, r2, r3 recorded)
    on Ackley, dims 12 and 10, 33 particles; all state after every step."""
    from evox.algorithms import SLPSOGS, SLPSOUS
    from evox.problems.numerical import Ackley
    from evox.workflows import StdWorkflow

    import evox.algorithms.so.pso_variants.sl_pso_gs as gmod
    import evox.algorithms.so.pso_variants.sl_pso_us as umod

    names = ["pop", "fit", "velocity", "global_best_location", "global_best_fit"]
    for kind, cls, mod in (("gs", SLPSOGS, gmod), ("us", SLPSOUS, umod)):
        for dim in (12, 10):
            pop_size, lo, hi = 33, -32.768, 32.768
            torch.manual_seed(31 + dim)
            algo = cls(pop_size, torch.full((dim,), lo), torch.full((dim,), hi), 0.2, 0.7)
            algo.velocity = 0.2 * algo.velocity
            wf = StdWorkflow(algo, Ackley())
            tag = f"slpso_{kind}_d{dim}"
            out[f"{tag}_bounds"] = np.asarray([lo, hi], dtype=np.float32)
            for n in names:
                out[f"{tag}_s0_{n}"] = _np(wf.algorithm.state_dict()[n])
            wf.init_step()
            for n in names:
                out[f"{tag}_s1_{n}"] = _np(wf.algorithm.state_dict()[n])
            gen = torch.Generator().manual_seed(17 + dim)
            for g in range(3):
                pick = torch.randn(pop_size, generator=gen) if kind == "gs" else torch.rand(pop_size, generator=gen)
                rs = [torch.rand(pop_size, dim, generator=gen) for _ in range(3)]
                # sl_pso_gs.py draws randn (demonstrator) then three rand; sl_pso_us.py draws rand (demonstrator) then three
                nq = [pick] if kind == "gs" else []
                uq = list(rs) if kind == "gs" else [pick] + list(rs)
                real_rand, real_randn = torch.rand, torch.randn
                mod.torch.rand = lambda *a, **k: uq.pop(0)
                mod.torch.randn = lambda *a, **k: nq.pop(0)
                try:
                    wf.step()
                finally:
                    mod.torch.rand, mod.torch.randn = real_rand, real_randn
                assert not nq and not uq
                out[f"{tag}_g{g}_pick"] = _np(pick)
                for j in range(3):
                    out[f"{tag}_g{g}_r{j + 1}"] = _np(rs[j])
                for n in names:
                    out[f"{tag}_s{g + 2}_{n}"] = _np(wf.algorithm.state_dict()[n])


def golden_rveaa(out: dict):
    """RVEAa's own pieces (algorithms/mo/rveaa.py:129-164): `_rv_regeneration` (the uniform draw recorded) and
    `_batch_truncation`, on objective sets with NaN rows as RVEA selection produces them."""
    from evox.algorithms import RVEAa

    import evox.algorithms.mo.rveaa as rmod

    g = torch.Generator().manual_seed(4242)
    algo = RVEAa(28, 3, torch.zeros(6), torch.ones(6))
    n = algo.pop_size
    obj = torch.rand(2 * n, 3, generator=g) + 0.1
    obj[torch.tensor([1, 5, 17, 30])] = float("nan")
    v = torch.rand(n, 3, generator=g)
    v[3] = torch.tensor([1.0, 0.0, 0.0]) * 1e-3  # a direction nobody is closest to is likely; keep a few odd ones
    draw = torch.rand(n, 3, generator=g)
    real = rmod.torch.rand
    rmod.torch.rand = lambda *a, **k: draw
    try:
        new_v = algo._rv_regeneration(obj, v)
    finally:
        rmod.torch.rand = real
    out["regen_obj"], out["regen_v"], out["regen_draw"], out["regen_new_v"] = _np(obj), _np(v), _np(draw), _np(new_v)
    pop = torch.rand(2 * n, 6, generator=g)
    pop[torch.isnan(obj).all(dim=1)] = float("nan")
    new_pop, new_obj = algo._batch_truncation(pop, obj)
    out["trunc_pop"], out["trunc_new_pop"], out["trunc_new_obj"] = _np(pop), _np(new_pop), _np(new_obj)


def golden_de(out: dict):
    """DE.init_step + 3 teacher-forced steps (index draws, crossover draws and forced dimensions recorded) with
    base vector "rand" and "best", one difference vector, on Ackley, dims 12 and 10, 29 individuals."""
    from evox.algorithms import DE
    from evox.problems.numerical import Ackley
    from evox.workflows import StdWorkflow

    import evox.algorithms.so.de_variants.de as dmod

    for base in ("rand", "best"):
        for dim in (12, 10):
            pop_size, lo, hi = 29, -32.768, 32.768
            torch.manual_seed(77 + dim)
            algo = DE(pop_size, torch.full((dim,), lo), torch.full((dim,), hi), base_vector=base, differential_weight=0.6,
                      cross_probability=0.7)
            wf = StdWorkflow(algo, Ackley())
            tag = f"de_{base}_d{dim}"
            out[f"{tag}_bounds"] = np.asarray([lo, hi], dtype=np.float32)
            out[f"{tag}_s0_pop"] = _np(wf.algorithm.state_dict()["pop"])
            wf.init_step()
            out[f"{tag}_s1_pop"], out[f"{tag}_s1_fit"] = _np(wf.algorithm.state_dict()["pop"]), _np(wf.algorithm.state_dict()["fit"])
            gen = torch.Generator().manual_seed(5 + dim)
            n_idx = 3 if base == "rand" else 2
            for g in range(3):
                idx = [torch.randint(0, pop_size, (pop_size,), generator=gen) for _ in range(n_idx)]
                cross = torch.rand(pop_size, dim, generator=gen)
                forced = torch.randint(0, dim, (pop_size, 1), generator=gen)
                iq, rq = list(idx) + [forced], [cross]
                real_rand, real_randint = torch.rand, torch.randint
                dmod.torch.rand = lambda *a, **k: rq.pop(0)
                dmod.torch.randint = lambda *a, **k: iq.pop(0)
                try:
                    wf.step()
                finally:
                    dmod.torch.rand, dmod.torch.randint = real_rand, real_randint
                assert not iq and not rq
                for j, t_ in enumerate(idx):
                    out[f"{tag}_g{g}_idx{j}"] = _np(t_)
                out[f"{tag}_g{g}_cross"], out[f"{tag}_g{g}_forced"] = _np(cross), _np(forced)
                out[f"{tag}_s{g + 2}_pop"], out[f"{tag}_s{g + 2}_fit"] = _np(wf.algorithm.state_dict()["pop"]), _np(wf.algorithm.state_dict()["fit"])


def golden_snes_des(out: dict):
    """SNES.step (both weight types) and DES.step with the normal draws fixed: three generations each on a
    shifted sphere; centre and sigma after every step."""
    from evox.algorithms import DES, SNES

    import evox.algorithms.so.es_variants.des as dmod
    import evox.algorithms.so.es_variants.snes as smod

    g = torch.Generator().manual_seed(8642)
    shift = torch.randn(18, generator=g)
    cases = [("snes_temp", lambda c: SNES(14, c, sigma=0.5, weight_type="temp"), smod),
             ("snes_recomb", lambda c: SNES(14, c, sigma=0.5, weight_type="recomb"), smod),
             ("des", lambda c: DES(14, c, sigma_init=0.3), dmod)]
    for tag, make, mod in cases:
        center = torch.randn(18, generator=g)
        algo = make(center.clone())
        algo.evaluate = lambda pop: ((pop - shift) ** 2).sum(dim=1)
        out[f"{tag}_center0"], out[f"{tag}_shift"] = _np(center), _np(shift)
        for k in range(3):
            z = torch.randn(14, 18, generator=g)
            real = mod.torch.randn
            mod.torch.randn = lambda *a, **kw: z
            try:
                algo.step()
            finally:
                mod.torch.randn = real
            out[f"{tag}_z{k}"], out[f"{tag}_center{k + 1}"], out[f"{tag}_sigma{k + 1}"] = _np(z), _np(algo.center), _np(algo.sigma)


def golden_hype(out: dict):
    """cal_hv (algorithms/mo/hype.py:12-39) with its uniform draw recorded, on objective sets with duplicates
    and with the population size given as a tensor (as the second call of HypE.step does); then HypE.init_step
    and two teacher-forced HypE.step on DTLZ2 (every rand / randint result recorded in call order)."""
    import evox.algorithms.mo.hype as hmod
    from evox.problems.numerical import DTLZ2
    from evox.workflows import StdWorkflow

    g = torch.Generator().manual_seed(909)
    cases = {"m3": (60, 3, 30, 500), "m2_tensor": (45, 2, torch.tensor(20), 300), "m6": (33, 6, 11, 257), "dup": (40, 3, 25, 400)}
    for tag, (n, m, pop_size, n_sample) in cases.items():
        fit = torch.rand(n, m, generator=g)
        if tag == "dup":
            fit = torch.round(fit * 4) / 4
        ref = torch.full((m,), float(fit.max()) * 1.2)
        draw = torch.rand(n_sample, m, generator=g)
        real = torch.rand
        hmod.torch.rand = lambda *a, **k: draw
        try:
            hv = hmod.cal_hv(fit, ref, pop_size, n_sample)
        finally:
            hmod.torch.rand = real
        out[f"hv_{tag}_fit"], out[f"hv_{tag}_ref"], out[f"hv_{tag}_draw"], out[f"hv_{tag}_out"] = _np(fit), _np(ref), _np(draw), _np(hv)
        out[f"hv_{tag}_pop_size"] = np.asarray(int(pop_size))

    pop_size, d, m, n_sample = 24, 8, 3, 300
    torch.manual_seed(31)
    algo = hmod.HypE(pop_size, m, torch.zeros(d), torch.ones(d), n_sample=n_sample)
    wf = StdWorkflow(algo, DTLZ2(d=d, m=m))
    out["step_s0_pop"] = _np(wf.algorithm.state_dict()["pop"])
    wf.init_step()
    out["step_s1_fit"], out["step_ref"] = _np(wf.algorithm.state_dict()["fit"]), _np(wf.algorithm.state_dict()["ref"])
    h = pop_size // 2
    for it in range(2):
        rec = {
            "samples_a": torch.rand(n_sample, m, generator=g), "parents": torch.randint(0, pop_size, (pop_size, 2), generator=g),
            "sbx_mu": torch.rand(h, d, generator=g), "sbx_sign": torch.randint(0, 2, (h, d), generator=g),
            "sbx_half": torch.rand(h, d, generator=g), "sbx_pc": torch.rand(h, d, generator=g),
            "pm_site": torch.rand(pop_size, d, generator=g) * 0.5, "pm_mu": torch.rand(pop_size, d, generator=g),
            "samples_b": torch.rand(n_sample, m, generator=g),
        }
        rq = [rec[k] for k in ("samples_a", "sbx_mu", "sbx_half", "sbx_pc", "pm_site", "pm_mu", "samples_b")]
        iq = [rec["parents"], rec["sbx_sign"]]
        real_rand, real_randint = torch.rand, torch.randint
        hmod.torch.rand = lambda *a, **k: rq.pop(0)
        hmod.torch.randint = lambda *a, **k: iq.pop(0)
        try:
            wf.step()
        finally:
            hmod.torch.rand, hmod.torch.randint = real_rand, real_randint
        assert not rq and not iq
        for k, v in rec.items():
            out[f"step_g{it}_{k}"] = _np(v)
        out[f"step_g{it}_pop"], out[f"step_g{it}_fit"] = _np(wf.algorithm.state_dict()["pop"]), _np(wf.algorithm.state_dict()["fit"])


def golden_nsga3(out: dict):
    """NSGA3.step (algorithms/mo/nsga3.py:155-266) on DTLZ2, the environmental part in isolation: per recorded
    generation the state before the step, the offspring and their objectives (taken at the `evaluate` call),
    the two permutations the step draws (merged population, reference points), and the state after it."""
    import evox.algorithms.mo.nsga3 as nmod
    from evox.problems.numerical import DTLZ2
    from evox.workflows import StdWorkflow

    for tag, (pop_size, d, m, gens, seed) in {"m3": (60, 12, 3, 4, 11), "m4": (84, 9, 4, 3, 12), "m2": (30, 6, 2, 3, 13)}.items():
        torch.manual_seed(seed)
        algo = nmod.NSGA3(pop_size, m, torch.zeros(d), torch.ones(d))
        wf = StdWorkflow(algo, DTLZ2(d=d, m=m))
        wf.init_step()
        out[f"{tag}_ref"] = _np(wf.algorithm.ref)
        out[f"{tag}_gens"] = np.asarray(gens)
        out[f"{tag}_pop_size"] = np.asarray(pop_size)  # the population itself may hold fewer rows (see oracle/nsga3.py)
        for g in range(gens):
            st = wf.algorithm.state_dict()
            out[f"{tag}_g{g}_pop"], out[f"{tag}_g{g}_fit"], out[f"{tag}_g{g}_rank"] = _np(st["pop"]), _np(st["fit"]), _np(st["rank"])
            perms, evals = [], []
            real_randperm, real_eval = torch.randperm, wf.algorithm.evaluate

            def randperm(*a, **k):
                perms.append(real_randperm(*a, **k))
                return perms[-1]

            def evaluate(x):
                f = real_eval(x)
                evals.append((x.clone(), f.clone()))
                return f

            nmod.torch.randperm = randperm
            wf.algorithm.evaluate = evaluate
            try:
                wf.step()
            finally:
                nmod.torch.randperm = real_randperm
                wf.algorithm.evaluate = real_eval
            assert len(perms) == 2 and len(evals) == 1
            out[f"{tag}_g{g}_offspring"], out[f"{tag}_g{g}_off_fit"] = _np(evals[0][0]), _np(evals[0][1])
            out[f"{tag}_g{g}_perm_merge"], out[f"{tag}_g{g}_perm_ref"] = _np(perms[0]), _np(perms[1])
            st = wf.algorithm.state_dict()
            out[f"{tag}_g{g}_next_pop"], out[f"{tag}_g{g}_next_fit"], out[f"{tag}_g{g}_next_rank"] = _np(st["pop"]), _np(st["fit"]), _np(st["rank"])


def golden_nds_large(out: dict):
    """Ranks at the sizes the benchmark quotes. 2N = 20,000 (benchmark configuration 1) comes from the reference
    itself (about 3 GB of temporaries and half a minute on CPU). 2N = 100,000 is beyond what the reference can
    hold (two (n, n, 3) boolean tensors = 60 GB): its ranks come from the blocked, bit-packed restatement in
    oracle/nds.py, which is first required to reproduce the reference's ranks at 20,000 bit for bit. The
    objectives are stored with the ranks because DTLZ2's sines and cosines may round differently on another
    host. Takes a few minutes; not part of a default run (ask for it with --only nds_large)."""
    from evox.operators.selection import non_dominate_rank

    sys.path.insert(0, str(HERE.parent.parent))
    from oracle import nds as onds

    for tag, n in (("config1", 20_000), ("metric", 100_000)):
        x = torch.rand(n, 12, generator=torch.Generator().manual_seed(0))
        f = onds.dtlz2_objectives(x, 3)
        if n <= 20_000:
            rank = non_dominate_rank(f)
            assert torch.equal(onds.non_dominate_rank(f), rank), "the restatement must reproduce the reference first"
        else:
            rank = onds.non_dominate_rank(f)
        assert int(rank.max()) < 127
        out[f"{tag}_f"] = _np(f)
        out[f"{tag}_rank"] = _np(rank).astype(np.int8)


GENERATORS = {"pso": golden_pso, "nds": golden_nds, "rvea": golden_rvea, "es": golden_es, "variation": golden_variation,
              "cso": golden_cso, "ars": golden_ars, "clpso": golden_clpso, "pes": golden_pes, "slpso": golden_slpso, "rveaa": golden_rveaa, "de": golden_de, "snes_des": golden_snes_des, "hype": golden_hype,
              "nsga3": golden_nsga3, "nds_large": golden_nds_large}
SLOW = {"nds_large"}  # only when named in --only


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="the src/ directory of an EMI-Group/evox checkout")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    torch.set_default_device("cpu")
    only = [s for s in args.only.split(",") if s]
    for name, fn in GENERATORS.items():
        if (only and name not in only) or (not only and name in SLOW):
            continue
        data: dict = {}
        fn(data)
        path = HERE / f"{name}.npz"
        np.savez_compressed(path, **data)
        print(f"wrote {path} ({path.stat().st_size} bytes, {len(data)} arrays)")


if __name__ == "__main__":
    main()
