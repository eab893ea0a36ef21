"""Mating selection, crossover and mutation on the CUDA kernels, with the reference's names and
arguments (evox/operators/selection/tournament_selection.py, crossover/sbx.py,
mutation/pm_mutation.py). Each function takes its random draws from torch's generator exactly as the
reference does unless they are passed in; `make_offspring` is the fused crossover + mutation + clamp
that NSGA2 / RVEA use."""

from __future__ import annotations

import torch

from .. import _cabi

__all__ = ["tournament_selection", "tournament_selection_multifit", "simulated_binary", "polynomial_mutation", "make_offspring"]

CROSSOVER, MUTATION, CLAMP = 1, 2, 4


def tournament_selection_multifit(n_round: int, fitnesses: list[torch.Tensor], tournament_size: int = 2,
                                  parents: torch.Tensor | None = None) -> torch.Tensor:
    fit = torch.stack([f.to(torch.float32) for f in fitnesses], dim=1).contiguous()
    dev = fit.device
    if parents is None:
        parents = torch.randint(0, fit.shape[0], (n_round, tournament_size), device=dev)
    parents = parents.to(torch.int64).contiguous()
    out = torch.empty(n_round, dtype=torch.int64, device=dev)
    _cabi.check(_cabi.lib.evox_tournament_multifit(_cabi.ptr(parents), n_round, tournament_size, _cabi.ptr(fit), fit.shape[0],
                                                   fit.shape[1], _cabi.ptr(out), _cabi.stream_ptr(dev)))
    return out


def tournament_selection(n_round: int, fitness: torch.Tensor, tournament_size: int = 2, parents: torch.Tensor | None = None) -> torch.Tensor:
    """The candidate with the smallest fitness of each round, the first one on ties
    (tournament_selection.py:32-54): the multi-key kernel with one key."""
    return tournament_selection_multifit(n_round, [fitness], tournament_size, parents)


def make_offspring(pop: torch.Tensor, lb: torch.Tensor, ub: torch.Tensor, mating_pool: torch.Tensor | None = None,
                   draws: dict | None = None, pro_c: float = 1.0, dis_c: float = 20.0, pro_m: float = 1.0, dis_m: float = 20.0,
                   flags: int = CROSSOVER | MUTATION | CLAMP, seed: int = 0, generation: int = 0) -> torch.Tensor:
    """clamp(polynomial_mutation(simulated_binary(pop[mating_pool]))) in one kernel. `draws`: dict with
    sbx_mu, sbx_sign, sbx_half, sbx_pc, pm_site, pm_mu (the reference's draws); None = Philox(seed, generation).
    Goes through the registered operator `evox_b200::offspring`, so a traced generation keeps it as one node."""
    from .. import ops

    d = draws or {}
    return ops.offspring(pop, lb, ub, mating_pool, d.get("sbx_mu"), d.get("sbx_sign"), d.get("sbx_half"), d.get("sbx_pc"),
                         d.get("pm_site"), d.get("pm_mu"), float(pro_c), float(dis_c), float(pro_m), float(dis_m), int(flags),
                         int(seed), int(generation))


def _make_offspring(pop, lb, ub, mating_pool, draws, pro_c, dis_c, pro_m, dis_m, flags, seed, generation) -> torch.Tensor:
    pop = pop.to(torch.float32).contiguous()
    dev = pop.device
    n = pop.shape[0] if mating_pool is None else mating_pool.shape[0]
    d = pop.shape[1]
    lb = lb.to(device=dev, dtype=torch.float32).reshape(-1).contiguous()
    ub = ub.to(device=dev, dtype=torch.float32).reshape(-1).contiguous()
    out = torch.empty(n // 2 * 2, d, dtype=torch.float32, device=dev)
    mp = None if mating_pool is None else mating_pool.to(torch.int64).contiguous()
    ptrs = [None] * 6
    keep = []
    if draws is not None:
        for i, (name, dt) in enumerate((("sbx_mu", torch.float32), ("sbx_sign", torch.int64), ("sbx_half", torch.float32),
                                        ("sbx_pc", torch.float32), ("pm_site", torch.float32), ("pm_mu", torch.float32))):
            t = draws[name].to(device=dev, dtype=dt).contiguous()
            keep.append(t)
            ptrs[i] = _cabi.ptr(t)
    _cabi.check(
        _cabi.lib.evox_offspring(_cabi.ptr(pop), _cabi.ptr(mp), n, d, _cabi.ptr(lb), _cabi.ptr(ub), *ptrs, pro_c, dis_c, pro_m, dis_m,
                                 flags, seed, generation, _cabi.ptr(out), _cabi.stream_ptr(dev))
    )
    return out


def simulated_binary(x: torch.Tensor, pro_c: float = 1.0, dis_c: float = 20.0) -> torch.Tensor:
    n, d = x.shape
    h, dev = n // 2, x.device
    draws = {"sbx_mu": torch.rand(h, d, device=dev), "sbx_sign": torch.randint(0, 2, (h, d), device=dev),
             "sbx_half": torch.rand(h, d, device=dev), "sbx_pc": torch.rand(h, d, device=dev),
             "pm_site": torch.ones(h * 2, d, device=dev), "pm_mu": torch.zeros(h * 2, d, device=dev)}
    inf = torch.full((d,), torch.inf, device=dev)
    return make_offspring(x, -inf, inf, draws=draws, pro_c=pro_c, dis_c=dis_c, flags=CROSSOVER)


def polynomial_mutation(x: torch.Tensor, lb: torch.Tensor, ub: torch.Tensor, pro_m: float = 1, dis_m: float = 20) -> torch.Tensor:
    n, d = x.shape
    dev = x.device
    if n % 2:  # the kernel works on pairs of rows: pad one row and drop it again
        return polynomial_mutation(torch.cat([x, x[-1:]]), lb, ub, pro_m, dis_m)[:n]
    h = n // 2
    z = torch.zeros(h, d, device=dev)
    draws = {"sbx_mu": z, "sbx_sign": torch.zeros(h, d, dtype=torch.int64, device=dev), "sbx_half": z, "sbx_pc": z,
             "pm_site": torch.rand(n, d, device=dev), "pm_mu": torch.rand(n, d, device=dev)}
    return make_offspring(x, lb, ub, draws=draws, pro_m=pro_m, dis_m=dis_m, flags=MUTATION)
