"""Oracle for the mating and variation step around NSGA-II / RVEA selection (test infrastructure;
see oracle/__init__.py).

Restates tournament_selection_multifit (operators/selection/tournament_selection.py:8-29),
simulated_binary (operators/crossover/sbx.py:4-39), polynomial_mutation
(operators/mutation/pm_mutation.py:6-68), the NaN-aware mating pool of RVEA
(algorithms/mo/rvea.py:118-125) and its reference-vector adaptation (:110-113), with every random
draw passed in as a tensor (the reference draws them from torch's global generator in the order
documented on each function).
"""

from __future__ import annotations

import torch

from .nds import lexsort
from .pso import relu_clamp


def tournament_multifit(parents: torch.Tensor, fitnesses: list[torch.Tensor]) -> torch.Tensor:
    """parents: (n_round, k) candidate indices (the reference's one randint draw). The winner of a
    round is the candidate that comes first when sorting by the LAST fitness, ties by the earlier
    ones, ties by position in the tournament."""
    fit = torch.stack(fitnesses, dim=1)
    order = lexsort(fit[parents].unbind(-1))
    return torch.gather(parents, 1, order[:, 0].unsqueeze(1)).squeeze(1)


def simulated_binary(x, mu, sign, r_half, r_pc, pro_c: float = 1.0, dis_c: float = 20.0):
    """Draw order in the reference: mu = rand, sign = randint(0, 2), r_half = rand, r_pc = rand,
    all (n // 2, d)."""
    n = x.shape[0]
    p1, p2 = x[: n // 2], x[n // 2 : n // 2 * 2]
    beta = torch.zeros_like(mu)
    beta = torch.where(mu <= 0.5, torch.pow(2 * mu, 1 / (dis_c + 1)), beta)
    beta = torch.where(mu > 0.5, torch.pow(2 - 2 * mu, -1 / (dis_c + 1)), beta)
    beta = beta * (1 - sign * 2)
    beta = torch.where(r_half < 0.5, 1, beta)
    beta = torch.where(r_pc > pro_c, 1, beta)
    return torch.cat([(p1 + p2) / 2 + beta * (p1 - p2) / 2, (p1 + p2) / 2 - beta * (p1 - p2) / 2])


def polynomial_mutation(x, lb, ub, r_site, mu, pro_m: float = 1, dis_m: float = 20):
    """Draw order in the reference: r_site = rand, mu = rand, both (n, d)."""
    n, d = x.shape
    site = r_site < pro_m / d
    temp = site & (mu <= 0.5)
    lower, upper = lb, ub
    hi = x - torch.relu(x - upper)  # minimum(x, upper), relu form
    pop = hi + torch.relu(lower - hi)  # maximum(., lower)
    norm = torch.where(temp, (pop - lower) / (upper - lower), 0.0)
    pop = torch.where(
        temp,
        pop + (upper - lower) * (torch.pow(2 * mu + (1 - 2 * mu) * torch.pow(1 - norm, dis_m + 1), 1 / (dis_m + 1)) - 1),
        pop,
    )
    temp = site & (mu > 0.5)
    norm = torch.where(temp, (upper - pop) / (upper - lower), torch.zeros_like(pop))
    pop = torch.where(
        temp,
        pop + (upper - lower) * (1 - torch.pow(2 * (1 - mu) + 2 * (mu - 0.5) * torch.pow(1 - norm, dis_m + 1), 1 / (dis_m + 1))),
        pop,
    )
    return pop


def offspring(parents_x, lb, ub, draws: dict) -> torch.Tensor:
    """crossover -> mutation -> clamp, as NSGA2.step / RVEA.step chain them (nsga2.py:95-97)."""
    c = simulated_binary(parents_x, draws["sbx_mu"], draws["sbx_sign"], draws["sbx_half"], draws["sbx_pc"])
    m = polynomial_mutation(c, lb, ub, draws["pm_site"], draws["pm_mu"])
    return relu_clamp(m, lb, ub)


def make_draws(n: int, d: int, seed: int) -> dict:
    g = torch.Generator().manual_seed(seed)
    h = n // 2
    return {
        "sbx_mu": torch.rand(h, d, generator=g), "sbx_sign": torch.randint(0, 2, (h, d), generator=g),
        "sbx_half": torch.rand(h, d, generator=g), "sbx_pc": torch.rand(h, d, generator=g),
        "pm_site": torch.rand(h * 2, d, generator=g), "pm_mu": torch.rand(h * 2, d, generator=g),
    }


def rvea_mating_pool(pop: torch.Tensor, picks: torch.Tensor) -> torch.Tensor:
    """rvea.py:118-125: `picks` in [0, number of rows that are not all-NaN) index the valid rows in
    their original order."""
    n = pop.shape[0]
    valid = ~torch.isnan(pop).all(dim=1)
    keyed = torch.where(valid, torch.arange(n), torch.iinfo(torch.int32).max)
    return pop[torch.argsort(keyed, stable=True)[picks]]


def rv_adaptation(init_v: torch.Tensor, fit: torch.Tensor) -> torch.Tensor:
    """rvea.py:110-113: scale the initial vectors by the NaN-ignoring range of each objective."""
    mx = torch.where(torch.isnan(fit), -torch.inf, fit).max(dim=0)[0]
    mn = torch.where(torch.isnan(fit), torch.inf, fit).min(dim=0)[0]
    return init_v * (mx - mn)
