"""Oracle for HypE (test infrastructure; see oracle/__init__.py).

Restates cal_hv, the Monte-Carlo hypervolume contribution (algorithms/mo/hype.py:12-39), and one HypE
generation (hype.py:124-149) with every random draw passed in. Pinned against outputs of the reference
recorded in tests/golden/hype.npz (tests/test_oracle_hype.py).

cal_hv here walks the samples in blocks instead of building the (n_sample, n) tables at once, so sizes the
reference cannot hold in memory still finish; the per-row sum is then taken in float64 and rounded once,
which differs from the reference's fp32 sum by a few ulp (the tests state the tolerance).
"""

from __future__ import annotations

import torch

from .nds import lexsort, non_dominate_rank
from .variation import offspring


def alpha_weights(n: int, pop_size) -> torch.Tensor:
    """hype.py:14-24: alpha[k] = prod_{j=1..k} (pop_size - j) / (n - j) / (k + 1), NaN -> 0."""
    j = torch.arange(1, n)
    alpha = torch.cumprod(torch.cat([torch.ones(1), (pop_size - j) / (n - j)]), dim=0) / torch.arange(1, n + 1)
    return torch.nan_to_num(alpha)


def cal_hv(fit: torch.Tensor, ref: torch.Tensor, pop_size, n_sample: int, draw: torch.Tensor, exact_order: bool = False) -> torch.Tensor:
    """`draw`: the (n_sample, m) uniform draw of hype.py:28. `exact_order=True` builds the reference's
    tables and sums them the way it does (bit-exact with it, small sizes only)."""
    n, m = fit.shape
    alpha = alpha_weights(n, pop_size)
    f_min = torch.min(fit, dim=0).values
    samples = draw * (ref - f_min) + f_min
    if exact_order:
        pds = (fit.unsqueeze(0) - samples.unsqueeze(1) <= 0).all(dim=2)  # (n_sample, n)
        ds = pds.sum(dim=1)
        ds = torch.where(ds == 0, ds, ds - 1)
        temp = torch.where(pds.T, ds.unsqueeze(0), -1)
        value = torch.where(temp != -1, alpha[temp], torch.tensor(0, dtype=torch.float32))
        f = torch.sum(value, dim=1)
    else:
        acc = torch.zeros(n, dtype=torch.float64)
        for s0 in range(0, n_sample, 512):
            blk = samples[s0 : s0 + 512]
            pds = (fit.unsqueeze(0) - blk.unsqueeze(1) <= 0).all(dim=2)
            ds = pds.sum(dim=1)
            w = torch.where(ds > 0, alpha[(ds - 1).clamp_min(0)], torch.zeros(()))
            acc += (pds.to(torch.float64) * w.to(torch.float64)[:, None]).sum(dim=0)
        f = acc.to(torch.float32)
    return f * torch.prod(ref - f_min) / n_sample


def tournament(parents: torch.Tensor, fitness: torch.Tensor) -> torch.Tensor:
    """tournament_selection (operators/selection/tournament_selection.py:32-54): argmin over each row of
    candidates, the first minimum on ties."""
    win = torch.argmin(fitness[parents], dim=1)
    return torch.gather(parents, 1, win.unsqueeze(1)).squeeze(1)


def select(rank: torch.Tensor, hv: torch.Tensor, pop_size: int) -> torch.Tensor:
    """hype.py:139-146 given the ranks and the contributions of the merged rows: row numbers kept."""
    dis = torch.where(selection_mask(rank, pop_size), hv, -torch.inf)
    return lexsort([-dis, rank])[:pop_size]


def selection_mask(rank: torch.Tensor, pop_size: int) -> torch.Tensor:
    order = torch.argsort(rank)
    return rank <= rank[order[pop_size - 1]]


def step(pop, fit, ref, lb, ub, evaluate, n_sample, sample_draws, parents, draws, exact_order=False):
    """One generation. sample_draws: the two (n_sample, m) draws; parents: (pop_size, 2); draws: the
    crossover / mutation draws of oracle.variation.offspring."""
    pop_size = pop.shape[0]
    hv = cal_hv(fit, ref, pop_size, n_sample, sample_draws[0], exact_order)
    mating = tournament(parents, -hv)
    off = offspring(pop[mating], lb, ub, draws)
    merge_pop, merge_fit = torch.cat([pop, off]), torch.cat([fit, evaluate(off)])
    rank = non_dominate_rank(merge_fit)
    mask = selection_mask(rank, pop_size)
    hv2 = cal_hv(merge_fit, ref, torch.sum(mask) - pop_size, n_sample, sample_draws[1], exact_order)
    keep = select(rank, hv2, pop_size)
    return merge_pop[keep], merge_fit[keep]
