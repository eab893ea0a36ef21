"""HypE: hypervolume-estimation based many-objective optimisation with every step of a generation on the
device.

Constructor arguments and state names follow the reference (evox/algorithms/mo/hype.py:42-149). A
generation is: Monte-Carlo hypervolume contributions (three kernels, no population x sample table) ->
binary tournament on them -> one fused crossover + mutation + clamp kernel -> `evaluate` -> the
non-dominated sort kernels -> contributions of the merged rows -> the first `pop_size` rows by (rank,
larger contribution)."""

from __future__ import annotations

from typing import Callable, Optional

import torch

from .. import _cabi
from ..core import Mutable
from ..operators.selection import _workspace, non_dominate_rank, raise_on_kernel_errors
from ..operators.variation import tournament_selection
from .mo import _MOBase

__all__ = ["HypE", "cal_hv"]


def cal_hv(fit: torch.Tensor, ref: torch.Tensor, pop_size, n_sample: int, draw: torch.Tensor | None = None) -> torch.Tensor:
    """Estimated hypervolume contribution of each row of `fit` (n, m) w.r.t. the reference point `ref`
    (hype.py:12-39). `pop_size` may be an int or a 0-dim device tensor (no host synchronisation either
    way); `draw` replaces the (n_sample, m) uniform draw of hype.py:28."""
    fit = fit.to(torch.float32).contiguous()
    n, m = fit.shape
    dev = fit.device
    j = torch.arange(1, n, device=dev)
    alpha = torch.cumprod(torch.cat([torch.ones(1, device=dev), (pop_size - j) / (n - j)]), dim=0) / torch.arange(1, n + 1, device=dev)
    alpha = torch.nan_to_num(alpha).to(torch.float32).contiguous()
    f_min = torch.min(fit, dim=0).values
    if draw is None:
        draw = torch.rand(n_sample, m, device=dev)
    span = ref.to(device=dev, dtype=torch.float32) - f_min
    samples = (draw.to(device=dev, dtype=torch.float32) * span + f_min).contiguous()
    volume = torch.prod(span).reshape(1)
    hv = torch.empty(n, dtype=torch.float32, device=dev)
    ws = _workspace("hv", dev, _cabi.lib.evox_hv_workspace_bytes(n, n_sample))
    _cabi.check(_cabi.lib.evox_hv_contribution(_cabi.ptr(fit), _cabi.ptr(samples), _cabi.ptr(alpha), _cabi.ptr(volume), n, m, n_sample,
                                               _cabi.ptr(hv), _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(dev)))
    return hv


class HypE(_MOBase):
    def __init__(self, pop_size: int, n_objs: int, lb: torch.Tensor, ub: torch.Tensor, n_sample: int = 10000,
                 selection_op: Optional[Callable] = None, mutation_op: Optional[Callable] = None,
                 crossover_op: Optional[Callable] = None, device: torch.device | None = None):
        """`selection_op` is accepted and ignored, as in the reference (hype.py:101: the binary tournament
        is always used)."""
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        self.pop_size = pop_size
        self.n_sample = n_sample
        self._setup(pop_size, n_objs, lb, ub, None, mutation_op, crossover_op, device)
        self.ref = Mutable(torch.ones(n_objs, device=device))
        self.pop = Mutable((self.ub - self.lb) * torch.rand(pop_size, self.dim, device=device) + self.lb)
        self.fit = Mutable(torch.full((pop_size, n_objs), torch.inf, device=device))

    def init_step(self):
        """hype.py:117-122: the reference point is 1.2 x the largest objective value of the first population."""
        self.fit = self.evaluate(self.pop)
        # the reference multiplies the Python float of the maximum (a double) and rounds once
        self.ref = (torch.max(self.fit).double() * 1.2).float().expand(self.n_objs).contiguous()

    def step(self, parents: torch.Tensor | None = None, draws: dict | None = None, sample_draws=None):
        """One generation (hype.py:124-149). `parents` (pop_size, 2), `draws` (crossover / mutation) and
        `sample_draws` (the two (n_sample, m) uniform draws) replace the random draws."""
        raise_on_kernel_errors()  # status of the previous generation's non-dominated sort
        sa, sb = sample_draws if sample_draws is not None else (None, None)
        hv = cal_hv(self.fit, self.ref, self.pop_size, self.n_sample, sa)
        mating_pool = tournament_selection(self.pop_size, -hv, parents=parents)
        offspring = self._variation(self.pop, mating_pool, draws)
        off_fit = self.evaluate(offspring)
        merge_pop = torch.cat([self.pop, offspring], dim=0)
        merge_fit = torch.cat([self.fit, off_fit], dim=0)
        rank = non_dominate_rank(merge_fit)
        worst_rank = torch.sort(rank).values[self.pop_size - 1]
        mask = rank <= worst_rank
        hv = cal_hv(merge_fit, self.ref, torch.sum(mask) - self.pop_size, self.n_sample, sb)
        dis = torch.where(mask, hv, -torch.inf)
        # lexsort([-dis, rank]): rank first, larger contribution first inside a rank, stable
        by_dis = torch.argsort(-dis, stable=True)
        keep = by_dis[torch.argsort(rank[by_dis], stable=True)][: self.pop_size]
        self._last_selection = (merge_fit, rank, hv, keep)  # for inspection; not part of the state
        self.pop = merge_pop[keep]
        self.fit = merge_fit[keep]
        self.generation += 1
