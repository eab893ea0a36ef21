"""Evaluation monitor: best-so-far tracking, optional histories, Pareto-front extraction.

Same constructor arguments and getters as the reference's `EvalMonitor`
(evox/workflows/eval_monitor.py:83-347; the plotting helpers are not provided). Differences that
follow from this package's design: the algorithms update their state in place, so everything the
monitor keeps beyond the current generation is copied (the reference relies on fresh tensors per
step); histories are plain Python lists; the Pareto front is ranked by the CUDA kernel
(`non_dominate_rank`) on the device the fitness lives on.
"""

from __future__ import annotations

import warnings
from typing import Dict, List, Tuple

import torch

from ..core import Monitor, Mutable

__all__ = ["EvalMonitor"]


class EvalMonitor(Monitor):
    def __init__(self, multi_obj: bool = False, full_fit_history: bool = True, full_sol_history: bool = False,
                 full_pop_history: bool = False, topk: int = 1, device: torch.device | None = None,
                 history_device: torch.device | None = None):
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        self.multi_obj = multi_obj
        self.full_fit_history = full_fit_history
        self.full_sol_history = full_sol_history
        self.full_pop_history = full_pop_history
        self.opt_direction = torch.tensor(1)
        self.topk = topk
        self.device = device
        self.history_device = torch.device("cpu") if history_device is None else torch.device(history_device)
        self.aux_keys: List[str] = []
        self.latest_solution = Mutable(torch.empty(0, device=device))
        self.latest_fitness = Mutable(torch.empty(0, device=device))
        self.topk_solutions = Mutable(torch.empty(0, device=device))
        self.topk_fitness = Mutable(torch.empty(0, device=device))
        self.fitness_history: List[torch.Tensor] = []
        self.solution_history: List[torch.Tensor] = []
        self.aux_history: Dict[str, List[torch.Tensor]] = {}

    # the reference's alternative spellings
    fit_history = property(lambda self: self.fitness_history)
    sol_history = property(lambda self: self.solution_history)
    auxiliary_history = property(lambda self: self.aux_history)

    def set_config(self, **config):
        for key in ("multi_obj", "full_fit_history", "full_sol_history", "topk", "opt_direction"):
            if key in config:
                setattr(self, key, config[key])
        return self

    def record_auxiliary(self, aux: Dict[str, torch.Tensor]):
        if self.full_pop_history:
            if not self.aux_keys:
                self.aux_keys = list(aux.keys())
            for key in self.aux_keys:
                self.aux_history.setdefault(key, []).append(aux[key].to(self.history_device, copy=True))

    def post_ask(self, candidate_solution: torch.Tensor):
        self.latest_solution = candidate_solution

    def pre_tell(self, fitness: torch.Tensor):
        self.latest_fitness = fitness
        if fitness.ndim == 1:
            self.multi_obj = False
            assert fitness.size(0) >= self.topk
            if self.topk_solutions.ndim <= 1:
                cand_sol, cand_fit = self.latest_solution, fitness
            else:
                cand_sol = torch.cat([self.topk_solutions, self.latest_solution])
                cand_fit = torch.cat([self.topk_fitness, fitness])
            best = torch.topk(cand_fit, self.topk, largest=False)[1]
            self.topk_fitness = cand_fit[best]
            # virtual populations hand over only the centre: keep fitness, skip the solutions
            if cand_sol.size(0) == cand_fit.size(0):
                self.topk_solutions = cand_sol[best]
        elif fitness.ndim == 2:
            self.multi_obj = True
        else:
            raise ValueError(f"Invalid fitness shape: {fitness.shape}")
        if self.full_sol_history:
            self.solution_history.append(self.latest_solution.to(self.history_device, copy=True))
        if self.full_fit_history:
            self.fitness_history.append(fitness.to(self.history_device, copy=True))

    # ---- getters (signs restored for opt_direction = "max") --------------------------------
    def _sign(self, device):
        return self.opt_direction.to(device)

    def get_latest_fitness(self) -> torch.Tensor:
        return self._sign(self.latest_fitness.device) * self.latest_fitness

    def get_latest_solution(self) -> torch.Tensor:
        return self.latest_solution

    def get_topk_fitness(self) -> torch.Tensor:
        return self._sign(self.topk_fitness.device) * self.topk_fitness

    def _single_objective_only(self, what: str):
        if self.multi_obj:
            raise ValueError(f"Multi-objective optimization does not have a single best {what}. Please use get_pf_{'solutions' if what == 'solution' else 'fitness'}")

    def get_topk_solutions(self) -> torch.Tensor:
        self._single_objective_only("solution")
        return self.topk_solutions

    def get_best_solution(self) -> torch.Tensor:
        self._single_objective_only("solution")
        return self.topk_solutions[0]

    def get_best_fitness(self) -> torch.Tensor:
        self._single_objective_only("fitness")
        return self._sign(self.topk_fitness.device) * self.topk_fitness[0]

    def _rank0(self, fitness: torch.Tensor) -> torch.Tensor:
        from ..operators.selection import non_dominate_rank

        dev = self.device if self.device.type == "cuda" else torch.device("cuda")
        return (non_dominate_rank(fitness.to(dev)) == 0).to(fitness.device)

    def get_pf_fitness(self, deduplicate: bool = True) -> torch.Tensor:
        if not self.multi_obj:
            raise ValueError("get_pf_fitness is only available for multi-objective optimization.")
        if not self.full_fit_history:
            warnings.warn("`get_pf_fitness` requires enabling `full_fit_history`.")
        fit = torch.cat(self.fitness_history, dim=0)
        if deduplicate:
            fit = torch.unique(fit, dim=0)
        return fit[self._rank0(fit)] * self._sign(fit.device)

    def get_pf(self, deduplicate: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
        if not self.multi_obj:
            raise ValueError("get_pf is only available for multi-objective optimization.")
        if not self.full_fit_history or not self.full_sol_history:
            warnings.warn("`get_pf` requires enabling both `full_sol_history` and `full_sol_history`.")
        sol = torch.cat(self.solution_history, dim=0)
        fit = torch.cat(self.fitness_history, dim=0)
        if deduplicate:
            _, inverse = torch.unique(sol, dim=0, return_inverse=True)
            first = torch.full((int(inverse.max()) + 1,), sol.shape[0], dtype=torch.int64, device=sol.device)
            first.scatter_reduce_(0, inverse, torch.arange(sol.shape[0], device=sol.device), reduce="amin")
            sol, fit = sol[first], fit[first]
        keep = self._rank0(fit)
        return sol[keep], fit[keep] * self._sign(fit.device)

    def get_pf_solutions(self, deduplicate: bool = True) -> torch.Tensor:
        return self.get_pf(deduplicate)[0]

    def get_fitness_history(self) -> List[torch.Tensor]:
        return [self._sign(f.device) * f for f in self.fitness_history]

    def get_solution_history(self) -> List[torch.Tensor]:
        return self.solution_history
