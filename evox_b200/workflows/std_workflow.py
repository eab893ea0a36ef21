"""The standard ask-evaluate-tell loop.

Constructor arguments, hook order and the virtual-population bypass follow the reference's
`StdWorkflow` (evox/workflows/std_workflow.py:20-227). Two things are new:

* an algorithm may ask whether the evaluation can be fused into its own kernel
  (`_workflow_fused_plan`): yes when the problem describes itself through `fused_fitness()`,
  no solution / fitness transform is installed and the direction is "min". The monitor hooks
  are then fired with the population and fitness tensors the kernel produced;
* `enable_distributed` evaluates this rank's `tensor_split` share and allgathers the fitness
  (std_workflow.py:167-189) — kept for problems that are not fused. Algorithms that shard
  their own state (e.g. `PSO(shard=True)`) do not need it.
"""

from __future__ import annotations

from typing import Any

import torch

from ..core import Algorithm, Monitor, Problem, Workflow

__all__ = ["StdWorkflow"]


class _Direction(torch.nn.Module):
    """Multiplies fitness by +1 (min) or -1 (max) before any user transform (std_workflow.py:10-17)."""

    def __init__(self, sign: torch.Tensor):
        super().__init__()
        self.sign = sign

    def forward(self, fitness: torch.Tensor) -> torch.Tensor:
        return fitness * self.sign


class StdWorkflow(Workflow):
    def __init__(
        self,
        algorithm: Algorithm,
        problem: Problem,
        monitor: Monitor | None = None,
        opt_direction: str | list[str] = "min",
        solution_transform: torch.nn.Module | None = None,
        fitness_transform: torch.nn.Module | None = None,
        device: str | torch.device | int | None = None,
        enable_distributed: bool = False,
        group: Any = None,
    ):
        super().__init__()
        if device is None:
            device = torch.get_default_device()
        directions = [opt_direction] if isinstance(opt_direction, str) else list(opt_direction)
        assert all(d in ("min", "max") for d in directions), (
            f"Expect optimization direction to be `min` or `max`, got {opt_direction}"
        )
        signs = [1 if d == "min" else -1 for d in directions]
        self.opt_direction = torch.tensor(signs[0] if isinstance(opt_direction, str) else signs, device=device)
        self._all_min = all(s == 1 for s in signs)
        self._plain_solution = solution_transform is None
        self._plain_fitness = fitness_transform is None
        solution_transform = torch.nn.Identity() if solution_transform is None else solution_transform
        user_fitness_transform = torch.nn.Identity() if fitness_transform is None else fitness_transform
        assert callable(solution_transform), f"Expect solution transform to be callable, got {solution_transform}"
        assert callable(user_fitness_transform), f"Expect fitness transform to be callable, got {fitness_transform}"
        fitness_transform = torch.nn.Sequential(_Direction(self.opt_direction), user_fitness_transform)
        for module in (solution_transform, fitness_transform):
            if isinstance(module, torch.nn.Module):
                module.to(device=device)
        if monitor is None:
            monitor = Monitor()
        else:
            monitor.set_config(opt_direction=self.opt_direction)
        algorithm.to(device=device)
        monitor.to(device=device)
        problem.to(device=device)

        self._has_init_ = type(algorithm).init_step is not Algorithm.init_step
        self._has_final_ = type(algorithm).final_step is not Algorithm.final_step
        # the algorithm reaches the problem only through these three callables
        object.__setattr__(algorithm, "evaluate", self._evaluate)
        object.__setattr__(algorithm, "_workflow_fused_plan", self._fused_plan)
        object.__setattr__(algorithm, "_workflow_fused_notify", self._fused_notify)

        self.algorithm = algorithm
        self.monitor = monitor
        self._monitor_has_record_auxiliary = "record_auxiliary" in type(monitor).__dict__
        self.problem = problem
        self.solution_transform = solution_transform
        self.fitness_transform = fitness_transform
        self.enable_distributed = enable_distributed
        self.group = group

    # -- fused evaluation protocol -------------------------------------------------------------
    def _fused_plan(self):
        if not (self._plain_solution and self._plain_fitness and self._all_min) or self.enable_distributed:
            return None
        describe = getattr(self.problem, "fused_fitness", None)
        return describe() if describe is not None else None

    def _fused_notify(self, population: torch.Tensor, fitness: torch.Tensor) -> None:
        m = self.monitor
        m.post_ask(population)
        m.pre_eval(population)
        m.post_eval(fitness)
        m.pre_tell(fitness)

    # -- the general path ----------------------------------------------------------------------
    def _evaluate(self, population):
        m = self.monitor
        if not isinstance(population, torch.Tensor):
            # virtual population: a (center, seeds, sigma) tuple goes to the problem untouched
            # (std_workflow.py:151-163); transforms of solutions are skipped
            center = population[0]
            center = center.unsqueeze(0) if center.ndim == 1 else center
            m.post_ask(center)
            m.pre_eval(center)
            fitness = self.problem.evaluate(population)
            m.post_eval(fitness)
            fitness = self.fitness_transform(fitness)
            m.pre_tell(fitness)
            return fitness

        m.post_ask(population)
        if self.enable_distributed:
            dist = torch.distributed
            rank = dist.get_rank(group=self.group)
            world_size = dist.get_world_size(group=self.group)
            pop_size = population.size(0)
            population = population.tensor_split(world_size, dim=0)[rank]
        population = self.solution_transform(population)
        m.pre_eval(population)
        if self.enable_distributed:
            with torch.random.fork_rng():
                fitness = self.problem.evaluate(population)
            gathered = torch.zeros(pop_size, *fitness.shape[1:], device=fitness.device, dtype=fitness.dtype)
            pieces = list(gathered.tensor_split(world_size, dim=0))
            dist.all_gather(pieces, fitness, group=self.group)
            fitness = torch.cat(pieces, dim=0)
        else:
            fitness = self.problem.evaluate(population)
        m.post_eval(fitness)
        fitness = self.fitness_transform(fitness)
        m.pre_tell(fitness)
        return fitness

    def _step(self, init: bool = False, final: bool = False):
        if init and self._has_init_:
            self.algorithm.init_step()
        elif final and self._has_final_:
            self.algorithm.final_step()
        else:
            self.algorithm.step()
        if self._monitor_has_record_auxiliary:
            self.monitor.record_auxiliary(self.algorithm.record_step())

    def init_step(self):
        self._step(init=True)

    def final_step(self):
        self._step(final=True)

    def step(self):
        self._step()
