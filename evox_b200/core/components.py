"""Roles of the generation loop (reference: evox/core/components.py:17-170)."""

from __future__ import annotations

from typing import Any, Dict

import torch

from .module import ModuleBase


class Algorithm(ModuleBase):
    """Proposes candidate solutions and consumes their fitness."""

    def step(self) -> None:
        pass

    def init_step(self) -> None:
        self.step()

    def final_step(self) -> None:
        self.step()

    def evaluate(self, pop: torch.Tensor) -> torch.Tensor:
        """Stand-in for `Problem.evaluate`; the workflow installs the real one."""
        raise NotImplementedError(
            "Evaluate function is not implemented. It is a proxy function of `Problem.evaluate` set by workflow."
        )

    def record_step(self) -> Dict[str, torch.Tensor]:
        return {"pop": self.pop, "fit": self.fit}


class Problem(ModuleBase):
    """Maps a population to fitness values."""

    def evaluate(self, pop: torch.Tensor) -> torch.Tensor:
        return torch.empty(0)


class Workflow(ModuleBase):
    def step(self) -> None:
        pass

    def init_step(self) -> None:
        return self.step()

    def final_step(self) -> None:
        return self.step()


class Monitor(ModuleBase):
    """Callbacks fired around every evaluation; the default ones do nothing."""

    def set_config(self, **config) -> "Monitor":
        return self

    def record_auxiliary(self, aux: Dict[str, torch.Tensor]) -> None:
        pass

    def post_ask(self, candidate_solution: torch.Tensor) -> None:
        pass

    def pre_eval(self, transformed_candidate_solution: Any) -> None:
        pass

    def post_eval(self, fitness: torch.Tensor) -> None:
        pass

    def pre_tell(self, transformed_fitness: torch.Tensor) -> None:
        pass
