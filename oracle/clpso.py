"""Oracle for the comprehensive-learning PSO step (test infrastructure; see oracle/__init__.py).

Restates CLPSO.step / CLPSO.init_step (algorithms/so/pso_variants/clpso.py:67-123) with the four random
draws of :92-95 passed in. State is a plain dict with the reference's buffer names.
"""

from __future__ import annotations

import torch

from .pso import min_by, relu_clamp


def init_step(state: dict, fitness) -> dict:
    """clpso.py:67-70 (the global best LOCATION is left as constructed)."""
    s = dict(state)
    s["fit"] = fitness(s["pop"])
    s["personal_best_fit"] = s["fit"]
    s["global_best_fit"] = torch.min(s["fit"])
    return s


def step(state: dict, coeff: torch.Tensor, i1: torch.Tensor, i2: torch.Tensor, poss: torch.Tensor, fitness) -> dict:
    """clpso.py:89-123."""
    s = dict(state)
    learning_index = torch.where(s["personal_best_fit"][i1] < s["personal_best_fit"][i2], i1, i2)
    compare = s["personal_best_fit"] > s["fit"]
    s["personal_best_location"] = torch.where(compare[:, None], s["pop"], s["personal_best_location"])
    s["personal_best_fit"] = torch.where(compare, s["fit"], s["personal_best_fit"])
    s["global_best_location"], s["global_best_fit"] = min_by(
        [s["global_best_location"][None, :], s["pop"]], [s["global_best_fit"].unsqueeze(0), s["fit"]]
    )
    learning_personal_best = s["personal_best_location"][learning_index, :]
    personal_best = torch.where((poss < s["P_c"][None])[:, None], learning_personal_best, s["personal_best_location"])
    velocity = s["w"] * s["velocity"] + s["c"] * coeff * (personal_best - s["pop"])
    s["velocity"] = relu_clamp(velocity, s["lb"], s["ub"])
    s["pop"] = relu_clamp(s["pop"] + velocity, s["lb"], s["ub"])
    s["fit"] = fitness(s["pop"])
    return s
