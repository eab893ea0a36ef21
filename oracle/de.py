"""Oracle for the differential-evolution step (test infrastructure; see oracle/__init__.py).

Restates DE.step / DE.init_step (algorithms/so/de_variants/de.py:92-157) for one difference vector with
the random draws passed in. State is a plain dict: `pop`, `fit`, `lb`, `ub`, `differential_weight`,
`cross_probability`.
"""

from __future__ import annotations

import torch

from .pso import relu_clamp


def init_step(state: dict, fitness) -> dict:
    s = dict(state)
    s["fit"] = fitness(s["pop"])
    return s


def step(state: dict, idx: list[torch.Tensor], cross: torch.Tensor, forced: torch.Tensor, fitness, best_vector: bool) -> dict:
    """de.py:105-157. `idx`: the randint draws of :112-113 (3 for base "rand", 2 for "best"), `cross` the uniform
    draw of :136, `forced` the (pop_size, 1) dimension that always crosses (:137)."""
    s = dict(state)
    pop, fit = s["pop"], s["fit"]
    if best_vector:
        base_vector = pop[torch.argmin(fit)][None, :]
        start = 0
    else:
        base_vector = pop[idx[0]]
        start = 1
    difference_vector = torch.stack([pop[idx[start]] - pop[idx[start + 1]]]).sum(dim=0)
    new_pop = base_vector + s["differential_weight"] * difference_vector
    mask = cross < s["cross_probability"]
    mask = mask.scatter(dim=1, index=forced, value=1)
    new_pop = torch.where(mask, new_pop, pop)
    new_pop = relu_clamp(new_pop, s["lb"], s["ub"])
    new_fitness = fitness(new_pop)
    compare = new_fitness < fit
    s["pop"] = torch.where(compare[:, None], new_pop, pop)
    s["fit"] = torch.where(compare, new_fitness, fit)
    s["trial"], s["trial_fit"] = new_pop, new_fitness
    return s
