"""Oracle for the competitive swarm optimiser step (test infrastructure; see oracle/__init__.py).

Restates CSO.step / CSO.init_step (algorithms/so/pso_variants/cso.py:68-105) with the random pairing
and the three uniform draws passed in. State is a plain dict with the reference's buffer names
(`pop`, `fit`, `velocity`, `lb`, `ub`, `phi`). The reference never writes the students' new velocity
back (cso.py:98-105 only stores positions and fitness); neither does this.
"""

from __future__ import annotations

import torch

from .pso import relu_clamp


def init_step(state: dict, fitness) -> dict:
    """cso.py:68-69."""
    s = dict(state)
    s["fit"] = fitness(s["pop"])
    return s


def step(state: dict, perm: torch.Tensor, lambdas: torch.Tensor, fitness) -> dict:
    """cso.py:79-105. `perm`: the randperm of :81, `lambdas`: the (3, pop_size // 2, dim) draw of :90."""
    s = dict(state)
    pop, fit, velocity = s["pop"].clone(), s["fit"].clone(), s["velocity"]
    lb, ub, phi = s["lb"], s["ub"], s["phi"]
    left, right = perm.view(2, -1)
    mask = fit[left] < fit[right]
    teachers = torch.where(mask, left, right)
    students = torch.where(mask, right, left)
    center = torch.mean(pop, dim=0)
    lambda1, lambda2, lambda3 = lambdas
    student_velocity = (
        lambda1 * velocity[students]
        + lambda2 * (pop[teachers] - pop[students])
        + phi * lambda3 * (center - pop[students])
    )
    vel_range = ub - lb
    student_velocity = relu_clamp(student_velocity, -vel_range, vel_range)
    candidates = relu_clamp(pop[students] + student_velocity, lb, ub)
    pop[students] = candidates
    fit[students] = fitness(candidates)
    s["pop"], s["fit"] = pop, fit
    return s
