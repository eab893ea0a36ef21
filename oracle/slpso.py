"""Oracle for the social-learning PSO steps (test infrastructure; see oracle/__init__.py).

Restates SLPSOGS.step (algorithms/so/pso_variants/sl_pso_gs.py:72-104) and SLPSOUS.step
(sl_pso_us.py:72-110) with their random draws passed in. State is a plain dict with the reference's buffer
names (`pop`, `fit`, `velocity`, `global_best_location`, `global_best_fit`) plus `lb`, `ub`,
`social_influence_factor`, `demonstrator_choice_factor`.
"""

from __future__ import annotations

import torch

from .pso import min_by, relu_clamp


def init_step(state: dict, fitness) -> dict:
    """sl_pso_gs.py:68-70."""
    s = dict(state)
    s["fit"] = fitness(s["pop"])
    s["global_best_fit"] = torch.min(s["fit"])
    return s


def demonstrator_rows_gs(fit: torch.Tensor, theta: torch.Tensor, pick: torch.Tensor) -> torch.Tensor:
    """Row of the swarm each particle learns from (sl_pso_gs.py:80-89); `pick`: the standard-normal draw."""
    n = fit.shape[0]
    order = torch.argsort(fit, descending=True)
    sigma = theta * (n - (torch.arange(n) + 1))
    normal_distribution = sigma * (-torch.abs(pick)) + n
    index_k = torch.clamp(normal_distribution, 1, n).to(dtype=torch.int64) - 1
    return order[index_k]


def clamp_int(a: torch.Tensor, lb: int, ub: int) -> torch.Tensor:
    """utils/jit_fix_operator.py clamp_int: relu-form clamp on integers / floats with scalar bounds."""
    return a + torch.relu(lb - a) - torch.relu(a - ub)


def demonstrator_rows_us(fit: torch.Tensor, theta: torch.Tensor, pick: torch.Tensor) -> torch.Tensor:
    """sl_pso_us.py:80-94; `pick`: the uniform draw."""
    n = fit.shape[0]
    order = torch.argsort(-fit)
    q = clamp_int(n - torch.ceil(theta * (n - (torch.arange(n) + 1) - 1)), 1, n)
    uniform_distribution = pick * (n + 1 - q) + q
    index_k = clamp_int(torch.floor(uniform_distribution).to(dtype=torch.int64) - 1, 0, n - 1)
    return order[index_k]


def step(state: dict, rows: torch.Tensor, r1: torch.Tensor, r2: torch.Tensor, r3: torch.Tensor, fitness) -> dict:
    """The part both variants share (sl_pso_gs.py:74-78, 90-104)."""
    s = dict(state)
    gbl, gbf = min_by([s["global_best_location"].unsqueeze(0), s["pop"]], [s["global_best_fit"].unsqueeze(0), s["fit"]])
    x_k = s["pop"][rows]
    x_avg = torch.mean(s["pop"], dim=0)
    velocity = r1 * s["velocity"] + r2 * (x_k - s["pop"]) + r3 * s["social_influence_factor"] * (x_avg - s["pop"])
    pop = relu_clamp(s["pop"] + velocity, s["lb"], s["ub"])
    s["velocity"] = relu_clamp(velocity, s["lb"], s["ub"])
    s["pop"] = pop
    s["global_best_location"], s["global_best_fit"] = gbl, gbf
    s["fit"] = fitness(pop)
    return s
