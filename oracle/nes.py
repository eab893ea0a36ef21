"""Oracle for SNES.step and DES.step (test infrastructure; see oracle/__init__.py).

Restates algorithms/so/es_variants/snes.py:36-95 and des.py:30-77 with the normal draws passed in.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def snes_weights(pop_size: int, weight_type: str, temperature: float = 12.5) -> torch.Tensor:
    """Per-rank weights (snes.py:57-62), one value per rank (the reference tiles them over the columns)."""
    if weight_type == "temp":
        w = torch.arange(pop_size) / (pop_size - 1) - 0.5
        return F.softmax(-20 * F.sigmoid(temperature * w), dim=0)
    w = torch.clip(math.log(pop_size / 2 + 1) - torch.log(torch.arange(1, pop_size + 1)), 0)
    return w / torch.sum(w) - 1 / pop_size


def snes_step(center, sigma, noise, fitness_fn, weights, lrate_mean, lrate_sigma):
    """snes.py:76-90. `weights`: per-rank weights; returns (center, sigma)."""
    dim = center.shape[0]
    population = center + noise * sigma.reshape(1, dim)
    fitness = fitness_fn(population)
    sorted_noise = noise[fitness.argsort()]
    wt = torch.tile(weights[:, None], (1, dim))
    grad_mean = (wt * sorted_noise).sum(dim=0)
    grad_sigma = (wt * (sorted_noise**2 - 1)).sum(dim=0)
    return center + lrate_mean * sigma * grad_mean, sigma * torch.exp(lrate_sigma / 2 * grad_sigma)


def des_step(center, sigma, noise, fitness_fn, temperature=torch.tensor(12.5), lrate_mean=torch.tensor(1.0), lrate_sigma=torch.tensor(0.1)):
    """des.py:57-72."""
    pop_size, dim = noise.shape
    ranks = torch.arange(pop_size) / (pop_size - 1) - 0.5
    population = center + noise * sigma
    fitness = fitness_fn(population)
    population = population[fitness.argsort()]
    weight = torch.tile(F.softmax(-20 * F.sigmoid(temperature * ranks), dim=0)[:, None], (1, dim))
    weight_mean = (weight * population).sum(dim=0)
    weight_sigma = torch.sqrt((weight * (population - center) ** 2).sum(dim=0) + 1e-6)
    return center + lrate_mean * (weight_mean - center), sigma + lrate_sigma * (weight_sigma - sigma)
