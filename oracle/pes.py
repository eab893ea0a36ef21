"""Oracle for PersistentES.step (test infrastructure; see oracle/__init__.py).

Restates algorithms/so/es_variants/persistent_es.py:74-112 with the normal draws passed in. State is a
plain dict with the reference's names (`center`, `sigma`, `pert_accum`, `inner_step_counter`, optional
`exp_avg` / `exp_avg_sq`); hyper-parameters are float32 tensors as the reference's Parameters are.
"""

from __future__ import annotations

import torch

from .lora import adam_single_tensor


def step(state: dict, z: torch.Tensor, fitness_fn, lr, T, K, sigma_decay, sigma_limit) -> dict:
    s = dict(state)
    pos_perts = z * s["sigma"]
    perts = torch.cat([pos_perts, -pos_perts], dim=0)
    pert_accum = s["pert_accum"] + perts
    population = s["center"] + perts
    fitness = fitness_fn(population)
    theta_grad = torch.mean(pert_accum * fitness.reshape(-1, 1) / (s["sigma"] ** 2), dim=0)
    if "exp_avg" in s:
        s["center"], s["exp_avg"], s["exp_avg_sq"] = adam_single_tensor(
            s["center"], theta_grad, s["exp_avg"], s["exp_avg_sq"], torch.tensor(0.9), torch.tensor(0.999), lr
        )
    else:
        s["center"] = s["center"] - lr * theta_grad
    # persistent_es.py:100-105: the counter that is STORED is the un-reset one (the reset value only lives in a
    # local), so once it has reached T the accumulator is cleared after every step
    counter = s["inner_step_counter"] + K
    s["inner_step_counter"] = counter
    reset = counter >= T
    s["pert_accum"] = torch.where(reset, torch.zeros_like(pert_accum), pert_accum)
    s["sigma"] = torch.maximum(sigma_decay * s["sigma"], sigma_limit)
    return s
