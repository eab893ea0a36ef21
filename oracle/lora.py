"""Oracle for the evolution-strategy paths (test infrastructure; see oracle/__init__.py).

Restates
  * philox_uniform / philox_normal (triton_kernels/kernels/philox.py:52-112): Philox4x32-10 keyed
    by a per-individual int64 seed, counter low word incremented per call WITHOUT carry, 24-bit
    uniforms, Box-Muller on consecutive pairs;
  * compute_counter_offsets, generate_lora_factors, lora_delta_output, lora_gradient
    (triton_kernels/kernels/lora_noise.py:58-196);
  * the layer loop of VirtualLoRAProblem._virtual_forward
    (problems/neuroevolution/virtual_lora_problem.py:126-201) for Linear + ReLU stacks;
  * OpenES.step (algorithms/so/es_variants/open_es.py:60-83), VirtualLoRAES.step
    (es_variants/virtual_lora_es.py:90-135) and adam_single_tensor (es_variants/adam_step.py:4-26).
"""

from __future__ import annotations

import math

import torch

from .pso import _MASK, philox4x32_10


def philox_uniform(seeds: torch.Tensor, n: int, counter: int = 0) -> torch.Tensor:
    pop = seeds.shape[0]
    n_calls = (n + 3) // 4
    idx = torch.arange(n_calls, dtype=torch.int64)[None, :].expand(pop, n_calls)
    c0 = ((counter & _MASK) + idx) & _MASK  # philox.py:80: the carry into c1 is dropped
    c1 = torch.full_like(c0, (counter >> 32) & _MASK)
    z = torch.zeros_like(c0)
    k0 = (seeds & _MASK)[:, None].expand(pop, n_calls)
    k1 = ((seeds >> 32) & _MASK)[:, None].expand(pop, n_calls)
    out = torch.stack(philox4x32_10(c0, c1, z, z, k0, k1), dim=2).reshape(pop, n_calls * 4)[:, :n]
    return ((out & _MASK) >> 8).to(torch.float32) * (1.0 / (1 << 24))


def philox_normal(seeds: torch.Tensor, n: int, counter: int = 0) -> torch.Tensor:
    n_pairs = (n + 1) // 2
    u = philox_uniform(seeds, 2 * n_pairs, counter).reshape(seeds.shape[0], n_pairs, 2)
    u1, u2 = u[..., 0], u[..., 1]
    r = torch.sqrt(-2.0 * torch.log(torch.clamp(u1, min=1e-10)))
    z1 = r * torch.cos(2.0 * math.pi * u2)
    z2 = r * torch.sin(2.0 * math.pi * u2)
    return torch.stack([z1, z2], dim=-1).reshape(seeds.shape[0], 2 * n_pairs)[:, :n]


def _ceil4(x: int) -> int:
    return (x + 3) // 4 * 4


def _as_2d(shape) -> tuple[int, int]:
    return int(math.prod(shape[:-1])), int(shape[-1])


def compute_counter_offsets(param_shapes, lora_rank: int) -> list[int]:
    """lora_noise.py:58-83."""
    offsets, cur = [], 0
    for shape in param_shapes:
        offsets.append(cur)
        if len(shape) == 1:
            n = shape[0]
        else:
            d, k = _as_2d(shape)
            n = lora_rank * k + d * lora_rank
        cur += _ceil4(n)
    return offsets


def generate_lora_factors(seeds, weight_shape, rank: int, counter: int):
    """lora_noise.py:86-127: A (pop, r, k) at `counter`, B (pop, d, r) at counter + ceil4(r k)."""
    pop = seeds.shape[0]
    if len(weight_shape) == 1:
        return philox_normal(seeds, weight_shape[0], counter)
    d, k = _as_2d(weight_shape)
    a = philox_normal(seeds, rank * k, counter).reshape(pop, rank, k)
    b = philox_normal(seeds, d * rank, counter + _ceil4(rank * k)).reshape(pop, d, rank)
    return a, b


def lora_delta_output(x, a, b, sigma):
    """lora_noise.py:151-153."""
    return sigma * torch.bmm(torch.bmm(x, a.transpose(-1, -2)), b.transpose(-1, -2))


def lora_gradient(fitness, a, b, pop_size, sigma, weight_shape):
    """lora_noise.py:188-196."""
    if b is None:
        return ((fitness / (pop_size * sigma)) @ a).reshape(weight_shape)
    return (torch.einsum("i,ijk,ikl->jl", fitness, b, a) / (pop_size * sigma)).reshape(weight_shape)


def adam_single_tensor(param, grad, exp_avg, exp_avg_sq, beta1=0.9, beta2=0.999, lr=1e-3, eps=1e-8):
    """adam_step.py:4-26 with weight_decay = 0 (no bias correction, as in the reference)."""
    exp_avg = torch.lerp(exp_avg, grad, 1 - beta1)
    exp_avg_sq = exp_avg_sq * beta2 + grad * grad * (1 - beta2)
    return param - lr * exp_avg / (exp_avg_sq.sqrt() + eps), exp_avg, exp_avg_sq


def virtual_forward(h, weights, biases, seeds, offsets, shapes, rank, sigma, relu_between=True):
    """Layer loop of _virtual_forward (virtual_lora_problem.py:160-193) for a stack of Linear
    layers with ReLU between them. `h` is (pop, batch, in) — per-individual inputs; the reference
    expands one shared batch to this shape (:158). `offsets` / `shapes` list the parameter blocks in
    order (weight, then bias when present)."""
    h = h.float()
    blk = 0
    n_layers = len(weights)
    for li, (w, bias) in enumerate(zip(weights, biases)):
        base = h @ w.float().t()
        if bias is not None:
            base = base + bias.float()
        a, b = generate_lora_factors(seeds, shapes[blk], rank, offsets[blk])
        out = base + lora_delta_output(h, a, b, sigma)
        blk += 1
        if bias is not None:
            noise = generate_lora_factors(seeds, shapes[blk], rank, offsets[blk])
            out = out + sigma * noise.unsqueeze(1)
            blk += 1
        h = torch.relu(out) if (relu_between and li + 1 < n_layers) else out
    return h


def centered_rank(fitness: torch.Tensor) -> torch.Tensor:
    """Fitness shaping used by the benchmark configuration (not part of the reference, which
    feeds raw fitness into the gradient): ranks in [0, P-1] scaled to [-0.5, 0.5]."""
    ranks = torch.argsort(torch.argsort(fitness, stable=True), stable=True).to(torch.float32)
    return ranks / (fitness.numel() - 1) - 0.5


def open_es_step(center, noise_half, fitness_fn, lr, sigma, mirrored=True, adam_state=None):
    """open_es.py:60-83 with the normal draws passed in."""
    noise = torch.cat([noise_half, -noise_half], dim=0) if mirrored else noise_half
    pop = center[None, :] + sigma * noise
    fitness = fitness_fn(pop)
    grad = noise.T @ fitness / noise.shape[0] / sigma
    if adam_state is None:
        return center - lr * grad, fitness, grad
    # the reference holds beta1 / beta2 as float32 tensors (open_es.py:57-58), so 1 - beta is rounded in fp32
    new_center, m, v = adam_single_tensor(center, grad, adam_state[0], adam_state[1], torch.tensor(0.9), torch.tensor(0.999), lr)
    return new_center, fitness, grad, (m, v)


def ars_step(center, z_plus, fitness_fn, lr, sigma, elite_pop_size, adam_state=None):
    """ARS.step (es_variants/ars.py:62-98) with the normal draws passed in."""
    half = z_plus.shape[0]
    noise = torch.cat([z_plus, -1.0 * z_plus])
    population = center + sigma * noise
    fitness = fitness_fn(population)
    fit_1, fit_2 = fitness[:half], fitness[half:]
    elite_idx = torch.minimum(fit_1, fit_2).argsort()[:elite_pop_size]
    fitness_elite = torch.cat([fit_1[elite_idx], fit_2[elite_idx]])
    sigma_fitness = torch.std(fitness_elite) + 1e-05
    fit_diff = fit_1[elite_idx] - fit_2[elite_idx]
    fit_diff_noise = noise[:half][elite_idx].T @ fit_diff
    theta_grad = 1.0 / (elite_pop_size * sigma_fitness) * fit_diff_noise
    if adam_state is None:
        return center - lr * theta_grad, theta_grad
    new_center, m, v = adam_single_tensor(center, theta_grad, adam_state[0], adam_state[1], torch.tensor(0.9), torch.tensor(0.999), lr)
    return new_center, theta_grad, (m, v)
