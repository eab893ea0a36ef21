"""`torch.ops.evox_b200.*`: the kernels as registered PyTorch operators.

The reference exposes its hand-written kernels as `torch.library.custom_op`s with a fake
(shape-only) implementation so that they survive tracing (evox/utils/op_register.py:54-132,
evox/triton_kernels/op_register.py:88-131). The same is done here: each operator has a CUDA
implementation (the C-ABI call) and a fake one; there is deliberately no CPU implementation.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _cabi
from . import lora_kernels as _lk
from .operators import selection as _sel

__all__ = ["nd_rank", "crowding_distance", "nd_environmental_selection", "ref_vec_guided", "philox_uniform", "philox_normal",
           "lora_delta_output", "lora_gradient", "eval_fitness", "pso_step", "pso_generation", "openes_ask", "openes_gradient",
           "es_update", "offspring", "lora_layer", "lora_layer_next", "lora_layer_neg_mse", "lora_gradient_seeds"]


@torch.library.custom_op("evox_b200::nd_rank", mutates_args=(), device_types="cuda")
def nd_rank(f: torch.Tensor) -> torch.Tensor:
    return _sel.non_dominate_rank(f)


@nd_rank.register_fake
def _(f):
    return f.new_empty(f.shape[0], dtype=torch.int32)


@torch.library.custom_op("evox_b200::crowding_distance", mutates_args=(), device_types="cuda")
def crowding_distance(costs: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return _sel.crowding_distance(costs, mask)


@crowding_distance.register_fake
def _(costs, mask):
    return costs.new_empty(costs.shape[0], dtype=torch.float32)


@torch.library.custom_op("evox_b200::nd_environmental_selection", mutates_args=(), device_types="cuda")
def nd_environmental_selection(x: torch.Tensor, f: torch.Tensor, topk: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return _sel.nd_environmental_selection(x, f, topk)


@nd_environmental_selection.register_fake
def _(x, f, topk):
    return (x.new_empty(topk, x.shape[1], dtype=torch.float32), f.new_empty(topk, f.shape[1], dtype=torch.float32),
            f.new_empty(topk, dtype=torch.int32), f.new_empty(topk, dtype=torch.float32))


@torch.library.custom_op("evox_b200::ref_vec_guided", mutates_args=(), device_types="cuda")
def ref_vec_guided(x: torch.Tensor, f: torch.Tensor, v: torch.Tensor, theta: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return _sel.ref_vec_guided(x, f, v, theta)


@ref_vec_guided.register_fake
def _(x, f, v, theta):
    return x.new_empty(v.shape[0], x.shape[1], dtype=torch.float32), f.new_empty(v.shape[0], f.shape[1], dtype=torch.float32)


@torch.library.custom_op("evox_b200::philox_uniform", mutates_args=(), device_types="cuda")
def philox_uniform(seeds: torch.Tensor, n: int, counter: int = 0) -> torch.Tensor:
    return _lk.philox_uniform(seeds, n, counter)


@philox_uniform.register_fake
def _(seeds, n, counter=0):
    return seeds.new_empty(seeds.shape[0], n, dtype=torch.float32)


@torch.library.custom_op("evox_b200::philox_normal", mutates_args=(), device_types="cuda")
def philox_normal(seeds: torch.Tensor, n: int, counter: int = 0) -> torch.Tensor:
    return _lk.philox_normal(seeds, n, counter)


@philox_normal.register_fake
def _(seeds, n, counter=0):
    return seeds.new_empty(seeds.shape[0], n, dtype=torch.float32)


@torch.library.custom_op("evox_b200::lora_delta_output", mutates_args=(), device_types="cuda")
def lora_delta_output(x: torch.Tensor, A: torch.Tensor, B: torch.Tensor, sigma: float) -> torch.Tensor:
    return _lk.lora_delta_output(x, A, B, sigma)


@lora_delta_output.register_fake
def _(x, A, B, sigma):
    return x.new_empty(x.shape[0], x.shape[1], B.shape[1], dtype=torch.float32)


@torch.library.custom_op("evox_b200::lora_gradient", mutates_args=(), device_types="cuda")
def lora_gradient(fitness: torch.Tensor, A: torch.Tensor, B: torch.Tensor, pop_size: int, sigma: float) -> torch.Tensor:
    return _lk.lora_gradient(fitness, A, B, pop_size, sigma, (B.shape[1], A.shape[2]))


@lora_gradient.register_fake
def _(fitness, A, B, pop_size, sigma):
    return A.new_empty(B.shape[1], A.shape[2], dtype=torch.float32)


# ---------------------------------------------------------------------------------------------
# Step-level operators: what PSO.step, OpenES.step, VirtualLoRAES.step and the offspring step of
# NSGA2 / RVEA launch. State tensors the kernels update in place are declared in `mutates_args`, so a
# traced program (torch.compile of `workflow.step`) keeps the calls in order and sees the updates.
# ---------------------------------------------------------------------------------------------
_pso_ws: dict[torch.device, torch.Tensor] = {}


def _pso_workspace(dev: torch.device) -> torch.Tensor:
    ws = _pso_ws.get(dev)
    if ws is None:
        ws = _pso_ws[dev] = torch.zeros(_cabi.lib.evox_pso_workspace_bytes(1, 1), dtype=torch.uint8, device=dev)
    return ws


@torch.library.custom_op("evox_b200::eval_fitness", mutates_args=(), device_types="cuda")
def eval_fitness(pop: torch.Tensor, fitness_id: int, params: Sequence[float]) -> torch.Tensor:
    """Ackley / Rastrigin / Sphere of every row (evox_eval_fitness)."""
    pop = pop.to(torch.float32).contiguous()
    fit = torch.empty(pop.shape[0], dtype=torch.float32, device=pop.device)
    _cabi.check(_cabi.lib.evox_eval_fitness(_cabi.ptr(pop), pop.shape[0], pop.shape[1], fitness_id, _cabi.host_floats(list(params)),
                                            _cabi.ptr(fit), _cabi.stream_ptr(pop.device)))
    return fit


@eval_fitness.register_fake
def _(pop, fitness_id, params):
    return pop.new_empty(pop.shape[0], dtype=torch.float32)


_PSO_STATE = ("pop", "velocity", "local_best_location", "local_best_fit", "fit", "global_best_location", "global_best_fit")


@torch.library.custom_op("evox_b200::pso_step", mutates_args=_PSO_STATE + ("generation",), device_types="cuda")
def pso_step(pop: torch.Tensor, velocity: torch.Tensor, local_best_location: torch.Tensor, local_best_fit: torch.Tensor,
             fit: torch.Tensor, global_best_location: torch.Tensor, global_best_fit: torch.Tensor, lb: torch.Tensor,
             ub: torch.Tensor, w: torch.Tensor, phi_p: torch.Tensor, phi_g: torch.Tensor, rg: Optional[torch.Tensor],
             rp: Optional[torch.Tensor], fitness_id: int, params: Sequence[float], seed: int, generation: torch.Tensor) -> None:
    """One whole single-GPU PSO generation that carries nothing from call to call (evox_pso_step: arg-min of
    `fit`, fold into the global best, update + fused evaluation). `generation` is a 0-d int64 HOST tensor: the
    position in the Philox stream, read and then incremented here."""
    dev = pop.device
    ws = _pso_workspace(dev)
    _cabi.check(
        _cabi.lib.evox_pso_step(
            _cabi.ptr(pop, torch.float32, "pop"), _cabi.ptr(velocity, torch.float32, "velocity"),
            _cabi.ptr(local_best_location, torch.float32), _cabi.ptr(local_best_fit, torch.float32), _cabi.ptr(fit, torch.float32),
            _cabi.ptr(global_best_location, torch.float32), _cabi.ptr(global_best_fit, torch.float32), _cabi.ptr(lb, torch.float32),
            _cabi.ptr(ub, torch.float32), _cabi.ptr(w, torch.float32), _cabi.ptr(phi_p, torch.float32), _cabi.ptr(phi_g, torch.float32),
            _cabi.ptr(rg, torch.float32), _cabi.ptr(rp, torch.float32), pop.shape[0], pop.shape[1], fitness_id,
            _cabi.host_floats(list(params)), seed, int(generation), _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(dev),
        )
    )
    generation += 1


@pso_step.register_fake
def _(*args):
    return None


@torch.library.custom_op("evox_b200::pso_generation", mutates_args=_PSO_STATE + ("record_out", "workspace"), device_types="cuda")
def pso_generation(pop: torch.Tensor, velocity: torch.Tensor, local_best_location: torch.Tensor, local_best_fit: torch.Tensor,
                   fit: torch.Tensor, global_best_location: torch.Tensor, global_best_fit: torch.Tensor, lb: torch.Tensor,
                   ub: torch.Tensor, w: torch.Tensor, phi_p: torch.Tensor, phi_g: torch.Tensor, rg: Optional[torch.Tensor],
                   rp: Optional[torch.Tensor], fitness_id: int, params: Sequence[float], seed: int, generation: int,
                   row_offset: int, records: torch.Tensor, n_records: int, record_out: torch.Tensor,
                   workspace: torch.Tensor) -> None:
    """One generation of a swarm shard in one launch (evox_pso_generation): folds `records` (the best-particle
    records the previous call left, gathered over the shards) into the global best, moves, evaluates, and leaves
    this shard's record of the new swarm in `record_out`."""
    dev = pop.device
    _cabi.check(
        _cabi.lib.evox_pso_generation(
            _cabi.ptr(pop, torch.float32, "pop"), _cabi.ptr(velocity, torch.float32, "velocity"),
            _cabi.ptr(local_best_location, torch.float32), _cabi.ptr(local_best_fit, torch.float32), _cabi.ptr(fit, torch.float32),
            _cabi.ptr(global_best_location, torch.float32), _cabi.ptr(global_best_fit, torch.float32), _cabi.ptr(lb, torch.float32),
            _cabi.ptr(ub, torch.float32), _cabi.ptr(w, torch.float32), _cabi.ptr(phi_p, torch.float32), _cabi.ptr(phi_g, torch.float32),
            _cabi.ptr(rg, torch.float32), _cabi.ptr(rp, torch.float32), pop.shape[0], pop.shape[1], fitness_id,
            _cabi.host_floats(list(params)), seed, generation, row_offset, _cabi.ptr(records), n_records, _cabi.ptr(record_out),
            _cabi.ptr(workspace), workspace.numel(), _cabi.stream_ptr(dev),
        )
    )


@pso_generation.register_fake
def _(*args):
    return None


@torch.library.custom_op("evox_b200::openes_ask", mutates_args=(), device_types="cuda")
def openes_ask(center: torch.Tensor, noise: torch.Tensor, noise_stdev: torch.Tensor, pop_size: int) -> torch.Tensor:
    """pop = center + sigma * [noise; -noise] (mirrored when noise has pop_size / 2 rows; open_es.py:63-68)."""
    dev = center.device
    noise = noise.to(torch.float32).contiguous()
    dim = center.shape[0]
    pop = torch.empty(pop_size, dim, dtype=torch.float32, device=dev)
    _cabi.check(_cabi.lib.evox_openes_ask(_cabi.ptr(center, torch.float32), _cabi.ptr(noise), _cabi.ptr(noise_stdev, torch.float32), pop_size,
                                          dim, noise.shape[0], _cabi.ptr(pop), _cabi.stream_ptr(dev)))
    return pop


@openes_ask.register_fake
def _(center, noise, noise_stdev, pop_size):
    return center.new_empty(pop_size, center.shape[0], dtype=torch.float32)


@torch.library.custom_op("evox_b200::openes_gradient", mutates_args=(), device_types="cuda")
def openes_gradient(noise: torch.Tensor, fitness: torch.Tensor, pop_size: int, sigma: float) -> torch.Tensor:
    """grad = noise^T fitness / pop_size / sigma over the (mirrored) noise rows (open_es.py:70)."""
    dev = noise.device
    noise = noise.to(torch.float32).contiguous()
    fitness = fitness.to(torch.float32).contiguous()
    grad = torch.empty(noise.shape[1], dtype=torch.float32, device=dev)
    _cabi.check(_cabi.lib.evox_openes_gradient(_cabi.ptr(noise), _cabi.ptr(fitness), pop_size, noise.shape[1], noise.shape[0], float(sigma),
                                               _cabi.ptr(grad), _cabi.stream_ptr(dev)))
    return grad


@openes_gradient.register_fake
def _(noise, fitness, pop_size, sigma):
    return noise.new_empty(noise.shape[1], dtype=torch.float32)


@torch.library.custom_op("evox_b200::es_update", mutates_args=("center", "exp_avg", "exp_avg_sq"), device_types="cuda")
def es_update(center: torch.Tensor, grad: torch.Tensor, learning_rate: torch.Tensor, exp_avg: Optional[torch.Tensor],
              exp_avg_sq: Optional[torch.Tensor], beta1: Optional[torch.Tensor], beta2: Optional[torch.Tensor], start: int,
              count: int) -> None:
    """center[start : start + count] -= lr * grad, or the reference's Adam step when the moment tensors are given
    (open_es.py:71-83, es_variants/adam_step.py:4-26)."""
    assert grad.numel() == count and grad.is_contiguous()

    def at(t):
        return None if t is None else _cabi.ptr(t, torch.float32) + 4 * start

    _cabi.check(
        _cabi.lib.evox_es_update(at(center), _cabi.ptr(grad, torch.float32, "grad"), _cabi.ptr(learning_rate, torch.float32), at(exp_avg),
                                 at(exp_avg_sq), _cabi.ptr(beta1), _cabi.ptr(beta2), 1e-8, count, _cabi.stream_ptr(center.device))
    )


@es_update.register_fake
def _(*args):
    return None


@torch.library.custom_op("evox_b200::offspring", mutates_args=(), device_types="cuda")
def offspring(pop: torch.Tensor, lb: torch.Tensor, ub: torch.Tensor, mating_pool: Optional[torch.Tensor],
              sbx_mu: Optional[torch.Tensor], sbx_sign: Optional[torch.Tensor], sbx_half: Optional[torch.Tensor],
              sbx_pc: Optional[torch.Tensor], pm_site: Optional[torch.Tensor], pm_mu: Optional[torch.Tensor], pro_c: float,
              dis_c: float, pro_m: float, dis_m: float, flags: int, seed: int, generation: int) -> torch.Tensor:
    """clamp(polynomial_mutation(simulated_binary(pop[mating_pool]))) in one kernel (evox_offspring; nsga2.py:95-97)."""
    from .operators import variation as _var

    draws = None
    if sbx_mu is not None:
        draws = {"sbx_mu": sbx_mu, "sbx_sign": sbx_sign, "sbx_half": sbx_half, "sbx_pc": sbx_pc, "pm_site": pm_site, "pm_mu": pm_mu}
    return _var._make_offspring(pop, lb, ub, mating_pool, draws, pro_c, dis_c, pro_m, dis_m, flags, seed, generation)


@offspring.register_fake
def _(pop, lb, ub, mating_pool, *rest):
    n = pop.shape[0] if mating_pool is None else mating_pool.shape[0]
    return pop.new_empty(n // 2 * 2, pop.shape[1], dtype=torch.float32)


@torch.library.custom_op("evox_b200::lora_layer", mutates_args=(), device_types="cuda")
def lora_layer(h: torch.Tensor, w: torch.Tensor, seeds: torch.Tensor, counter: int, sigma: float, bias: Optional[torch.Tensor],
               bias_counter: Optional[int], relu: bool, t: Optional[torch.Tensor]) -> torch.Tensor:
    """One virtual-LoRA Linear layer on the tensor cores -> bf16 activations (virtual_lora_problem.py:160-193)."""
    return _lk.lora_layer_bf16(h, w, seeds, counter, sigma, bias=bias, bias_counter=bias_counter, relu=relu, t=t)


@lora_layer.register_fake
def _(h, w, seeds, counter, sigma, bias, bias_counter, relu, t):
    return h.new_empty(h.shape[0], h.shape[1], w.shape[0], dtype=torch.bfloat16)


@torch.library.custom_op("evox_b200::lora_layer_next", mutates_args=(), device_types="cuda")
def lora_layer_next(h: torch.Tensor, w: torch.Tensor, seeds: torch.Tensor, counter: int, sigma: float, bias: Optional[torch.Tensor],
                    bias_counter: Optional[int], relu: bool, t: Optional[torch.Tensor],
                    next_counter: int) -> tuple[torch.Tensor, torch.Tensor]:
    """lora_layer that also returns the next layer's down-projection of its own output."""
    y, t_next = _lk.lora_layer_bf16(h, w, seeds, counter, sigma, bias=bias, bias_counter=bias_counter, relu=relu, t=t,
                                     next_counter=next_counter)
    return y, t_next


@lora_layer_next.register_fake
def _(h, w, seeds, counter, sigma, bias, bias_counter, relu, t, next_counter):
    return (h.new_empty(h.shape[0], h.shape[1], w.shape[0], dtype=torch.bfloat16),
            h.new_empty(h.shape[0], h.shape[1], 8, dtype=torch.float32))


@torch.library.custom_op("evox_b200::lora_layer_neg_mse", mutates_args=(), device_types="cuda")
def lora_layer_neg_mse(h: torch.Tensor, w: torch.Tensor, seeds: torch.Tensor, counter: int, sigma: float,
                       bias: Optional[torch.Tensor], bias_counter: Optional[int], t: Optional[torch.Tensor],
                       target: torch.Tensor) -> torch.Tensor:
    """Last layer fused with the loss: -mean((y - target)^2) per individual, y never written."""
    return _lk.lora_layer_bf16(h, w, seeds, counter, sigma, bias=bias, bias_counter=bias_counter, t=t, target=target)


@lora_layer_neg_mse.register_fake
def _(h, w, seeds, counter, sigma, bias, bias_counter, t, target):
    return h.new_empty(h.shape[0], dtype=torch.float32)


@torch.library.custom_op("evox_b200::lora_gradient_seeds", mutates_args=(), device_types="cuda")
def lora_gradient_seeds(fitness: torch.Tensor, seeds: torch.Tensor, d: int, k: int, rank: int, counter: int, pop_size: int,
                        sigma: float, passes: int) -> torch.Tensor:
    """sum_i f_i B_i A_i / (pop_size sigma) with the factors regenerated from the seeds (lora_noise.py:157-196)."""
    return _lk.lora_gradient_from_seeds(fitness, seeds, (d, k), rank, counter, pop_size, sigma, passes=passes)


@lora_gradient_seeds.register_fake
def _(fitness, seeds, d, k, rank, counter, pop_size, sigma, passes):
    return fitness.new_empty(d, k, dtype=torch.float32)


# ---------------------------------------------------------------------------------------------
# vmap rules: the reference's programming model maps whole workflows over a batch dimension
# (evox/utils/op_register.py:54-132 asks every custom op for a `vmap_fn`). A batched call runs the
# kernel once per slice — the kernels take one problem instance — and stacks the results on dim 0.
# ---------------------------------------------------------------------------------------------
def _slices(batch: int, args, in_dims):
    """Per-slice argument tuples; unbatched arguments (in_dim None) are passed to every slice as they are."""
    moved = [a if d is None else a.movedim(d, 0) for a, d in zip(args, in_dims)]
    return [tuple(m if d is None else m[i] for m, d in zip(moved, in_dims)) for i in range(batch)]


def _register_loop_vmap(op, n_out: int):
    def rule(info, in_dims, *args):
        outs = [op(*one) for one in _slices(info.batch_size, args, in_dims)]
        if n_out == 1:
            return torch.stack(outs), 0
        return tuple(torch.stack([o[k] for o in outs]) for k in range(n_out)), tuple(0 for _ in range(n_out))

    torch.library.register_vmap(op, rule)


_register_loop_vmap(nd_rank, 1)
_register_loop_vmap(crowding_distance, 1)
_register_loop_vmap(nd_environmental_selection, 4)
_register_loop_vmap(ref_vec_guided, 2)
_register_loop_vmap(philox_uniform, 1)
_register_loop_vmap(philox_normal, 1)
_register_loop_vmap(lora_delta_output, 1)
_register_loop_vmap(lora_gradient, 1)
