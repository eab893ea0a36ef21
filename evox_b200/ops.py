"""`torch.ops.evox_b200.*`: the kernels as registered PyTorch operators.

The reference exposes its hand-written kernels as `torch.library.custom_op`s with a fake
(shape-only) implementation so that they survive tracing (evox/utils/op_register.py:54-132,
evox/triton_kernels/op_register.py:88-131). The same is done here: each operator has a CUDA
implementation (the C-ABI call) and a fake one; there is deliberately no CPU implementation.
"""

from __future__ import annotations

import torch

from . import lora_kernels as _lk
from .operators import selection as _sel

__all__ = ["nd_rank", "crowding_distance", "nd_environmental_selection", "ref_vec_guided", "philox_uniform", "philox_normal",
           "lora_delta_output", "lora_gradient"]


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
