"""`use_state` and `vmap` over modules whose steps run in-place CUDA kernels.

The reference turns a module method into a function of the module's state and maps it over stacked
states with `torch.func` (evox/core/module.py:153-260; used as
`vmap(use_state(workflow.step), randomness="different")` over `torch.func.stack_module_state([workflow] * n)`
in unit_test/algorithms/test_base.py:52-65 and unit_test/workflows/test_std_workflow.py:94-103).
`torch.vmap` cannot batch a kernel that updates its operands in place, so here

* `use_state(method)` gives `fn(state, *args) -> new_state | (new_state, out)`: the module's parameters and
  buffers are swapped for COPIES of `state` for the duration of the call (the caller's tensors are never
  written), the method runs its usual kernels on the copies, and the copies come back as the new state;
* `vmap(fn)` maps over the leading dimension of every tensor argument by running the slices one after the
  other on the current stream (each call already fills the GPU) and stacking the results. With
  `randomness="different"` slice b draws from its own random stream (`replica_seed`); with "same" all slices
  share one. The non-tensor part of a module's state (the position in its random stream, kept in
  `get_extra_state`) is wound back before every slice, so that a mapped call advances it once, not once per slice.
"""

from __future__ import annotations

import contextlib
from typing import Any, Callable

import torch
from torch import nn
from torch.utils import _pytree as pytree

_REPLICA = 0  # slice number of the enclosing `vmap(..., randomness="different")`, 0 outside


def replica_seed(seed: int) -> int:
    """The seed a kernel uses: `seed` itself outside `vmap`, a slice-specific one inside
    `vmap(..., randomness="different")` (an odd 64-bit multiplier spreads neighbouring slices)."""
    if _REPLICA == 0:
        return seed
    return (seed ^ (_REPLICA * 0x9E3779B97F4A7C15)) & ((1 << 62) - 1)


def _owner(module: nn.Module, name: str) -> tuple[nn.Module, str]:
    *path, attr = name.split(".")
    for p in path:
        module = getattr(module, p)
    return module, attr


def _named_state(module: nn.Module) -> dict[str, torch.Tensor]:
    out = dict(module.named_parameters(remove_duplicate=False))
    out.update(dict(module.named_buffers(remove_duplicate=False)))
    return out


def _bind(owner: nn.Module, attr: str, value: torch.Tensor) -> None:
    if attr in owner._parameters:
        owner._parameters[attr] = value if isinstance(value, nn.Parameter) else nn.Parameter(value, requires_grad=False)
    else:
        owner._buffers[attr] = value


def use_state(stateful_func: Callable | nn.Module, tie_weights: bool = True, strict: bool = False) -> Callable:
    """`fn(params_and_buffers, *args, **kwargs) -> params_and_buffers | (params_and_buffers, returns)` of a
    module or of a bound method of one (evox/core/module.py:178-260). `tie_weights` is accepted for the
    signature; tied tensors are copied per name."""
    if isinstance(stateful_func, nn.Module):
        module, func = stateful_func, stateful_func.forward
    else:
        module = getattr(stateful_func, "__self__", None)
        func = stateful_func
        if not isinstance(module, nn.Module):
            raise TypeError("use_state expects a torch.nn.Module or a bound method of one")

    def state_fn(state: dict[str, torch.Tensor], *args, **kwargs):
        current = _named_state(module)
        if strict:
            missing, unexpected = set(current) - set(state), set(state) - set(current)
            if missing or unexpected:
                raise KeyError(f"use_state(strict=True): missing {sorted(missing)}, unexpected {sorted(unexpected)}")
        try:
            for name, value in state.items():
                if name in current:
                    owner, attr = _owner(module, name)
                    _bind(owner, attr, value.detach().clone())
            out = func(*args, **kwargs)
            new_state = {name: t.detach() for name, t in _named_state(module).items()}
        finally:
            for name, value in current.items():
                owner, attr = _owner(module, name)
                _bind(owner, attr, value)
        return new_state if out is None else (new_state, out)

    state_fn.__wrapped__ = func
    state_fn._evox_module = module
    return state_fn


def _extra_states(module: nn.Module) -> list[tuple[nn.Module, Any]]:
    snap = []
    for sub in module.modules():
        if type(sub).get_extra_state is not nn.Module.get_extra_state:
            snap.append((sub, sub.get_extra_state()))
    return snap


@contextlib.contextmanager
def _replica(index: int):
    global _REPLICA
    old, _REPLICA = _REPLICA, index
    try:
        yield
    finally:
        _REPLICA = old


def vmap(func: Callable, in_dims: int | tuple = 0, out_dims: int | tuple = 0, randomness: str = "error", *,
         chunk_size: int | None = None) -> Callable:
    """Map `func` over dimension `in_dims` of its tensor arguments, slice by slice (see the module text).
    `in_dims` / `out_dims`: one integer or `None` for all arguments / results, or a tuple with one entry
    per positional argument / result; an entry applies to every tensor inside that argument. `chunk_size` is
    accepted for `torch.vmap`'s signature; the slices run one at a time whatever it says."""
    del chunk_size
    if randomness not in ("error", "different", "same"):
        raise ValueError(f"randomness must be 'error', 'different' or 'same', got {randomness!r}")
    module = getattr(func, "_evox_module", None)

    def mapped(*args):
        dims = in_dims if isinstance(in_dims, tuple) else (in_dims,) * len(args)
        if len(dims) != len(args):
            raise ValueError(f"in_dims has {len(dims)} entries for {len(args)} arguments")
        sizes = set()
        for a, d in zip(args, dims):
            if d is None:
                continue
            for leaf in pytree.tree_leaves(a):
                if isinstance(leaf, torch.Tensor):
                    sizes.add(leaf.shape[d])
        if len(sizes) != 1:
            raise ValueError(f"vmap: the mapped dimensions must have one common size, got {sorted(sizes)}")
        (n,) = sizes
        snap = _extra_states(module) if module is not None else []
        results = []
        for b in range(n):
            sliced = [
                a if d is None else pytree.tree_map(lambda t: t.select(d, b) if isinstance(t, torch.Tensor) else t, a)
                for a, d in zip(args, dims)
            ]
            for sub, extra in snap:
                sub.set_extra_state(extra)
            with _replica(b + 1 if randomness == "different" else 0):
                results.append(func(*sliced))
        flat0, spec = pytree.tree_flatten(results[0])
        flats = [pytree.tree_flatten(r)[0] for r in results]
        if isinstance(out_dims, tuple):
            if not isinstance(results[0], tuple) or len(out_dims) != len(results[0]):
                raise ValueError("out_dims must have one entry per result")
            per_leaf = []
            for part, d in zip(results[0], out_dims):
                per_leaf += [d] * len(pytree.tree_leaves(part))
        else:
            per_leaf = [out_dims] * len(flat0)
        stacked = []
        for i, d in enumerate(per_leaf):
            column = [f[i] for f in flats]
            if isinstance(column[0], torch.Tensor) and d is not None:
                stacked.append(torch.stack(column, dim=d))
            else:
                stacked.append(column[0])
        return pytree.tree_unflatten(stacked, spec)

    mapped.__wrapped__ = func
    return mapped
