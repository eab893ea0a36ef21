"""Differential evolution (rand/1/bin, best/1/bin) with the generation in two kernel launches.

Drop-in for the reference's `DE` (evox/algorithms/so/de_variants/de.py:8-157) with one difference
vector: same constructor arguments, state names (`pop`, `fit`) and update rule. The index draws stay
`torch.randint` on the device (pop_size scalars each, with replacement as in the reference); mutation,
binomial crossover, clamp and the evaluation of the trials are one kernel, the one-to-one selection a
second one. The crossover draws come from a Philox4x32-10 stream keyed by (`seed`, generation) unless
`step(...)` is given the reference's tensors.
"""

from __future__ import annotations

from typing import Literal

import torch

from .. import _cabi
from ..core import Algorithm, Mutable, Parameter
from ..core.functional import replica_seed
from ..problems.numerical import _relu_clamp_rows

__all__ = ["DE"]


class DE(Algorithm):
    def __init__(
        self,
        pop_size: int,
        lb: torch.Tensor,
        ub: torch.Tensor,
        base_vector: Literal["best", "rand"] = "rand",
        num_difference_vectors: int = 1,
        differential_weight: float | torch.Tensor = 0.5,
        cross_probability: float = 0.9,
        mean: torch.Tensor | None = None,
        stdev: torch.Tensor | None = None,
        device: torch.device | None = None,
        seed: int | None = None,
    ):
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        assert pop_size >= 4
        assert 0 < cross_probability <= 1
        assert base_vector in ["rand", "best"]
        assert lb.shape == ub.shape and lb.ndim == 1 and ub.ndim == 1 and lb.dtype == ub.dtype
        assert lb.dtype == torch.float32, "the DE kernels compute in float32"
        if num_difference_vectors != 1:
            raise _cabi.EvoxKernelError("evox_b200.DE supports one difference vector (rand/1 and best/1)")
        assert isinstance(differential_weight, float)
        self.pop_size = pop_size
        self.dim = lb.shape[0]
        self.best_vector = base_vector == "best"
        self.num_difference_vectors = 1
        self.seed = int(torch.randint(0, 2**62, (), device="cpu")) if seed is None else int(seed)
        self.generation = 0
        self.differential_weight = Parameter(differential_weight, dtype=torch.float32, device=device)
        self.cross_probability = Parameter(cross_probability, dtype=torch.float32, device=device)
        self.lb = lb[None, :].to(device=device).contiguous()
        self.ub = ub[None, :].to(device=device).contiguous()
        if mean is not None and stdev is not None:
            pop = mean.to(device) + stdev.to(device) * torch.randn(pop_size, self.dim, device=device)
            pop = _relu_clamp_rows(pop, self.lb, self.ub)
        else:
            pop = torch.rand(pop_size, self.dim, device=device) * (self.ub - self.lb) + self.lb
        self.pop = Mutable(pop.contiguous())
        self.fit = Mutable(torch.full((pop_size,), torch.inf, device=device))
        self._trial: torch.Tensor | None = None
        self._trial_fit: torch.Tensor | None = None

    def get_extra_state(self):
        return {"seed": self.seed, "generation": self.generation}

    def set_extra_state(self, state):
        self.seed = int(state["seed"])
        self.generation = int(state["generation"])

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        if "_extra_state" not in state_dict:  # a state_dict written by the reference
            state_dict = dict(state_dict)
            state_dict["_extra_state"] = self.get_extra_state()
        return super().load_state_dict(state_dict, strict=strict, assign=assign)

    def _fused_plan(self):
        planner = getattr(self, "_workflow_fused_plan", None)
        return planner() if planner is not None else None

    def _notify(self, pop, fit):
        notify = getattr(self, "_workflow_fused_notify", None)
        if notify is not None:
            notify(pop, fit)

    def _ready(self) -> torch.device:
        dev = self.pop.device
        if dev.type != "cuda":
            raise _cabi.EvoxKernelError("DE.step needs its state on a CUDA device; evox_b200 has no CPU path")
        for name in ("pop", "fit"):
            t = getattr(self, name)
            if not t.is_contiguous() or t.dtype != torch.float32:
                setattr(self, name, t.to(torch.float32).contiguous())
        if self._trial is None or self._trial.device != dev:
            self._trial = torch.empty_like(self.pop)
            self._trial_fit = torch.empty_like(self.fit)
        return dev

    def init_step(self):
        """de.py:92-99."""
        dev = self._ready()
        plan = self._fused_plan()
        if plan is None:
            self.fit = self.evaluate(self.pop)
            return
        fitness_id, params = plan
        _cabi.check(_cabi.lib.evox_eval_fitness(_cabi.ptr(self.pop), self.pop_size, self.dim, fitness_id, _cabi.host_floats(params),
                                                _cabi.ptr(self.fit), _cabi.stream_ptr(dev)))
        self._notify(self.pop, self.fit)

    def step(self, random_choices: list[torch.Tensor] | None = None, cross_prob: torch.Tensor | None = None,
             random_dim: torch.Tensor | None = None):
        """One generation (de.py:101-157). `random_choices`: the index draws of de.py:112-113 (three tensors for
        base "rand", two for "best"); `cross_prob`: the (pop_size, dim) uniform draw; `random_dim`: the
        (pop_size, 1) column that always crosses over."""
        dev = self._ready()
        plan = self._fused_plan()
        n = self.pop_size
        n_idx = 2 if self.best_vector else 3
        if random_choices is None:
            random_choices = [torch.randint(0, n, (n,), device=dev) for _ in range(n_idx)]
        idx = [r.to(device=dev, dtype=torch.int64).contiguous() for r in random_choices]
        assert len(idx) == n_idx and all(r.shape == (n,) for r in idx)
        forced = torch.randint(0, self.dim, (n, 1), device=dev) if random_dim is None else random_dim.to(device=dev, dtype=torch.int64)
        forced = forced.reshape(n).contiguous()
        if cross_prob is not None:
            cross_prob = cross_prob.to(device=dev, dtype=torch.float32).contiguous()
            assert cross_prob.shape == self.pop.shape
        best = torch.argmin(self.fit).reshape(1) if self.best_vector else None
        base_rows = None if self.best_vector else idx[0]
        rows_a, rows_b = (idx[0], idx[1]) if self.best_vector else (idx[1], idx[2])
        fitness_id, params = plan if plan is not None else (-1, (0.0, 0.0, 0.0))
        lib, s = _cabi.lib, _cabi.stream_ptr(dev)
        _cabi.check(
            lib.evox_de_trial(
                _cabi.ptr(self.pop), _cabi.ptr(self._trial), _cabi.ptr(self._trial_fit), _cabi.ptr(base_rows), _cabi.ptr(best),
                _cabi.ptr(rows_a), _cabi.ptr(rows_b), _cabi.ptr(forced), _cabi.ptr(self.lb, torch.float32, "lb"),
                _cabi.ptr(self.ub, torch.float32, "ub"), _cabi.ptr(self.differential_weight, torch.float32, "differential_weight"),
                _cabi.ptr(self.cross_probability, torch.float32, "cross_probability"), _cabi.ptr(cross_prob), n, self.dim,
                fitness_id, _cabi.host_floats(params), replica_seed(self.seed), self.generation, s,
            )
        )
        self.generation += 1
        if plan is None:
            self._trial_fit = self.evaluate(self._trial).to(torch.float32).contiguous()
        else:
            self._notify(self._trial, self._trial_fit)
        _cabi.check(lib.evox_de_select(_cabi.ptr(self._trial), _cabi.ptr(self._trial_fit), _cabi.ptr(self.pop), _cabi.ptr(self.fit), n,
                                       self.dim, s))
