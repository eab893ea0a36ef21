"""Competitive swarm optimiser with the generation in two kernel launches.

Drop-in for the reference's `CSO` (evox/algorithms/so/pso_variants/cso.py:8-105): same constructor
arguments, same state names (`pop`, `fit`, `velocity`), same update rule — including the fact that the
reference never stores the students' new velocities. What differs:

* the students' rows of `pop` / `fit` are updated in place by the kernel;
* when the workflow reports that the problem is one the kernel can evaluate itself (Ackley /
  Rastrigin / Sphere without shift, affine or transforms) the evaluation is fused into the update;
* the three uniform draws come from a Philox4x32-10 stream keyed by (`seed`, generation) unless
  `step(perm=..., lambdas=...)` supplies them; the random pairing is `torch.randperm` on the device;
* the swarm's mean position for the next generation is accumulated by the update kernel itself
  whenever rows have at most 1,024 floats, so the swarm is not read a second time for it.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _cabi
from ..core import Algorithm, Mutable, Parameter
from ..core.functional import replica_seed
from ..problems.numerical import _relu_clamp_rows

__all__ = ["CSO"]


class CSO(Algorithm):
    def __init__(
        self,
        pop_size: int,
        lb: torch.Tensor,
        ub: torch.Tensor,
        phi: float = 0.0,
        mean: torch.Tensor | None = None,
        stdev: torch.Tensor | None = None,
        device: torch.device | None = None,
        seed: int | None = None,
        store_velocity: bool = False,
    ):
        """
        :param pop_size: number of particles; must be even (the reference pairs all of them).
        :param lb, ub: 1-D lower / upper position bounds of equal shape, float32.
        :param phi: weight of the pull towards the swarm's mean position.
        :param mean, stdev: if both given, the initial swarm is normal(mean, stdev) clamped to the bounds.
        :param seed: key of the in-kernel random stream; drawn from torch's CPU generator if None.
        :param store_velocity: False (default) reproduces the reference, which never writes the students'
            new velocities back (cso.py:98-105), so the initial velocities act in every generation and the
            swarm does not contract; True stores them, as the original algorithm does.
        """
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        assert lb.shape == ub.shape and lb.ndim == 1 and ub.ndim == 1 and lb.dtype == ub.dtype
        assert lb.dtype == torch.float32, "the CSO kernels compute in float32"
        assert pop_size % 2 == 0 and pop_size >= 2, "CSO pairs the whole swarm: pop_size must be even"
        self.pop_size = pop_size
        self.dim = lb.shape[0]
        self.seed = int(torch.randint(0, 2**62, (), device="cpu")) if seed is None else int(seed)
        self.generation = 0
        self.store_velocity = bool(store_velocity)
        self.phi = Parameter(phi, dtype=torch.float32, device=device)
        lb = lb[None, :].to(device=device).contiguous()
        ub = ub[None, :].to(device=device).contiguous()
        length = ub - lb
        self.lb = lb
        self.ub = ub
        if mean is not None and stdev is not None:
            pop = mean.to(device) + stdev.to(device) * torch.randn(pop_size, self.dim, device=device)
            pop = _relu_clamp_rows(pop, lb, ub)
        else:
            pop = torch.rand(pop_size, self.dim, device=device) * (ub - lb) + lb
        velocity = 2 * length * torch.rand(pop_size, self.dim, device=device) - length
        self.pop = Mutable(pop.contiguous())
        self.fit = Mutable(torch.empty(pop_size, device=device))
        self.velocity = Mutable(velocity.contiguous())
        self._ws: torch.Tensor | None = None
        self._center_stamp = None  # (data_ptr, version) of pop when the workspace holds its mean

    def get_extra_state(self):
        return {"seed": self.seed, "generation": self.generation}

    def set_extra_state(self, state):
        self.seed = int(state["seed"])
        self.generation = int(state["generation"])
        self._center_stamp = None

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        if "_extra_state" not in state_dict:  # a state_dict written by the reference
            state_dict = dict(state_dict)
            state_dict["_extra_state"] = self.get_extra_state()
        self._center_stamp = None
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
            raise _cabi.EvoxKernelError("CSO.step needs its state on a CUDA device; evox_b200 has no CPU path")
        for name in ("pop", "fit", "velocity"):
            t = getattr(self, name)
            if not t.is_contiguous() or t.dtype != torch.float32:
                setattr(self, name, t.to(torch.float32).contiguous())
                self._center_stamp = None
        if self._ws is None or self._ws.device != dev:
            nbytes = _cabi.lib.evox_cso_workspace_bytes(self.pop_size, self.dim)
            self._ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            self._center_stamp = None
        return dev

    def init_step(self):
        """cso.py:68-69."""
        dev = self._ready()
        plan = self._fused_plan()
        if plan is None:
            self.fit = self.evaluate(self.pop)
            return
        fitness_id, params = plan
        _cabi.check(
            _cabi.lib.evox_eval_fitness(
                _cabi.ptr(self.pop), self.pop_size, self.dim, fitness_id, _cabi.host_floats(params),
                _cabi.ptr(self.fit), _cabi.stream_ptr(dev),
            )
        )
        self._notify(self.pop, self.fit)

    def step(self, perm: torch.Tensor | None = None, lambdas: torch.Tensor | None = None):
        """One generation (cso.py:71-105). `perm`: optional permutation of range(pop_size) (int64);
        `lambdas`: optional (3, pop_size // 2, dim) uniform draws."""
        dev = self._ready()
        plan = self._fused_plan()
        half = self.pop_size // 2
        if perm is None:
            perm = torch.randperm(self.pop_size, device=dev)
        perm = perm.to(device=dev, dtype=torch.int64).contiguous()
        assert perm.shape == (self.pop_size,)
        if lambdas is not None:
            lambdas = lambdas.to(device=dev, dtype=torch.float32).contiguous()
            assert lambdas.shape == (3, half, self.dim)
        candidates = students = None
        if plan is None:
            fitness_id, params = -1, (0.0, 0.0, 0.0)
            candidates = torch.empty(half, self.dim, dtype=torch.float32, device=dev)
            students = torch.empty(half, dtype=torch.int64, device=dev)
        else:
            fitness_id, params = plan
        stamp = (self.pop.data_ptr(), self.pop._version)
        next_ready = ctypes.c_int32(0)
        _cabi.check(
            _cabi.lib.evox_cso_step(
                _cabi.ptr(self.pop), _cabi.ptr(self.velocity), int(self.store_velocity), _cabi.ptr(self.fit), _cabi.ptr(perm),
                _cabi.ptr(self.lb, torch.float32, "lb"), _cabi.ptr(self.ub, torch.float32, "ub"),
                _cabi.ptr(self.phi, torch.float32, "phi"), _cabi.ptr(lambdas), self.pop_size, self.dim, fitness_id,
                _cabi.host_floats(params), replica_seed(self.seed), self.generation, int(self._center_stamp == stamp),
                _cabi.ptr(candidates), _cabi.ptr(students), _cabi.ptr(self._ws), self._ws.numel(),
                ctypes.byref(next_ready), _cabi.stream_ptr(dev),
            )
        )
        self.generation += 1
        # the kernel wrote through raw pointers: torch's version counter of pop did not move
        self._center_stamp = stamp if next_ready.value else None
        if plan is None:
            self.fit[students] = self.evaluate(candidates)
        else:
            self._notify(self.pop, self.fit)
