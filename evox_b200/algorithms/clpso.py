"""Comprehensive-learning PSO with the generation in four small-to-large kernel launches.

Drop-in for the reference's `CLPSO` (evox/algorithms/so/pso_variants/clpso.py:8-123): same constructor
arguments, state names (`pop`, `fit`, `velocity`, `personal_best_location`, `personal_best_fit`,
`global_best_location`, `global_best_fit`) and update rule. The exemplar bookkeeping (two random
indices per particle, one comparison, one probability test: pop_size scalars) stays in torch ops on the
device; the personal-best update and the move with the fused evaluation are kernels. The uniform
coefficients come from a Philox4x32-10 stream keyed by (`seed`, generation) unless `step(...)` is given
the reference's draws.
"""

from __future__ import annotations

import torch

from .. import _cabi
from ..core import Algorithm, Mutable, Parameter
from ..core.functional import replica_seed

__all__ = ["CLPSO"]


class CLPSO(Algorithm):
    def __init__(
        self,
        pop_size: int,
        lb: torch.Tensor,
        ub: torch.Tensor,
        inertia_weight: float = 0.5,
        const_coefficient: float = 1.5,
        learning_probability: float = 0.05,
        device: torch.device | None = None,
        seed: int | None = None,
    ):
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        assert lb.shape == ub.shape and lb.ndim == 1 and ub.ndim == 1 and lb.dtype == ub.dtype
        assert lb.dtype == torch.float32, "the CLPSO kernels compute in float32"
        self.pop_size = pop_size
        self.dim = lb.shape[0]
        self.seed = int(torch.randint(0, 2**62, (), device="cpu")) if seed is None else int(seed)
        self.generation = 0
        self.lb = lb[None, :].to(device=device).contiguous()
        self.ub = ub[None, :].to(device=device).contiguous()
        self.w = Parameter(inertia_weight, dtype=torch.float32, device=device)
        self.c = Parameter(const_coefficient, dtype=torch.float32, device=device)
        self.P_c = Parameter(learning_probability, dtype=torch.float32, device=device)
        length = self.ub - self.lb
        pop = length * torch.rand(pop_size, self.dim, device=device) + self.lb
        velocity = 2 * length * torch.rand(pop_size, self.dim, device=device) - length
        self.pop = Mutable(pop.contiguous())
        self.fit = Mutable(torch.empty(pop_size, device=device))
        self.velocity = Mutable(velocity.contiguous())
        self.personal_best_location = Mutable(pop.clone())
        self.personal_best_fit = Mutable(torch.full((pop_size,), torch.inf, device=device))
        self.global_best_location = Mutable(pop[0].clone())
        self.global_best_fit = Mutable(torch.tensor(torch.inf, device=device))
        self._scratch: dict[str, torch.Tensor] = {}

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
            raise _cabi.EvoxKernelError("CLPSO.step needs its state on a CUDA device; evox_b200 has no CPU path")
        for name in ("pop", "fit", "velocity", "personal_best_location", "personal_best_fit", "global_best_location", "global_best_fit"):
            t = getattr(self, name)
            if not t.is_contiguous() or t.dtype != torch.float32:
                setattr(self, name, t.to(torch.float32).contiguous())
        if self.personal_best_location.data_ptr() == self.pop.data_ptr():
            # a loaded reference state may alias the two (clpso.py:58-62 wraps the same tensor twice)
            self.personal_best_location = self.personal_best_location.clone()
        if "ws" not in self._scratch or self._scratch["ws"].device != dev:
            nbytes = _cabi.lib.evox_pso_workspace_bytes(self.pop_size, self.dim)
            self._scratch["ws"] = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
            self._scratch["cand"] = torch.zeros(_cabi.lib.evox_pso_candidate_words(self.dim), dtype=torch.int32, device=dev)
        return dev

    def _evaluate_into_fit(self, dev, plan):
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

    def init_step(self):
        """clpso.py:67-70."""
        dev = self._ready()
        self._evaluate_into_fit(dev, self._fused_plan())
        self._ready()
        self.personal_best_fit.copy_(self.fit)
        self.global_best_fit.copy_(torch.min(self.fit))

    def step(self, random_coefficient: torch.Tensor | None = None, rand1_index: torch.Tensor | None = None,
             rand2_index: torch.Tensor | None = None, rand_possibility: torch.Tensor | None = None):
        """One generation (clpso.py:72-123); the four optional arguments are the draws of :92-95."""
        dev = self._ready()
        plan = self._fused_plan()
        n = self.pop_size
        lib, s = _cabi.lib, _cabi.stream_ptr(dev)
        r1 = torch.randint(0, n, (n,), device=dev) if rand1_index is None else rand1_index.to(device=dev, dtype=torch.int64)
        r2 = torch.randint(0, n, (n,), device=dev) if rand2_index is None else rand2_index.to(device=dev, dtype=torch.int64)
        poss = torch.rand(n, device=dev) if rand_possibility is None else rand_possibility.to(device=dev, dtype=torch.float32)
        if random_coefficient is not None:
            random_coefficient = random_coefficient.to(device=dev, dtype=torch.float32).contiguous()
            assert random_coefficient.shape == self.pop.shape
        # exemplar of every particle, from the personal bests BEFORE this generation's update (clpso.py:95-99)
        learning_index = torch.where(self.personal_best_fit[r1] < self.personal_best_fit[r2], r1, r2)
        source_rows = torch.where(poss < self.P_c, learning_index, torch.arange(n, device=dev)).contiguous()
        # global best: tracked only (clpso.py:105-108), same rule as PSO's
        ws, cand = self._scratch["ws"], self._scratch["cand"]
        _cabi.check(lib.evox_pso_local_best(_cabi.ptr(self.fit), _cabi.ptr(self.pop), n, self.dim, 0, _cabi.ptr(cand), _cabi.ptr(ws), ws.numel(), s))
        _cabi.check(lib.evox_pso_merge_best(_cabi.ptr(cand), 1, self.dim, 1, _cabi.ptr(self.global_best_location), _cabi.ptr(self.global_best_fit), s))
        _cabi.check(lib.evox_clpso_update_pbest(_cabi.ptr(self.pop), _cabi.ptr(self.fit), _cabi.ptr(self.personal_best_location),
                                                _cabi.ptr(self.personal_best_fit), n, self.dim, s))
        fitness_id, params = plan if plan is not None else (-1, (0.0, 0.0, 0.0))
        _cabi.check(
            lib.evox_clpso_move_eval(
                _cabi.ptr(self.pop), _cabi.ptr(self.velocity), _cabi.ptr(self.personal_best_location), _cabi.ptr(self.fit),
                _cabi.ptr(source_rows), _cabi.ptr(self.lb, torch.float32, "lb"), _cabi.ptr(self.ub, torch.float32, "ub"),
                _cabi.ptr(self.w, torch.float32, "w"), _cabi.ptr(self.c, torch.float32, "c"), _cabi.ptr(random_coefficient),
                n, self.dim, fitness_id, _cabi.host_floats(params), replica_seed(self.seed), self.generation, s,
            )
        )
        self.generation += 1
        if plan is None:
            self.fit = self.evaluate(self.pop)
        else:
            self._notify(self.pop, self.fit)
