"""Social-learning PSO (Gaussian and uniform demonstrator sampling) with the update in one kernel launch.

Drop-ins for the reference's `SLPSOGS` and `SLPSOUS` (evox/algorithms/so/pso_variants/sl_pso_gs.py:8-104,
sl_pso_us.py:9-110): same constructor arguments, state names (`pop`, `fit`, `velocity`,
`global_best_location`, `global_best_fit`) and update rule. The demonstrator choice (a sort of the fitness
and pop_size scalars of arithmetic) stays in the reference's torch ops on the device; the update, the
clamps, the evaluation and the NEXT generation's mean position are one kernel. A particle learns from
another particle's position before the update, so the kernel writes the new swarm to a second buffer and
`pop` is rebound to it each generation (as the reference rebinds `self.pop`).
"""

from __future__ import annotations

import ctypes

import torch

from .. import _cabi
from ..core import Algorithm, Mutable, Parameter
from ..core.functional import replica_seed

__all__ = ["SLPSOGS", "SLPSOUS"]


class _SLPSO(Algorithm):
    def __init__(self, pop_size: int, lb: torch.Tensor, ub: torch.Tensor, social_influence_factor: float = 0.2,
                 demonstrator_choice_factor: float = 0.7, device: torch.device | None = None, seed: int | None = None):
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        assert lb.shape == ub.shape and lb.ndim == 1 and ub.ndim == 1 and lb.dtype == ub.dtype
        assert lb.dtype == torch.float32, "the SL-PSO kernel computes in float32"
        self.dim = lb.shape[0]
        self.pop_size = pop_size
        self.seed = int(torch.randint(0, 2**62, (), device="cpu")) if seed is None else int(seed)
        self.generation = 0
        self.social_influence_factor = Parameter(social_influence_factor, dtype=torch.float32, device=device)
        self.demonstrator_choice_factor = Parameter(demonstrator_choice_factor, dtype=torch.float32, device=device)
        self.lb = lb[None, :].to(device=device).contiguous()
        self.ub = ub[None, :].to(device=device).contiguous()
        length = self.ub - self.lb
        pop = length * torch.rand(pop_size, self.dim, device=device) + self.lb
        velocity = 2 * length * torch.rand(pop_size, self.dim, device=device) - length
        self.pop = Mutable(pop.contiguous())
        self.fit = Mutable(torch.empty(pop_size, device=device))
        self.velocity = Mutable(velocity.contiguous())
        self.global_best_location = Mutable(pop[0].clone())
        self.global_best_fit = Mutable(torch.tensor(torch.inf, device=device))
        self._scratch: dict[str, torch.Tensor] = {}
        self._center_stamp = None  # (data_ptr, version) of the pop whose mean the workspace holds

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
            raise _cabi.EvoxKernelError(f"{type(self).__name__}.step needs its state on a CUDA device; evox_b200 has no CPU path")
        for name in ("pop", "fit", "velocity", "global_best_location", "global_best_fit"):
            t = getattr(self, name)
            if not t.is_contiguous() or t.dtype != torch.float32:
                setattr(self, name, t.to(torch.float32).contiguous())
                self._center_stamp = None
        sc = self._scratch
        if "ws" not in sc or sc["ws"].device != dev:
            sc["ws"] = torch.empty(_cabi.lib.evox_slpso_workspace_bytes(self.pop_size, self.dim), dtype=torch.uint8, device=dev)
            sc["best_ws"] = torch.zeros(_cabi.lib.evox_pso_workspace_bytes(self.pop_size, self.dim), dtype=torch.uint8, device=dev)
            sc["cand"] = torch.zeros(_cabi.lib.evox_pso_candidate_words(self.dim), dtype=torch.int32, device=dev)
            sc["other"] = torch.empty_like(self.pop)
            self._center_stamp = None
        return dev

    def init_step(self):
        """sl_pso_gs.py:68-70."""
        dev = self._ready()
        plan = self._fused_plan()
        if plan is None:
            self.fit = self.evaluate(self.pop)
            self._ready()
        else:
            fitness_id, params = plan
            _cabi.check(_cabi.lib.evox_eval_fitness(_cabi.ptr(self.pop), self.pop_size, self.dim, fitness_id, _cabi.host_floats(params),
                                                    _cabi.ptr(self.fit), _cabi.stream_ptr(dev)))
            self._notify(self.pop, self.fit)
        self.global_best_fit.copy_(torch.min(self.fit))

    def _demonstrator_rows(self, pick: torch.Tensor | None, dev: torch.device) -> torch.Tensor:
        raise NotImplementedError

    def step(self, pick: torch.Tensor | None = None, r1: torch.Tensor | None = None, r2: torch.Tensor | None = None,
             r3: torch.Tensor | None = None, demonstrator_rows: torch.Tensor | None = None):
        """One generation. `pick`: the (pop_size,) draw of the demonstrator choice (standard normal for the
        Gaussian variant, uniform for the uniform one); `r1`, `r2`, `r3`: the three (pop_size, dim) uniform draws;
        `demonstrator_rows`: the chosen rows themselves (int64), bypassing the choice."""
        dev = self._ready()
        plan = self._fused_plan()
        n, sc = self.pop_size, self._scratch
        lib, s = _cabi.lib, _cabi.stream_ptr(dev)
        # global best: tracked only (sl_pso_gs.py:74-78), same rule as PSO's
        _cabi.check(lib.evox_pso_local_best(_cabi.ptr(self.fit), _cabi.ptr(self.pop), n, self.dim, 0, _cabi.ptr(sc["cand"]),
                                            _cabi.ptr(sc["best_ws"]), sc["best_ws"].numel(), s))
        _cabi.check(lib.evox_pso_merge_best(_cabi.ptr(sc["cand"]), 1, self.dim, 1, _cabi.ptr(self.global_best_location),
                                            _cabi.ptr(self.global_best_fit), s))
        if demonstrator_rows is None:
            rows = self._demonstrator_rows(pick, dev).contiguous()
        else:
            rows = demonstrator_rows.to(device=dev, dtype=torch.int64).contiguous()
            assert rows.shape == (n,)
        draws = [None if r is None else r.to(device=dev, dtype=torch.float32).contiguous() for r in (r1, r2, r3)]
        assert all(r is None for r in draws) or all(r is not None and r.shape == self.pop.shape for r in draws)
        fitness_id, params = plan if plan is not None else (-1, (0.0, 0.0, 0.0))
        stamp = (self.pop.data_ptr(), self.pop._version)
        new_pop = sc["other"]
        next_ready = ctypes.c_int32(0)
        _cabi.check(
            lib.evox_slpso_step(
                _cabi.ptr(self.pop), _cabi.ptr(new_pop), _cabi.ptr(self.velocity), _cabi.ptr(self.fit), _cabi.ptr(rows),
                _cabi.ptr(self.lb, torch.float32, "lb"), _cabi.ptr(self.ub, torch.float32, "ub"),
                _cabi.ptr(self.social_influence_factor, torch.float32, "social_influence_factor"),
                _cabi.ptr(draws[0]), _cabi.ptr(draws[1]), _cabi.ptr(draws[2]), n, self.dim, fitness_id, _cabi.host_floats(params),
                replica_seed(self.seed), self.generation, int(self._center_stamp == stamp), _cabi.ptr(sc["ws"]), sc["ws"].numel(),
                ctypes.byref(next_ready), s,
            )
        )
        self.generation += 1
        sc["other"] = self.pop.detach()
        self.pop = new_pop
        self._center_stamp = (self.pop.data_ptr(), self.pop._version) if next_ready.value else None
        if plan is None:
            self.fit = self.evaluate(self.pop)
        else:
            self._notify(self.pop, self.fit)


class SLPSOGS(_SLPSO):
    """Demonstrators drawn by Gaussian sampling over the fitness-sorted swarm (sl_pso_gs.py:80-89)."""

    def _demonstrator_rows(self, pick, dev):
        n = self.pop_size
        order = torch.argsort(self.fit, descending=True)
        sigma = self.demonstrator_choice_factor * (n - (torch.arange(n, device=dev) + 1))
        pick = torch.randn(n, device=dev) if pick is None else pick.to(device=dev, dtype=torch.float32)
        normal_distribution = sigma * (-torch.abs(pick)) + n
        index_k = torch.clamp(normal_distribution, 1, n).to(dtype=torch.int64) - 1
        return order[index_k]


class SLPSOUS(_SLPSO):
    """Demonstrators drawn uniformly from the better part of the fitness-sorted swarm (sl_pso_us.py:80-94)."""

    def _demonstrator_rows(self, pick, dev):
        n = self.pop_size
        order = torch.argsort(-self.fit)
        q = torch.clamp(n - torch.ceil(self.demonstrator_choice_factor * (n - (torch.arange(n, device=dev) + 1) - 1)), 1, n)
        pick = torch.rand(n, device=dev) if pick is None else pick.to(device=dev, dtype=torch.float32)
        uniform_distribution = pick * (n + 1 - q) + q
        index_k = torch.clamp(torch.floor(uniform_distribution).to(dtype=torch.int64) - 1, 0, n - 1)
        return order[index_k]
