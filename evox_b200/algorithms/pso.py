"""Particle swarm optimisation with the whole generation in one kernel launch.

Drop-in for the reference's `PSO` (evox/algorithms/so/pso_variants/pso.py:9-115): same
constructor arguments, same state names (`pop`, `velocity`, `fit`, `local_best_location`,
`local_best_fit`, `global_best_location`, `global_best_fit`), same update rule. What differs:

* the state tensors are updated in place by the kernels instead of being rebound each step;
* when the workflow reports that the problem is one the update kernel can evaluate itself
  (Ackley / Rastrigin / Sphere without shift, affine or transforms) the evaluation is fused
  into the update and `Problem.evaluate` is not called;
* the uniform draws come from a Philox4x32-10 stream keyed by (`seed`, generation) unless
  `step(rg=..., rp=...)` supplies them (pso.py:96-97 draws rg first, then rp);
* with `shard=True` under an initialised `torch.distributed` group each rank holds only its
  rows; one allgather of a (dim + 4)-word best-particle record per generation keeps the
  global best identical on all ranks.

The global-best search of generation g + 1 (min_by over the fitness generation g produced,
pso.py:92-95) rides on the kernel of generation g: its tail leaves this shard's best-particle
record, the head of the next launch folds the records into the running best. The record is
only trusted while `pop` and `fit` are the tensors the kernel left (same storage, same
version counter); after a `load_state_dict`, a torch-side write or an evaluation outside the
kernel it is rebuilt from `fit` with one extra launch.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _cabi
from ..core import Algorithm, Mutable, Parameter
from ..core.functional import replica_seed
from ..problems.numerical import FIT_SPHERE
from ..sharding import allgather_records, group_info, shard_bounds

_INIT_GENERATION = (1 << 64) - 1  # Philox generation slot reserved for the initial swarm


class PSO(Algorithm):
    def __init__(
        self,
        pop_size: int,
        lb: torch.Tensor,
        ub: torch.Tensor,
        w: float = 0.6,
        phi_p: float = 2.5,
        phi_g: float = 0.8,
        device: torch.device | None = None,
        shard: bool = False,
        group=None,
        seed: int | None = None,
        peer_exchange: bool = True,
    ):
        """
        :param pop_size: number of particles (of the WHOLE swarm when `shard=True`).
        :param lb, ub: 1-D lower / upper position bounds of equal shape and dtype float32.
        :param w, phi_p, phi_g: inertia, cognitive and social weights.
        :param device: where the state lives; must be a CUDA device to step.
        :param shard: split the particles over the ranks of `group`.
        :param peer_exchange: sharded swarms only: let the generation kernels write their best-particle records
            straight into the other GPUs' memory (one launch per generation, no collective call); falls back to
            one NCCL allgather per generation when the ranks cannot map each other's memory.
        :param seed: key of the in-kernel random stream; drawn from torch's CPU generator if None,
            so `torch.manual_seed` makes runs repeatable (and equal on every rank).
        """
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        assert lb.shape == ub.shape and lb.ndim == 1 and ub.ndim == 1 and lb.dtype == ub.dtype
        assert lb.dtype == torch.float32, "the PSO kernels compute in float32"
        self.pop_size = pop_size
        self.dim = lb.shape[0]
        self.group = group
        self.rank, self.world_size = group_info(group) if shard else (0, 1)
        self.row_start, self.row_end = shard_bounds(pop_size, self.world_size, self.rank)
        self.local_size = self.row_end - self.row_start
        assert self.local_size > 0, "every rank needs at least one particle"
        self.seed = int(torch.randint(0, 2**62, (), device="cpu")) if seed is None else int(seed)
        # position in the random stream: a 0-d HOST tensor, so that a traced step can hand it to the operator
        # that reads and advances it (`generation` below is its integer view)
        self._generation = torch.zeros((), dtype=torch.int64)
        # hyper-parameters stay 0-d device tensors: the kernels read them without a host sync
        self.w = Parameter(w, dtype=torch.float32, device=device)
        self.phi_p = Parameter(phi_p, dtype=torch.float32, device=device)
        self.phi_g = Parameter(phi_g, dtype=torch.float32, device=device)
        lb = lb[None, :].to(device=device).contiguous()
        ub = ub[None, :].to(device=device).contiguous()
        length = ub - lb
        n, d = self.local_size, self.dim
        if device.type == "cuda":
            u_pop = torch.empty(n, d, dtype=torch.float32, device=device)
            u_vel = torch.empty(n, d, dtype=torch.float32, device=device)
            for which, out in ((0, u_pop), (1, u_vel)):
                _cabi.check(
                    _cabi.lib.evox_pso_fill_uniform(
                        _cabi.ptr(out), n, d, self.seed, _INIT_GENERATION, which, self.row_start, _cabi.stream_ptr(device)
                    )
                )
        else:  # host-only construction (state inspection, checkpoints); stepping needs CUDA
            u_pop = torch.rand(n, d, device=device)
            u_vel = torch.rand(n, d, device=device)
        pop = length * u_pop + lb
        velocity = 2 * length * u_vel - length
        self.lb = lb
        self.ub = ub
        self.pop = Mutable(pop)
        self.velocity = Mutable(velocity)
        self.fit = Mutable(torch.full((n,), torch.inf, device=device))
        self.local_best_location = Mutable(pop.clone())
        self.local_best_fit = Mutable(torch.full((n,), torch.inf, device=device))
        self.global_best_location = Mutable(pop[0].clone())
        self.global_best_fit = Mutable(torch.tensor(torch.inf, device=device))
        self._scratch: dict[str, torch.Tensor] = {}
        self._checked_ptrs = None  # storage addresses of the state the last argument check saw
        self._cur = 0              # which of the two record buffers holds this shard's latest record
        self._pending = None       # (swarm key, gathered records) left by the last fused generation
        # sharded swarm: the records are exchanged by the kernels themselves over peer memory when the ranks can
        # map each other's exchange buffers (None: not tried yet, False: unavailable -> NCCL allgather)
        self.peer_exchange = peer_exchange
        self._peer = None
        # measurement hook: when a list, step() appends a (start, end) CUDA-event pair around the
        # generation kernel (on several GPUs the allgather that follows stays outside the pair)
        self._kernel_events: list | None = None

    @property
    def generation(self) -> int:
        return int(self._generation)

    @generation.setter
    def generation(self, value: int) -> None:
        self._generation.fill_(int(value))

    # -- checkpointing of the random stream position ------------------------------------------
    def get_extra_state(self):
        return {"seed": self.seed, "generation": self.generation}

    def set_extra_state(self, state):
        self.seed = int(state["seed"])
        self.generation = int(state["generation"])

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        # a state_dict written by the reference has no random-stream entry: keep ours
        if "_extra_state" not in state_dict:
            state_dict = dict(state_dict)
            state_dict["_extra_state"] = self.get_extra_state()
        return super().load_state_dict(state_dict, strict=strict, assign=assign)

    # -- kernel plumbing -----------------------------------------------------------------------
    _STATE = ("pop", "velocity", "local_best_location", "local_best_fit", "fit", "global_best_location", "global_best_fit")

    def _buffers_ready(self) -> torch.device:
        dev = self.pop.device
        if dev.type != "cuda":
            raise _cabi.EvoxKernelError("PSO.step needs its state on a CUDA device; evox_b200 has no CPU path")
        for name in self._STATE:
            t = getattr(self, name)
            if not t.is_contiguous() or t.dtype != torch.float32:
                setattr(self, name, t.to(torch.float32).contiguous())
        if self.local_best_location.data_ptr() == self.pop.data_ptr():
            # a loaded reference state may alias the two (pso.py:63-66 wraps the same tensor twice)
            self.local_best_location = self.local_best_location.clone()
        if "ws" not in self._scratch or self._scratch["ws"].device != dev:
            nbytes = _cabi.lib.evox_pso_workspace_bytes(self.local_size, self.dim)
            self._scratch["ws"] = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
            words = _cabi.lib.evox_pso_candidate_words(self.dim)
            # two records of this shard (the kernel reads one generation's while it writes the next one's)
            self._scratch["cand"] = torch.zeros(2, words, dtype=torch.int32, device=dev)
            self._scratch["gathered"] = torch.zeros(self.world_size, words, dtype=torch.int32, device=dev)
            self._pending = None
        return dev

    def _fused_plan(self):
        planner = getattr(self, "_workflow_fused_plan", None)
        return planner() if planner is not None else None

    def _swarm_key(self):
        pop, fit = self.pop, self.fit
        return (pop.data_ptr(), pop._version, fit.data_ptr(), fit._version)

    def _gather(self, record: torch.Tensor) -> torch.Tensor:
        """Every shard's record in rank order: the record itself on one GPU, one allgather otherwise."""
        if self.world_size == 1:
            return record
        return allgather_records(record, self.group, out=self._scratch["gathered"])

    def _setup_peer_exchange(self, dev: torch.device) -> None:
        """Exchange buffers the ranks can write into each other (torch's symmetric memory: plain peer mappings
        over NVLink; no multicast object is bound). Every rank ends with the same answer."""
        import os

        import torch.distributed as dist

        ok, peer = 1, None
        try:
            if self.world_size > 16:
                raise RuntimeError("the peer exchange serves at most 16 ranks")
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem

            words = (_cabi.lib.evox_pso_exchange_words(self.dim, self.world_size) + 3) // 4 * 4
            buf = symm_mem.empty(words, dtype=torch.int32, device=dev)
            handle = symm_mem.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
            buf.zero_()
            ptrs = [int(p) for p in handle.buffer_ptrs]
            if len(ptrs) != self.world_size or any(p == 0 for p in ptrs):
                raise RuntimeError("symmetric memory gave no peer addresses")
            peer = {"buf": buf, "handle": handle, "ptrs": (ctypes.c_uint64 * self.world_size)(*ptrs),
                    "status": torch.zeros(1, dtype=torch.int32, device=dev), "tag": 1}
        except Exception as exc:  # unavailable on this machine / build: the NCCL path serves
            ok, self._peer_error = 0, f"{type(exc).__name__}: {exc}"
        flag = torch.tensor([ok], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)  # also orders the zero-fill before any peer write
        torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)
        self._peer = peer if int(flag.item()) == 1 else False

    def exchange_status(self) -> int:
        """0, or 1 when a kernel's wait for another GPU's record ran out (synchronises the device)."""
        return int(self._peer["status"]) if self._peer else 0

    def _rebuild_records(self, dev: torch.device) -> torch.Tensor:
        """This shard's best-particle record from `fit` and `pop` as they are now, gathered."""
        ws, cand = self._scratch["ws"], self._scratch["cand"][self._cur]
        _cabi.check(
            _cabi.lib.evox_pso_local_best(
                _cabi.ptr(self.fit), _cabi.ptr(self.pop), self.local_size, self.dim, self.row_start,
                _cabi.ptr(cand), _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(dev),
            )
        )
        return self._gather(cand)

    def _update_global_best(self, dev: torch.device, have_previous: bool) -> torch.Tensor:
        records = self._rebuild_records(dev)
        _cabi.check(
            _cabi.lib.evox_pso_merge_best(
                _cabi.ptr(records), self.world_size, self.dim, int(have_previous),
                _cabi.ptr(self.global_best_location), _cabi.ptr(self.global_best_fit), _cabi.stream_ptr(dev),
            )
        )
        return records

    def step(self, rg: torch.Tensor | None = None, rp: torch.Tensor | None = None):
        """One generation (pso.py:71-106). `rg`, `rp`: optional (local_size, dim) uniform draws."""
        if torch.compiler.is_compiling():
            return self._step_traced(rg, rp)
        ptrs = tuple(getattr(self, n).data_ptr() for n in self._STATE)
        if ptrs != self._checked_ptrs:
            dev = self._buffers_ready()
            self._checked_ptrs = tuple(getattr(self, n).data_ptr() for n in self._STATE)
            self._static_args = (
                _cabi.ptr(self.lb, torch.float32, "lb"), _cabi.ptr(self.ub, torch.float32, "ub"),
                _cabi.ptr(self.w, torch.float32, "w"), _cabi.ptr(self.phi_p, torch.float32, "phi_p"),
                _cabi.ptr(self.phi_g, torch.float32, "phi_g"),
            )
            self._device = dev
        dev = self._device
        plan = self._fused_plan()
        fitness_id, params = plan if plan is not None else (FIT_SPHERE, (0.0, 0.0, 0.0))
        if (rg is None) != (rp is None):
            raise _cabi.EvoxKernelError("rg and rp must be given together")
        if rg is not None:
            rg, rp = rg.contiguous(), rp.contiguous()
            assert rg.shape == self.pop.shape and rp.shape == self.pop.shape
        lib, s = _cabi.lib, _cabi.stream_ptr(dev)
        ws = self._scratch["ws"]
        state = tuple(_cabi.ptr(getattr(self, n)) for n in self._STATE)
        args = (
            *self._static_args, _cabi.ptr(rg, torch.float32, "rg"), _cabi.ptr(rp, torch.float32, "rp"),
            self.local_size, self.dim, fitness_id, _cabi.host_floats(params), replica_seed(self.seed), self.generation,
        )
        if plan is None:
            # the problem is evaluated outside: two launches, nothing carried to the next generation
            self._update_global_best(dev, have_previous=True)
            _cabi.check(lib.evox_pso_move_eval(*state[:6], *args, self.row_start, s))
            self._pending = None
        else:
            if self.world_size > 1 and self.peer_exchange and self._peer is None:
                self._setup_peer_exchange(dev)
            stale = self._pending is None or self._pending[0] != self._swarm_key()
            if self.world_size > 1 and self._peer:
                peer = self._peer
                tag = peer["tag"]
                if stale or self._pending[1] is not None:
                    # The records are not in the exchange buffer (first generation, or the swarm was written
                    # between generations): take them from init_step or rebuild them (one launch + one NCCL
                    # allgather, which also orders every rank's earlier kernels before this write) and place them
                    # where the kernel's head looks: slot (tag & 1) of this rank's buffer, flags = tag. Every rank
                    # must take this branch in the same generation, as with any collective.
                    records = self._rebuild_records(dev) if stale else self._pending[1]
                    words, g = records.shape[1], self.world_size
                    base = (tag & 1) * g * words
                    peer["buf"][base : base + g * words].copy_(records.view(-1))
                    flags = 2 * g * words + (tag & 1) * g
                    peer["buf"][flags : flags + g].fill_(tag if tag < 2**31 else tag - 2**32)
                if self._kernel_events is not None:
                    pair = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    pair[0].record()
                _cabi.check(
                    lib.evox_pso_generation_peer(
                        *state, *args, self.row_start, peer["ptrs"], self.world_size, self.rank, tag, _cabi.ptr(peer["status"]),
                        _cabi.ptr(ws), ws.numel(), s,
                    )
                )
                if self._kernel_events is not None:
                    pair[1].record()
                    self._kernel_events.append(pair)
                peer["tag"] = 1 if tag == 2**32 - 1 else tag + 1
                self._pending = (self._swarm_key(), None)
                if self.generation % 256 == 255 and int(peer["status"]) != 0:  # one host read per 256 generations
                    raise _cabi.EvoxKernelError("PSO: a wait for another GPU's best-particle record timed out")
            else:
                records = self._rebuild_records(dev) if stale else self._pending[1]
                self._cur ^= 1
                out = self._scratch["cand"][self._cur]
                if self._kernel_events is not None:
                    pair = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    pair[0].record()
                _cabi.check(
                    lib.evox_pso_generation(
                        *state, *args, self.row_start, _cabi.ptr(records), self.world_size, _cabi.ptr(out),
                        _cabi.ptr(ws), ws.numel(), s,
                    )
                )
                if self._kernel_events is not None:
                    pair[1].record()
                    self._kernel_events.append(pair)
                self._pending = (self._swarm_key(), self._gather(out))
        self.generation += 1
        if plan is None:
            self.fit = self.evaluate(self.pop)
        else:
            self._workflow_notify(self.pop, self.fit)

    def _step_traced(self, rg, rp):
        """The generation as ONE registered operator (`evox_b200::pso_step`), for torch.compile: no storage
        addresses, version counters or Python integers are read here. It is the two-launch form, which carries
        nothing between calls; the operator bumps the version counters of the state it writes, so an eager step
        afterwards rebuilds its best-particle record."""
        from .. import ops

        if self.world_size != 1:
            raise _cabi.EvoxKernelError("a traced PSO.step runs on one GPU; step a sharded swarm eagerly")
        plan = self._fused_plan()
        fitness_id, params = plan if plan is not None else (FIT_SPHERE, (0.0, 0.0, 0.0))
        ops.pso_step(self.pop, self.velocity, self.local_best_location, self.local_best_fit, self.fit, self.global_best_location,
                     self.global_best_fit, self.lb, self.ub, self.w, self.phi_p, self.phi_g, rg, rp, fitness_id,
                     [float(p) for p in params], self.seed, self._generation)
        if plan is None:
            self.fit = self.evaluate(self.pop)
        else:
            self._workflow_notify(self.pop, self.fit)

    def init_step(self):
        """First generation (pso.py:108-115): evaluate, seed the personal and global bests."""
        dev = self._buffers_ready()
        plan = self._fused_plan()
        if plan is None:
            self.fit = self.evaluate(self.pop)
            self._buffers_ready()
        else:
            fitness_id, params = plan
            _cabi.check(
                _cabi.lib.evox_eval_fitness(
                    _cabi.ptr(self.pop), self.local_size, self.dim, fitness_id, _cabi.host_floats(params),
                    _cabi.ptr(self.fit), _cabi.stream_ptr(dev),
                )
            )
            self._workflow_notify(self.pop, self.fit)
        self.local_best_fit.copy_(self.fit)
        records = self._update_global_best(dev, have_previous=False)
        # the first generation folds the same records again: a tie, which the stored best wins
        self._pending = (self._swarm_key(), records) if plan is not None else None

    def _workflow_notify(self, pop: torch.Tensor, fit: torch.Tensor) -> None:
        notify = getattr(self, "_workflow_fused_notify", None)
        if notify is not None:
            notify(pop, fit)
