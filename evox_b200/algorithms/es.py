"""OpenES, ARS and VirtualLoRAES with the reference's constructor arguments and state names
(evox/algorithms/so/es_variants/open_es.py:10-86, ars.py:8-101, virtual_lora_es.py:18-138)."""

from __future__ import annotations

from typing import Literal

import torch

import torch.distributed as dist

from .. import _cabi
from ..core import Algorithm, Mutable, Parameter
from ..lora_kernels import compute_counter_offsets, lora_gradient_from_seeds
from ..sharding import group_info, shard_bounds


def _update_center(algo, grad: torch.Tensor, start: int = 0, count: int | None = None, lr: torch.Tensor | None = None) -> None:
    """center[start : start + count] -= lr * grad (or the Adam step) — `grad` holds `count` values."""
    dev = algo.center.device
    lr = algo.learning_rate if lr is None else lr
    adam = algo.optimizer == "adam"
    count = algo.center.numel() - start if count is None else count
    if torch.compiler.is_compiling():  # traced: one registered operator that declares what it updates in place
        from .. import ops

        ops.es_update(algo.center, grad, lr, algo.exp_avg if adam else None, algo.exp_avg_sq if adam else None,
                      algo.beta1 if adam else None, algo.beta2 if adam else None, start, count)
        return
    assert grad.numel() == count and grad.is_contiguous()

    def at(t):
        return None if t is None else _cabi.ptr(t, torch.float32) + 4 * start

    _cabi.check(
        _cabi.lib.evox_es_update(
            at(algo.center), _cabi.ptr(grad, torch.float32, "grad"),
            _cabi.ptr(lr, torch.float32, "learning_rate"),
            at(algo.exp_avg) if adam else None, at(algo.exp_avg_sq) if adam else None,
            _cabi.ptr(algo.beta1) if adam else None, _cabi.ptr(algo.beta2) if adam else None,
            1e-8, count, _cabi.stream_ptr(dev),
        )
    )


class _ESBase(Algorithm):
    def _common_init(self, pop_size, center_init, learning_rate, noise_stdev, optimizer, device):
        assert noise_stdev > 0, "noise_stdev must be greater than 0."
        assert learning_rate > 0, "learning_rate must be greater than 0."
        assert pop_size > 0, "pop_size must be greater than 0."
        assert optimizer in [None, "adam"], "optimizer must be None or 'adam'."
        self.learning_rate = Parameter(learning_rate, dtype=torch.float32, device=device)
        self.noise_stdev = Parameter(noise_stdev, dtype=torch.float32, device=device)
        self._sigma_host = float(noise_stdev)
        self.pop_size = pop_size
        self.optimizer = optimizer
        self.center = Mutable(center_init.to(device=device, dtype=torch.float32).contiguous().clone())
        if optimizer == "adam":
            self.exp_avg = Mutable(torch.zeros_like(self.center))
            self.exp_avg_sq = Mutable(torch.zeros_like(self.center))
            self.beta1 = Parameter(0.9, dtype=torch.float32, device=device)
            self.beta2 = Parameter(0.999, dtype=torch.float32, device=device)

    def sigma(self) -> float:
        """Host copy of noise_stdev; refreshed (one sync) when the parameter was modified in place OR rebound to
        another tensor (a fresh tensor's version counter can equal the cached one, so the key also holds the
        tensor's identity and storage address)."""
        if torch.compiler.is_compiling():
            return self._sigma_host  # a traced step cannot look at storage or version counters; it uses the last value read
        t = self.noise_stdev
        key = (id(t), t.data_ptr(), t._version)
        if getattr(self, "_sigma_key", None) != key:
            self._sigma_host = float(t)
            self._sigma_key = key
        return self._sigma_host

    def record_step(self):
        return {"center": self.center}


class OpenES(_ESBase):
    """OpenAI-ES: mirrored Gaussian sampling, score-function gradient, SGD or Adam."""

    def __init__(
        self,
        pop_size: int,
        center_init: torch.Tensor,
        learning_rate: float,
        noise_stdev: float,
        optimizer: Literal["adam"] | None = None,
        mirrored_sampling: bool = True,
        device: torch.device | None = None,
    ):
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        if mirrored_sampling is True:
            assert pop_size % 2 == 0, "When mirrored_sampling is True, pop_size must be a multiple of 2."
        self._common_init(pop_size, center_init, learning_rate, noise_stdev, optimizer, device)
        self.dim = center_init.shape[0]
        self.mirrored_sampling = mirrored_sampling

    def step(self, noise: torch.Tensor | None = None):
        """One generation (open_es.py:60-83). `noise`: optional (pop/2 or pop, dim) standard-normal
        draws; by default they come from torch.randn like the reference's."""
        dev = self.center.device
        rows = self.pop_size // 2 if self.mirrored_sampling else self.pop_size
        if noise is None:
            noise = torch.randn(rows, self.dim, device=dev)
        noise = noise.to(torch.float32).contiguous()
        assert noise.shape == (rows, self.dim)
        if torch.compiler.is_compiling():  # traced: the same three kernels as registered operators
            from .. import ops

            pop = ops.openes_ask(self.center, noise, self.noise_stdev, self.pop_size)
            fitness = self.evaluate(pop)
            _update_center(self, ops.openes_gradient(noise, fitness, self.pop_size, self.sigma()))
            return
        pop = torch.empty(self.pop_size, self.dim, dtype=torch.float32, device=dev)
        lib, s = _cabi.lib, _cabi.stream_ptr(dev)
        _cabi.check(lib.evox_openes_ask(_cabi.ptr(self.center), _cabi.ptr(noise), _cabi.ptr(self.noise_stdev), self.pop_size, self.dim, rows, _cabi.ptr(pop), s))
        fitness = self.evaluate(pop).to(torch.float32).contiguous()
        grad = torch.empty(self.dim, dtype=torch.float32, device=dev)
        _cabi.check(lib.evox_openes_gradient(_cabi.ptr(noise), _cabi.ptr(fitness), self.pop_size, self.dim, rows, self.sigma(), _cabi.ptr(grad), s))
        _update_center(self, grad)


class ARS(Algorithm):
    """Augmented random search (ars.py:8-101): mirrored sampling, the `elite_pop_size` best directions
    (by the better of their two evaluations) weighted by their fitness difference, scaled by the elite's
    fitness spread. The population and the weighted sum of directions run on the OpenES kernels; the
    elite bookkeeping works on pop_size / 2 scalars with torch ops on the device."""

    def __init__(
        self,
        pop_size: int,
        center_init: torch.Tensor,
        elite_ratio: float = 0.1,
        lr: float = 0.05,
        sigma: float = 0.03,
        optimizer: Literal["adam"] | None = None,
        device: torch.device | None = None,
    ):
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        assert pop_size > 1 and pop_size % 2 == 0, "ARS mirrors its samples: pop_size must be even"
        assert 0 <= elite_ratio <= 1
        assert optimizer in [None, "adam"]
        self.lr = Parameter(lr, dtype=torch.float32, device=device)
        self.sigma = Parameter(sigma, dtype=torch.float32, device=device)
        self.dim = center_init.shape[0]
        self.pop_size = pop_size
        self.optimizer = optimizer
        self.elite_pop_size = max(1, int(pop_size / 2 * elite_ratio))
        self.center = Mutable(center_init.to(device=device, dtype=torch.float32).contiguous().clone())
        if optimizer == "adam":
            self.exp_avg = Mutable(torch.zeros_like(self.center))
            self.exp_avg_sq = Mutable(torch.zeros_like(self.center))
            self.beta1 = Parameter(0.9, dtype=torch.float32, device=device)
            self.beta2 = Parameter(0.999, dtype=torch.float32, device=device)

    def step(self, z_plus: torch.Tensor | None = None):
        """One generation (ars.py:62-98). `z_plus`: optional (pop_size / 2, dim) standard-normal draws."""
        dev = self.center.device
        half, k = self.pop_size // 2, self.elite_pop_size
        if z_plus is None:
            z_plus = torch.randn(half, self.dim, device=dev)
        z_plus = z_plus.to(device=dev, dtype=torch.float32).contiguous()
        assert z_plus.shape == (half, self.dim)
        lib, s = _cabi.lib, _cabi.stream_ptr(dev)
        pop = torch.empty(self.pop_size, self.dim, dtype=torch.float32, device=dev)
        _cabi.check(lib.evox_openes_ask(_cabi.ptr(self.center), _cabi.ptr(z_plus), _cabi.ptr(self.sigma), self.pop_size, self.dim, half, _cabi.ptr(pop), s))
        fitness = self.evaluate(pop).to(torch.float32)
        fit_1, fit_2 = fitness[:half], fitness[half:]
        elite_idx = torch.minimum(fit_1, fit_2).argsort()[:k]
        sigma_fitness = torch.std(torch.cat([fit_1[elite_idx], fit_2[elite_idx]])) + 1e-05
        # weights of all pop_size / 2 directions: the elite's fitness difference, zero elsewhere, pre-scaled so
        # that the kernel's division by its row count leaves 1 / (k * sigma_fitness)
        weights = torch.zeros(half, dtype=torch.float32, device=dev)
        weights[elite_idx] = (fit_1[elite_idx] - fit_2[elite_idx]) * (half / (k * sigma_fitness))
        grad = torch.empty(self.dim, dtype=torch.float32, device=dev)
        _cabi.check(lib.evox_openes_gradient(_cabi.ptr(z_plus), _cabi.ptr(weights), half, self.dim, half, 1.0, _cabi.ptr(grad), s))
        _update_center(self, grad, lr=self.lr)

    def record_step(self):
        return {"center": self.center}


class PersistentES(Algorithm):
    """Persistent evolution strategies (persistent_es.py:9-115): mirrored perturbations are accumulated
    over the inner steps of an unrolled problem and the gradient estimate uses the ACCUMULATED
    perturbations. One kernel forms the population and adds the perturbations to `pert_accum`; the
    weighted row sum and the centre update are the OpenES kernels. As in the reference, the stored
    `inner_step_counter` is never reset (only a local copy is, persistent_es.py:100-105): once it has
    reached T the accumulator is cleared after every step."""

    def __init__(
        self,
        pop_size: int,
        center_init: torch.Tensor,
        optimizer: Literal["adam"] | None = None,
        lr: float = 0.05,
        sigma: float = 0.03,
        T: int = 100,
        K: int = 10,
        sigma_decay: float = 1.0,
        sigma_limit: float = 0.01,
        device: torch.device | None = None,
    ):
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        assert pop_size > 1 and pop_size % 2 == 0
        assert optimizer in [None, "adam"]
        self.lr = Parameter(lr, dtype=torch.float32, device=device)
        self.T = Parameter(T, device=device)
        self.K = Parameter(K, device=device)
        self.sigma_decay = Parameter(sigma_decay, dtype=torch.float32, device=device)
        self.sigma_limit = Parameter(sigma_limit, dtype=torch.float32, device=device)
        self.dim = center_init.shape[0]
        self.pop_size = pop_size
        self.optimizer = optimizer
        self.sigma = Mutable(torch.tensor(sigma, dtype=torch.float32, device=device))
        self.center = Mutable(center_init.to(device=device, dtype=torch.float32).contiguous().clone())
        self.inner_step_counter = Mutable(torch.tensor(0.0, device=device))
        self.pert_accum = Mutable(torch.zeros(pop_size, self.dim, device=device))
        if optimizer == "adam":
            self.exp_avg = Mutable(torch.zeros_like(self.center))
            self.exp_avg_sq = Mutable(torch.zeros_like(self.center))
            self.beta1 = Parameter(0.9, dtype=torch.float32, device=device)
            self.beta2 = Parameter(0.999, dtype=torch.float32, device=device)

    def step(self, z: torch.Tensor | None = None):
        """One generation (persistent_es.py:74-112). `z`: optional (pop_size / 2, dim) standard-normal draws."""
        dev = self.center.device
        half = self.pop_size // 2
        if z is None:
            z = torch.randn(half, self.dim, device=dev)
        z = z.to(device=dev, dtype=torch.float32).contiguous()
        assert z.shape == (half, self.dim)
        if not self.pert_accum.is_contiguous():
            self.pert_accum = self.pert_accum.contiguous()
        lib, s = _cabi.lib, _cabi.stream_ptr(dev)
        pop = torch.empty(self.pop_size, self.dim, dtype=torch.float32, device=dev)
        _cabi.check(lib.evox_pes_ask(_cabi.ptr(self.center), _cabi.ptr(z), _cabi.ptr(self.sigma, torch.float32, "sigma"), self.pop_size,
                                     self.dim, _cabi.ptr(self.pert_accum, torch.float32, "pert_accum"), _cabi.ptr(pop), s))
        fitness = self.evaluate(pop).to(torch.float32).contiguous()
        # mean over the population of pert_accum * fitness / sigma^2: the division rides on the weights, which
        # keeps sigma on the device (it decays every generation)
        weights = fitness / (self.sigma**2)
        grad = torch.empty(self.dim, dtype=torch.float32, device=dev)
        _cabi.check(lib.evox_openes_gradient(_cabi.ptr(self.pert_accum), _cabi.ptr(weights), self.pop_size, self.dim, self.pop_size, 1.0,
                                             _cabi.ptr(grad), s))
        _update_center(self, grad, lr=self.lr)
        self.inner_step_counter = self.inner_step_counter + self.K
        # scalar bookkeeping on the device, no host synchronisation: clear the accumulator when the counter
        # has reached T (an in-place masked fill with a 0-d mask)
        self.pert_accum.masked_fill_(self.inner_step_counter >= self.T, 0.0)
        self.sigma = torch.maximum(self.sigma_decay * self.sigma, self.sigma_limit)

    def record_step(self):
        return {"center": self.center, "sigma": self.sigma}


def _rank_weighted_step(algo, noise, weights_by_rank, x_is_population: bool):
    """Shared by SNES and DES: sample with per-coordinate step sizes, evaluate, give every row the weight of
    its fitness rank and reduce the two weighted column sums in one pass. Returns (first, second)."""
    dev = algo.center.device
    pop_size, dim = algo.pop_size, algo.dim
    if noise is None:
        noise = torch.randn(pop_size, dim, device=dev)
    noise = noise.to(device=dev, dtype=torch.float32).contiguous()
    assert noise.shape == (pop_size, dim)
    lib, s = _cabi.lib, _cabi.stream_ptr(dev)
    pop = torch.empty(pop_size, dim, dtype=torch.float32, device=dev)
    _cabi.check(lib.evox_es_ask_diag(_cabi.ptr(algo.center, torch.float32, "center"), _cabi.ptr(noise), _cabi.ptr(algo.sigma, torch.float32, "sigma"),
                                     pop_size, dim, _cabi.ptr(pop), s))
    fitness = algo.evaluate(pop)
    row_weights = torch.empty(pop_size, dtype=torch.float32, device=dev)
    row_weights[fitness.argsort()] = weights_by_rank
    first = torch.empty(dim, dtype=torch.float32, device=dev)
    second = torch.empty(dim, dtype=torch.float32, device=dev)
    x, shift, offset = (pop, algo.center, 0.0) if x_is_population else (noise, None, -1.0)
    _cabi.check(lib.evox_rank_weighted_moments(_cabi.ptr(x), _cabi.ptr(row_weights), _cabi.ptr(shift), offset, pop_size, dim,
                                               _cabi.ptr(first), _cabi.ptr(second), s))
    return first, second


class SNES(Algorithm):
    """Separable natural evolution strategy (snes.py:12-95): per-coordinate step sizes, rank-based weights."""

    def __init__(self, pop_size: int, center_init: torch.Tensor, sigma: float = 1.0, lrate_mean: float = 1.0,
                 temperature: float = 12.5, weight_type: Literal["recomb", "temp"] = "temp", device: torch.device | None = None):
        import math

        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        assert pop_size > 1
        dim = center_init.shape[0]
        self.lrate_mean = Parameter(lrate_mean, dtype=torch.float32, device=device)
        self.lrate_sigma = Parameter((3 + math.log(dim)) / (5 * math.sqrt(dim)), dtype=torch.float32, device=device)
        self.temperature = Parameter(temperature, dtype=torch.float32, device=device)
        self.dim = dim
        self.pop_size = pop_size
        if weight_type == "temp":
            w = torch.arange(pop_size, device=device) / (pop_size - 1) - 0.5
            w = torch.nn.functional.softmax(-20 * torch.sigmoid(temperature * w), dim=0)
        else:
            w = torch.clip(math.log(pop_size / 2 + 1) - torch.log(torch.arange(1, pop_size + 1, device=device)), 0)
            w = w / torch.sum(w) - 1 / pop_size
        # the reference keeps the weights tiled over the columns (pop_size, dim); one value per rank carries the same information
        self.weights = Mutable(w.to(torch.float32).contiguous())
        self.center = Mutable(center_init.to(device=device, dtype=torch.float32).contiguous().clone())
        self.sigma = Mutable(sigma * torch.ones(dim, device=device))

    def step(self, noise: torch.Tensor | None = None):
        """One generation (snes.py:70-90). `noise`: optional (pop_size, dim) standard-normal draws."""
        grad_mean, grad_sigma = _rank_weighted_step(self, noise, self.weights, x_is_population=False)
        self.center = self.center + self.lrate_mean * self.sigma * grad_mean
        self.sigma = self.sigma * torch.exp(self.lrate_sigma / 2 * grad_sigma)

    def record_step(self):
        return {"center": self.center, "sigma": self.sigma}


class DES(Algorithm):
    """Discovered evolution strategy (des.py:11-77): softmax rank weights, weighted mean and deviation."""

    def __init__(self, pop_size: int, center_init: torch.Tensor, temperature: float = 12.5, sigma_init: float = 0.1,
                 device: torch.device | None = None):
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        assert pop_size > 1
        self.temperature = Parameter(temperature, dtype=torch.float32, device=device)
        self.sigma_init = Parameter(sigma_init, dtype=torch.float32, device=device)
        self.lrate_mean = Parameter(1.0, dtype=torch.float32, device=device)
        self.lrate_sigma = Parameter(0.1, dtype=torch.float32, device=device)
        self.dim = center_init.shape[0]
        self.pop_size = pop_size
        self.ranks = torch.arange(pop_size, device=device) / (pop_size - 1) - 0.5
        self.center = Mutable(center_init.to(device=device, dtype=torch.float32).contiguous().clone())
        self.sigma = Mutable(sigma_init * torch.ones(self.dim, device=device))

    def step(self, noise: torch.Tensor | None = None):
        """One generation (des.py:57-72). `noise`: optional (pop_size, dim) standard-normal draws."""
        weight = torch.nn.functional.softmax(-20 * torch.sigmoid(self.temperature * self.ranks), dim=0)
        weight_mean, weight_sq = _rank_weighted_step(self, noise, weight, x_is_population=True)
        weight_sigma = torch.sqrt(weight_sq + 1e-6)
        self.center = self.center + self.lrate_mean * (weight_mean - self.center)
        self.sigma = self.sigma + self.lrate_sigma * (weight_sigma - self.sigma)

    def record_step(self):
        return {"center": self.center, "sigma": self.sigma}


class VirtualLoRAES(_ESBase):
    """ES over a virtual population: only the centre and one int64 seed per individual exist;
    perturbations are rank-r factors regenerated from the seeds."""

    def __init__(
        self,
        param_shapes: list[tuple],
        lora_rank: int,
        pop_size: int,
        center_init: torch.Tensor,
        learning_rate: float,
        noise_stdev: float,
        optimizer: Literal["adam"] | None = None,
        device: torch.device | None = None,
        shard: bool = False,
        group=None,
        gradient_passes: int = 3,
    ):
        """`gradient_passes`: tensor-core passes of the population gradient (3 = fp32-accurate, the
        default; 1 = bf16 operands; see `lora_gradient_from_seeds`).
        `shard=True` (under an initialised torch.distributed group): every rank keeps the whole
        centre, but the gradient and update of each 2-D block are computed for this rank's rows only
        and the updated rows are allgathered; seeds are broadcast from rank 0 each generation."""
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        self.group = group
        self.gradient_passes = gradient_passes
        self.rank, self.world_size = group_info(group) if shard else (0, 1)
        assert lora_rank > 0, "lora_rank must be greater than 0."
        self._common_init(pop_size, center_init, learning_rate, noise_stdev, optimizer, device)
        self.param_shapes = [tuple(s) for s in param_shapes]
        self.lora_rank = lora_rank
        self.dim = sum(int(torch.tensor(s).prod()) for s in self.param_shapes)
        self.counter_offsets = compute_counter_offsets(self.param_shapes, lora_rank)
        assert center_init.shape[0] == self.dim, (
            "center_init length must equal the total number of parameters (sum of element counts over param_shapes)."
        )
        self.seeds = Mutable(torch.randint(0, 2**31, (pop_size,), device=device, dtype=torch.int64))

    def step(self, seeds: torch.Tensor | None = None):
        """One generation (virtual_lora_es.py:90-135). `seeds`: optional int64 (pop,) to use
        instead of fresh torch.randint draws."""
        dev = self.center.device
        self.seeds = torch.randint(0, 2**31, (self.pop_size,), device=dev, dtype=torch.int64) if seeds is None else seeds.to(dev)
        if self.world_size > 1:
            dist.broadcast(self.seeds, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0, group=self.group)
        sigma = self.sigma()
        fitness = self.evaluate((self.center, self.seeds, sigma)).to(torch.float32).contiguous()
        start = 0
        for shape, offset in zip(self.param_shapes, self.counter_offsets):
            n = int(torch.tensor(shape).prod())
            rows = self._row_shard(shape)
            if rows is None:  # whole block on every rank (identical arithmetic everywhere)
                grad = torch.empty(n, dtype=torch.float32, device=dev)
                lora_gradient_from_seeds(fitness, self.seeds, shape, self.lora_rank, offset, self.pop_size, sigma, out=grad, passes=self.gradient_passes)
                _update_center(self, grad, start, n)
            else:
                r0, r1 = rows
                k = int(shape[-1])
                grad = torch.empty((r1 - r0) * k, dtype=torch.float32, device=dev)
                lora_gradient_from_seeds(fitness, self.seeds, shape, self.lora_rank, offset, self.pop_size, sigma, out=grad, rows=rows, passes=self.gradient_passes)
                _update_center(self, grad, start + r0 * k, (r1 - r0) * k)
                block = self.center[start : start + n]
                dist.all_gather_into_tensor(block, block[r0 * k : r1 * k].clone(), group=self.group)
            start += n

    def _row_shard(self, shape) -> tuple[int, int] | None:
        """This rank's rows of a 2-D block, or None when the block is not sharded (1-D blocks, a
        single rank, or row counts the tensor-core gradient cannot split evenly)."""
        if self.world_size == 1 or len(shape) < 2:
            return None
        d = int(torch.tensor(shape[:-1]).prod())
        if d % (128 * self.world_size) != 0:
            return None
        if not _cabi.lib.evox_lora_gradient_tc_supported(self.pop_size, d // self.world_size, int(shape[-1]), self.lora_rank):
            return None
        return shard_bounds(d, self.world_size, self.rank)
