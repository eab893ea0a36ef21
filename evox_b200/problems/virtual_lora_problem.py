"""Fitness of a virtual LoRA-perturbed population of an `nn.Sequential` of Linear layers.

Same constructor and payload protocol as the reference's `VirtualLoRAProblem`
(evox/problems/neuroevolution/virtual_lora_problem.py:33-272): `evaluate` receives
`(center_flat, seeds, sigma)`; weights are slices of the flat centre in `named_parameters()`
order; per layer `h <- act(h W^T + b + sigma (h A^T) B^T + sigma * bias_noise)` with the factors
regenerated from the seeds. Inputs may be one shared batch (batch, in) as in the reference, or one
batch per individual (pop, batch, in).
"""

from __future__ import annotations

import warnings

import torch
from torch import nn

from .. import _cabi
from ..core import Problem
from ..lora_kernels import compute_counter_offsets, generate_lora_factors, lora_layer_bf16, raise_on_kernel_errors
from ..sharding import group_info, shard_bounds

__all__ = ["VirtualLoRAProblem"]

_ACTIVATIONS = (nn.ReLU, nn.Tanh, nn.Sigmoid, nn.GELU, nn.LeakyReLU, nn.ELU, nn.Softmax, nn.Identity)


class VirtualLoRAProblem(Problem):
    def __init__(self, model: nn.Sequential, data_loader, criterion, lora_rank: int, n_batch_per_eval: int = 1,
                 device: torch.device | None = None, reduction: str = "mean", compute_dtype: torch.dtype = torch.float32,
                 shard: bool = False, group=None):
        """`compute_dtype=torch.bfloat16` runs every Linear layer whose shape the tensor-core kernel
        supports (rank 8, batch 64 or 128 per individual, feature sizes multiples of 256) with bf16
        operands and fp32 accumulation; other layers and the default use the fp32 kernels."""
        super().__init__()
        self.compute_dtype = compute_dtype
        # shard=True: this rank evaluates only its tensor_split share of the individuals and the
        # fitness values are allgathered (the reference's one collective, std_workflow.py:185-189)
        self.group = group
        self.rank, self.world_size = group_info(group) if shard else (0, 1)
        if not isinstance(model, nn.Sequential):
            raise TypeError(f"VirtualLoRAProblem requires an nn.Sequential model, got {type(model).__name__}.")
        self.device = torch.get_default_device() if device is None else torch.device(device)
        self.model = model
        self.data_loader = data_loader
        self.data_loader_iter = iter(data_loader)
        self.criterion = criterion
        self.lora_rank = lora_rank
        self.n_batch_per_eval = n_batch_per_eval
        self.reduction = reduction
        named = list(model.named_parameters())
        self.param_names = [n for n, _ in named]
        self.param_shapes = [tuple(p.shape) for _, p in named]
        self.counter_offsets = compute_counter_offsets(self.param_shapes, lora_rank)
        starts, cur = [], 0
        for shape in self.param_shapes:
            starts.append(cur)
            cur += int(torch.tensor(shape).prod())
        self._starts = starts
        self.dim = cur
        for module in model.children():
            if not isinstance(module, (nn.Linear, *_ACTIVATIONS)):
                raise NotImplementedError(
                    f"Layer type {type(module).__name__} is not supported by VirtualLoRAProblem. Supported types: "
                    "nn.Linear and common activation modules (ReLU, Tanh, Sigmoid, GELU, LeakyReLU, ELU, Softmax, Identity)."
                )

    def _param(self, center: torch.Tensor, name: str) -> tuple[torch.Tensor, int]:
        i = self.param_names.index(name)
        n = int(torch.tensor(self.param_shapes[i]).prod())
        return center[self._starts[i] : self._starts[i] + n].view(self.param_shapes[i]), i

    def _virtual_forward(self, inputs: torch.Tensor, center: torch.Tensor, seeds: torch.Tensor, sigma: float, pop_size: int,
                         mse_target: torch.Tensor | None = None):
        """Activations of the last layer, (pop, batch, out) fp32. With `mse_target` (batch, out) and a
        last Linear layer on the tensor-core path, the squared error is reduced inside that layer's
        epilogue and a `("mse", per-individual mean squared error)` tuple is returned instead."""
        dev = center.device
        shared = inputs.ndim == 2
        h = inputs.to(device=dev).contiguous()
        if self.compute_dtype != torch.bfloat16 or h.dtype != torch.bfloat16:
            h = h.to(torch.float32)
        batch = h.shape[-2]
        children = list(self.model.named_children())
        lib, s = _cabi.lib, _cabi.stream_ptr(dev)
        skip = False
        pending_t = None  # next layer's h A^T, accumulated by the previous tensor-core layer's epilogue
        for pos, (name, module) in enumerate(children):
            if skip:
                skip = False
                continue
            if isinstance(module, nn.Linear):
                weight, wi = self._param(center, f"{name}.weight")
                d, k = weight.shape
                relu = pos + 1 < len(children) and isinstance(children[pos + 1][1], nn.ReLU)
                if (self.compute_dtype == torch.bfloat16 and not shared
                        and lib.evox_lora_gemm_supported(pop_size, batch, k, d, self.lora_rank)):
                    bias = bias_counter = None
                    if module.bias is not None:
                        bias, bi = self._param(center, f"{name}.bias")
                        bias_counter = self.counter_offsets[bi]
                    nxt = pos + (2 if relu else 1)
                    last = nxt >= len(children)
                    t_now, pending_t = pending_t, None
                    if last and not relu and mse_target is not None:
                        neg = lora_layer_bf16(h.to(torch.bfloat16), weight.to(torch.bfloat16), seeds, self.counter_offsets[wi], sigma,
                                              bias=bias, bias_counter=bias_counter, target=mse_target, t=t_now)
                        return "mse", -neg
                    # if the next layer is a tensor-core Linear too, let this layer's epilogue project for it
                    next_counter = None
                    if not last and isinstance(children[nxt][1], nn.Linear):
                        nd, nk = children[nxt][1].weight.shape
                        if nk == d and lib.evox_lora_gemm_supported(pop_size, batch, nk, nd, self.lora_rank):
                            next_counter = self.counter_offsets[self.param_names.index(f"{children[nxt][0]}.weight")]
                    res = lora_layer_bf16(
                        h.to(torch.bfloat16), weight.to(torch.bfloat16), seeds, self.counter_offsets[wi], sigma, bias=bias,
                        bias_counter=bias_counter, relu=relu, out_dtype=torch.float32 if last else torch.bfloat16, t=t_now,
                        next_counter=next_counter,
                    )
                    h, pending_t = res if isinstance(res, tuple) else (res, None)
                    skip = relu
                    continue
                pending_t = None
                a, b = generate_lora_factors(seeds, (d, k), self.lora_rank, self.counter_offsets[wi])
                bias = bias_noise = None
                if module.bias is not None:
                    bias, bi = self._param(center, f"{name}.bias")
                    bias_noise = generate_lora_factors(seeds, (d,), self.lora_rank, self.counter_offsets[bi])
                t = torch.empty(pop_size, batch, self.lora_rank, dtype=torch.float32, device=dev)
                h = h.to(torch.float32)
                _cabi.check(lib.evox_lora_down(_cabi.ptr(h), int(shared), _cabi.ptr(a), pop_size, batch, k, self.lora_rank, _cabi.ptr(t), s))
                out = torch.empty(pop_size, batch, d, dtype=torch.float32, device=dev)
                _cabi.check(
                    lib.evox_lora_linear_forward(
                        _cabi.ptr(h), int(shared), _cabi.ptr(weight.contiguous()), _cabi.ptr(bias), _cabi.ptr(t), _cabi.ptr(b),
                        _cabi.ptr(bias_noise), float(sigma), pop_size, batch, k, d, self.lora_rank, int(relu), _cabi.ptr(out), s,
                    )
                )
                h, shared, skip = out, False, relu
            else:
                if shared:
                    h = h.unsqueeze(0).expand(pop_size, -1, -1).contiguous()
                    shared = False
                h = module(h)
        if shared:
            h = h.unsqueeze(0).expand(pop_size, -1, -1).contiguous()
        return h.to(torch.float32)

    def evaluate(self, payload) -> torch.Tensor:
        center_flat, seeds, sigma = payload
        raise_on_kernel_errors()  # status words of the previous generation's tensor-core launches
        if self.world_size > 1:
            return self._evaluate_sharded(center_flat, seeds, sigma)
        return self._evaluate_local(center_flat, seeds, sigma, None)

    def _evaluate_sharded(self, center_flat, seeds, sigma) -> torch.Tensor:
        import torch.distributed as dist

        pop = seeds.shape[0]
        a, b = shard_bounds(pop, self.world_size, self.rank)
        local = self._evaluate_local(center_flat, seeds[a:b].contiguous(), sigma, (a, b, pop)).contiguous()
        if pop % self.world_size == 0:
            out = torch.empty(pop, dtype=local.dtype, device=local.device)
            dist.all_gather_into_tensor(out, local, group=self.group)
            return out
        pieces = [torch.empty(shard_bounds(pop, self.world_size, r)[1] - shard_bounds(pop, self.world_size, r)[0],
                              dtype=local.dtype, device=local.device) for r in range(self.world_size)]
        dist.all_gather(pieces, local, group=self.group)
        return torch.cat(pieces)

    def _evaluate_local(self, center_flat, seeds, sigma, span) -> torch.Tensor:
        """Fitness of the individuals in `seeds`; `span = (a, b, pop)` says they are rows a..b of a
        population of `pop`, so per-individual inputs are sliced the same way."""
        pop_size = seeds.shape[0]
        center = center_flat.to(torch.float32).contiguous()
        if self.n_batch_per_eval == -1:
            batches = list(self.data_loader)
        else:
            batches = []
            for _ in range(self.n_batch_per_eval):
                try:
                    batches.append(next(self.data_loader_iter))
                except StopIteration:
                    self.data_loader_iter = iter(self.data_loader)
                    batches.append(next(self.data_loader_iter))
        per_individual = []
        for inputs, labels in batches:
            inputs = inputs.to(device=self.device, non_blocking=True)
            labels = labels.to(device=self.device, non_blocking=True)
            if span is not None and inputs.ndim == 3 and inputs.shape[0] == span[2]:
                inputs = inputs[span[0] : span[1]]
            fuse = (isinstance(self.criterion, nn.MSELoss) and self.criterion.reduction == "none" and labels.ndim == 2
                    and self.reduction == "mean")
            logits = self._virtual_forward(inputs, center, seeds, sigma, pop_size, mse_target=labels if fuse else None)
            if isinstance(logits, tuple):  # the last layer already reduced (y - target)^2 per individual
                per_individual.append(logits[1])
                continue
            batch = logits.shape[1]
            flat_logits = logits.reshape(pop_size * batch, -1)
            if labels.ndim == 1:  # class labels shared by the population (virtual_lora_problem.py:247)
                flat_labels = labels.unsqueeze(0).expand(pop_size, -1).reshape(-1)
            else:  # regression targets (batch, out) shared by the population
                flat_labels = labels.unsqueeze(0).expand(pop_size, *labels.shape).reshape(pop_size * batch, -1)
            flat_loss = self.criterion(flat_logits, flat_labels)
            if flat_loss.ndim == 0:
                warnings.warn(
                    "Criterion output is a scalar. We recommend setting `reduction` to 'none' "
                    "for the criterion and letting VirtualLoRAProblem handle the reduction."
                )
                loss = flat_loss.expand(pop_size)
            else:
                if flat_loss.ndim == 2:
                    flat_loss = flat_loss.mean(dim=1)
                per_sample = flat_loss.reshape(pop_size, batch)
                loss = per_sample.mean(dim=1) if self.reduction == "mean" else per_sample.sum(dim=1)
            per_individual.append(loss)
        losses = torch.stack(per_individual, dim=1)
        return losses.mean(dim=1) if self.reduction == "mean" else losses.sum(dim=1)
