"""Philox streams and virtual-LoRA operators on the CUDA kernels.

Same function names, argument order and shapes as the reference's `evox.triton_kernels`
(kernels/philox.py:274-311, kernels/lora_noise.py:58-196).
"""

from __future__ import annotations

import math

import torch

from . import _cabi

__all__ = [
    "philox_uniform", "philox_normal", "compute_counter_offsets", "generate_lora_factors",
    "lora_delta_output", "lora_gradient", "lora_gradient_from_seeds", "lora_layer_bf16", "raise_on_kernel_errors",
]

_grad_ws: dict[torch.device, torch.Tensor] = {}

# Error flags of tensor-core launches that have not been looked at yet. The kernels bound every wait
# and report an expired one through a device word; reading it needs a host synchronisation, so the
# flags are collected here and examined by `raise_on_kernel_errors()` (the problem / algorithm
# classes call it once per generation, on the flags of the previous one).
_pending_flags: list[tuple[str, torch.Tensor]] = []


def raise_on_kernel_errors() -> None:
    """Synchronise on and check every tensor-core launch since the last call; raise if a bounded
    device-side wait expired (1 producer, 2 / 3 issuer, 4 epilogue) or shared memory was misaligned (5)."""
    pending, _pending_flags[:] = list(_pending_flags), []
    for what, flag in pending:
        code = int(flag)
        if code != 0:
            raise _cabi.EvoxKernelError(f"{what}: the tensor-core kernel gave up with status {code} (a bounded wait expired)")


def _seeds(seeds: torch.Tensor) -> torch.Tensor:
    if seeds.ndim != 1 or seeds.dtype != torch.int64:
        raise _cabi.EvoxKernelError("seeds must be a 1-D int64 tensor")
    return seeds.contiguous()


def _fill(fn, seeds: torch.Tensor, n: int, counter: int) -> torch.Tensor:
    seeds = _seeds(seeds)
    out = torch.empty(seeds.shape[0], n, dtype=torch.float32, device=seeds.device)
    if out.numel():
        _cabi.check(fn(_cabi.ptr(seeds), seeds.shape[0], n, counter & (2**64 - 1), _cabi.ptr(out), _cabi.stream_ptr(seeds.device)))
    return out


def philox_uniform(seeds: torch.Tensor, n: int, counter: int = 0) -> torch.Tensor:
    """(pop, n) uniforms in [0, 1) from per-individual Philox4x32-10 streams."""
    return _fill(_cabi.lib.evox_philox_uniform, seeds, n, counter)


def philox_normal(seeds: torch.Tensor, n: int, counter: int = 0) -> torch.Tensor:
    """(pop, n) standard normals (Box-Muller on the uniform stream)."""
    return _fill(_cabi.lib.evox_philox_normal, seeds, n, counter)


def _ceil4(x: int) -> int:
    return (x + 3) // 4 * 4


def _as_2d(shape) -> tuple[int, int]:
    return int(math.prod(shape[:-1])), int(shape[-1])


def compute_counter_offsets(param_shapes: list[tuple], lora_rank: int) -> list[int]:
    """Disjoint Philox counter ranges for a list of parameter blocks (host arithmetic)."""
    offsets, cur = [], 0
    for shape in param_shapes:
        offsets.append(cur)
        if len(shape) == 1:
            n = shape[0]
        else:
            d, k = _as_2d(shape)
            n = lora_rank * k + d * lora_rank
        cur += _ceil4(n)
    return offsets


def generate_lora_factors(seeds: torch.Tensor, weight_shape: tuple, rank: int, counter: int):
    """Flat noise (pop, n) for a 1-D block; (A (pop, r, k), B (pop, d, r)) otherwise."""
    pop = seeds.shape[0]
    if len(weight_shape) == 1:
        return philox_normal(seeds, weight_shape[0], counter)
    d, k = _as_2d(weight_shape)
    a = philox_normal(seeds, rank * k, counter).reshape(pop, rank, k)
    b = philox_normal(seeds, d * rank, counter + _ceil4(rank * k)).reshape(pop, d, rank)
    return a, b


def lora_delta_output(x: torch.Tensor, A: torch.Tensor, B: torch.Tensor, sigma: float) -> torch.Tensor:
    """sigma * (x @ A^T) @ B^T for x (pop, batch, k), A (pop, r, k), B (pop, d, r)."""
    x, A, B = x.float().contiguous(), A.float().contiguous(), B.float().contiguous()
    pop, batch, k = x.shape
    r, d = A.shape[1], B.shape[1]
    if A.shape != (pop, r, k) or B.shape != (pop, d, r):
        raise _cabi.EvoxKernelError(f"shape mismatch: x {tuple(x.shape)}, A {tuple(A.shape)}, B {tuple(B.shape)}")
    out = torch.empty(pop, batch, d, dtype=torch.float32, device=x.device)
    t = torch.empty(pop, batch, r, dtype=torch.float32, device=x.device)
    _cabi.check(
        _cabi.lib.evox_lora_delta_output(
            _cabi.ptr(x), _cabi.ptr(A), _cabi.ptr(B), float(sigma), pop, batch, k, r, d, _cabi.ptr(out), _cabi.ptr(t),
            _cabi.stream_ptr(x.device),
        )
    )
    return out


def lora_gradient(fitness: torch.Tensor, A: torch.Tensor, B: torch.Tensor | None, pop_size: int, sigma, weight_shape: tuple) -> torch.Tensor:
    """Population gradient of one parameter block, reshaped to `weight_shape`."""
    fitness = fitness.float().contiguous()
    A = A.float().contiguous()
    sigma = float(sigma)
    dev = fitness.device
    if B is None:
        n = A.shape[1]
        grad = torch.empty(n, dtype=torch.float32, device=dev)
        _cabi.check(_cabi.lib.evox_lora_gradient(_cabi.ptr(fitness), _cabi.ptr(A), None, pop_size, sigma, 1, n, 1, _cabi.ptr(grad), _cabi.stream_ptr(dev)))
    else:
        B = B.float().contiguous()
        r, k = A.shape[1], A.shape[2]
        d = B.shape[1]
        grad = torch.empty(d, k, dtype=torch.float32, device=dev)
        _cabi.check(_cabi.lib.evox_lora_gradient(_cabi.ptr(fitness), _cabi.ptr(A), _cabi.ptr(B), pop_size, sigma, d, k, r, _cabi.ptr(grad), _cabi.stream_ptr(dev)))
    return grad.reshape(weight_shape)


def lora_layer_bf16(h: torch.Tensor, w: torch.Tensor, seeds: torch.Tensor, counter: int, sigma: float, *,
                    bias: torch.Tensor | None = None, bias_counter: int | None = None, relu: bool = False,
                    out_dtype: torch.dtype = torch.bfloat16, target: torch.Tensor | None = None, lora: bool = True,
                    t: torch.Tensor | None = None, next_counter: int | None = None):
    """One virtual-LoRA Linear layer on the tensor cores: h (pop, batch, k) bf16, w (d, k) bf16.

    Returns y (pop, batch, d) in `out_dtype`, or, with `target` (batch, d) given, the per-individual
    fitness -mean((y - target)^2) without ever writing y. `counter` is the weight block's Philox
    counter (A at `counter`, B at `counter + ceil4(8 k)`), `bias_counter` the bias block's.
    `t` (pop, batch, 8): this layer's h A_p^T if already known (skips the projection kernel).
    `next_counter`: counter of the NEXT layer's weight block (whose row length is d); the kernel then
    also accumulates that layer's projection from its own bf16 output and `(y, t_next)` is returned."""
    rank = 8
    pop, batch, k = h.shape
    d = w.shape[0]
    dev = h.device
    if h.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise _cabi.EvoxKernelError("lora_layer_bf16 needs bf16 activations and weights")
    if not _cabi.lib.evox_lora_gemm_supported(pop, batch, k, d, rank):
        raise _cabi.EvoxKernelError(f"layer shape (pop {pop}, batch {batch}, k {k}, d {d}) is not supported by the tensor-core path")
    h, w, seeds = h.contiguous(), w.contiguous(), _seeds(seeds)
    lib, s = _cabi.lib, _cabi.stream_ptr(dev)
    if not lora:
        t = None
    elif t is not None:
        t = t.contiguous()
    elif lora:
        t = torch.empty(pop, batch, rank, dtype=torch.float32, device=dev)
        _cabi.check(lib.evox_lora_down_bf16(_cabi.ptr(h), _cabi.ptr(seeds), counter, pop, batch, k, rank, _cabi.ptr(t), s))
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    out_bf16 = out_f32 = partial = None
    if target is not None:
        target = target.to(device=dev, dtype=torch.float32).contiguous()
        partial = torch.empty(pop * batch, d // 128, dtype=torch.float32, device=dev)
    elif out_dtype == torch.bfloat16:
        out_bf16 = torch.empty(pop, batch, d, dtype=torch.bfloat16, device=dev)
    else:
        out_f32 = torch.empty(pop, batch, d, dtype=torch.float32, device=dev)
    bias_f = None if bias is None else bias.to(device=dev, dtype=torch.float32).contiguous()
    t_partial = None
    if next_counter is not None and out_bf16 is not None and lora:
        t_partial = torch.empty(pop * batch, 2 * (d // 256), rank, dtype=torch.float32, device=dev)
    _cabi.check(
        lib.evox_lora_gemm_bf16(
            _cabi.ptr(h), _cabi.ptr(w), _cabi.ptr(bias_f), _cabi.ptr(t), _cabi.ptr(seeds), counter + _ceil4(rank * k),
            int(bias is not None and bias_counter is not None and lora), bias_counter or 0, float(sigma), pop, batch, k, d, rank,
            int(relu), _cabi.ptr(out_bf16), _cabi.ptr(out_f32), _cabi.ptr(target), _cabi.ptr(partial), _cabi.ptr(t_partial),
            next_counter or 0, _cabi.ptr(err), s,
        )
    )
    lora_layer_bf16.last_error_flag = err
    _pending_flags.append(("lora_layer_bf16", err))
    del _pending_flags[:-256]
    if target is not None:
        fitness = torch.empty(pop, dtype=torch.float32, device=dev)
        _cabi.check(lib.evox_neg_mse_from_partials(_cabi.ptr(partial), pop, batch, d, _cabi.ptr(fitness), s))
        return fitness
    if t_partial is not None:
        t_next = torch.empty(pop, batch, rank, dtype=torch.float32, device=dev)
        _cabi.check(lib.evox_lora_t_from_partials(_cabi.ptr(t_partial), pop * batch, d, _cabi.ptr(t_next), s))
        return out_bf16, t_next
    return out_bf16 if out_bf16 is not None else out_f32


def lora_gradient_from_seeds(fitness: torch.Tensor, seeds: torch.Tensor, weight_shape: tuple, rank: int, counter: int,
                             pop_size: int, sigma: float, out: torch.Tensor | None = None,
                             rows: tuple[int, int] | None = None, passes: int = 3) -> torch.Tensor:
    """`lora_gradient(fitness, *generate_lora_factors(seeds, weight_shape, rank, counter), ...)` without
    the factors ever existing in fp32: on supported shapes the tensor-core kernel regenerates them;
    otherwise this falls back to generating them and calling `lora_gradient`. `out`: optional flat
    fp32 destination of prod(weight_shape) elements. `rows = (begin, end)` computes only those rows
    of a 2-D block (tensor-core path only) and returns that slice; `out` then has (end - begin) * k
    elements. `passes`: 3 (default) = operands split into two fp16 pieces, three tensor-core products,
    about 1e-6 relative error; 6 = three bf16 pieces, six products, same accuracy at twice the work;
    1 = bf16 operands, about 4e-3."""
    fitness = fitness.float().contiguous()
    seeds = _seeds(seeds)
    dev = fitness.device
    n = int(math.prod(weight_shape))
    if rows is not None:
        n = (rows[1] - rows[0]) * int(weight_shape[-1])
    if out is None:
        out = torch.empty(n, dtype=torch.float32, device=dev)
    if len(weight_shape) >= 2:
        d, k = _as_2d(weight_shape)
        r0, r1 = rows if rows is not None else (0, d)
        if rows is not None and not _cabi.lib.evox_lora_gradient_tc_supported(pop_size, r1 - r0, k, rank):
            raise _cabi.EvoxKernelError("a row range needs the tensor-core gradient path")
        if _cabi.lib.evox_lora_gradient_tc_supported(pop_size, r1 - r0, k, rank) and out.data_ptr() % 16 == 0:
            d = r1 - r0
            nbytes = _cabi.lib.evox_lora_gradient_tc_workspace_bytes(pop_size, d, k)
            ws = _grad_ws.get(dev)
            if ws is None or ws.numel() < nbytes:
                ws = _grad_ws[dev] = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            err = torch.zeros(1, dtype=torch.int32, device=dev)
            _cabi.check(
                _cabi.lib.evox_lora_gradient_tc(
                    _cabi.ptr(fitness), _cabi.ptr(seeds), counter, pop_size, float(sigma), r0, d, k, rank, passes, _cabi.ptr(out),
                    _cabi.ptr(ws), ws.numel(), _cabi.ptr(err), _cabi.stream_ptr(dev),
                )
            )
            lora_gradient_from_seeds.last_error_flag = err
            _pending_flags.append(("lora_gradient_from_seeds", err))
            return out.view(d, k) if rows is not None else out.view(weight_shape)
        a, b = generate_lora_factors(seeds, weight_shape, rank, counter)
        out.copy_(lora_gradient(fitness, a, b, pop_size, sigma, weight_shape).reshape(-1))
        return out.view(weight_shape)
    noise = generate_lora_factors(seeds, weight_shape, rank, counter)
    out.copy_(lora_gradient(fitness, noise, None, pop_size, sigma, weight_shape).reshape(-1))
    return out.view(weight_shape)
