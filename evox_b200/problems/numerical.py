"""Numerical test problems evaluated by the row-reduction kernel `evox_eval_fitness`.

Same classes and constructor arguments as the reference (evox/problems/numerical/basic.py:27-131):
an optional `shift` vector and `affine` matrix are applied before the test function. With
neither, a problem can also describe itself to an algorithm (`fused_fitness`) so that the
evaluation is fused into the algorithm's own update kernel.
"""

from __future__ import annotations

import math

import torch

from .. import _cabi
from ..core import Problem

FIT_ACKLEY, FIT_RASTRIGIN, FIT_SPHERE = 0, 1, 2

__all__ = ["ShiftAffineNumericalProblem", "Ackley", "Rastrigin", "Sphere", "DTLZ2", "ackley_func", "rastrigin_func", "sphere_func"]


def _relu_clamp_rows(a: torch.Tensor, lb: torch.Tensor, ub: torch.Tensor) -> torch.Tensor:
    """The reference's relu-form clamp (utils/jit_fix_operator.py:42-44) for the rare path where user
    operators produce the offspring; the fused kernels apply it themselves."""
    return a + torch.relu(lb - a) - torch.relu(a - ub)


def _eval_rows(fitness_id: int, params: tuple[float, float, float], x: torch.Tensor) -> torch.Tensor:
    if x.ndim != 2:
        raise _cabi.EvoxKernelError(f"population must be 2-D (pop_size, dim), got shape {tuple(x.shape)}")
    if torch.compiler.is_compiling():  # a traced program keeps the evaluation as one registered operator
        from .. import ops

        return ops.eval_fitness(x, fitness_id, [float(p) for p in params])
    x = x.contiguous()
    out = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    if x.shape[0] == 0:
        return out
    _cabi.check(
        _cabi.lib.evox_eval_fitness(
            _cabi.ptr(x, torch.float32, "pop"),
            x.shape[0],
            x.shape[1],
            fitness_id,
            _cabi.host_floats(params),
            _cabi.ptr(out),
            _cabi.stream_ptr(x.device),
        )
    )
    return out


def ackley_func(a: float, b: float, c: float, x: torch.Tensor) -> torch.Tensor:
    """-a exp(-b sqrt(mean x^2)) - exp(mean cos(c x)) + a + e per row (basic.py:66-69)."""
    return _eval_rows(FIT_ACKLEY, (a, b, c), x)


def rastrigin_func(x: torch.Tensor) -> torch.Tensor:
    """10 d + sum(x^2 - 10 cos(2 pi x)) per row (basic.py:115-116)."""
    return _eval_rows(FIT_RASTRIGIN, (0.0, 0.0, 0.0), x)


def sphere_func(x: torch.Tensor) -> torch.Tensor:
    return _eval_rows(FIT_SPHERE, (0.0, 0.0, 0.0), x)


class ShiftAffineNumericalProblem(Problem):
    """Applies `x + shift` then `x @ affine` before the test function (basic.py:27-63)."""

    def __init__(self, shift: torch.Tensor | None = None, affine: torch.Tensor | None = None):
        super().__init__()
        if affine is not None:
            assert affine.ndim == 2 and affine.shape[0] == affine.shape[1], "affine must be a square matrix"
            self.affine = affine[None, :, :]
        else:
            self.affine = None
        if shift is not None:
            assert shift.ndim == 1, "shift must be a vector"
            if affine is not None:
                assert affine.shape[0] == shift.shape[0], "affine and shift must have the same dimension"
            self.shift = shift[None, :]
        else:
            self.shift = None

    def evaluate(self, pop: torch.Tensor) -> torch.Tensor:
        if self.shift is not None:
            pop = pop + self.shift.to(pop.device)
        if self.affine is not None:
            pop = torch.matmul(pop[:, None, :], self.affine.to(pop.device)).squeeze(1)
        return self._true_evaluate(pop)

    def fused_fitness(self) -> tuple[int, tuple[float, float, float]] | None:
        """(fitness id, parameters) when an update kernel may evaluate this problem itself."""
        if self.shift is not None or self.affine is not None:
            return None
        return self._descriptor()

    def _descriptor(self):
        return None


class Ackley(ShiftAffineNumericalProblem):
    def __init__(self, a: float = 20.0, b: float = 0.2, c: float = 2 * math.pi, **kwargs):
        super().__init__(**kwargs)
        self.a, self.b, self.c = a, b, c

    def _true_evaluate(self, x: torch.Tensor) -> torch.Tensor:
        return ackley_func(self.a, self.b, self.c, x)

    def _descriptor(self):
        return FIT_ACKLEY, (float(self.a), float(self.b), float(self.c))


class Rastrigin(ShiftAffineNumericalProblem):
    def _true_evaluate(self, x: torch.Tensor) -> torch.Tensor:
        return rastrigin_func(x)

    def _descriptor(self):
        return FIT_RASTRIGIN, (0.0, 0.0, 0.0)


class Sphere(ShiftAffineNumericalProblem):
    def _true_evaluate(self, x: torch.Tensor) -> torch.Tensor:
        return sphere_func(x)

    def _descriptor(self):
        return FIT_SPHERE, (0.0, 0.0, 0.0)


class DTLZ2(Problem):
    """DTLZ2 test problem (problems/numerical/dtlz.py:93-127): objectives on the unit sphere scaled by
    1 + g, g = sum over the last d - m + 1 variables of (x - 0.5)^2. Used to build benchmark inputs and
    to exercise NSGA-II / RVEA end to end; a handful of elementwise torch ops, not a kernel."""

    def __init__(self, d: int = 12, m: int = 3):
        super().__init__()
        self.d, self.m = d, m

    def evaluate(self, X: torch.Tensor) -> torch.Tensor:
        m = self.m
        n = X.shape[0]
        g = torch.sum((X[:, m - 1 :] - 0.5) ** 2, dim=1, keepdim=True)
        ones = torch.ones(n, 1, device=X.device)
        cosines = torch.cat([ones, torch.clamp_min(torch.cos(X[:, : m - 1] * torch.pi / 2), 0.0)], dim=1)
        sines = torch.cat([ones, torch.sin(torch.flip(X[:, : m - 1], dims=[1]) * torch.pi / 2)], dim=1)
        return (1 + g) * torch.flip(torch.cumprod(cosines, dim=1), dims=[1]) * sines
