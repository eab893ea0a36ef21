"""Oracle for the particle swarm step (test infrastructure; see oracle/__init__.py).

Restates PSO.step / PSO.init_step (algorithms/so/pso_variants/pso.py:71-115), min_by
(pso_variants/utils.py:6-25), the relu-form clamp (utils/jit_fix_operator.py:24-44) and the
Ackley / Rastrigin test functions (problems/numerical/basic.py:66-69, 115-116).
State is a plain dict with the reference's buffer names.
"""

from __future__ import annotations

import math

import torch


def relu_clamp(a: torch.Tensor, lb: torch.Tensor, ub: torch.Tensor) -> torch.Tensor:
    """jit_fix_operator.py:42-44 — not bit-equal to torch.clamp."""
    return a + torch.relu(lb - a) - torch.relu(a - ub)


def ackley(x: torch.Tensor, a: float = 20.0, b: float = 0.2, c: float = 2 * math.pi) -> torch.Tensor:
    """basic.py:66-69."""
    return -a * torch.exp(-b * torch.sqrt(torch.mean(x**2, dim=1))) - torch.exp(torch.mean(torch.cos(c * x), dim=1)) + a + math.e


def rastrigin(x: torch.Tensor) -> torch.Tensor:
    """basic.py:115-116."""
    return 10 * x.size(1) + torch.sum(x**2 - 10 * torch.cos(2 * math.pi * x), dim=1)


def sphere(x: torch.Tensor) -> torch.Tensor:
    return torch.sum(x**2, dim=1)


FITNESS = {"ackley": ackley, "rastrigin": rastrigin, "sphere": sphere}


def min_by(values: list[torch.Tensor], keys: list[torch.Tensor]):
    """utils.py:18-25 — first minimum of the concatenated keys and the row it belongs to."""
    v = torch.cat(values, dim=0)
    k = torch.cat(keys, dim=0)
    i = torch.argmin(k)
    return v[i], k[i]


def init_step(state: dict, fitness) -> dict:
    """pso.py:108-115."""
    s = dict(state)
    s["fit"] = fitness(s["pop"])
    s["local_best_fit"] = s["fit"]
    s["global_best_location"], s["global_best_fit"] = min_by([s["pop"]], [s["fit"]])
    return s


def step(state: dict, rg: torch.Tensor, rp: torch.Tensor, fitness) -> dict:
    """pso.py:89-106 with the two uniform draws passed in (rg is drawn first, :96-97)."""
    s = dict(state)
    better = s["local_best_fit"] > s["fit"]
    s["local_best_location"] = torch.where(better[:, None], s["pop"], s["local_best_location"])
    s["local_best_fit"] = torch.where(better, s["fit"], s["local_best_fit"])
    s["global_best_location"], s["global_best_fit"] = min_by(
        [s["global_best_location"][None], s["pop"]], [s["global_best_fit"][None], s["fit"]]
    )
    lb, ub = s["lb"], s["ub"]
    velocity = (
        s["w"] * s["velocity"]
        + s["phi_p"] * rp * (s["local_best_location"] - s["pop"])
        + s["phi_g"] * rg * (s["global_best_location"] - s["pop"])
    )
    pop = s["pop"] + velocity
    s["pop"] = relu_clamp(pop, lb, ub)
    s["velocity"] = relu_clamp(velocity, lb, ub)
    s["fit"] = fitness(s["pop"])
    return s


def make_state(pop_size: int, dim: int, lb: float, ub: float, w: float, phi_p: float, phi_g: float, seed: int) -> dict:
    """Initial swarm of the benchmark configurations: positions uniform in [lb, ub), velocities
    uniform in +-0.2 * (ub - lb); personal / global bests unset (+inf), as PSO.__init__ leaves them."""
    g = torch.Generator().manual_seed(seed)
    span = ub - lb
    pop = lb + span * torch.rand(pop_size, dim, generator=g)
    vel = 0.2 * span * (2 * torch.rand(pop_size, dim, generator=g) - 1)
    return {
        "pop": pop,
        "velocity": vel,
        "fit": torch.full((pop_size,), torch.inf),
        "local_best_location": pop.clone(),
        "local_best_fit": torch.full((pop_size,), torch.inf),
        "global_best_location": pop[0].clone(),
        "global_best_fit": torch.tensor(torch.inf),
        "lb": torch.full((1, dim), lb),
        "ub": torch.full((1, dim), ub),
        "w": torch.tensor(w),
        "phi_p": torch.tensor(phi_p),
        "phi_g": torch.tensor(phi_g),
    }


def draws(pop_size: int, dim: int, seed: int):
    """rg then rp for one generation."""
    g = torch.Generator().manual_seed(seed)
    rg = torch.rand(pop_size, dim, generator=g)
    rp = torch.rand(pop_size, dim, generator=g)
    return rg, rp


# ---------------------------------------------------------------------------------------------
# Philox stream of the in-kernel generator (defined by this repository, not by the reference):
# key = seed, counter = (q lo, q hi, generation lo, which + 2 * generation hi),
# q = global_row * ceil(dim / 4) + column // 4; outputs c0..c3 -> columns 4q..4q+3.
# The round function and the 24-bit conversion restate triton_kernels/kernels/philox.py:52-112.
# ---------------------------------------------------------------------------------------------
_M0, _M1, _W0, _W1, _MASK = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Vectorised over int64 tensors holding uint32 values."""
    for _ in range(10):
        p0 = c0 * _M0  # < 2^64: exact in uint64 arithmetic, taken modulo 2^64 by int64 wraparound
        p1 = c2 * _M1
        hi0, lo0 = (p0 >> 32) & _MASK, p0 & _MASK
        hi1, lo1 = (p1 >> 32) & _MASK, p1 & _MASK
        c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
        k0 = (k0 + _W0) & _MASK
        k1 = (k1 + _W1) & _MASK
    return c0, c1, c2, c3


def pso_uniform(pop_size: int, dim: int, seed: int, generation: int, which: int, row_offset: int = 0) -> torch.Tensor:
    n_call = (dim + 3) // 4
    q = (torch.arange(pop_size, dtype=torch.int64)[:, None] + row_offset) * n_call + torch.arange(n_call, dtype=torch.int64)[None, :]
    c0, c1 = q & _MASK, (q >> 32) & _MASK
    c2 = torch.full_like(q, generation & _MASK)
    c3 = torch.full_like(q, (which + 2 * ((generation >> 32) & _MASK)) & _MASK)
    k0 = torch.full_like(q, seed & _MASK)
    k1 = torch.full_like(q, (seed >> 32) & _MASK)
    out = torch.stack(philox4x32_10(c0, c1, c2, c3, k0, k1), dim=2).reshape(pop_size, n_call * 4)[:, :dim]
    return ((out & _MASK) >> 8).to(torch.float32) * (1.0 / (1 << 24))


# ---------------------------------------------------------------------------------------------
# Sharded swarm: the best-particle record each rank contributes and how the records are merged.
# Layout as in include/evox_b200.h (evox_pso_local_best): word 0 fitness bits, words 1-2 global
# row index (int64), word 3 zero, then the row. min_by's tie rules (utils.py:18-25) decide.
# ---------------------------------------------------------------------------------------------
def candidate_record(fit: torch.Tensor, pop: torch.Tensor, row_offset: int) -> torch.Tensor:
    i = int(torch.argmin(fit))
    d = pop.shape[1]
    rec = torch.zeros(4 + d, dtype=torch.int32)
    rec[0] = fit[i : i + 1].view(torch.int32)[0]
    rec[1:3] = torch.tensor([i + row_offset], dtype=torch.int64).view(torch.int32)  # little endian: lo, hi
    rec[4:] = pop[i].view(torch.int32)
    return rec


def merge_records(records: torch.Tensor, world: int, d: int, gbest_loc: torch.Tensor, gbest_fit: torch.Tensor, have_previous: bool = True):
    """Pick the winner the way argmin over cat([old best, all particles]) would."""
    recs = records.view(world, 4 + d)
    fits = recs[:, 0].contiguous().view(torch.float32)
    idx = (recs[:, 1].to(torch.int64) & 0xFFFFFFFF) | (recs[:, 2].to(torch.int64) << 32)
    order = sorted(range(world), key=lambda r: int(idx[r]))  # global row order = concatenation order
    keys = torch.stack([fits[r] for r in order])
    rows = torch.stack([recs[r, 4:].contiguous().view(torch.float32) for r in order])
    if have_previous:
        return min_by([gbest_loc[None], rows], [gbest_fit[None], keys])
    return min_by([rows], [keys])
