"""Oracle for NSGA-II environmental selection (test infrastructure; see oracle/__init__.py).

Restates dominate_relation, the front-peeling loop of non_dominate_rank, crowding_distance and
nd_environmental_selection (operators/selection/non_dominate.py:6-26, 151-195, 198-231, 234-254)
and the stable lexsort they rely on (utils/jit_fix_operator.py:216-252).

`non_dominate_rank` here holds the dominance matrix bit-packed and builds it in row blocks, so
that sizes the reference cannot hold in memory (it materialises two (n, n, m) boolean tensors)
still finish; for sizes the reference can run, tests/golden pins that both give the same ranks.
"""

from __future__ import annotations

import numpy as np
import torch


def dominate_relation(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """A[i, j] = x_i dominates y_j: all(x_i <= y_j) and any(x_i < y_j) (non_dominate.py:16-24)."""
    le = (x[:, None, :] <= y[None, :, :]).all(dim=2)
    lt = (x[:, None, :] < y[None, :, :]).any(dim=2)
    return le & lt


def non_dominate_rank(f: torch.Tensor, block: int = 2048) -> torch.Tensor:
    """Rank 0 = non-dominated; each pass removes the current front and decrements the dominated
    counts of what it dominates (non_dominate.py:29-59, 162-168, 186-194)."""
    n = f.shape[0]
    words = (n + 7) // 8
    packed = np.zeros((n, words), dtype=np.uint8)  # row i: bit j set iff i dominates j
    count = torch.zeros(n, dtype=torch.int64)
    for a in range(0, n, block):
        d = dominate_relation(f[a : a + block], f)
        count += d.sum(dim=0)
        packed[a : a + block] = np.packbits(d.numpy(), axis=1, bitorder="little")
    rank = torch.zeros(n, dtype=torch.int32)
    front = count == 0
    current = 0
    while bool(front.any()):
        rank = torch.where(front, current, rank).to(torch.int32)
        idx = torch.nonzero(front).flatten().numpy()
        dec = torch.zeros(n, dtype=torch.int64)
        for a in range(0, len(idx), block):
            rows = np.unpackbits(packed[idx[a : a + block]], axis=1, count=n, bitorder="little")
            dec += torch.from_numpy(rows.sum(axis=0, dtype=np.int64))
        count = count - dec - front.to(torch.int64)
        current += 1
        front = count == 0
    return rank


def lexsort(keys: list[torch.Tensor], dim: int = -1) -> torch.Tensor:
    """Last key is the primary one; every pass is a stable argsort (jit_fix_operator.py:246-252)."""
    order = torch.argsort(keys[0], dim=dim, stable=True)
    for key in keys[1:]:
        order = order.gather(dim, torch.argsort(key.gather(dim, order), dim=dim, stable=True))
    return order


def crowding_distance(costs: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """non_dominate.py:198-231. Rows outside `mask` get -inf; per objective the masked rows are
    sorted (stable), interior rows get (next - previous) / (last - first), the two ends +inf."""
    n, m = costs.shape
    n_valid = int(mask.sum())
    inv = (~mask)[:, None].expand(-1, m).to(costs.dtype)
    order = lexsort([costs, inv], dim=0)
    sorted_costs = torch.gather(costs, 0, order)
    span = sorted_costs[n_valid - 1] - sorted_costs[0]
    dist = torch.zeros(n, m, dtype=costs.dtype)  # the reference leaves one masked-out slot uninitialised
    dist = dist.scatter(0, order[1:-1], (sorted_costs[2:] - sorted_costs[:-2]) / span)
    # advanced indexing with the (m,) index rows: a row that is first or last in ANY objective
    # becomes +inf in EVERY column (non_dominate.py:226-227)
    dist[order[0], :] = torch.inf
    dist[order[n_valid - 1], :] = torch.inf
    dist = torch.where(mask[:, None], dist, -torch.inf)
    return dist.sum(dim=1)


def nd_environmental_selection(x: torch.Tensor, f: torch.Tensor, topk: int, rank: torch.Tensor | None = None):
    """non_dominate.py:234-254. Also returns the selected row indices (the reference returns only
    the gathered rows)."""
    if rank is None:
        rank = non_dominate_rank(f)
    worst = torch.topk(rank, topk, largest=False)[0][-1]
    mask = rank == worst
    crowd = crowding_distance(f, mask)
    order = lexsort([-crowd, rank])[:topk]
    return x[order], f[order], rank[order], crowd[order], order


def dtlz2_objectives(x: torch.Tensor, m: int = 3) -> torch.Tensor:
    """Objective values of the DTLZ2 shape used by the benchmark configuration: g = sum over the
    last (d - m + 1) variables of (x - 0.5)^2, points on the unit sphere scaled by (1 + g)
    (problems/numerical/dtlz.py:97-127)."""
    n = x.shape[0]
    g = torch.sum((x[:, m - 1 :] - 0.5) ** 2, dim=1, keepdim=True)
    ang = x[:, : m - 1] * (torch.pi / 2)
    cosines = torch.cat([torch.ones(n, 1), torch.cos(ang).clamp_min(0.0)], dim=1)
    cum = torch.flip(torch.cumprod(cosines, dim=1), [1])
    sines = torch.cat([torch.ones(n, 1), torch.sin(torch.flip(ang, [1]))], dim=1)
    return (1 + g) * cum * sines
