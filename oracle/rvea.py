"""Oracle for RVEA's reference-vector-guided selection (test infrastructure; see oracle/__init__.py).

Restates ref_vec_guided and apd_fn (operators/selection/rvea_selection.py:7-99) with the relu-form
helpers they call: nanmin (utils/jit_fix_operator.py:255-292), maximum (:108-123), clamp_float
(:47-66). Cosines come from torch.nn.functional.cosine_similarity, the same ATen routine the
reference calls (:63, :75). Besides the reference's outputs the intermediate association, APD
matrix and selected row numbers are returned so that tests can reason about near-ties.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def _relu_clamp01(a: torch.Tensor) -> torch.Tensor:
    return a + torch.relu(0.0 - a) - torch.relu(a - 1.0)


def ref_vec_guided(x: torch.Tensor, f: torch.Tensor, v: torch.Tensor, theta: torch.Tensor):
    n, nv, m = f.size(0), v.size(0), f.size(1)
    zmin = torch.where(torch.isnan(f), torch.inf, f).min(dim=0, keepdim=True)[0]
    obj = f - zmin
    obj = obj + torch.relu(torch.tensor(1e-32) - obj)
    cos_vv = F.cosine_similarity(v.unsqueeze(1), v.unsqueeze(0), dim=-1)
    cos_vv = torch.where(torch.eye(nv, dtype=torch.bool), 0, cos_vv)
    gamma = torch.min(torch.acos(_relu_clamp01(cos_vv)), dim=1)[0]
    angle = torch.acos(_relu_clamp01(F.cosine_similarity(obj.unsqueeze(1), v.unsqueeze(0), dim=-1)))
    nan_mask = torch.isnan(obj).any(dim=1)
    associate = torch.where(nan_mask, -1, torch.argmin(angle, dim=1))
    member = associate[:, None] == torch.arange(nv)[None, :]
    empty = member.sum(dim=0) == 0
    norm = torch.linalg.vector_norm(obj, dim=1)
    # rvea_selection.py:25-29: (1 + m * theta * angle) / gamma * |obj|
    apd = (1 + m * theta * angle) / gamma[None, :] * norm[:, None]
    apd = torch.where(member, apd, torch.inf)
    next_ind = torch.argmin(apd, dim=0)
    next_x = torch.where(empty[:, None], torch.nan, x[next_ind])
    next_f = torch.where(empty[:, None], torch.nan, f[next_ind])
    return {
        "next_x": next_x, "next_f": next_f, "next_ind": torch.where(empty, -1, next_ind), "associate": associate,
        "apd": apd, "angle": angle, "gamma": gamma, "empty": empty,
    }


def simplex_lattice(h: int, m: int) -> torch.Tensor:
    """All m-part compositions of h divided by h: the Das-Dennis design the benchmark
    configuration's reference vectors come from (H = 3, M = 10 gives 220 of the 275 vectors; the
    inner layer is added by two_layer_vectors)."""
    rows = []

    def rec(prefix, left, slots):
        if slots == 1:
            rows.append(prefix + [left])
            return
        for k in range(left + 1):
            rec(prefix + [k], left - k, slots - 1)

    rec([], h, m)
    return torch.tensor(rows, dtype=torch.float32) / h


def two_layer_vectors(h1: int, h2: int, m: int) -> torch.Tensor:
    """Outer lattice + inner lattice shrunk halfway towards the centre (275 vectors for
    h1 = 3, h2 = 2, m = 10, as operators/sampling/uniform.py:8-51 produces)."""
    outer = simplex_lattice(h1, m)
    if h2 <= 0:
        return outer
    inner = simplex_lattice(h2, m) / 2 + 1 / (2 * m)
    return torch.cat([outer, inner], dim=0)


def config2_inputs(n: int = 50_000, m: int = 10, dx: int = 19, seed: int = 0):
    """benchmark configuration 2: objectives uniform in [0,1] + 0.05 |N(0,1)|, 275 simplex-lattice vectors."""
    g = torch.Generator().manual_seed(seed)
    f = torch.rand(n, m, generator=g) + 0.05 * torch.randn(n, m, generator=g).abs()
    x = torch.rand(n, dx, generator=g)
    v = two_layer_vectors(3, 2, m)
    return x, f, v, torch.tensor(0.25)


def _nanmin0(x: torch.Tensor) -> torch.Tensor:
    return torch.where(torch.isnan(x), torch.inf, x).min(dim=0).values


def _nanmax0(x: torch.Tensor) -> torch.Tensor:
    return torch.where(torch.isnan(x), -torch.inf, x).max(dim=0).values


def rv_regeneration(pop_obj: torch.Tensor, v: torch.Tensor, draw: torch.Tensor) -> torch.Tensor:
    """RVEAa._rv_regeneration (algorithms/mo/rveaa.py:129-142): reference vectors of the second set that no
    individual is closest to are redrawn inside the objectives' current range; `draw` is the uniform draw."""
    import torch.nn.functional as F

    pop_obj = pop_obj - _nanmin0(pop_obj)
    cosine = F.cosine_similarity(pop_obj.unsqueeze(1), v.unsqueeze(0), dim=-1)
    filled = torch.where(torch.isnan(cosine), -torch.inf, cosine)
    associate = filled.max(dim=1).indices
    associate = torch.where(filled[:, 0] == -torch.inf, -1, associate)
    taken = torch.sum(associate.unsqueeze(1) == torch.arange(v.size(0)), dim=0)
    return torch.where((taken == 0).unsqueeze(1), draw * _nanmax0(pop_obj), v)


def batch_truncation(pop: torch.Tensor, obj: torch.Tensor):
    """RVEAa._batch_truncation (rveaa.py:144-164): rank the rows by the cosine to their nearest other row
    (most crowded first) and blank the first half with NaN."""
    import torch.nn.functional as F

    n = pop.size(0) // 2
    cosine = F.cosine_similarity(obj.unsqueeze(1), obj.unsqueeze(0), dim=-1)
    not_all_nan_rows = ~torch.isnan(cosine).all(dim=1)
    cosine = torch.where(torch.eye(cosine.size(0), dtype=torch.bool) & not_all_nan_rows.unsqueeze(1), 0, cosine)
    sorted_values, _ = torch.sort(-cosine, dim=1)
    nearest = torch.where(torch.isnan(sorted_values[:, 0]), -torch.inf, sorted_values[:, 0])
    rank = torch.argsort(nearest)  # computed by the reference and then not used: the mask below is by POSITION
    keep = (torch.arange(rank.size(0)) >= n).unsqueeze(1)
    return torch.where(keep, pop, torch.nan), torch.where(keep, obj, torch.nan)
