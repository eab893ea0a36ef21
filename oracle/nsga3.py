"""CPU restatement of NSGA-III's environmental selection, TEST INFRASTRUCTURE only (never imported by the
package): plain loops over reference points, following evox/algorithms/mo/nsga3.py:155-266 step by step.

Pinned against tests/golden/nsga3.npz, which tests/golden/make_golden.py records from the reference's own
`NSGA3.step` (state before, offspring, the two permutations it draws, state after).
"""

from __future__ import annotations

import torch

from . import nds as onds


def perpendicular_distances(fit: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """|f| * sqrt(1 - cos^2) of every (solution, reference point) pair (nsga3.py:272-286)."""
    mag = torch.norm(fit, dim=1, keepdim=True).clamp_min(1e-10)
    fn = fit / mag
    rn = ref / torch.norm(ref, dim=1, keepdim=True).clamp_min(1e-10)
    cos = torch.matmul(fn, rn.T)
    return mag * torch.sqrt((1 - cos**2).clamp_min(1e-10))


def normalise(fit: torch.Tensor) -> torch.Tensor:
    """Translate by the ideal point and divide by the hyperplane intercepts of the extreme points
    (achievement scalarising weights eye + 1e-6), or by the largest value per objective when the
    extreme points are degenerate (nsga3.py:176-188)."""
    m = fit.shape[1]
    f = fit - fit.min(dim=0).values
    w = torch.eye(m, dtype=f.dtype) + 1e-6
    extreme = torch.stack([f[torch.argmin((f / w[j]).max(dim=1).values)] for j in range(m)])
    if int(torch.linalg.matrix_rank(extreme)) == m:
        intercepts = 1.0 / torch.linalg.solve(extreme, torch.ones(m, dtype=f.dtype))
    else:
        intercepts = f.max(dim=0).values
    return f / intercepts


def masked_assign(target: list, index: list, mask: list, value) -> list:
    """The reference's `_masked_assign` (nsga3.py:56-72) as the CPU executes it: every entry writes to its
    index clamped into the target, `value` where the mask holds and the target's OLD entry elsewhere, one
    after the other, so that among entries meeting at one index the last one stands. An entry outside the
    mask can therefore undo an assignment made at the index it is clamped to (index 0 for reference points
    without a candidate in the first stage, the last index for exhausted ones afterwards)."""
    n = len(target)
    out = list(target)
    for idx, m in zip(index, mask):
        j = min(max(int(idx), 0), n - 1)
        out[j] = value if m else target[j]
    return out


def environmental_selection(pop, fit, offspring, off_fit, perm_merge, perm_ref, ref, pop_size):
    """-> (pop, fit, rank) of the next generation (nsga3.py:163-266), the reference's bookkeeping restated with
    plain lists: `rho` = members admitted per reference point, `rho_last` = candidates of the last front left
    per reference point, `big` = the sentinel the reference calls upper_bound."""
    merge_pop = torch.cat([pop, offspring])[perm_merge]
    merge_fit = torch.cat([fit, off_fit])[perm_merge]
    rank_t = onds.non_dominate_rank(merge_fit)
    worst = int(torch.sort(rank_t).values[pop_size])  # rank of the (pop_size + 1)-th best
    keep = torch.nonzero(rank_t <= worst).flatten()
    merge_pop, merge_fit, rank_t = merge_pop[keep], merge_fit[keep], rank_t[keep]
    c, n_ref = merge_pop.shape[0], ref.shape[0]
    dist = perpendicular_distances(normalise(merge_fit), ref[perm_ref])
    group_dist_t, group_id_t = dist.min(dim=1)
    group_dist, rank = group_dist_t.tolist(), [int(r) for r in rank_t]
    big = c + merge_pop.shape[1] + merge_fit.shape[1] + 1
    rho, rho_last = [0] * n_ref, [0] * n_ref
    for i in range(c):
        (rho if rank[i] < worst else rho_last)[int(group_id_t[i])] += 1
    selected_num = sum(rho)
    rho = [big if rho_last[r] == 0 else rho[r] for r in range(n_ref)]
    group_id = [int(group_id_t[i]) if rank[i] == worst else big for i in range(c)]

    # first stage: reference points nobody was admitted for take their closest candidate (first minimum);
    # the others "take" the first minimum of an all-infinite column, index 0, outside the mask
    selected_ref = [rho[r] == 0 for r in range(n_ref)]
    candi = []
    for r in range(n_ref):
        col = [group_dist[i] if (selected_ref[r] and group_id[i] == r) else float("inf") for i in range(c)]
        candi.append(min(range(c), key=lambda i: (col[i], i)))
    rank = masked_assign(rank, candi, selected_ref, worst - 1)
    for r in range(n_ref):
        if selected_ref[r]:
            rho_last[r] -= 1
            rho[r] = 1
        if rho_last[r] == 0:
            rho[r] = big
    selected_num += sum(selected_ref)

    # second stage: per reference point the remaining candidates in index order
    group_id = masked_assign(group_id, candi, selected_ref, big)
    table = [[i for i in range(c) if group_id[i] == r] + [big] * c for r in range(n_ref)]
    cursor = [0] * n_ref
    while selected_num < pop_size:
        level = min(rho)
        selected_ref = [rho[r] == level for r in range(n_ref)]
        candi = [table[r][cursor[r]] for r in range(n_ref)]
        rank = masked_assign(rank, candi, selected_ref, worst - 1)
        for r in range(n_ref):
            if selected_ref[r]:
                cursor[r] += 1
                rho_last[r] -= 1
                rho[r] = level + 1
            if rho_last[r] == 0:
                rho[r] = big
        selected_num += sum(selected_ref)

    # the last round may admit too many: its lowest indices leave again
    dif = selected_num - pop_size
    order = sorted(candi[r] if selected_ref[r] else big for r in range(n_ref))
    rank = masked_assign(rank, order, [p < dif for p in range(n_ref)], worst)

    final = torch.tensor([r < worst for r in rank])
    return merge_pop[final], merge_fit[final], torch.tensor(rank, dtype=rank_t.dtype)[final]
