"""NSGA-II and RVEA with every step of a generation on the device.

Constructor arguments and state names follow the reference (evox/algorithms/mo/nsga2.py:27-102,
rvea.py:28-154). With the default operators a generation is: mating selection kernel -> one fused
crossover + mutation + clamp kernel -> `evaluate` -> the environmental-selection kernels. Custom
`selection_op` / `mutation_op` / `crossover_op` callables are honoured as in the reference."""

from __future__ import annotations

from typing import Callable, Optional

import torch

from ..core import Algorithm, Mutable, Parameter
from ..core.functional import replica_seed
from ..operators.selection import nd_environmental_selection, non_dominate_rank, raise_on_kernel_errors, ref_vec_guided
from ..operators.variation import make_offspring, tournament_selection_multifit
from ..problems.numerical import _relu_clamp_rows

__all__ = ["NSGA2", "RVEA", "RVEAa", "uniform_sampling"]


def uniform_sampling(n: int, m: int) -> tuple[torch.Tensor, int]:
    """Das-Dennis two-layer simplex-lattice reference vectors (host arithmetic, done once): the
    largest design with at most `n` points, as evox/operators/sampling/uniform.py:8-51 builds it."""
    from itertools import combinations
    from math import comb

    h1 = 1
    while comb(h1 + m, m - 1) <= n:
        h1 += 1

    def lattice(h):
        rows = []
        for c in combinations(range(1, h + m), m - 1):
            prev, parts = 0, []
            for x in c:
                parts.append(x - prev - 1)
                prev = x
            parts.append(h + m - 1 - prev)
            rows.append(parts)
        return torch.tensor(rows, dtype=torch.float32) / h

    w = lattice(h1)
    if h1 < m:
        h2 = 0
        while comb(h1 + m - 1, m - 1) + comb(h2 + m, m - 1) <= n:
            h2 += 1
        if h2 > 0:
            w = torch.cat([w, lattice(h2) / 2 + 1 / (2 * m)], dim=0)
    w = torch.maximum(w, torch.tensor(1e-6))
    return w, w.shape[0]


class _MOBase(Algorithm):
    def _setup(self, pop_size, n_objs, lb, ub, selection_op, mutation_op, crossover_op, device):
        assert lb.shape == ub.shape and lb.ndim == 1 and ub.ndim == 1
        assert lb.dtype == ub.dtype and lb.device == ub.device
        self.n_objs = n_objs
        self.dim = lb.shape[0]
        self.lb = lb.to(device=device, dtype=torch.float32)
        self.ub = ub.to(device=device, dtype=torch.float32)
        self.selection, self.mutation, self.crossover = selection_op, mutation_op, crossover_op
        self.seed = int(torch.randint(0, 2**62, (), device="cpu"))
        self.generation = 0

    # -- checkpointing: the position in the random stream travels with the state_dict --------------
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
        # some populations change their row count while they run (RVEAa keeps 2 * pop_size rows after its first
        # generation, rveaa.py:189-212): a buffer whose stored shape differs is re-created before the copy
        for name, buf in list(self.named_buffers(recurse=False)):
            src = state_dict.get(name)
            if isinstance(src, torch.Tensor) and src.shape != buf.shape:
                setattr(self, name, torch.empty(src.shape, dtype=buf.dtype, device=buf.device))
        out = super().load_state_dict(state_dict, strict=strict, assign=assign)
        self._after_load()
        return out

    def _after_load(self) -> None:
        pass

    def _variation(self, pop: torch.Tensor, mating_pool: torch.Tensor | None, draws: dict | None) -> torch.Tensor:
        """crossover -> mutation -> clamp (nsga2.py:95-97). Fused kernel unless custom operators are set."""
        if self.crossover is None and self.mutation is None:
            return make_offspring(pop, self.lb, self.ub, mating_pool, draws, seed=replica_seed(self.seed), generation=self.generation)
        from ..operators.variation import polynomial_mutation, simulated_binary

        parents = pop if mating_pool is None else pop[mating_pool]
        crossed = (self.crossover or simulated_binary)(parents)
        mutated = (self.mutation or polynomial_mutation)(crossed, self.lb, self.ub)
        return _relu_clamp_rows(mutated, self.lb, self.ub)


class NSGA2(_MOBase):
    def __init__(self, pop_size: int, n_objs: int, lb: torch.Tensor, ub: torch.Tensor, selection_op: Optional[Callable] = None,
                 mutation_op: Optional[Callable] = None, crossover_op: Optional[Callable] = None, device: torch.device | None = None):
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        self.pop_size = pop_size
        self._setup(pop_size, n_objs, lb, ub, selection_op, mutation_op, crossover_op, device)
        pop = (self.ub - self.lb) * torch.rand(pop_size, self.dim, device=device) + self.lb
        self.pop = Mutable(pop)
        self.fit = Mutable(torch.full((pop_size, n_objs), torch.inf, device=device))
        self.rank = Mutable(torch.full((pop_size,), torch.inf, device=device))
        self.dis = Mutable(torch.full((pop_size,), -torch.inf, device=device))

    def init_step(self):
        self.fit = self.evaluate(self.pop)
        _, _, self.rank, self.dis = nd_environmental_selection(self.pop, self.fit, self.pop_size)

    def step(self, parents: torch.Tensor | None = None, draws: dict | None = None):
        """One generation (nsga2.py:92-102). `parents` (pop_size, 2) and `draws` replace the random
        draws of the tournament and of crossover / mutation."""
        raise_on_kernel_errors()  # status of the previous generation's non-dominated sort
        select = self.selection or tournament_selection_multifit
        kwargs = {"parents": parents} if (self.selection is None and parents is not None) else {}
        mating_pool = select(self.pop_size, [-self.dis, self.rank.to(torch.float32)], **kwargs)
        offspring = self._variation(self.pop, mating_pool, draws)
        off_fit = self.evaluate(offspring)
        merge_pop = torch.cat([self.pop, offspring], dim=0)
        merge_fit = torch.cat([self.fit, off_fit], dim=0)
        self.pop, self.fit, self.rank, self.dis = nd_environmental_selection(merge_pop, merge_fit, self.pop_size)
        self.generation += 1


def _masked_assign(target: torch.Tensor, index: torch.Tensor, mask: torch.Tensor, value) -> torch.Tensor:
    """`target` with `value` written at `index[mask]`, INCLUDING what the reference's helper of that name does
    with the entries outside the mask (nsga3.py:56-72): every entry writes to its index clamped into the
    target, the target's old value where the mask does not hold, and among entries that meet at one index the
    LAST one stands, as on the reference's sequential CPU path (a plain `index_copy` with duplicates is not
    deterministic on a GPU). An assignment can thus be undone by a later entry outside the mask that is
    clamped onto the same index; generations of the reference depend on it."""
    n = target.shape[0]
    idx = index.clamp(0, n - 1).to(torch.int64)
    pos = torch.arange(idx.shape[0], device=target.device)
    last = torch.full((n,), -1, dtype=torch.int64, device=target.device).scatter_reduce(0, idx, pos, "amax", include_self=True)
    wins = last[idx] == pos
    write = torch.where(mask, torch.as_tensor(value, dtype=target.dtype, device=target.device), target[idx])
    out = target.clone()
    out[idx[wins]] = write[wins]
    return out


class NSGA3(_MOBase):
    """NSGA-III (algorithms/mo/nsga3.py:75-286): non-dominated rank by the dominance / peel kernels, then
    reference-point niching over the last admitted front. Constructor arguments and state names are the
    reference's; `data_type` other than float32 is not supported."""

    def __init__(self, pop_size: int, n_objs: int, lb: torch.Tensor, ub: torch.Tensor, selection_op: Optional[Callable] = None,
                 mutation_op: Optional[Callable] = None, crossover_op: Optional[Callable] = None,
                 data_type: Optional[torch.dtype] = None, device: torch.device | None = None):
        super().__init__()
        assert data_type in (None, torch.float32), "NSGA3: only float32 decision variables"
        device = torch.get_default_device() if device is None else torch.device(device)
        self.pop_size = pop_size
        self._setup(pop_size, n_objs, lb, ub, selection_op, mutation_op, crossover_op, device)
        pop = (self.ub - self.lb) * torch.rand(pop_size, self.dim, device=device) + self.lb
        self.pop = Mutable(pop)
        self.fit = Mutable(torch.full((pop_size, n_objs), torch.inf, device=device))
        self.rank = Mutable(torch.full((pop_size,), torch.inf, device=device))
        self.ref = uniform_sampling(pop_size, n_objs)[0].to(device)

    def init_step(self):
        self.fit = self.evaluate(self.pop)
        self.rank = non_dominate_rank(self.fit)

    def step(self, parents: torch.Tensor | None = None, draws: dict | None = None, perm_merge: torch.Tensor | None = None,
             perm_ref: torch.Tensor | None = None):
        """One generation (nsga3.py:155-266). `parents`, `draws`, `perm_merge`, `perm_ref` replace the random
        draws of the tournament, of crossover / mutation and of the two permutations."""
        raise_on_kernel_errors()
        select = self.selection or tournament_selection_multifit
        kwargs = {"parents": parents} if (self.selection is None and parents is not None) else {}
        mating_pool = select(self.pop_size, [self.rank.to(torch.float32)], **kwargs)
        offspring = self._variation(self.pop, mating_pool, draws)
        off_fit = self.evaluate(offspring)
        self.environmental_selection(offspring, off_fit, perm_merge, perm_ref)
        self.generation += 1

    @staticmethod
    def _normalise(fit: torch.Tensor) -> torch.Tensor:
        """Ideal-point translation and hyperplane intercepts of the extreme points (nsga3.py:176-188)."""
        m = fit.shape[1]
        f = fit - fit.min(dim=0).values
        w = torch.eye(m, device=f.device) + 1e-6
        # per objective j the row with the smallest achievement value max_k f[i, k] / w[j, k]
        extreme = f[(f.unsqueeze(0) / w.unsqueeze(1)).max(dim=2).values.argmin(dim=1)]
        if int(torch.linalg.matrix_rank(extreme)) == m:
            intercepts = 1.0 / torch.linalg.solve(extreme, torch.ones(m, device=f.device))
        else:
            intercepts = f.max(dim=0).values
        return f / intercepts

    @staticmethod
    def _distances(fit: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
        """|f| * sqrt(1 - cos^2) of every (row, reference point) pair (nsga3.py:272-286)."""
        mag = torch.norm(fit, dim=1, keepdim=True).clamp_min(1e-10)
        cos = torch.matmul(fit / mag, (ref / torch.norm(ref, dim=1, keepdim=True).clamp_min(1e-10)).T)
        return mag * torch.sqrt((1 - cos**2).clamp_min(1e-10))

    def environmental_selection(self, offspring: torch.Tensor, off_fit: torch.Tensor, perm_merge: torch.Tensor | None = None,
                                perm_ref: torch.Tensor | None = None) -> None:
        dev, n_keep = self.pop.device, self.pop_size
        merge_pop = torch.cat([self.pop, offspring], dim=0)
        merge_fit = torch.cat([self.fit, off_fit], dim=0)
        perm_merge = torch.randperm(merge_pop.shape[0], device=dev) if perm_merge is None else perm_merge.to(dev)
        merge_pop, merge_fit = merge_pop[perm_merge], merge_fit[perm_merge]
        rank = non_dominate_rank(merge_fit)
        worst = torch.sort(rank).values[n_keep]  # rank of the (pop_size + 1)-th best row
        keep = torch.nonzero(rank <= worst).flatten()
        merge_pop, merge_fit, rank = merge_pop[keep], merge_fit[keep], rank[keep]
        c, n_ref = merge_pop.shape[0], self.ref.shape[0]
        perm_ref = torch.randperm(n_ref, device=dev) if perm_ref is None else perm_ref.to(dev)
        group_dist, group_id = self._distances(self._normalise(merge_fit), self.ref[perm_ref]).min(dim=1)
        big = c + merge_pop.shape[1] + merge_fit.shape[1] + 1  # the reference's upper_bound sentinel
        in_last = rank == worst
        zeros = torch.zeros(n_ref, dtype=torch.int64, device=dev)
        rho = zeros.scatter_add(0, group_id, (~in_last).to(torch.int64))  # rows already admitted, per reference point
        rho_last = zeros.scatter_add(0, group_id, in_last.to(torch.int64))  # candidates of the last front
        selected_num = int(rho.sum())
        rho = torch.where(rho_last == 0, big, rho)
        group_id = torch.where(in_last, group_id, big)
        rows = torch.arange(c, device=dev)

        # first stage: reference points nobody was admitted for take their closest candidate (first minimum);
        # candidates ordered by (reference point, distance, index): a group's first entry is that minimum
        selected_ref = rho == 0
        by_dist = torch.argsort(group_dist, stable=True)
        order = by_dist[torch.argsort(group_id[by_dist], stable=True)]
        first = torch.full((n_ref + 1,), c, dtype=torch.int64, device=dev).scatter_reduce(
            0, group_id[order].clamp(max=n_ref), rows, "amin", include_self=True)[:n_ref]
        candi = torch.where(selected_ref, order[first.clamp(max=c - 1)], 0)  # the others: argmin of an all-inf column = 0
        rank = _masked_assign(rank, candi, selected_ref, worst - 1)
        rho_last = torch.where(selected_ref, rho_last - 1, rho_last)
        rho = torch.where(selected_ref, 1, rho)
        rho = torch.where(rho_last == 0, big, rho)
        selected_num += int(selected_ref.sum())

        # second stage: per reference point its remaining candidates in index order, one per round for the
        # reference points with the fewest admitted rows
        group_id = _masked_assign(group_id, candi, selected_ref, big)
        order = torch.argsort(group_id, stable=True)  # by (reference point, index); rows outside the last front at the end
        counts = zeros.scatter_add(0, group_id.clamp(max=n_ref - 1), (group_id < big).to(torch.int64))
        start = torch.cumsum(counts, 0) - counts
        cursor = torch.zeros_like(counts)
        while selected_num < n_keep:
            selected_ref = rho == rho.min()
            level = rho.min()
            candi = torch.where(cursor < counts, order[(start + cursor).clamp(max=c - 1)], big)
            rank = _masked_assign(rank, candi, selected_ref, worst - 1)
            cursor = torch.where(selected_ref, cursor + 1, cursor)
            rho_last = torch.where(selected_ref, rho_last - 1, rho_last)
            rho = torch.where(selected_ref, level + 1, rho)
            rho = torch.where(rho_last == 0, big, rho)
            selected_num += int(selected_ref.sum())

        # the last round may admit too many: its lowest indices leave again
        dif = selected_num - n_keep
        leaving = torch.sort(torch.where(selected_ref, candi, big)).values
        rank = _masked_assign(rank, leaving, torch.arange(n_ref, device=dev) < dif, worst)
        final = rank < worst
        self.pop, self.fit, self.rank = merge_pop[final], merge_fit[final], rank[final]


class RVEA(_MOBase):
    def __init__(self, pop_size: int, n_objs: int, lb: torch.Tensor, ub: torch.Tensor, alpha: float = 2.0, fr: float = 0.1,
                 max_gen: int = 100, selection_op: Optional[Callable] = None, mutation_op: Optional[Callable] = None,
                 crossover_op: Optional[Callable] = None, device: torch.device | None = None):
        super().__init__()
        device = torch.get_default_device() if device is None else torch.device(device)
        self._setup(pop_size, n_objs, lb, ub, selection_op, mutation_op, crossover_op, device)
        self.alpha = Parameter(alpha, dtype=torch.float32, device=device)
        self.fr = Parameter(fr, dtype=torch.float32, device=device)
        self.max_gen = Parameter(max_gen, dtype=torch.float32, device=device)
        self._schedule = None  # host copies of (generation count, adaptation period, last generation)
        v, n = uniform_sampling(pop_size, n_objs)
        v = v.to(device)
        self.pop_size = n
        self.pop = Mutable((self.ub - self.lb) * torch.rand(n, self.dim, device=device) + self.lb)
        self.fit = Mutable(torch.full((n, n_objs), torch.inf, device=device))
        self.reference_vector = Mutable(v.clone())
        self.init_v = v
        self.gen = Mutable(torch.tensor(0, dtype=torch.int64, device=device))

    def _sync_schedule(self) -> None:
        """Host copies of what decides WHEN vectors adapt and when RVEAa truncates: the `gen` buffer and the
        `fr` / `max_gen` Parameters (rvea.py:107: the period is recomputed from `fr` in init_step; rveaa.py:181
        compares `gen` with `max_gen`). Read once here — in init_step and after a load_state_dict — and counted
        on the host afterwards, so a generation needs no device-to-host copy."""
        period = torch.max(torch.round(1 / self.fr), torch.tensor(1.0, device=self.fr.device))
        self._gen_host = int(self.gen)
        self._adapt_every = int(period)
        self._max_gen_host = int(self.max_gen)
        self._schedule = True

    def _after_load(self) -> None:
        self._schedule = None  # gen, fr or max_gen may have changed

    def init_step(self):
        self._sync_schedule()
        self.fit = self.evaluate(self.pop)

    def _mating_rows(self, picks: torch.Tensor | None) -> torch.Tensor:
        """Row numbers of the mating pool: uniform picks among the rows that are not all-NaN
        (rvea.py:118-125)."""
        n, rows = self.pop_size, self.pop.shape[0]  # RVEAa keeps 2 * pop_size rows after its first generation
        valid = ~torch.isnan(self.pop).all(dim=1)
        order = torch.argsort(torch.where(valid, torch.arange(rows, device=self.pop.device), torch.iinfo(torch.int32).max), stable=True)
        if picks is None:
            picks = (torch.rand(n, device=self.pop.device) * valid.sum()).long().clamp_(max=rows - 1)
        return order[picks]

    def step(self, picks: torch.Tensor | None = None, draws: dict | None = None):
        """One generation (rvea.py:135-154). `picks` (pop_size,) in [0, #valid rows) and `draws` replace
        the random draws of the mating pool and of crossover / mutation."""
        if self._schedule is None:
            self._sync_schedule()
        self.gen = self.gen + 1
        self._gen_host += 1
        mating = self._mating_rows(picks)
        # NaN rows never enter the pool, so the fused kernel can gather straight from pop
        offspring = self._variation(self.pop, mating, draws)
        off_fit = self.evaluate(offspring)
        merge_pop = torch.cat([self.pop, offspring], dim=0)
        merge_fit = torch.cat([self.fit, off_fit], dim=0)
        theta = (self.gen / self.max_gen) ** self.alpha
        select = self.selection or ref_vec_guided
        self.pop, self.fit = select(merge_pop, merge_fit, self.reference_vector, theta)
        if self._gen_host % self._adapt_every == 0:  # rvea.py:110-113, 127-133
            f = self.fit
            mx = torch.where(torch.isnan(f), -torch.inf, f).max(dim=0)[0]
            mn = torch.where(torch.isnan(f), torch.inf, f).min(dim=0)[0]
            self.reference_vector = self.init_v * (mx - mn)
        self.generation += 1


class RVEAa(RVEA):
    """RVEA with reference-vector regeneration (evox/algorithms/mo/rveaa.py:17-212): a second set of
    pop_size random reference vectors is selected against together with the lattice; vectors of that
    set that no survivor is closest to are redrawn every generation; only non-dominated rows of the
    merged population compete; the very last generation blanks half of the (2 * pop_size) rows.
    Ranking and selection are the P2 / P3 kernels; the regeneration and truncation bookkeeping are
    (pop_size x 2 pop_size) cosine tables in torch ops, as in the reference."""

    def __init__(self, pop_size: int, n_objs: int, lb: torch.Tensor, ub: torch.Tensor, alpha: float = 2.0, fr: float = 0.1,
                 max_gen: int = 100, selection_op: Optional[Callable] = None, mutation_op: Optional[Callable] = None,
                 crossover_op: Optional[Callable] = None, device: torch.device | None = None):
        super().__init__(pop_size, n_objs, lb, ub, alpha, fr, max_gen, selection_op, mutation_op, crossover_op, device)
        extra = torch.rand(self.pop_size, n_objs, device=self.reference_vector.device)
        self.reference_vector = Mutable(torch.cat([self.reference_vector, extra], dim=0))

    @staticmethod
    def _rv_regeneration(pop_obj: torch.Tensor, v: torch.Tensor, draw: torch.Tensor | None = None) -> torch.Tensor:
        """rveaa.py:129-142. `draw`: optional (len(v), n_objs) uniform draw."""
        finite_min = torch.where(torch.isnan(pop_obj), torch.inf, pop_obj).min(dim=0).values
        shifted = pop_obj - finite_min
        cosine = torch.nn.functional.cosine_similarity(shifted.unsqueeze(1), v.unsqueeze(0), dim=-1)
        cosine = torch.where(torch.isnan(cosine), -torch.inf, cosine)
        nearest = cosine.max(dim=1).indices
        nearest = torch.where(cosine[:, 0] == -torch.inf, -1, nearest)  # rows without objectives join nobody
        joined = torch.zeros(v.size(0) + 1, dtype=torch.int64, device=v.device).index_add_(0, nearest + 1, torch.ones_like(nearest))[1:]
        if draw is None:
            draw = torch.rand(v.shape, device=v.device)
        upper = torch.where(torch.isnan(shifted), -torch.inf, shifted).max(dim=0).values
        return torch.where((joined == 0).unsqueeze(1), draw * upper, v)

    @staticmethod
    def _batch_truncation(pop: torch.Tensor, obj: torch.Tensor):
        """rveaa.py:144-164: the reference ranks the rows by crowding and then masks by POSITION — the first
        half of the rows becomes NaN whatever the ranking says; reproduced as is."""
        keep = (torch.arange(pop.size(0), device=pop.device) >= pop.size(0) // 2).unsqueeze(1)
        return torch.where(keep, pop, torch.nan), torch.where(keep, obj, torch.nan)

    def step(self, picks: torch.Tensor | None = None, draws: dict | None = None, regeneration_draw: torch.Tensor | None = None):
        """One generation (rveaa.py:189-212)."""
        from ..operators.selection import non_dominate_rank

        if self._schedule is None:
            self._sync_schedule()
        self.gen = self.gen + 1
        self._gen_host += 1
        mating = self._mating_rows(picks)
        offspring = self._variation(self.pop, mating, draws)
        off_fit = self.evaluate(offspring)
        merge_pop = torch.cat([self.pop, offspring], dim=0)
        merge_fit = torch.cat([self.fit, off_fit], dim=0)
        front = (non_dominate_rank(merge_fit) == 0).unsqueeze(1)
        merge_fit = torch.where(front, merge_fit, torch.nan)
        merge_pop = torch.where(front, merge_pop, torch.nan)
        theta = (self.gen / self.max_gen) ** self.alpha
        select = self.selection or ref_vec_guided
        survivor, survivor_fit = select(merge_pop, merge_fit, self.reference_vector, theta)
        n = self.pop_size
        v_regen = self._rv_regeneration(survivor_fit, self.reference_vector[n:], regeneration_draw)
        if self._gen_host % self._adapt_every == 0:
            mx = torch.where(torch.isnan(survivor_fit), -torch.inf, survivor_fit).max(dim=0)[0]
            mn = torch.where(torch.isnan(survivor_fit), torch.inf, survivor_fit).min(dim=0)[0]
            v_adapt = self.init_v * (mx - mn)
        else:
            v_adapt = self.reference_vector[:n].clone()
        if self._gen_host == self._max_gen_host:
            self.pop, self.fit = self._batch_truncation(survivor, survivor_fit)
        else:
            self.pop, self.fit = survivor, survivor_fit
        self.reference_vector = torch.cat([v_adapt, v_regen], dim=0)
        self.generation += 1
