"""Mating / variation kernels and whole NSGA-II / RVEA generations against the reference's recorded
outputs and the oracle. Index outputs (tournament winners, selected rows) must be exact; offspring
values go through device powf: relative 1e-5 of the variable's range."""
import pytest
import torch

from oracle import nds as onds
from oracle import rvea as orvea
from oracle import variation as ov

pytestmark = pytest.mark.gpu


def t(a):
    return torch.from_numpy(a)


def close(got, want, scale, rel=1e-5):
    err = (got.cpu().double() - want.double()).abs().max().item()
    assert err <= rel * scale, err


def test_variation_golden(golden, cuda):
    from evox_b200.operators.variation import CROSSOVER, MUTATION, make_offspring, tournament_selection_multifit

    g = golden("variation")
    x, lb, ub = t(g["var_x"]), t(g["var_lb"]), t(g["var_ub"])
    draws = {k: t(g[f"var_{k}"]) for k in ("sbx_mu", "sbx_sign", "sbx_half", "sbx_pc", "pm_site", "pm_mu")}
    inf = torch.full_like(lb, float("inf"))
    crossed = make_offspring(x.to(cuda), -inf, inf, draws=draws, flags=CROSSOVER)
    close(crossed, t(g["var_crossed"]), 4.0)
    mutated = make_offspring(t(g["var_crossed"]).to(cuda), lb, ub, draws=draws, flags=MUTATION)
    close(mutated, t(g["var_mutated"]), 4.0)
    fused = make_offspring(x.to(cuda), lb, ub, draws=draws)
    close(fused, ov.offspring(x, lb, ub, draws), 4.0)
    picked = tournament_selection_multifit(40, [-t(g["ts_dis"]).to(cuda), t(g["ts_rank"]).to(cuda)], parents=t(g["ts_parents"]).to(cuda))
    assert torch.equal(picked.cpu(), t(g["ts_selected"]))


def test_variation_standalone_functions_and_philox(cuda):
    from evox_b200.operators.variation import make_offspring, polynomial_mutation, simulated_binary

    lb, ub = torch.zeros(5, device=cuda), torch.ones(5, device=cuda)
    x = torch.rand(33, 5, device=cuda)
    c = simulated_binary(x)
    assert c.shape == (32, 5) and torch.isfinite(c).all()
    m = polynomial_mutation(x, lb, ub)
    assert m.shape == (33, 5) and (m >= 0).all() and (m <= 1).all()
    a = make_offspring(x, lb, ub, seed=5, generation=2)
    b = make_offspring(x, lb, ub, seed=5, generation=2)
    c2 = make_offspring(x, lb, ub, seed=5, generation=3)
    assert torch.equal(a, b) and not torch.equal(a, c2)
    assert (a >= -1e-6).all() and (a <= 1 + 1e-6).all()


def test_nsga2_generation_vs_oracle(cuda):
    """One teacher-forced NSGA-II generation on DTLZ2: tournament -> offspring -> evaluate -> merge ->
    environmental selection, with all draws injected."""
    from evox_b200.algorithms import NSGA2
    from evox_b200.problems.numerical import DTLZ2
    from evox_b200.workflows import StdWorkflow

    n, d, m = 200, 12, 3
    g = torch.Generator().manual_seed(4)
    lb, ub = torch.zeros(d), torch.ones(d)
    algo = NSGA2(n, m, lb, ub, device=cuda)
    wf = StdWorkflow(algo, DTLZ2(d, m), device=cuda)
    pop0 = torch.rand(n, d, generator=g)
    wf.algorithm.pop = pop0.to(cuda)
    wf.init_step()
    fit0 = onds.dtlz2_objectives(pop0, m)
    _, _, rank0, dis0, _ = onds.nd_environmental_selection(pop0, fit0, n)
    assert torch.equal(wf.algorithm.rank.cpu(), rank0)
    parents = torch.randint(0, n, (n, 2), generator=g)
    draws = ov.make_draws(n, d, 9)
    wf.algorithm.step(parents=parents.to(cuda), draws=draws)
    # oracle: the selection sorts the rows, so state after init is pop0 in selected order
    x0, f0, r0, d0, _ = onds.nd_environmental_selection(pop0, fit0, n)
    # the reference keeps pop unsorted after init_step (only rank / dis come from the selection)
    mating = ov.tournament_multifit(parents, [-dis0, rank0.float()])
    off = ov.offspring(pop0[mating], lb, ub, draws)
    # evaluate the DEVICE offspring so that the selection sees identical objectives on both sides
    merge_pop = torch.cat([pop0, off])
    dev_off = wf.problem.evaluate(make_dev(off, cuda)).cpu()
    close(dev_off, onds.dtlz2_objectives(off, m), 4.0)
    want = onds.nd_environmental_selection(merge_pop, torch.cat([fit0, onds.dtlz2_objectives(off, m)]), n)
    got_pop = wf.algorithm.pop.cpu()
    close(got_pop, want[0], 1.0, rel=1e-4)
    assert torch.equal(wf.algorithm.rank.cpu(), want[2])


def make_dev(x, cuda):
    return x.to(cuda)


def test_nsga2_and_rvea_improve(cuda):
    """Default (Philox / torch draws) runs: the populations move towards the DTLZ2 front, where
    sum(f^2) = 1."""
    from evox_b200.algorithms import NSGA2, RVEA
    from evox_b200.problems.numerical import DTLZ2
    from evox_b200.workflows import StdWorkflow

    d, m = 12, 3
    lb, ub = torch.zeros(d), torch.ones(d)
    torch.manual_seed(0)
    for algo in (NSGA2(100, m, lb, ub, device=cuda), RVEA(100, m, lb, ub, max_gen=60, device=cuda)):
        wf = StdWorkflow(algo, DTLZ2(d, m), device=cuda)
        wf.init_step()
        f = wf.algorithm.fit
        before = torch.nanmean((f**2).sum(dim=1).sqrt())
        for _ in range(60):
            wf.step()
        f = wf.algorithm.fit
        after = torch.nanmean((f**2).sum(dim=1).sqrt())
        assert after < before and after < 1.15, (type(algo).__name__, float(before), float(after))
        assert wf.algorithm.pop.shape[0] == wf.algorithm.pop_size


def test_rvea_generation_vs_oracle(cuda):
    """One teacher-forced RVEA generation (mating pool picks and variation draws injected), including a
    NaN slot in the population as RVEA produces for empty vectors."""
    from evox_b200.algorithms import RVEA
    from evox_b200.problems.numerical import DTLZ2
    from evox_b200.workflows import StdWorkflow

    d, m = 12, 3
    lb, ub = torch.zeros(d), torch.ones(d)
    algo = RVEA(91, m, lb, ub, max_gen=50, device=cuda)
    n = algo.pop_size
    wf = StdWorkflow(algo, DTLZ2(d, m), device=cuda)
    g = torch.Generator().manual_seed(8)
    pop0 = torch.rand(n, d, generator=g)
    pop0[7] = float("nan")
    wf.algorithm.pop = pop0.to(cuda)
    wf.init_step()
    fit0 = wf.algorithm.fit.cpu()
    picks = torch.randint(0, n - 1, (n,), generator=g)
    draws = ov.make_draws(n, d, 3)
    wf.algorithm.step(picks=picks.to(cuda), draws=draws)
    parents = ov.rvea_mating_pool(pop0, picks)
    off = ov.offspring(parents, lb, ub, draws)
    dev_off_fit = wf.problem.evaluate(off.to(cuda)).cpu()
    merge_pop, merge_fit = torch.cat([pop0, off]), torch.cat([fit0, dev_off_fit])
    theta = (torch.tensor(1.0) / 50.0) ** 2.0
    want = orvea.ref_vec_guided(merge_pop, merge_fit, wf.algorithm.init_v.cpu(), theta)
    got = wf.algorithm.pop.cpu()
    assert torch.equal(torch.isnan(got), torch.isnan(want["next_x"]))
    close(torch.nan_to_num(got), torch.nan_to_num(want["next_x"]), 1.0, rel=1e-4)


def test_eval_monitor_single_and_multi_objective(cuda):
    """EvalMonitor with the fused PSO step (best-so-far must never get worse and must equal the
    swarm's own global best) and with NSGA-II (the extracted front is non-dominated)."""
    from evox_b200.algorithms import NSGA2, PSO
    from evox_b200.problems.numerical import DTLZ2, Ackley
    from evox_b200.workflows import EvalMonitor, StdWorkflow

    d = 30
    mon = EvalMonitor(topk=3, full_sol_history=False, device=cuda)
    wf = StdWorkflow(PSO(256, torch.full((d,), -32.768), torch.full((d,), 32.768), device=cuda, seed=3), Ackley(), monitor=mon, device=cuda)
    wf.init_step()
    best = [float(mon.get_best_fitness())]
    for _ in range(15):
        wf.step()
        best.append(float(mon.get_best_fitness()))
    assert all(b <= a + 1e-12 for a, b in zip(best, best[1:]))
    assert mon.get_topk_fitness().shape == (3,) and mon.get_topk_solutions().shape == (3, d)
    assert len(mon.fitness_history) == 16
    # the swarm's global best lags the monitor by one evaluation (it is folded in at the next step)
    assert float(wf.algorithm.global_best_fit) >= best[-1] - 1e-6

    mon = EvalMonitor(full_sol_history=True, device=cuda)
    wf = StdWorkflow(NSGA2(64, 3, torch.zeros(12), torch.ones(12), device=cuda), DTLZ2(12, 3), monitor=mon, device=cuda)
    wf.init_step()
    for _ in range(5):
        wf.step()
    sol, fit = mon.get_pf()
    assert sol.shape[0] == fit.shape[0] > 0
    assert int(onds.non_dominate_rank(fit.cpu()).max()) == 0
    with pytest.raises(ValueError):
        mon.get_best_fitness()


def test_rveaa_pieces_and_generation(golden, cuda):
    """RVEAa: regeneration and truncation against the reference's recorded outputs; one teacher-forced
    generation against the oracle composition (rank kernel -> NaN masking -> selection kernel over the
    doubled vector set -> regeneration); then a short run that must keep a non-dominated population."""
    from evox_b200.algorithms import RVEAa
    from evox_b200.problems.numerical import DTLZ2
    from evox_b200.workflows import StdWorkflow

    g = golden("rveaa")
    new_v = RVEAa._rv_regeneration(t(g["regen_obj"]).to(cuda), t(g["regen_v"]).to(cuda), t(g["regen_draw"]).to(cuda))
    close(new_v, t(g["regen_new_v"]), 1.0, rel=1e-6)
    new_pop, new_obj = RVEAa._batch_truncation(t(g["trunc_pop"]).to(cuda), t(g["regen_obj"]).to(cuda))
    assert torch.equal(torch.nan_to_num(new_pop.cpu(), nan=-7.0), torch.nan_to_num(t(g["trunc_new_pop"]), nan=-7.0))
    assert torch.equal(torch.nan_to_num(new_obj.cpu(), nan=-7.0), torch.nan_to_num(t(g["trunc_new_obj"]), nan=-7.0))

    d, m = 12, 3
    lb, ub = torch.zeros(d), torch.ones(d)
    torch.manual_seed(11)
    algo = RVEAa(91, m, lb, ub, max_gen=50, device=cuda)
    n = algo.pop_size
    assert algo.reference_vector.shape == (2 * n, m)
    wf = StdWorkflow(algo, DTLZ2(d, m), device=cuda)
    gen = torch.Generator().manual_seed(8)
    pop0 = torch.rand(n, d, generator=gen)
    wf.algorithm.pop = pop0.to(cuda)
    wf.init_step()
    fit0 = wf.algorithm.fit.cpu()
    v_all = wf.algorithm.reference_vector.cpu().clone()
    picks = torch.randint(0, n, (n,), generator=gen)
    draws = ov.make_draws(n, d, 3)
    regen = torch.rand(n, m, generator=gen)
    wf.algorithm.step(picks=picks.to(cuda), draws=draws, regeneration_draw=regen.to(cuda))
    off = ov.offspring(ov.rvea_mating_pool(pop0, picks), lb, ub, draws)
    off_fit = wf.problem.evaluate(off.to(cuda)).cpu()
    merge_pop, merge_fit = torch.cat([pop0, off]), torch.cat([fit0, off_fit])
    front = (onds.non_dominate_rank(merge_fit) == 0).unsqueeze(1)
    merge_pop, merge_fit = torch.where(front, merge_pop, torch.nan), torch.where(front, merge_fit, torch.nan)
    want = orvea.ref_vec_guided(merge_pop, merge_fit, v_all, (torch.tensor(1.0) / 50.0) ** 2.0)
    got = wf.algorithm.pop.cpu()
    assert got.shape == (2 * n, d)
    assert torch.equal(torch.isnan(got), torch.isnan(want["next_x"]))
    close(torch.nan_to_num(got), torch.nan_to_num(want["next_x"]), 1.0, rel=1e-4)
    want_v = orvea.rv_regeneration(want["next_f"], v_all[n:], regen)
    close(wf.algorithm.reference_vector[n:], want_v, 1.0, rel=1e-4)
    assert torch.equal(wf.algorithm.reference_vector[:n].cpu(), v_all[:n])
    for _ in range(12):
        wf.step()
    fit = wf.algorithm.fit
    alive = ~torch.isnan(fit).any(dim=1)
    assert int(alive.sum()) >= 10
    assert int(onds.non_dominate_rank(fit[alive].cpu()).max()) == 0


@pytest.mark.parametrize("name", ["RVEA", "RVEAa", "NSGA2"])
def test_checkpoint_resume_equals_uninterrupted_run(cuda, name):
    """state_dict -> fresh object -> load_state_dict -> continue: the resumed run must land where the
    uninterrupted one does. Covers what lives outside the tensors: the position in the random stream and, for
    RVEA / RVEAa, the schedule of the reference-vector adaptation (period 1 / fr, rvea.py:107) and RVEAa's
    final truncation at gen == max_gen (rveaa.py:181) — with fr = 0.25 the adaptation falls on generations
    4 and 8 and the truncation on generation 8, all after the checkpoint at generation 3."""
    from evox_b200 import algorithms
    from evox_b200.problems.numerical import DTLZ2
    from evox_b200.workflows import StdWorkflow

    d, m = 12, 3
    lb, ub = torch.zeros(d), torch.ones(d)

    def make():
        torch.manual_seed(5)  # the constructors draw the seed of their random stream from torch's generator
        cls = getattr(algorithms, name)
        algo = cls(60, m, lb, ub, device=cuda) if name == "NSGA2" else cls(60, m, lb, ub, fr=0.25, max_gen=8, device=cuda)
        return StdWorkflow(algo, DTLZ2(d, m), device=cuda)

    def run(wf, gens):
        for g in gens:
            torch.manual_seed(100 + g)  # draws taken from torch's generator (mating picks, regeneration)
            wf.step()

    full = make()
    full.init_step()
    run(full, range(8))
    first = make()
    first.init_step()
    run(first, range(3))
    saved = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in first.algorithm.state_dict().items()}
    torch.manual_seed(999)
    second = make()
    second.algorithm.seed = 1  # whatever the fresh object drew must not matter after the load
    second.algorithm.load_state_dict(saved)
    run(second, range(3, 8))
    a, b = full.algorithm.state_dict(), second.algorithm.state_dict()
    for k in a:
        if isinstance(a[k], torch.Tensor):
            assert torch.equal(torch.nan_to_num(a[k].float(), nan=-1.0), torch.nan_to_num(b[k].float(), nan=-1.0)), k
    assert full.algorithm.generation == second.algorithm.generation == 8
