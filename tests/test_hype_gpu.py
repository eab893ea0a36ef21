"""HypE on the device: the hypervolume-contribution kernels against the reference's recorded outputs and
the oracle, and whole generations against the reference's recorded states.

The cover counts and every index decision are exact; a contribution is a sum of fp32 weights whose order
differs from the reference's, so values are compared to 1e-5 relative."""

import numpy as np
import pytest
import torch

from oracle import hype as ohype
from oracle import nds as onds

pytestmark = pytest.mark.gpu

CASES = ["m3", "m2_tensor", "m6", "dup"]


def close(got, want, rel=1e-5, abs_=1e-9):
    got, want = got.cpu().double(), want.cpu().double()
    err = (got - want).abs()
    assert bool((err <= rel * want.abs() + abs_).all()), float((err / (want.abs() + 1e-30)).max())


@pytest.mark.parametrize("tag", CASES)
def test_cal_hv_golden(golden, cuda, tag):
    from evox_b200.algorithms.hype import cal_hv

    g = golden("hype")
    fit, ref, draw = (torch.from_numpy(g[f"hv_{tag}_{k}"]).to(cuda) for k in ("fit", "ref", "draw"))
    pop_size = int(g[f"hv_{tag}_pop_size"])
    if tag == "m2_tensor":
        pop_size = torch.tensor(pop_size, device=cuda)
    got = cal_hv(fit, ref, pop_size, draw.shape[0], draw)
    close(got, torch.from_numpy(g[f"hv_{tag}_out"]))


@pytest.mark.parametrize("n,m,n_sample,pop_size", [(1, 3, 40, 1), (257, 2, 1000, 100), (1000, 3, 4097, 500), (3000, 4, 2500, 1500),
                                                  (700, 5, 999, 350), (300, 7, 1300, 100), (400, 8, 900, 100), (350, 10, 800, 100), (129, 32, 300, 64), (5000, 3, 10000, 2500)])
def test_cal_hv_vs_oracle(cuda, n, m, n_sample, pop_size):
    from evox_b200.algorithms.hype import cal_hv

    gen = torch.Generator().manual_seed(n + m)
    fit = torch.rand(n, m, generator=gen)
    if m > 5:
        fit = fit * 0.3  # keep a useful share of the samples covered when there are many objectives
    if n == 257:
        fit = torch.round(fit * 8) / 8
    ref = torch.full((m,), 1.1)
    draw = torch.rand(n_sample, m, generator=gen)
    want = ohype.cal_hv(fit, ref, pop_size, n_sample, draw)
    got = cal_hv(fit.to(cuda), ref.to(cuda), pop_size, n_sample, draw.to(cuda))
    close(got, want, rel=2e-5)
    assert float(want.max()) > 0


def test_cal_hv_rejects_too_many_objectives(cuda):
    from evox_b200 import _cabi
    from evox_b200.algorithms.hype import cal_hv

    with pytest.raises(_cabi.EvoxKernelError):
        cal_hv(torch.rand(10, 33, device=cuda), torch.ones(33, device=cuda), 5, 10)


def test_generations_match_reference(golden, cuda):
    """HypE.init_step + two teacher-forced generations against the reference's recorded populations. The
    first generation must agree row by row. In the second one two survivors have contributions that the
    reference's summation order separates by one ulp and the kernel's does not, so their two rows may swap
    places: that generation is compared as a set of rows (sorted by the first variable)."""
    from evox_b200.algorithms import HypE
    from evox_b200.problems.numerical import DTLZ2
    from evox_b200.workflows import StdWorkflow

    g = golden("hype")
    pop0 = torch.from_numpy(g["step_s0_pop"])
    d, m, n = pop0.shape[1], 3, pop0.shape[0]
    algo = HypE(n, m, torch.zeros(d), torch.ones(d), n_sample=300, device=cuda)
    wf = StdWorkflow(algo, DTLZ2(d, m), device=cuda)
    wf.algorithm.pop = pop0.to(cuda)
    wf.init_step()
    assert torch.equal(wf.algorithm.ref.cpu(), torch.from_numpy(g["step_ref"]))
    close(wf.algorithm.fit, torch.from_numpy(g["step_s1_fit"]), rel=1e-5, abs_=1e-6)
    for it in range(2):
        draws = {k: torch.from_numpy(g[f"step_g{it}_{k}"]) for k in ("sbx_mu", "sbx_sign", "sbx_half", "sbx_pc", "pm_site", "pm_mu")}
        wf.algorithm.step(parents=torch.from_numpy(g[f"step_g{it}_parents"]).to(cuda), draws=draws,
                          sample_draws=[torch.from_numpy(g[f"step_g{it}_samples_{s}"]).to(cuda) for s in "ab"])
        got_pop, got_fit = wf.algorithm.pop.cpu(), wf.algorithm.fit.cpu()
        want_pop, want_fit = torch.from_numpy(g[f"step_g{it}_pop"]), torch.from_numpy(g[f"step_g{it}_fit"])
        if it == 1:
            a, b = torch.argsort(got_pop[:, 0]), torch.argsort(want_pop[:, 0])
            assert int((a != b).sum()) <= 2
            got_pop, got_fit, want_pop, want_fit = got_pop[a], got_fit[a], want_pop[b], want_fit[b]
        close(got_pop, want_pop, rel=1e-4, abs_=1e-6)
        close(got_fit, want_fit, rel=1e-4, abs_=1e-6)


def test_selection_is_the_oracles_given_device_values(cuda):
    """The index work of a generation (rank, last admitted front, order by rank then contribution) is exact:
    recompute it with the oracle from the contributions the device produced."""
    from evox_b200.algorithms import HypE
    from evox_b200.problems.numerical import DTLZ2
    from evox_b200.workflows import StdWorkflow

    n, d, m = 300, 12, 3
    torch.manual_seed(8)
    algo = HypE(n, m, torch.zeros(d), torch.ones(d), n_sample=2000, device=cuda)
    wf = StdWorkflow(algo, DTLZ2(d, m), device=cuda)
    wf.init_step()
    for _ in range(3):
        wf.step()
        merge_fit, rank, hv, keep = wf.algorithm._last_selection
        assert torch.equal(rank.cpu(), onds.non_dominate_rank(merge_fit.cpu()))
        assert torch.equal(keep.cpu(), ohype.select(rank.cpu(), hv.cpu(), n))
        assert torch.equal(wf.algorithm.fit, merge_fit[keep])


def test_hype_improves(cuda):
    """Mean distance of the population's objective vectors to DTLZ2's unit sphere shrinks."""
    from evox_b200.algorithms import HypE
    from evox_b200.problems.numerical import DTLZ2
    from evox_b200.workflows import StdWorkflow

    n, d, m = 200, 12, 3
    torch.manual_seed(3)
    wf = StdWorkflow(HypE(n, m, torch.zeros(d), torch.ones(d), n_sample=4000, device=cuda), DTLZ2(d, m), device=cuda)
    wf.init_step()
    before = float((wf.algorithm.fit.norm(dim=1) - 1).abs().mean())
    for _ in range(40):
        wf.step()
    after = float((wf.algorithm.fit.norm(dim=1) - 1).abs().mean())
    assert after < 0.3 * before
