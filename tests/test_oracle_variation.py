"""The mating / variation oracle reproduces outputs recorded from the reference (CPU only)."""
import torch

from oracle import variation as ov


def t(a):
    return torch.from_numpy(a)


def test_sbx_pm_tournament(golden):
    g = golden("variation")
    crossed = ov.simulated_binary(t(g["var_x"]), t(g["var_sbx_mu"]), t(g["var_sbx_sign"]), t(g["var_sbx_half"]), t(g["var_sbx_pc"]))
    assert torch.equal(crossed, t(g["var_crossed"]))
    mutated = ov.polynomial_mutation(crossed, t(g["var_lb"]), t(g["var_ub"]), t(g["var_pm_site"]), t(g["var_pm_mu"]))
    assert torch.equal(mutated, t(g["var_mutated"]))
    assert (mutated != crossed).sum() > 20  # the mutation really fired
    picked = ov.tournament_multifit(t(g["ts_parents"]), [-t(g["ts_dis"]), t(g["ts_rank"])])
    assert torch.equal(picked, t(g["ts_selected"]))


def test_rvea_mating_pool_skips_nan_rows():
    pop = torch.arange(12.0).reshape(6, 2)
    pop[1] = float("nan")
    pop[4] = float("nan")
    got = ov.rvea_mating_pool(pop, torch.tensor([0, 1, 2, 3, 3, 0]))
    assert torch.equal(got[:, 0], torch.tensor([0.0, 4.0, 6.0, 10.0, 10.0, 0.0]))
