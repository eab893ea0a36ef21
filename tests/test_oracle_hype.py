"""The HypE oracle against golden vectors produced by the reference (tests/golden/make_golden.py)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import hype as ohype
from oracle import nds as onds

GOLD = np.load(Path(__file__).parent / "golden" / "hype.npz")
CASES = ["m3", "m2_tensor", "m6", "dup"]


def t(name):
    return torch.from_numpy(GOLD[name])


@pytest.mark.parametrize("tag", CASES)
def test_cal_hv_matches_reference(tag):
    fit, ref, draw = t(f"hv_{tag}_fit"), t(f"hv_{tag}_ref"), t(f"hv_{tag}_draw")
    pop_size = int(GOLD[f"hv_{tag}_pop_size"])
    want = t(f"hv_{tag}_out")
    got = ohype.cal_hv(fit, ref, pop_size, draw.shape[0], draw, exact_order=True)
    assert torch.equal(got, want)
    # the blocked form (float64 row sums, rounded once): same up to the reference's own fp32 summation error
    blocked = ohype.cal_hv(fit, ref, pop_size, draw.shape[0], draw)
    assert torch.allclose(blocked, want, rtol=1e-5, atol=1e-7)
    assert float(want.max()) > 0


def test_step_matches_reference():
    pop = t("step_s0_pop")
    d, m = pop.shape[1], 3
    fit = onds.dtlz2_objectives(pop, m)
    assert torch.equal(fit, t("step_s1_fit"))
    ref = t("step_ref")
    assert torch.equal(ref, torch.full((m,), float(fit.max()) * 1.2))
    lb, ub = torch.zeros(d), torch.ones(d)
    for g in range(2):
        draws = {k: t(f"step_g{g}_{k}") for k in ("sbx_mu", "sbx_sign", "sbx_half", "sbx_pc", "pm_site", "pm_mu")}
        pop, fit = ohype.step(pop, fit, ref, lb, ub, lambda x: onds.dtlz2_objectives(x, m), 300,
                              [t(f"step_g{g}_samples_a"), t(f"step_g{g}_samples_b")], t(f"step_g{g}_parents"), draws, exact_order=True)
        assert torch.equal(pop, t(f"step_g{g}_pop")), g
        assert torch.equal(fit, t(f"step_g{g}_fit")), g
