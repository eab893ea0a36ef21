"""The SL-PSO oracle against golden vectors produced by the reference (tests/golden/make_golden.py)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import pso as opso
from oracle import slpso as oslpso

GOLD = np.load(Path(__file__).parent / "golden" / "slpso.npz")
NAMES = ["pop", "fit", "velocity", "global_best_location", "global_best_fit"]


def load_state(tag: str, step: int) -> dict:
    lo, hi = GOLD[f"{tag}_bounds"]
    s = {n: torch.from_numpy(GOLD[f"{tag}_s{step}_{n}"]) for n in NAMES}
    dim = s["pop"].shape[1]
    s.update(lb=torch.full((1, dim), float(lo)), ub=torch.full((1, dim), float(hi)), social_influence_factor=torch.tensor(0.2),
             demonstrator_choice_factor=torch.tensor(0.7))
    return s


@pytest.mark.parametrize("kind", ["gs", "us"])
@pytest.mark.parametrize("dim", [12, 10])
def test_oracle_reproduces_reference_steps(kind, dim):
    tag = f"slpso_{kind}_d{dim}"
    s = oslpso.init_step(load_state(tag, 0), opso.ackley)
    for n in NAMES:
        assert torch.equal(s[n], torch.from_numpy(GOLD[f"{tag}_s1_{n}"])), n
    choose = oslpso.demonstrator_rows_gs if kind == "gs" else oslpso.demonstrator_rows_us
    for g in range(3):
        rows = choose(s["fit"], s["demonstrator_choice_factor"], torch.from_numpy(GOLD[f"{tag}_g{g}_pick"]))
        rs = [torch.from_numpy(GOLD[f"{tag}_g{g}_r{j}"]) for j in (1, 2, 3)]
        s = oslpso.step(s, rows, *rs, opso.ackley)
        for n in NAMES:
            assert torch.equal(s[n], torch.from_numpy(GOLD[f"{tag}_s{g + 2}_{n}"])), (g, n)
