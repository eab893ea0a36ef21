"""The CLPSO oracle against golden vectors produced by the reference (tests/golden/make_golden.py)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import clpso as oclpso
from oracle import pso as opso

GOLD = np.load(Path(__file__).parent / "golden" / "clpso.npz")
NAMES = ["pop", "fit", "velocity", "personal_best_location", "personal_best_fit", "global_best_location", "global_best_fit"]


def load_state(tag: str, step: int) -> dict:
    lo, hi = GOLD[f"{tag}_bounds"]
    s = {n: torch.from_numpy(GOLD[f"{tag}_s{step}_{n}"]) for n in NAMES}
    dim = s["pop"].shape[1]
    s.update(lb=torch.full((1, dim), float(lo)), ub=torch.full((1, dim), float(hi)), w=torch.tensor(0.5), c=torch.tensor(1.5),
             P_c=torch.tensor(0.3))
    return s


@pytest.mark.parametrize("prob", ["ackley", "sphere"])
@pytest.mark.parametrize("dim", [12, 10])
def test_oracle_reproduces_reference_steps(prob, dim):
    tag = f"clpso_{prob}_d{dim}"
    fitness = opso.FITNESS[prob]
    s = oclpso.init_step(load_state(tag, 0), fitness)
    for n in NAMES:
        assert torch.equal(s[n], torch.from_numpy(GOLD[f"{tag}_s1_{n}"])), n
    for g in range(3):
        draws = [torch.from_numpy(GOLD[f"{tag}_g{g}_{k}"]) for k in ("coeff", "i1", "i2", "poss")]
        s = oclpso.step(s, *draws, fitness)
        for n in NAMES:
            assert torch.equal(s[n], torch.from_numpy(GOLD[f"{tag}_s{g + 2}_{n}"])), (g, n)
