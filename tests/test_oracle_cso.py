"""The CSO oracle against golden vectors produced by the reference (tests/golden/make_golden.py)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import cso as ocso
from oracle import pso as opso

GOLD = np.load(Path(__file__).parent / "golden" / "cso.npz")


def load_state(tag: str, step: int) -> dict:
    lo, hi = GOLD[f"{tag}_bounds"]
    s = {n: torch.from_numpy(GOLD[f"{tag}_s{step}_{n}"]) for n in ("pop", "fit", "velocity")}
    dim = s["pop"].shape[1]
    s["lb"] = torch.full((1, dim), float(lo))
    s["ub"] = torch.full((1, dim), float(hi))
    s["phi"] = torch.tensor(float(GOLD[f"{tag}_phi"]))
    return s


@pytest.mark.parametrize("prob", ["ackley", "sphere"])
@pytest.mark.parametrize("dim", [12, 10])
def test_oracle_reproduces_reference_steps(prob, dim):
    tag = f"cso_{prob}_d{dim}"
    fitness = opso.FITNESS[prob]
    s = ocso.init_step(load_state(tag, 0), fitness)
    assert torch.equal(s["fit"], torch.from_numpy(GOLD[f"{tag}_s1_fit"]))
    for g in range(3):
        perm = torch.from_numpy(GOLD[f"{tag}_g{g}_perm"])
        lambdas = torch.from_numpy(GOLD[f"{tag}_g{g}_lambdas"])
        s = ocso.step(s, perm, lambdas, fitness)
        for n in ("pop", "fit", "velocity"):
            assert torch.equal(s[n], torch.from_numpy(GOLD[f"{tag}_s{g + 2}_{n}"])), (g, n)
