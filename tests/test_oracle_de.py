"""The DE oracle against golden vectors produced by the reference (tests/golden/make_golden.py)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import de as ode
from oracle import pso as opso

GOLD = np.load(Path(__file__).parent / "golden" / "de.npz")


def load_state(tag: str) -> dict:
    lo, hi = GOLD[f"{tag}_bounds"]
    pop = torch.from_numpy(GOLD[f"{tag}_s0_pop"])
    dim = pop.shape[1]
    return {"pop": pop, "lb": torch.full((1, dim), float(lo)), "ub": torch.full((1, dim), float(hi)),
            "differential_weight": torch.tensor(0.6), "cross_probability": torch.tensor(0.7)}


@pytest.mark.parametrize("base", ["rand", "best"])
@pytest.mark.parametrize("dim", [12, 10])
def test_oracle_reproduces_reference_steps(base, dim):
    tag = f"de_{base}_d{dim}"
    s = ode.init_step(load_state(tag), opso.ackley)
    assert torch.equal(s["fit"], torch.from_numpy(GOLD[f"{tag}_s1_fit"]))
    for g in range(3):
        idx = [torch.from_numpy(GOLD[f"{tag}_g{g}_idx{j}"]) for j in range(3 if base == "rand" else 2)]
        s = ode.step(s, idx, torch.from_numpy(GOLD[f"{tag}_g{g}_cross"]), torch.from_numpy(GOLD[f"{tag}_g{g}_forced"]), opso.ackley,
                     best_vector=base == "best")
        assert torch.equal(s["pop"], torch.from_numpy(GOLD[f"{tag}_s{g + 2}_pop"])), g
        assert torch.equal(s["fit"], torch.from_numpy(GOLD[f"{tag}_s{g + 2}_fit"])), g
