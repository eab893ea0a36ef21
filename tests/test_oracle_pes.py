"""The PersistentES oracle against golden vectors produced by the reference (tests/golden/make_golden.py)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import pes

GOLD = np.load(Path(__file__).parent / "golden" / "pes.npz")
HYPER = dict(lr=torch.tensor(0.05), T=torch.tensor(30), K=torch.tensor(10), sigma_decay=torch.tensor(0.9), sigma_limit=torch.tensor(0.075))


@pytest.mark.parametrize("opt", [None, "adam"])
def test_oracle_reproduces_reference_steps(opt):
    tag = f"pes_{opt}"
    shift = torch.from_numpy(GOLD[f"{tag}_shift"])
    center = torch.from_numpy(GOLD[f"{tag}_center0"])
    s = {"center": center, "sigma": torch.tensor(0.1), "pert_accum": torch.zeros(12, 20), "inner_step_counter": torch.tensor(0.0)}
    if opt:
        s["exp_avg"], s["exp_avg_sq"] = torch.zeros(20), torch.zeros(20)
    for k in range(4):
        s = pes.step(s, torch.from_numpy(GOLD[f"{tag}_z{k}"]), lambda pop: ((pop - shift) ** 2).sum(dim=1), **HYPER)
        assert torch.equal(s["center"], torch.from_numpy(GOLD[f"{tag}_center{k + 1}"])), k
        assert torch.equal(s["pert_accum"], torch.from_numpy(GOLD[f"{tag}_accum{k + 1}"])), k
        assert torch.equal(s["sigma"], torch.from_numpy(GOLD[f"{tag}_sigma{k + 1}"])), k
        assert float(s["inner_step_counter"]) == float(GOLD[f"{tag}_counter{k + 1}"]), k
