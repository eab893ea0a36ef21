"""The ARS oracle against golden vectors produced by the reference (tests/golden/make_golden.py)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import lora

GOLD = np.load(Path(__file__).parent / "golden" / "ars.npz")


@pytest.mark.parametrize("opt", [None, "adam"])
def test_oracle_reproduces_reference_steps(opt):
    tag = f"ars_{opt}"
    shift = torch.from_numpy(GOLD[f"{tag}_shift"])
    center = torch.from_numpy(GOLD[f"{tag}_center0"])
    fitness = lambda pop: ((pop - shift) ** 2).sum(dim=1)  # noqa: E731
    state = (torch.zeros_like(center), torch.zeros_like(center)) if opt else None
    for k in range(2):
        z = torch.from_numpy(GOLD[f"{tag}_z{k}"])
        res = lora.ars_step(center, z, fitness, torch.tensor(0.05), torch.tensor(0.1), 4, state)
        center = res[0]
        if opt:
            state = res[2]
        assert torch.equal(center, torch.from_numpy(GOLD[f"{tag}_center{k + 1}"])), k
    if opt:
        assert torch.equal(state[0], torch.from_numpy(GOLD[f"{tag}_exp_avg"]))
        assert torch.equal(state[1], torch.from_numpy(GOLD[f"{tag}_exp_avg_sq"]))
