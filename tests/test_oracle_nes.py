"""The SNES / DES oracle against golden vectors produced by the reference (tests/golden/make_golden.py)."""

import math
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import nes

GOLD = np.load(Path(__file__).parent / "golden" / "snes_des.npz")


@pytest.mark.parametrize("tag", ["snes_temp", "snes_recomb", "des"])
def test_oracle_reproduces_reference_steps(tag):
    shift = torch.from_numpy(GOLD[f"{tag}_shift"])
    center = torch.from_numpy(GOLD[f"{tag}_center0"])
    fit = lambda pop: ((pop - shift) ** 2).sum(dim=1)  # noqa: E731
    dim = center.shape[0]
    sigma = (0.3 if tag == "des" else 0.5) * torch.ones(dim)
    for k in range(3):
        z = torch.from_numpy(GOLD[f"{tag}_z{k}"])
        if tag == "des":
            center, sigma = nes.des_step(center, sigma, z, fit)
        else:
            w = nes.snes_weights(14, tag.split("_")[1])
            center, sigma = nes.snes_step(center, sigma, z, fit, w, torch.tensor(1.0), torch.tensor((3 + math.log(dim)) / (5 * math.sqrt(dim))))
        assert torch.equal(center, torch.from_numpy(GOLD[f"{tag}_center{k + 1}"])), k
        assert torch.equal(sigma, torch.from_numpy(GOLD[f"{tag}_sigma{k + 1}"])), k
