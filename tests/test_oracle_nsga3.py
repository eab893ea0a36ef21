"""The NSGA-III restatement (oracle/nsga3.py) against the reference's recorded generations."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import nsga3 as onsga3

GOLDEN = np.load(Path(__file__).parent / "golden" / "nsga3.npz")


def case(tag, g):
    t = lambda k: torch.from_numpy(GOLDEN[f"{tag}_g{g}_{k}"])  # noqa: E731
    return {k: t(k) for k in ("pop", "fit", "offspring", "off_fit", "perm_merge", "perm_ref", "next_pop", "next_fit", "next_rank")}


CASES = [(tag, g) for tag in ("m3", "m4", "m2") for g in range(int(GOLDEN[f"{tag}_gens"]))]


@pytest.mark.parametrize("tag,g", CASES)
def test_oracle_reproduces_reference_generation(tag, g):
    c = case(tag, g)
    ref = torch.from_numpy(GOLDEN[f"{tag}_ref"])
    pop, fit, rank = onsga3.environmental_selection(c["pop"], c["fit"], c["offspring"], c["off_fit"], c["perm_merge"],
                                                    c["perm_ref"], ref, int(GOLDEN[f"{tag}_pop_size"]))
    assert torch.equal(pop, c["next_pop"])
    assert torch.equal(fit, c["next_fit"])
    assert torch.equal(rank.to(c["next_rank"].dtype), c["next_rank"])


def test_generations_chain():
    """Each recorded generation starts from the state the previous one left."""
    for tag in ("m3", "m4", "m2"):
        for g in range(1, int(GOLDEN[f"{tag}_gens"])):
            assert np.array_equal(GOLDEN[f"{tag}_g{g}_pop"], GOLDEN[f"{tag}_g{g - 1}_next_pop"])
