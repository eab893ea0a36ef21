"""NSGA3 (evox_b200/algorithms/mo.py) against the reference's recorded generations (tests/golden/nsga3.npz):
the niching logic on CPU with the oracle's ranks standing in for the rank kernel, and the whole environmental
selection on the GPU. The recorded generations include ones where the reference's population ends one row short
(see `_masked_assign`); those must be reproduced too."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import nds as onds

GOLDEN = np.load(Path(__file__).parent / "golden" / "nsga3.npz")
CASES = [(tag, g) for tag in ("m3", "m4", "m2") for g in range(int(GOLDEN[f"{tag}_gens"]))]


def load(tag, g, dev):
    return {k: torch.from_numpy(GOLDEN[f"{tag}_g{g}_{k}"]).to(dev)
            for k in ("pop", "fit", "rank", "offspring", "off_fit", "perm_merge", "perm_ref", "next_pop", "next_fit", "next_rank")}


def run_generation(tag, g, dev):
    from evox_b200.algorithms import NSGA3

    c = load(tag, g, dev)
    d, m = c["pop"].shape[1], c["fit"].shape[1]
    algo = NSGA3(int(GOLDEN[f"{tag}_pop_size"]), m, torch.zeros(d), torch.ones(d), device=dev)
    assert torch.allclose(algo.ref.cpu(), torch.from_numpy(GOLDEN[f"{tag}_ref"]))
    algo.ref = torch.from_numpy(GOLDEN[f"{tag}_ref"]).to(dev)
    algo.pop, algo.fit, algo.rank = c["pop"], c["fit"], c["rank"]
    algo.environmental_selection(c["offspring"], c["off_fit"], c["perm_merge"], c["perm_ref"])
    return algo, c


@pytest.mark.parametrize("tag,g", CASES)
def test_niching_on_cpu_with_oracle_ranks(monkeypatch, tag, g):
    import evox_b200.algorithms.mo as mo

    monkeypatch.setattr(mo, "non_dominate_rank", onds.non_dominate_rank)
    monkeypatch.setattr(mo, "raise_on_kernel_errors", lambda: None)
    algo, c = run_generation(tag, g, torch.device("cpu"))
    assert torch.equal(algo.pop, c["next_pop"])
    assert torch.equal(algo.fit, c["next_fit"])
    assert torch.equal(algo.rank.to(c["next_rank"].dtype), c["next_rank"])


def test_masked_assign_last_writer_wins():
    from evox_b200.algorithms.mo import _masked_assign

    target = torch.tensor([10, 11, 12, 13])
    # entry 0 assigns index 3, entry 2 (outside the mask, clamped from 99 to 3) writes the old value back
    out = _masked_assign(target, torch.tensor([3, 1, 99]), torch.tensor([True, True, False]), 7)
    assert out.tolist() == [10, 7, 12, 13]
    # the other order keeps the assignment
    out = _masked_assign(target, torch.tensor([99, 1, 3]), torch.tensor([False, True, True]), 7)
    assert out.tolist() == [10, 7, 12, 7]
    assert target.tolist() == [10, 11, 12, 13]


@pytest.mark.gpu
@pytest.mark.parametrize("tag,g", CASES)
def test_environmental_selection_on_gpu(cuda, tag, g):
    algo, c = run_generation(tag, g, cuda)
    assert torch.equal(algo.pop, c["next_pop"])
    assert torch.equal(algo.fit, c["next_fit"])
    assert torch.equal(algo.rank.to(c["next_rank"].dtype), c["next_rank"])


@pytest.mark.gpu
def test_workflow_runs_and_improves(cuda):
    """StdWorkflow(NSGA3, DTLZ2) with its own random draws: the population keeps (about) its size, every row is
    finite and the mean distance to the front shrinks."""
    from evox_b200.algorithms import NSGA3
    from evox_b200.problems.numerical import DTLZ2
    from evox_b200.workflows import StdWorkflow

    torch.manual_seed(5)
    d, m, n = 12, 3, 91
    wf = StdWorkflow(NSGA3(n, m, torch.zeros(d), torch.ones(d), device=cuda), DTLZ2(d=d, m=m), device=cuda)
    wf.init_step()
    first = (wf.algorithm.fit.norm(dim=1) - 1).abs().mean().item()
    for _ in range(30):
        wf.step()
    a = wf.algorithm
    assert n - 5 <= a.pop.shape[0] <= n + 1 and a.fit.shape == (a.pop.shape[0], m)
    assert torch.isfinite(a.fit).all()
    assert (a.fit.norm(dim=1) - 1).abs().mean().item() < 0.5 * first
