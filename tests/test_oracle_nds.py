"""The NSGA-II selection oracle reproduces outputs recorded from the reference (CPU only)."""
import numpy as np
import pytest
import torch

from oracle import nds

CASES = ["dtlz2", "ties_m2", "nan_m5", "flat_objective", "single_front", "tiny"]


def same(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Bit-equal, treating NaNs at the same positions as equal."""
    return torch.equal(torch.isnan(a), torch.isnan(b)) and torch.equal(torch.nan_to_num(a, nan=0.0), torch.nan_to_num(b, nan=0.0))


@pytest.mark.parametrize("case", CASES)
def test_rank_crowding_selection(golden, case):
    g = golden("nds")
    f = torch.from_numpy(g[f"{case}_f"])
    topk = int(g[f"{case}_topk"])
    rank = nds.non_dominate_rank(f, block=64)
    assert rank.dtype == torch.int32
    assert torch.equal(rank, torch.from_numpy(g[f"{case}_rank"]))
    mask = torch.from_numpy(g[f"{case}_mask"])
    assert same(nds.crowding_distance(f, mask), torch.from_numpy(g[f"{case}_crowd"]))
    x = torch.arange(f.shape[0], dtype=torch.float32)[:, None].repeat(1, 2)
    sx, sf, srank, scrowd, order = nds.nd_environmental_selection(x, f, topk)
    assert np.array_equal(order.numpy(), g[f"{case}_sel_index"])
    assert same(sf, torch.from_numpy(g[f"{case}_sel_f"]))
    assert torch.equal(srank, torch.from_numpy(g[f"{case}_sel_rank"]))
    assert same(scrowd, torch.from_numpy(g[f"{case}_sel_crowd"]))


def test_blocking_does_not_change_ranks():
    f = nds.dtlz2_objectives(torch.rand(700, 12, generator=torch.Generator().manual_seed(1)))
    assert torch.equal(nds.non_dominate_rank(f, block=37), nds.non_dominate_rank(f, block=4096))
