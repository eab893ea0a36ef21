"""The RVEA selection oracle reproduces outputs recorded from the reference (CPU only)."""
import pytest
import torch

from oracle import rvea


def same(a, b):
    return torch.equal(torch.isnan(a), torch.isnan(b)) and torch.equal(torch.nan_to_num(a), torch.nan_to_num(b))


@pytest.mark.parametrize("case", ["unit", "m10", "m3"])
def test_matches_reference(golden, case):
    g = golden("rvea")
    x, f, v, theta = (torch.from_numpy(g[f"{case}_{k}"]) for k in ("x", "f", "v", "theta"))
    o = rvea.ref_vec_guided(x, f, v, theta)
    assert same(o["next_x"], torch.from_numpy(g[f"{case}_next_x"]))
    assert same(o["next_f"], torch.from_numpy(g[f"{case}_next_f"]))
    assert o["next_x"].shape[0] == v.shape[0]  # one slot per reference vector (the reference's own test)


def test_lattice_counts():
    assert rvea.simplex_lattice(3, 10).shape == (220, 10)
    v = rvea.two_layer_vectors(3, 2, 10)
    assert v.shape == (275, 10)
    assert torch.allclose(v.sum(dim=1), torch.ones(275), atol=1e-6)
