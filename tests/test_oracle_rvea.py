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


def test_rveaa_pieces_match_reference():
    """RVEAa's vector regeneration and final truncation against outputs recorded from the reference."""
    import numpy as np
    from pathlib import Path

    g = np.load(Path(__file__).parent / "golden" / "rveaa.npz")
    t = torch.from_numpy
    new_v = rvea.rv_regeneration(t(g["regen_obj"]), t(g["regen_v"]), t(g["regen_draw"]))
    assert torch.equal(new_v, t(g["regen_new_v"]))
    assert not torch.equal(new_v, t(g["regen_v"]))  # the case does regenerate something
    new_pop, new_obj = rvea.batch_truncation(t(g["trunc_pop"]), t(g["regen_obj"]))
    assert torch.equal(torch.nan_to_num(new_pop, nan=-7.0), torch.nan_to_num(t(g["trunc_new_pop"]), nan=-7.0))
    assert torch.equal(torch.nan_to_num(new_obj, nan=-7.0), torch.nan_to_num(t(g["trunc_new_obj"]), nan=-7.0))
