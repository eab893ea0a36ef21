"""The PSO oracle reproduces the reference's recorded states bit for bit (CPU only)."""
import pytest
import torch

from oracle import pso as opso

NAMES = ["pop", "velocity", "fit", "local_best_location", "local_best_fit", "global_best_location", "global_best_fit"]


def load_state(g, tag, k):
    s = {n: torch.from_numpy(g[f"{tag}_s{k}_{n}"]) for n in NAMES}
    lo, hi = g[f"{tag}_bounds"]
    dim = s["pop"].shape[1]
    s["lb"] = torch.full((1, dim), float(lo))
    s["ub"] = torch.full((1, dim), float(hi))
    w, pp, pg = g[f"{tag}_hyper"]
    s["w"], s["phi_p"], s["phi_g"] = torch.tensor(w), torch.tensor(pp), torch.tensor(pg)
    return s


@pytest.mark.parametrize("prob", ["ackley", "rastrigin"])
@pytest.mark.parametrize("dim", [12, 10])
def test_oracle_matches_reference_states(golden, prob, dim):
    g = golden("pso")
    tag = f"pso_{prob}_d{dim}"
    fitness = opso.FITNESS[prob]
    s = opso.init_step(load_state(g, tag, 0), fitness)
    want = load_state(g, tag, 1)
    for n in NAMES:
        assert torch.equal(s[n], want[n]), f"init_step {n}"
    for gen in range(3):
        s = load_state(g, tag, gen + 1)  # teacher forcing: start from the reference's own state
        rg = torch.from_numpy(g[f"{tag}_g{gen}_rg"])
        rp = torch.from_numpy(g[f"{tag}_g{gen}_rp"])
        s = opso.step(s, rg, rp, fitness)
        want = load_state(g, tag, gen + 2)
        for n in NAMES:
            assert torch.equal(s[n], want[n]), f"gen {gen} {n}"


def test_relu_clamp_is_not_torch_clamp():
    # the reference's clamp can land one ulp off the bound; the oracle must keep that quirk
    a = torch.tensor([40.123456], dtype=torch.float32)
    lb, ub = torch.tensor([-32.768]), torch.tensor([32.768])
    got = opso.relu_clamp(a, lb, ub)
    assert torch.allclose(got, torch.clamp(a, lb, ub), rtol=1e-6)


def test_philox_stream_shapes_and_range():
    u = opso.pso_uniform(5, 10, seed=7, generation=3, which=1)
    assert u.shape == (5, 10) and u.dtype == torch.float32
    assert (u >= 0).all() and (u < 1).all()
    # row_offset shifts the stream exactly by rows (sharding invariance)
    full = opso.pso_uniform(8, 10, seed=7, generation=3, which=1)
    part = opso.pso_uniform(3, 10, seed=7, generation=3, which=1, row_offset=5)
    assert torch.equal(full[5:], part)


def test_philox_matches_known_answer():
    # Philox4x32-10 known-answer vectors published with the Random123 library (kat_vectors):
    # counter = key = 0 and counter = key = all ones.
    z = torch.zeros(1, dtype=torch.int64)
    out = opso.philox4x32_10(z, z, z, z, z, z)
    assert [int(o) for o in out] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    f = torch.full((1,), 0xFFFFFFFF, dtype=torch.int64)
    out = opso.philox4x32_10(f, f, f, f, f, f)
    assert [int(o) for o in out] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
