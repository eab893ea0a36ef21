"""Edge cases through the public wrappers: empty and single-row inputs, all-masked and all-NaN
inputs, duplicates, infinities — each against the oracle (which is pinned to the reference)."""
import math

import pytest
import torch

from oracle import nds as onds
from oracle import pso as opso
from oracle import rvea as orvea

pytestmark = pytest.mark.gpu


def same(a, b):
    a, b = a.cpu(), b.cpu()
    return torch.equal(torch.isnan(a), torch.isnan(b)) and torch.equal(torch.nan_to_num(a, nan=0.0), torch.nan_to_num(b, nan=0.0))


def test_rank_empty_and_single(cuda):
    from evox_b200.operators.selection import non_dominate_rank

    assert non_dominate_rank(torch.empty(0, 3, device=cuda)).shape == (0,)
    assert non_dominate_rank(torch.tensor([[1.0, 2.0]], device=cuda)).tolist() == [0]


def test_rank_all_duplicates_and_all_nan(cuda):
    from evox_b200.operators.selection import non_dominate_rank

    f = torch.ones(100, 3)
    assert torch.equal(non_dominate_rank(f.to(cuda), check=True).cpu(), onds.non_dominate_rank(f))  # nobody dominates a copy of itself
    f = torch.full((65, 2), float("nan"))
    assert torch.equal(non_dominate_rank(f.to(cuda), check=True).cpu(), onds.non_dominate_rank(f))
    f = torch.rand(300, 2, generator=torch.Generator().manual_seed(0))
    f[::7] = float("inf")
    f[5, 0] = float("-inf")
    assert torch.equal(non_dominate_rank(f.to(cuda), check=True).cpu(), onds.non_dominate_rank(f))


def test_crowding_masks(cuda):
    from evox_b200.operators.selection import crowding_distance

    f = torch.rand(50, 3, generator=torch.Generator().manual_seed(1))
    for mask in (torch.zeros(50, dtype=torch.bool), torch.arange(50) == 13, torch.arange(50) < 2):
        if int(mask.sum()) == 0:
            got = crowding_distance(f.to(cuda), mask.to(cuda))
            assert torch.isinf(got).all() and (got < 0).all()  # the reference would index element -1 here; all rows are outside the mask
            continue
        assert same(crowding_distance(f.to(cuda), mask.to(cuda)), onds.crowding_distance(f, mask))


def test_selection_keeps_everything_or_one(cuda):
    from evox_b200.operators.selection import nd_environmental_selection

    g = torch.Generator().manual_seed(2)
    f, x = torch.rand(64, 2, generator=g), torch.rand(64, 3, generator=g)
    for topk in (64, 1):
        want = onds.nd_environmental_selection(x, f, topk)
        got = nd_environmental_selection(x.to(cuda), f.to(cuda), topk, return_index=True, check=True)
        assert torch.equal(got[4].cpu(), want[4]) and same(got[3], want[3])


def test_rvea_all_nan_and_single_row(cuda):
    from evox_b200.operators.selection import ref_vec_guided

    v = orvea.two_layer_vectors(4, 0, 3)
    x, f = torch.rand(20, 4), torch.full((20, 3), float("nan"))
    nx, nf = ref_vec_guided(x.to(cuda), f.to(cuda), v.to(cuda), 0.5)
    assert torch.isnan(nx).all() and torch.isnan(nf).all()  # nobody can be associated: every slot empty
    x, f = torch.rand(1, 4), torch.rand(1, 3)
    nx, nf, idx = ref_vec_guided(x.to(cuda), f.to(cuda), v.to(cuda), 0.5, return_index=True)
    o = orvea.ref_vec_guided(x, f, v, torch.tensor(0.5))
    assert torch.equal(idx.cpu(), o["next_ind"])


def test_pso_single_particle_and_odd_dims(cuda):
    from evox_b200.algorithms import PSO
    from evox_b200.problems.numerical import Ackley
    from evox_b200.workflows import StdWorkflow

    for P, d in ((1, 1), (3, 7), (2, 1025)):
        state = opso.init_step(opso.make_state(P, d, -32.768, 32.768, 0.6, 2.5, 0.8, seed=P + d), opso.ackley)
        algo = PSO(P, torch.full((d,), -32.768), torch.full((d,), 32.768), device=cuda, seed=1)
        wf = StdWorkflow(algo, Ackley(), device=cuda)
        names = ["pop", "velocity", "fit", "local_best_location", "local_best_fit", "global_best_location", "global_best_fit"]
        wf.algorithm.load_state_dict({**{n: state[n] for n in names}, "w": state["w"], "phi_p": state["phi_p"], "phi_g": state["phi_g"]})
        rg, rp = opso.draws(P, d, 5)
        wf.algorithm.step(rg=rg.to(cuda), rp=rp.to(cuda))
        want = opso.step(state, rg, rp, opso.ackley)
        got = wf.algorithm.state_dict()
        for n in ("pop", "velocity", "local_best_location", "global_best_location"):
            assert torch.equal(got[n].cpu(), want[n]), (P, d, n)
        assert torch.allclose(got["fit"].cpu(), want["fit"], rtol=1e-5)


def test_pso_inf_and_nan_fitness_state(cuda):
    """Fresh swarm (all fitness +inf, as PSO.__init__ leaves it) stepped without init_step, like the
    reference allows: nothing improves, the global best stays particle 0 (+inf ties keep the old best)."""
    P, d = 40, 8
    state = opso.make_state(P, d, -1.0, 1.0, 0.6, 2.5, 0.8, seed=3)
    rg, rp = opso.draws(P, d, 1)
    want = opso.step(state, rg, rp, opso.sphere)
    from tests.test_pso_gpu import Swarm

    sw = Swarm(state, cuda)
    sw.step("sphere", rg, rp)
    for n in ("pop", "velocity", "local_best_location", "global_best_location", "local_best_fit", "global_best_fit"):
        assert same(sw.t[n], want[n]), n
    assert math.isinf(sw.t["global_best_fit"].item())
