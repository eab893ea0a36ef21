"""CSO kernels against the oracle / the reference's golden vectors (teacher-forced pairing and draws)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import cso as ocso
from oracle import pso as opso

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "cso.npz")
RTOL = 1e-5  # fp32 tolerance of the path (positions are bit-exact in practice, the mean and fitness are not)


def close(a, b, scale=None):
    a, b = a.detach().cpu().double(), torch.as_tensor(b).double()
    s = b.abs().max() if scale is None else scale
    return float((a - b).abs().max()) <= RTOL * float(max(s, 1e-30))


def build(tag, prob_cls, cuda, step=1, **kw):
    from evox_b200.algorithms import CSO
    from evox_b200.workflows import StdWorkflow

    lo, hi = GOLD[f"{tag}_bounds"]
    pop = torch.from_numpy(GOLD[f"{tag}_s{step}_pop"])
    n, d = pop.shape
    algo = CSO(n, torch.full((d,), float(lo)), torch.full((d,), float(hi)), phi=float(GOLD[f"{tag}_phi"]), device=cuda, seed=5)
    algo.pop.copy_(pop)
    algo.velocity.copy_(torch.from_numpy(GOLD[f"{tag}_s{step}_velocity"]))
    if step >= 1:
        algo.fit.copy_(torch.from_numpy(GOLD[f"{tag}_s{step}_fit"]))
    return StdWorkflow(algo, prob_cls(), device=cuda, **kw)


@pytest.mark.parametrize("prob", ["ackley", "sphere"])
@pytest.mark.parametrize("dim", [12, 10])
@pytest.mark.parametrize("fused", [True, False])
def test_teacher_forced_generations_match_reference(cuda, prob, dim, fused):
    from evox_b200.problems.numerical import Ackley, Sphere

    tag = f"cso_{prob}_d{dim}"
    cls = {"ackley": Ackley, "sphere": Sphere}[prob]
    kw = {} if fused else {"fitness_transform": torch.nn.Identity()}  # any transform switches the fusion off
    wf = build(tag, cls, cuda, step=0, **kw)
    wf.init_step()
    assert close(wf.algorithm.fit, GOLD[f"{tag}_s1_fit"])
    for g in range(3):
        wf.algorithm.step(perm=torch.from_numpy(GOLD[f"{tag}_g{g}_perm"]), lambdas=torch.from_numpy(GOLD[f"{tag}_g{g}_lambdas"]))
        lo, hi = GOLD[f"{tag}_bounds"]
        assert close(wf.algorithm.pop, GOLD[f"{tag}_s{g + 2}_pop"], scale=float(hi - lo)), g
        assert close(wf.algorithm.fit, GOLD[f"{tag}_s{g + 2}_fit"]), g
        assert torch.equal(wf.algorithm.velocity.cpu(), torch.from_numpy(GOLD[f"{tag}_s{g + 2}_velocity"]))


@pytest.mark.parametrize("n,d", [(2, 4), (64, 1000), (250, 1024), (100, 1028), (30, 7), (4096, 64)])
def test_random_swarms_against_oracle(cuda, n, d):
    """Two generations on seeded swarms (row lengths on both sides of the register-resident column sums,
    scalar path, a single pair), draws supplied; the second generation uses the mean the kernel accumulated."""
    from evox_b200.algorithms import CSO
    from evox_b200.problems.numerical import Ackley
    from evox_b200.workflows import StdWorkflow

    g = torch.Generator().manual_seed(n * 31 + d)
    lb, ub = torch.full((d,), -32.0), torch.full((d,), 32.0)
    algo = CSO(n, lb, ub, phi=0.15, device=cuda, seed=1)
    wf = StdWorkflow(algo, Ackley(), device=cuda)
    wf.init_step()
    s = {"pop": algo.pop.cpu().clone(), "velocity": algo.velocity.cpu().clone(), "lb": lb[None], "ub": ub[None], "phi": torch.tensor(0.15)}
    s = ocso.init_step(s, opso.ackley)
    assert close(algo.fit, s["fit"])
    for _ in range(2):
        perm = torch.randperm(n, generator=g)
        lam = torch.rand(3, n // 2, d, generator=g)
        # the pairing decision compares fitness values: give the kernel the oracle's (they agree to 1e-5,
        # which a near-tie could still turn into a swapped teacher and student)
        algo.fit.copy_(s["fit"])
        algo.step(perm=perm, lambdas=lam)
        s = ocso.step(s, perm, lam, opso.ackley)
        assert close(algo.pop, s["pop"], scale=64.0)
        assert close(algo.fit, s["fit"])


def test_in_kernel_stream_properties(cuda):
    """Philox mode: repeatable for a seed, inside the bounds, the best never gets worse; with the
    students' velocities stored (the original rule, not the reference's) the swarm contracts on Sphere."""
    from evox_b200.algorithms import CSO
    from evox_b200.problems.numerical import Sphere
    from evox_b200.workflows import EvalMonitor, StdWorkflow

    def run(seed, store=False):
        torch.manual_seed(3)
        algo = CSO(512, torch.full((40,), -10.0), torch.full((40,), 10.0), phi=0.1, device=cuda, seed=seed, store_velocity=store)
        mon = EvalMonitor(device=cuda)
        wf = StdWorkflow(algo, Sphere(), monitor=mon, device=cuda)
        wf.init_step()
        first = float(algo.fit.min())
        for _ in range(60):
            wf.step()
        return algo.pop.clone(), first, float(algo.fit.min()), mon

    a, first, last, mon = run(11)
    b, _, _, _ = run(11)
    c, _, _, _ = run(12)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert float(a.min()) >= -10.0 and float(a.max()) <= 10.0
    assert last <= first
    assert float(mon.get_best_fitness()) <= last + 1e-6
    _, first, last, _ = run(11, store=True)
    assert last < 0.05 * first


def test_outside_change_of_the_swarm_recomputes_the_mean(cuda):
    """The cached mean is dropped when torch-side code wrote to `pop` between two steps."""
    from evox_b200.algorithms import CSO
    from evox_b200.problems.numerical import Sphere
    from evox_b200.workflows import StdWorkflow

    n, d = 64, 16
    g = torch.Generator().manual_seed(0)
    lb, ub = torch.full((d,), -4.0), torch.full((d,), 4.0)
    algo = CSO(n, lb, ub, phi=0.5, device=cuda, seed=2)
    wf = StdWorkflow(algo, Sphere(), device=cuda)
    wf.init_step()
    perm, lam = torch.randperm(n, generator=g), torch.rand(3, n // 2, d, generator=g)
    algo.step(perm=perm, lambdas=lam)
    algo.pop.mul_(0.5)  # outside change
    wf.init_step()
    s = {"pop": algo.pop.cpu().clone(), "fit": algo.fit.cpu().clone(), "velocity": algo.velocity.cpu().clone(),
         "lb": lb[None], "ub": ub[None], "phi": torch.tensor(0.5)}
    perm, lam = torch.randperm(n, generator=g), torch.rand(3, n // 2, d, generator=g)
    algo.step(perm=perm, lambdas=lam)
    s = ocso.step(s, perm, lam, opso.sphere)
    assert close(algo.pop, s["pop"], scale=8.0)


def test_odd_swarm_is_rejected(cuda):
    from evox_b200.algorithms import CSO

    with pytest.raises(AssertionError):
        CSO(7, torch.zeros(3), torch.ones(3), device=cuda)
