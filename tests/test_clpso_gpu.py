"""CLPSO kernels against the reference's golden vectors and the oracle (teacher-forced draws)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import clpso as oclpso
from oracle import pso as opso

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "clpso.npz")
NAMES = ["pop", "fit", "velocity", "personal_best_location", "personal_best_fit", "global_best_location", "global_best_fit"]
RTOL = 1e-5


def close(a, b, scale=None):
    a, b = a.detach().cpu().double(), torch.as_tensor(b).double()
    s = b.abs().max() if scale is None else scale
    return float((a - b).abs().max()) <= RTOL * float(max(s, 1e-30))


@pytest.mark.parametrize("prob", ["ackley", "sphere"])
@pytest.mark.parametrize("dim", [12, 10])
@pytest.mark.parametrize("fused", [True, False])
def test_teacher_forced_generations_match_reference(cuda, prob, dim, fused):
    from evox_b200.algorithms import CLPSO
    from evox_b200.problems.numerical import Ackley, Sphere
    from evox_b200.workflows import StdWorkflow

    tag = f"clpso_{prob}_d{dim}"
    lo, hi = GOLD[f"{tag}_bounds"]
    algo = CLPSO(37, torch.full((dim,), float(lo)), torch.full((dim,), float(hi)), 0.5, 1.5, 0.3, device=cuda, seed=3)
    for n in NAMES:
        getattr(algo, n).copy_(torch.from_numpy(GOLD[f"{tag}_s0_{n}"]))
    kw = {} if fused else {"fitness_transform": torch.nn.Identity()}
    wf = StdWorkflow(algo, {"ackley": Ackley, "sphere": Sphere}[prob](), device=cuda, **kw)
    wf.init_step()
    for g in range(-1, 3):
        if g >= 0:
            draws = [torch.from_numpy(GOLD[f"{tag}_g{g}_{k}"]) for k in ("coeff", "i1", "i2", "poss")]
            wf.algorithm.step(*draws)
        for n in NAMES:
            want = GOLD[f"{tag}_s{g + 2}_{n}"]
            scale = float(hi - lo) if want.ndim >= 1 and n not in ("fit", "personal_best_fit") else None
            assert close(getattr(wf.algorithm, n), want, scale=scale), (g, n)


@pytest.mark.parametrize("n,d", [(1, 4), (300, 1000), (64, 7), (2048, 64)])
def test_random_swarms_against_oracle(cuda, n, d):
    from evox_b200.algorithms import CLPSO
    from evox_b200.problems.numerical import Rastrigin
    from evox_b200.workflows import StdWorkflow

    g = torch.Generator().manual_seed(n + d)
    lb, ub = torch.full((d,), -5.12), torch.full((d,), 5.12)
    algo = CLPSO(n, lb, ub, 0.6, 1.4, 0.25, device=cuda, seed=9)
    algo.velocity.mul_(0.2)
    wf = StdWorkflow(algo, Rastrigin(), device=cuda)
    wf.init_step()
    s = {k: getattr(algo, k).cpu().clone() for k in NAMES}
    s.update(lb=lb[None], ub=ub[None], w=torch.tensor(0.6), c=torch.tensor(1.4), P_c=torch.tensor(0.25))
    for _ in range(2):
        coeff = torch.rand(n, d, generator=g)
        i1, i2 = torch.randint(0, n, (n,), generator=g), torch.randint(0, n, (n,), generator=g)
        poss = torch.rand(n, generator=g)
        # decisions compare fitness values: hand the kernel the oracle's so that near-ties cannot flip them
        algo.fit.copy_(s["fit"])
        algo.personal_best_fit.copy_(s["personal_best_fit"])
        algo.step(coeff, i1, i2, poss)
        s = oclpso.step(s, coeff, i1, i2, poss, opso.rastrigin)
        assert close(algo.pop, s["pop"], scale=10.24)
        assert close(algo.velocity, s["velocity"], scale=10.24)
        assert close(algo.fit, s["fit"])
        assert torch.equal(algo.personal_best_location.cpu(), s["personal_best_location"])


def test_in_kernel_stream_improves_and_repeats(cuda):
    from evox_b200.algorithms import CLPSO
    from evox_b200.problems.numerical import Sphere
    from evox_b200.workflows import StdWorkflow

    def run(seed):
        torch.manual_seed(5)
        algo = CLPSO(256, torch.full((30,), -10.0), torch.full((30,), 10.0), device=cuda, seed=seed)
        wf = StdWorkflow(algo, Sphere(), device=cuda)
        wf.init_step()
        first = float(algo.global_best_fit)
        for _ in range(150):
            wf.step()
        return algo.pop.clone(), first, float(algo.global_best_fit)

    a, first, last = run(1)
    b, _, _ = run(1)
    assert torch.equal(a, b)
    assert last < 0.1 * first
    assert float(a.min()) >= -10.0 and float(a.max()) <= 10.0
