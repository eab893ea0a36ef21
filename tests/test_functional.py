"""`use_state` / `vmap` over modules (the reference's usage: unit_test/algorithms/test_base.py:52-65,
unit_test/workflows/test_std_workflow.py:94-103): CPU checks of the mechanism on a pure-torch algorithm,
and a GPU check that three mapped PSO workflows equal three separate ones."""

import pytest
import torch

from evox_b200.core import Algorithm, Mutable, Parameter, Problem, use_state, vmap
from evox_b200.core import functional


class Toy(Algorithm):
    """Rebinds one buffer, writes the other in place, keeps a draw counter outside the tensors."""

    def __init__(self, n=4, d=3):
        super().__init__()
        self.pop = Mutable(torch.arange(n * d, dtype=torch.float32).reshape(n, d))
        self.fit = Mutable(torch.zeros(n))
        self.gain = Parameter(2.0)
        self.seed, self.draws = 5, 0
        self.seen_seeds = []

    def get_extra_state(self):
        return {"draws": self.draws}

    def set_extra_state(self, state):
        self.draws = int(state["draws"])

    def step(self):
        self.seen_seeds.append(functional.replica_seed(self.seed))
        self.draws += 1
        self.pop = self.pop * self.gain + self.draws  # a new tensor
        self.fit.copy_((self.pop**2).sum(-1))  # in place

    def best(self, shift):
        return (self.fit + shift).min()


def test_use_state_is_functional():
    algo = Toy()
    before = {k: v.clone() for k, v in algo.state_dict().items() if isinstance(v, torch.Tensor)}
    state = {k: v.clone() for k, v in before.items()}
    state["pop"] += 1.0
    given = {k: v.clone() for k, v in state.items()}
    fn = use_state(algo.step)
    new = fn(state)
    assert set(new) == {"pop", "fit", "gain"}
    assert torch.equal(new["pop"], given["pop"] * 2.0 + 1)
    assert torch.equal(new["fit"], (new["pop"] ** 2).sum(-1))
    for k in given:  # the caller's tensors are not written
        assert torch.equal(state[k], given[k]), k
    for k in before:  # nor is the module's own state (its buffers are the same objects as before)
        assert torch.equal(algo.state_dict()[k], before[k]), k
    # a method with a return value gives (state, value); extra arguments pass through
    new2, val = use_state(algo.best)(new, 3.0)
    assert torch.equal(val, new["fit"].min() + 3.0) and torch.equal(new2["fit"], new["fit"])
    with pytest.raises(KeyError):
        use_state(algo.step, strict=True)({"pop": state["pop"]})
    with pytest.raises(TypeError):
        use_state(lambda: None)


@pytest.mark.parametrize("randomness", ["different", "same"])
def test_vmap_over_stacked_state(randomness):
    algo = Toy()
    params, buffers = torch.func.stack_module_state([algo] * 3)
    state = params | buffers
    state["pop"] = state["pop"] + torch.arange(3.0).view(3, 1, 1)  # three different replicas
    step = vmap(use_state(algo.step), randomness=randomness)
    out = step(state)
    assert out["pop"].shape == (3, 4, 3) and out["fit"].shape == (3, 4) and out["gain"].shape == (3,)
    for b in range(3):
        assert torch.equal(out["pop"][b], state["pop"][b] * 2.0 + 1)  # every slice saw draws == 1
    assert algo.draws == 1  # the mapped call advanced the counter once
    seeds = algo.seen_seeds
    assert len(seeds) == 3
    assert (len(set(seeds)) == 3) if randomness == "different" else (set(seeds) == {5})
    out2 = step(out)
    assert algo.draws == 2
    assert torch.equal(out2["pop"][1], out["pop"][1] * 2.0 + 2)
    assert functional.replica_seed(5) == 5  # outside vmap


def test_vmap_dims_and_plain_functions():
    f = vmap(lambda x, y: (x * y, (x + y).sum()), in_dims=(0, None), out_dims=(1, 0))
    x, y = torch.arange(6.0).view(3, 2), torch.tensor([10.0, 100.0])
    a, b = f(x, y)
    assert torch.equal(a, (x * y).t()) and torch.equal(b, (x + y).sum(-1))
    with pytest.raises(ValueError):
        vmap(lambda x, y: x + y)(torch.zeros(2, 1), torch.zeros(3, 1))
    with pytest.raises(ValueError):
        vmap(lambda x: x, randomness="sometimes")


@pytest.mark.gpu
def test_vmapped_pso_workflows_equal_separate_ones(cuda):
    from evox_b200.algorithms import PSO
    from evox_b200.problems.numerical import Ackley
    from evox_b200.workflows import StdWorkflow

    d = 40
    lb, ub = torch.full((d,), -32.768), torch.full((d,), 32.768)
    wf = StdWorkflow(PSO(300, lb, ub, device=cuda, seed=21), Ackley(), device=cuda)
    params, buffers = torch.func.stack_module_state([wf] * 3)
    state = params | buffers
    # three different swarms
    state["algorithm.pop"] = state["algorithm.pop"] * torch.tensor([1.0, 0.5, 0.25], device=cuda).view(3, 1, 1)
    given = {k: v.clone() for k, v in state.items()}
    init = vmap(use_state(wf.init_step), randomness="different")
    step = vmap(use_state(wf.step), randomness="different")
    out = init(state)
    for _ in range(3):
        out = step(out)
    for k in given:
        assert torch.equal(state[k], given[k]), k
    assert wf.algorithm.generation == 3
    for b in range(3):
        with functional._replica(b + 1):
            seed_b = functional.replica_seed(21)
        ref = StdWorkflow(PSO(300, lb, ub, device=cuda, seed=21), Ackley(), device=cuda)
        ref.algorithm.pop.copy_(given["algorithm.pop"][b])
        ref.algorithm.seed = seed_b
        ref.init_step()
        for _ in range(3):
            ref.step()
        for name, t in ref.state_dict().items():
            if isinstance(t, torch.Tensor):
                assert torch.equal(out[name][b], t), (b, name)
    # the swarms differ from one another and improved
    assert not torch.equal(out["algorithm.pop"][0], out["algorithm.pop"][1])
