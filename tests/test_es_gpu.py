"""Parity of the CUDA evolution-strategy kernels with the reference's recorded outputs and the oracle.

Uniform streams are integer work and must be bit-exact. Normals go through device logf / sincosf
instead of the CPU's: absolute 2e-6. Products, gradients and centre updates: relative 1e-5
(measured against the largest magnitude of the tensor, since individual entries can cancel).
"""
import numpy as np
import pytest
import torch
from torch import nn

from oracle import lora

pytestmark = pytest.mark.gpu


def t(a):
    return torch.from_numpy(a)


def close(got, want, rel=1e-5):
    got, want = got.detach().cpu().double(), want.detach().double()
    scale = want.abs().max().clamp_min(1e-30)
    err = (got - want).abs().max() / scale
    assert err <= rel, f"max error {err:.3e} of scale {scale:.3e}"


def test_philox_golden(golden, cuda):
    from evox_b200.lora_kernels import philox_normal, philox_uniform

    g = golden("es")
    seeds = t(g["seeds"]).to(cuda)
    for key in g:
        if key.startswith("uniform_n"):
            n, c = int(key.split("_")[1][1:]), int(key.split("_c")[1])
            assert torch.equal(philox_uniform(seeds, n, c).cpu(), t(g[key])), key
            z = philox_normal(seeds, n, c).cpu()
            assert (z - t(g[key.replace("uniform", "normal")])).abs().max() <= 2e-6


@pytest.mark.parametrize("pop,n,counter", [(1, 1, 0), (3, 5, 7), (64, 32768, 12345), (1024, 1001, (5 << 32) + 3), (7, 4096, (1 << 32) - 8)])
def test_philox_vs_oracle(cuda, pop, n, counter):
    from evox_b200.lora_kernels import philox_normal, philox_uniform

    seeds = torch.randint(0, 2**31, (pop,), generator=torch.Generator().manual_seed(pop), dtype=torch.int64)
    if pop > 2:
        seeds[2] = (9 << 32) + 77
    assert torch.equal(philox_uniform(seeds.to(cuda), n, counter).cpu(), lora.philox_uniform(seeds, n, counter))
    z, zr = philox_normal(seeds.to(cuda), n, counter).cpu(), lora.philox_normal(seeds, n, counter)
    assert (z - zr).abs().max() <= 2e-6
    if n >= 1000:  # the reference's own moment checks (test_philox.py:150-185)
        assert abs(z.mean()) < 0.1 and abs(z.std() - 1) < 0.1


def test_factors_delta_gradient_golden(golden, cuda):
    from evox_b200.lora_kernels import compute_counter_offsets, generate_lora_factors, lora_delta_output, lora_gradient

    g = golden("es")
    assert compute_counter_offsets([(10,), (4, 3), (2, 5)], 2) == [0, 12, 28]
    seeds = t(g["seeds"]).to(cuda)
    a, b = generate_lora_factors(seeds, (12, 20), 4, 40)
    assert a.shape == (6, 4, 20) and b.shape == (6, 12, 4)
    assert (a.cpu() - t(g["factors_A"])).abs().max() <= 2e-6 and (b.cpu() - t(g["factors_B"])).abs().max() <= 2e-6
    # feed the reference's own factors so that only the product is compared
    A, B = t(g["factors_A"]).to(cuda), t(g["factors_B"]).to(cuda)
    close(lora_delta_output(t(g["delta_x"]).to(cuda), A, B, 0.1), t(g["delta_out"]))
    fit = t(g["grad_fitness"]).to(cuda)
    close(lora_gradient(fit, A, B, 6, 0.1, (12, 20)), t(g["grad_out"]))
    close(lora_gradient(fit, t(g["bias_noise"]).to(cuda), None, 6, 0.1, (9,)), t(g["grad_bias"]))


@pytest.mark.parametrize("pop,batch,k,d,r", [(16, 7, 33, 50, 4), (64, 64, 256, 192, 8), (5, 1, 8, 3, 16)])
def test_delta_and_gradient_vs_oracle(cuda, pop, batch, k, d, r):
    from evox_b200.lora_kernels import lora_delta_output, lora_gradient

    g = torch.Generator().manual_seed(k)
    x, A, B = torch.randn(pop, batch, k, generator=g), torch.randn(pop, r, k, generator=g), torch.randn(pop, d, r, generator=g)
    fit = torch.randn(pop, generator=g)
    close(lora_delta_output(x.to(cuda), A.to(cuda), B.to(cuda), 0.02), lora.lora_delta_output(x, A, B, 0.02))
    close(lora_gradient(fit.to(cuda), A.to(cuda), B.to(cuda), pop, 0.02, (d, k)), lora.lora_gradient(fit, A, B, pop, 0.02, (d, k)))


@pytest.mark.parametrize("opt", [None, "adam"])
def test_virtual_lora_es_step_golden(golden, cuda, opt):
    from evox_b200.algorithms import VirtualLoRAES
    from evox_b200.core import Problem
    from evox_b200.workflows import StdWorkflow

    g = golden("es")
    tag = f"vlora_{opt}"
    shapes = [(8, 6), (8,), (3, 8), (3,)]
    fitness = t(g[f"{tag}_fitness"]).to(cuda)
    seen = {}

    class Fixed(Problem):
        def evaluate(self, payload):
            seen["payload"] = payload
            return fitness

    algo = VirtualLoRAES(shapes, 2, 10, t(g[f"{tag}_center0"]), 0.05, 0.1, optimizer=opt, device=cuda)
    wf = StdWorkflow(algo, Fixed(), device=cuda)
    wf.algorithm.step(seeds=t(g[f"{tag}_seeds"]).to(cuda))
    center, seeds, sigma = seen["payload"]  # the tuple reaches the problem untouched
    assert center.shape == (sum(int(np.prod(s)) for s in shapes),) and seeds.dtype == torch.int64 and abs(sigma - 0.1) < 1e-7
    close(wf.algorithm.center, t(g[f"{tag}_center1"]))
    if opt:
        close(wf.algorithm.exp_avg, t(g[f"{tag}_exp_avg"]))
        close(wf.algorithm.exp_avg_sq, t(g[f"{tag}_exp_avg_sq"]))


@pytest.mark.parametrize("opt", [None, "adam"])
def test_open_es_step_golden(golden, cuda, opt):
    from evox_b200.algorithms import OpenES
    from evox_b200.core import Problem
    from evox_b200.workflows import StdWorkflow

    g = golden("es")
    tag = f"openes_{opt}"

    class Sphere(Problem):
        def evaluate(self, pop):
            return (pop**2).sum(dim=1)

    algo = OpenES(8, t(g[f"{tag}_center0"]), 0.05, 0.1, optimizer=opt, device=cuda)
    wf = StdWorkflow(algo, Sphere(), device=cuda)
    wf.algorithm.step(noise=t(g[f"{tag}_noise"]).to(cuda))
    close(wf.algorithm.center, t(g[f"{tag}_center1"]))
    wf.step()  # default path draws its own noise


@pytest.mark.parametrize("opt", [None, "adam"])
def test_ars_steps_golden(golden, cuda, opt):
    """ARS on the OpenES kernels: two teacher-forced generations against the reference's centres; then a
    run with its own draws on a larger problem must reduce the fitness of the centre."""
    from evox_b200.algorithms import ARS
    from evox_b200.core import Problem
    from evox_b200.workflows import StdWorkflow

    g = golden("ars")
    tag = f"ars_{opt}"
    shift = t(g[f"{tag}_shift"]).to(cuda)

    class ShiftedSphere(Problem):
        def evaluate(self, pop):
            return ((pop - shift) ** 2).sum(dim=1)

    algo = ARS(16, t(g[f"{tag}_center0"]), elite_ratio=0.5, lr=0.05, sigma=0.1, optimizer=opt, device=cuda)
    wf = StdWorkflow(algo, ShiftedSphere(), device=cuda)
    for k in range(2):
        wf.algorithm.step(z_plus=t(g[f"{tag}_z{k}"]))
        close(wf.algorithm.center, t(g[f"{tag}_center{k + 1}"]))
    if opt:
        close(wf.algorithm.exp_avg, t(g[f"{tag}_exp_avg"]))
        close(wf.algorithm.exp_avg_sq, t(g[f"{tag}_exp_avg_sq"]))
    before = float(((wf.algorithm.center - shift) ** 2).sum())
    for _ in range(200):
        wf.step()
    assert float(((wf.algorithm.center - shift) ** 2).sum()) < 0.5 * before


@pytest.mark.parametrize("opt", [None, "adam"])
def test_persistent_es_steps_golden(golden, cuda, opt):
    """PersistentES: four teacher-forced generations (accumulator, reset at T, decaying sigma) against the
    reference's recorded centres, accumulators and sigmas."""
    from evox_b200.algorithms import PersistentES
    from evox_b200.core import Problem
    from evox_b200.workflows import StdWorkflow

    g = golden("pes")
    tag = f"pes_{opt}"
    shift = t(g[f"{tag}_shift"]).to(cuda)

    class ShiftedSphere(Problem):
        def evaluate(self, pop):
            return ((pop - shift) ** 2).sum(dim=1)

    algo = PersistentES(12, t(g[f"{tag}_center0"]), optimizer=opt, lr=0.05, sigma=0.1, T=30, K=10, sigma_decay=0.9, sigma_limit=0.075,
                        device=cuda)
    wf = StdWorkflow(algo, ShiftedSphere(), device=cuda)
    for k in range(4):
        wf.algorithm.step(z=t(g[f"{tag}_z{k}"]))
        close(wf.algorithm.center, t(g[f"{tag}_center{k + 1}"]))
        assert torch.equal(wf.algorithm.pert_accum.cpu(), t(g[f"{tag}_accum{k + 1}"]))
        assert torch.equal(wf.algorithm.sigma.cpu(), t(g[f"{tag}_sigma{k + 1}"]))
        assert float(wf.algorithm.inner_step_counter) == float(g[f"{tag}_counter{k + 1}"])
    wf.step()  # default path draws its own noise


@pytest.mark.parametrize("tag", ["snes_temp", "snes_recomb", "des"])
def test_snes_des_steps_golden(golden, cuda, tag):
    """SNES (both weight types) and DES: three teacher-forced generations against the reference's centres and
    step sizes; then a run with its own draws must approach the optimum."""
    from evox_b200.algorithms import DES, SNES
    from evox_b200.core import Problem
    from evox_b200.workflows import StdWorkflow

    g = golden("snes_des")
    shift = t(g[f"{tag}_shift"]).to(cuda)

    class ShiftedSphere(Problem):
        def evaluate(self, pop):
            return ((pop - shift) ** 2).sum(dim=1)

    c0 = t(g[f"{tag}_center0"])
    algo = DES(14, c0, sigma_init=0.3, device=cuda) if tag == "des" else SNES(14, c0, sigma=0.5, weight_type=tag.split("_")[1], device=cuda)
    wf = StdWorkflow(algo, ShiftedSphere(), device=cuda)
    for k in range(3):
        wf.algorithm.step(noise=t(g[f"{tag}_z{k}"]))
        close(wf.algorithm.center, t(g[f"{tag}_center{k + 1}"]))
        close(wf.algorithm.sigma, t(g[f"{tag}_sigma{k + 1}"]))
    before = float(((wf.algorithm.center - shift) ** 2).sum())
    for _ in range(150):
        wf.step()
    assert float(((wf.algorithm.center - shift) ** 2).sum()) < 0.2 * before


@pytest.mark.parametrize("pop,dim", [(200, 1000), (64, 32768), (33, 20001), (7, 5)])
def test_weighted_column_sums_vs_torch(cuda, pop, dim):
    """Both tilings (32 columns, and float4 tiles of 128 for long aligned rows) of the two reductions behind
    OpenES / ARS / PersistentES (noise^T fitness) and SNES / DES (two rank-weighted moments)."""
    from evox_b200 import _cabi as c

    g = torch.Generator().manual_seed(pop + dim)
    x = torch.randn(pop, dim, generator=g).to(cuda)
    w = torch.randn(pop, generator=g).to(cuda)
    shift = torch.randn(dim, generator=g).to(cuda)
    first, second = torch.empty(dim, device=cuda), torch.empty(dim, device=cuda)
    for sh, off in ((None, -1.0), (shift, 0.0)):
        c.check(c.lib.evox_rank_weighted_moments(c.ptr(x), c.ptr(w), c.ptr(sh), off, pop, dim, c.ptr(first), c.ptr(second), c.stream_ptr(cuda)))
        xd, wd = x.double(), w.double()
        close(first, (wd[:, None] * xd).sum(0).cpu())
        dv = xd - (0 if sh is None else sh.double())
        close(second, (wd[:, None] * (dv * dv + off)).sum(0).cpu())
    if pop % 2 == 0:
        grad = torch.empty(dim, device=cuda)
        half = x[: pop // 2].contiguous()
        c.check(c.lib.evox_openes_gradient(c.ptr(half), c.ptr(w), pop, dim, pop // 2, 0.25, c.ptr(grad), c.stream_ptr(cuda)))
        close(grad, ((torch.cat([half, -half]).double().T @ w.double()) / pop / 0.25).cpu())


def make_mlp(sizes, bias, gen):
    layers = []
    for i in range(len(sizes) - 1):
        lin = nn.Linear(sizes[i], sizes[i + 1], bias=bias)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(lin.weight.shape, generator=gen) / sizes[i] ** 0.5)
            if bias:
                lin.bias.copy_(torch.randn(lin.bias.shape, generator=gen) * 0.1)
        layers.append(lin)
        if i + 2 < len(sizes):
            layers.append(nn.ReLU())
    return nn.Sequential(*layers)


@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("shared", [True, False])
def test_virtual_forward_vs_oracle(cuda, bias, shared):
    from evox_b200.problems import VirtualLoRAProblem

    gen = torch.Generator().manual_seed(3)
    sizes, pop, batch, r, sigma = [20, 33, 17, 6], 12, 9, 4, 0.1
    model = make_mlp(sizes, bias, gen)
    x = torch.randn(batch, sizes[0], generator=gen) if shared else torch.randn(pop, batch, sizes[0], generator=gen)
    prob = VirtualLoRAProblem(model, [(x, torch.zeros(batch, dtype=torch.long))], nn.CrossEntropyLoss(reduction="none"), r, device=cuda)
    center = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    seeds = torch.randint(0, 2**31, (pop,), generator=gen, dtype=torch.int64)
    got = prob._virtual_forward(x.to(cuda), center.to(cuda), seeds.to(cuda), sigma, pop)
    weights = [m.weight.detach() for m in model if isinstance(m, nn.Linear)]
    biases = [m.bias.detach() if bias else None for m in model if isinstance(m, nn.Linear)]
    h0 = x.unsqueeze(0).expand(pop, -1, -1) if shared else x
    want = lora.virtual_forward(h0, weights, biases, seeds, prob.counter_offsets, prob.param_shapes, r, sigma)
    close(got, want)
    # sigma = 0 reproduces the plain model (the reference's invariant, test_virtual_lora_problem.py:67-100)
    plain = prob._virtual_forward(x.to(cuda), center.to(cuda), seeds.to(cuda), 0.0, pop)
    close(plain, model(h0.float()).detach())


def test_virtual_lora_workflow_learns(cuda):
    """VirtualLoRAES + VirtualLoRAProblem through StdWorkflow on a tiny regression: the loss drops."""
    from evox_b200.algorithms import VirtualLoRAES
    from evox_b200.problems import VirtualLoRAProblem
    from evox_b200.transforms import CenteredRank
    from evox_b200.workflows import StdWorkflow

    assert torch.equal(CenteredRank()(torch.tensor([3.0, 1.0, 2.0])), lora.centered_rank(torch.tensor([3.0, 1.0, 2.0])))
    gen = torch.Generator().manual_seed(0)
    model = make_mlp([8, 16, 4], True, gen)
    x = torch.randn(32, 8, generator=gen)
    y = torch.randn(32, 4, generator=gen)
    prob = VirtualLoRAProblem(model, [(x, y)], nn.MSELoss(reduction="none"), 2, device=cuda)
    center = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    torch.manual_seed(1)
    algo = VirtualLoRAES(prob.param_shapes, 2, 64, center, 0.02, 0.05, device=cuda)
    wf = StdWorkflow(algo, prob, device=cuda, fitness_transform=CenteredRank())

    def loss_of(c):
        return float(prob.evaluate((c, torch.zeros(1, dtype=torch.int64, device=cuda), 0.0))[0])

    before = loss_of(wf.algorithm.center)
    for _ in range(100):
        wf.step()
    after = loss_of(wf.algorithm.center)
    assert after < before, (before, after)
