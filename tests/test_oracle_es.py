"""The evolution-strategy oracle reproduces outputs recorded from the reference (CPU only)."""
import numpy as np
import torch

from oracle import lora


def t(a):
    return torch.from_numpy(a)


def test_philox_streams(golden):
    g = golden("es")
    seeds = t(g["seeds"])
    for key in g:
        if key.startswith("uniform_n"):
            n, c = int(key.split("_")[1][1:]), int(key.split("_c")[1])
            assert torch.equal(lora.philox_uniform(seeds, n, c), t(g[key]))
            assert torch.equal(lora.philox_normal(seeds, n, c), t(g[key.replace("uniform", "normal")]))


def test_counter_offsets_known_answer(golden):
    # the one hard-coded expectation of the reference's own test (test_lora_noise.py:111-112)
    assert lora.compute_counter_offsets([(10,), (4, 3), (2, 5)], 2) == [0, 12, 28]
    assert list(golden("es")["offsets_kat"]) == [0, 12, 28]


def test_factors_delta_gradient(golden):
    g = golden("es")
    seeds = t(g["seeds"])
    a, b = lora.generate_lora_factors(seeds, (12, 20), 4, 40)
    assert torch.equal(a, t(g["factors_A"])) and torch.equal(b, t(g["factors_B"]))
    assert torch.equal(lora.lora_delta_output(t(g["delta_x"]), a, b, 0.1), t(g["delta_out"]))
    fit = t(g["grad_fitness"])
    assert torch.equal(lora.lora_gradient(fit, a, b, 6, 0.1, (12, 20)), t(g["grad_out"]))
    noise = lora.generate_lora_factors(seeds, (9,), 4, 3)
    assert torch.equal(noise, t(g["bias_noise"]))
    assert torch.equal(lora.lora_gradient(fit, noise, None, 6, 0.1, (9,)), t(g["grad_bias"]))
    # the delta equals sigma * x @ (B A)^T (the reference's own check, test_lora_noise.py:168-181)
    x = t(g["delta_x"])
    explicit = 0.1 * torch.einsum("pbk,pdk->pbd", x, torch.bmm(b, a))
    assert torch.allclose(lora.lora_delta_output(x, a, b, 0.1), explicit, atol=1e-5)


def vlora_step(g, tag, opt):
    shapes = [(8, 6), (8,), (3, 8), (3,)]
    offsets = lora.compute_counter_offsets(shapes, 2)
    seeds, fit, center = t(g[f"{tag}_seeds"]), t(g[f"{tag}_fitness"]), t(g[f"{tag}_center0"])
    parts = []
    for shape, off in zip(shapes, offsets):
        f = lora.generate_lora_factors(seeds, shape, 2, off)
        if isinstance(f, tuple):
            parts.append(lora.lora_gradient(fit, f[0], f[1], 10, torch.tensor(0.1), shape).reshape(-1))
        else:
            parts.append(lora.lora_gradient(fit, f, None, 10, torch.tensor(0.1), shape).reshape(-1))
    grad = torch.cat(parts)
    if opt is None:
        return center - torch.tensor(0.05) * grad, None
    z = torch.zeros_like(center)
    return lora.adam_single_tensor(center, grad, z, z, torch.tensor(0.9), torch.tensor(0.999), torch.tensor(0.05))


def test_virtual_lora_es_step(golden):
    g = golden("es")
    new_center, _ = vlora_step(g, "vlora_None", None)
    assert torch.equal(new_center, t(g["vlora_None_center1"]))
    c, m, v = vlora_step(g, "vlora_adam", "adam")
    assert torch.equal(c, t(g["vlora_adam_center1"]))
    assert torch.equal(m, t(g["vlora_adam_exp_avg"])) and torch.equal(v, t(g["vlora_adam_exp_avg_sq"]))


def test_open_es_step(golden):
    g = golden("es")
    c0, noise = t(g["openes_None_center0"]), t(g["openes_None_noise"])
    new_center, *_ = lora.open_es_step(c0, noise, lambda pop: (pop**2).sum(dim=1), torch.tensor(0.05), torch.tensor(0.1))
    assert torch.equal(new_center, t(g["openes_None_center1"]))
    c0, noise = t(g["openes_adam_center0"]), t(g["openes_adam_noise"])
    z = torch.zeros_like(c0)
    new_center, *_ = lora.open_es_step(c0, noise, lambda pop: (pop**2).sum(dim=1), torch.tensor(0.05), torch.tensor(0.1), adam_state=(z, z))
    assert torch.equal(new_center, t(g["openes_adam_center1"]))
