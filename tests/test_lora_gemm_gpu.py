"""The tensor-core (tcgen05) virtual-LoRA layer against fp32 math on the same bf16-rounded inputs.

Tolerance: 2e-2 relative to the largest output magnitude (bf16 operands, fp32 accumulation, bf16
output rounding). The kernel's error flag must stay zero (no bounded wait expired).
"""
import pytest
import torch

from oracle import lora

pytestmark = pytest.mark.gpu


def reference_layer(h, w, seeds, counter, sigma, bias, bias_counter, relu, rank=8):
    pop, batch, k = h.shape
    d = w.shape[0]
    a, b = lora.generate_lora_factors(seeds, (d, k), rank, counter)
    y = h.float() @ w.float().t() + lora.lora_delta_output(h.float(), a, b, sigma)
    if bias is not None:
        y = y + bias
        if bias_counter is not None:
            y = y + sigma * lora.generate_lora_factors(seeds, (d,), rank, bias_counter).unsqueeze(1)
    return torch.relu(y) if relu else y


def rel_err(got, want):
    return float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max())


@pytest.mark.parametrize("pop,batch,k,d,bias,relu", [
    (2, 64, 256, 256, False, False),
    (4, 64, 512, 512, True, True),
    (3, 128, 256, 768, False, True),
    (128, 64, 256, 2048, False, True),   # 256 pair tiles: every CTA pair walks several tiles and both accumulators
    (130, 64, 1024, 1024, True, True),   # 8,320 rows = 65 x 128: single-CTA tiles, 16 k-blocks through the 4-stage ring
    (64, 128, 1024, 512, True, False),   # pairs, 16 k-blocks through the 6-stage ring
])
def test_layer_vs_fp32(cuda, pop, batch, k, d, bias, relu):
    from evox_b200.lora_kernels import lora_layer_bf16

    g = torch.Generator().manual_seed(pop * 1000 + k)
    h = torch.randn(pop, batch, k, generator=g).bfloat16()
    w = (torch.randn(d, k, generator=g) / k**0.5).bfloat16()
    seeds = torch.randint(0, 2**31, (pop,), generator=g, dtype=torch.int64)
    b = torch.randn(d, generator=g) * 0.1 if bias else None
    counter, bias_counter, sigma = 40, (4096 if bias else None), 0.05
    want = reference_layer(h, w, seeds, counter, sigma, b, bias_counter, relu)
    for out_dtype in (torch.float32, torch.bfloat16):
        got = lora_layer_bf16(h.to(cuda), w.to(cuda), seeds.to(cuda), counter, sigma, bias=None if b is None else b.to(cuda),
                              bias_counter=bias_counter, relu=relu, out_dtype=out_dtype)
        torch.cuda.synchronize()
        assert int(lora_layer_bf16.last_error_flag) == 0
        assert got.dtype == out_dtype
        err = rel_err(got.float(), want)
        assert err <= (2e-2 if out_dtype == torch.bfloat16 else 5e-3), err
    # without the correction: the plain product
    plain = lora_layer_bf16(h.to(cuda), w.to(cuda), seeds.to(cuda), counter, 0.0, out_dtype=torch.float32, lora=False)
    assert rel_err(plain, h.float() @ w.float().t()) <= 1e-3


@pytest.mark.parametrize("pop", [6, 8])  # 384 rows: one CTA per tile; 512 rows: CTA pairs
def test_fused_negative_mse(cuda, pop):
    from evox_b200.lora_kernels import lora_layer_bf16

    g = torch.Generator().manual_seed(5)
    batch, k, d = 64, 256, 512
    h = torch.randn(pop, batch, k, generator=g).bfloat16()
    w = (torch.randn(d, k, generator=g) / k**0.5).bfloat16()
    seeds = torch.randint(0, 2**31, (pop,), generator=g, dtype=torch.int64)
    target = torch.randn(batch, d, generator=g)
    want = -((reference_layer(h, w, seeds, 8, 0.02, None, None, False) - target) ** 2).mean(dim=(1, 2))
    got = lora_layer_bf16(h.to(cuda), w.to(cuda), seeds.to(cuda), 8, 0.02, target=target.to(cuda))
    torch.cuda.synchronize()
    assert int(lora_layer_bf16.last_error_flag) == 0
    assert rel_err(got, want) <= 2e-3


def test_unsupported_shape_is_rejected(cuda):
    from evox_b200 import _cabi
    from evox_b200.lora_kernels import lora_layer_bf16

    h = torch.zeros(2, 48, 256, dtype=torch.bfloat16, device=cuda)
    w = torch.zeros(256, 256, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(_cabi.EvoxKernelError):
        lora_layer_bf16(h, w, torch.zeros(2, dtype=torch.int64, device=cuda), 0, 0.1)


@pytest.mark.parametrize("pop,d,k", [(8, 128, 256), (64, 256, 512), (256, 512, 256), (1024, 256, 512)])
def test_tensor_core_gradient_vs_fp32(cuda, pop, d, k):
    """Split-precision tensor-core gradient against the fp32 einsum: 1e-5 of the largest entry."""
    from evox_b200.lora_kernels import lora_gradient_from_seeds

    g = torch.Generator().manual_seed(d + k)
    seeds = torch.randint(0, 2**31, (pop,), generator=g, dtype=torch.int64)
    fit = torch.rand(pop, generator=g) - 0.5
    a, b = lora.generate_lora_factors(seeds, (d, k), 8, 24)
    want = torch.einsum("i,ijk,ikl->jl", fit.double(), b.double(), a.double()) / (pop * 0.02)
    got = lora_gradient_from_seeds(fit.to(cuda), seeds.to(cuda), (d, k), 8, 24, pop, 0.02)
    torch.cuda.synchronize()
    assert int(lora_gradient_from_seeds.last_error_flag) == 0
    assert rel_err(got, want) <= 1e-5
    # the three-piece bf16 scheme (twice the work) and the single bf16 pass
    got6 = lora_gradient_from_seeds(fit.to(cuda), seeds.to(cuda), (d, k), 8, 24, pop, 0.02, passes=6)
    got1 = lora_gradient_from_seeds(fit.to(cuda), seeds.to(cuda), (d, k), 8, 24, pop, 0.02, passes=1)
    assert rel_err(got6, want) <= 1e-5 and rel_err(got1, want) <= 2e-2
    # fitness of any magnitude: the fp16 pieces are formed after a power-of-two normalisation
    for scale in (3.0e7, 1.0e-9):
        got_s = lora_gradient_from_seeds((fit * scale).to(cuda), seeds.to(cuda), (d, k), 8, 24, pop, 0.02)
        assert rel_err(got_s, want * scale) <= 1e-5


def test_problem_bf16_path_with_fused_mse(cuda):
    """VirtualLoRAProblem(compute_dtype=bf16): three tensor-core layers, the last one reducing the
    squared error in its epilogue, against the fp32 oracle forward on the bf16-rounded operands."""
    from torch import nn

    from evox_b200.problems import VirtualLoRAProblem

    g = torch.Generator().manual_seed(9)
    pop, batch, width, rank, sigma = 4, 64, 256, 8, 0.05
    layers = []
    for i in range(3):
        lin = nn.Linear(width, width, bias=False)
        with torch.no_grad():
            lin.weight.copy_((torch.randn(width, width, generator=g) / width**0.5).bfloat16().float())
        layers += [lin] + ([nn.ReLU()] if i < 2 else [])
    model = nn.Sequential(*layers)
    x = torch.randn(pop, batch, width, generator=g).bfloat16()
    target = torch.randn(batch, width, generator=g)
    prob = VirtualLoRAProblem(model, [(x, target)], nn.MSELoss(reduction="none"), rank, device=cuda, compute_dtype=torch.bfloat16)
    center = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    seeds = torch.randint(0, 2**31, (pop,), generator=g, dtype=torch.int64)
    got = prob.evaluate((center.to(cuda), seeds.to(cuda), sigma))
    weights = [m.weight.detach() for m in model if isinstance(m, nn.Linear)]
    # the oracle keeps activations in fp32; the kernel rounds them to bf16 between layers
    out = lora.virtual_forward(x.float(), weights, [None] * 3, seeds, prob.counter_offsets, prob.param_shapes, rank, sigma)
    want = ((out - target) ** 2).mean(dim=(1, 2))
    assert got.shape == (pop,)
    assert rel_err(got, want) <= 2e-2


@pytest.mark.parametrize("pop", [6, 8])
def test_fused_next_layer_projection(cuda, pop):
    """The epilogue's projection for the next layer equals the standalone projection kernel run on
    the bf16 output (same factors, fp32 accumulation; only the summation order differs)."""
    from evox_b200 import _cabi
    from evox_b200.lora_kernels import lora_layer_bf16

    g = torch.Generator().manual_seed(17)
    batch, k, d = 64, 256, 512
    h = torch.randn(pop, batch, k, generator=g).bfloat16().to(cuda)
    w = (torch.randn(d, k, generator=g) / k**0.5).bfloat16().to(cuda)
    seeds = torch.randint(0, 2**31, (pop,), generator=g, dtype=torch.int64).to(cuda)
    next_counter = 123456
    y, t_next = lora_layer_bf16(h, w, seeds, 40, 0.05, relu=True, next_counter=next_counter)
    torch.cuda.synchronize()
    assert int(lora_layer_bf16.last_error_flag) == 0
    want = torch.empty(pop, batch, 8, dtype=torch.float32, device=cuda)
    _cabi.check(_cabi.lib.evox_lora_down_bf16(_cabi.ptr(y), _cabi.ptr(seeds), next_counter, pop, batch, d, 8, _cabi.ptr(want),
                                              _cabi.stream_ptr(cuda)))
    assert rel_err(t_next, want.cpu()) <= 1e-4
    # and against the oracle's factors
    a, _ = lora.generate_lora_factors(seeds.cpu(), (d, d), 8, next_counter)
    ref = torch.bmm(y.float().cpu(), a.transpose(1, 2))
    assert rel_err(t_next, ref) <= 1e-4


# ---------------------------------------------------------------------------------------------
# The layer shape of the virtual-LoRA benchmark configuration: K = N = 4096 (64 k-blocks per tile,
# 16 column tiles, 32 slices of the fused next-layer projection), few individuals so that the fp32
# oracle stays cheap.
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("pop", [8, 6])  # 512 rows: CTA pairs; 384 rows: single-CTA tiles
def test_layer_at_benchmark_width(cuda, pop):
    from evox_b200.lora_kernels import lora_layer_bf16

    g = torch.Generator().manual_seed(4096 + pop)
    batch, k, d, sigma, counter, next_counter = 64, 4096, 4096, 0.02, 65536, 131072
    h = torch.randn(pop, batch, k, generator=g).bfloat16()
    w = (torch.randn(d, k, generator=g) / k**0.5).bfloat16()
    seeds = torch.randint(0, 2**31, (pop,), generator=g, dtype=torch.int64)
    want = reference_layer(h, w, seeds, counter, sigma, None, None, True)
    y, t_next = lora_layer_bf16(h.to(cuda), w.to(cuda), seeds.to(cuda), counter, sigma, relu=True, next_counter=next_counter)
    torch.cuda.synchronize()
    assert int(lora_layer_bf16.last_error_flag) == 0
    assert rel_err(y.float(), want) <= 2e-2
    # the projection for the next layer, from the bf16 activations the kernel stored
    a, _ = lora.generate_lora_factors(seeds, (d, d), 8, next_counter)
    assert rel_err(t_next, torch.bmm(y.float().cpu(), a.transpose(1, 2))) <= 1e-4
    # fused squared error of a last layer of that width
    target = torch.randn(batch, d, generator=g)
    want_mse = -((reference_layer(h, w, seeds, counter, sigma, None, None, False) - target) ** 2).mean(dim=(1, 2))
    got_mse = lora_layer_bf16(h.to(cuda), w.to(cuda), seeds.to(cuda), counter, sigma, target=target.to(cuda))
    torch.cuda.synchronize()
    assert int(lora_layer_bf16.last_error_flag) == 0
    assert rel_err(got_mse, want_mse) <= 2e-3


def test_problem_at_benchmark_width(cuda):
    """Three 4096 -> 4096 layers with ReLU between them, eight individuals with their own 64 x 4096 batch, the
    squared error reduced in the last layer's epilogue: the benchmark configuration's network, against the fp32
    oracle forward on the same bf16-rounded operands (2e-2 relative on the fitness)."""
    from torch import nn

    from evox_b200.lora_kernels import lora_layer_bf16
    from evox_b200.problems import VirtualLoRAProblem

    g = torch.Generator().manual_seed(11)
    pop, batch, width, rank, sigma = 8, 64, 4096, 8, 0.02
    layers = []
    for i in range(3):
        lin = nn.Linear(width, width, bias=False)
        with torch.no_grad():
            lin.weight.copy_((torch.randn(width, width, generator=g) / width**0.5).bfloat16().float())
        layers += [lin] + ([nn.ReLU()] if i < 2 else [])
    model = nn.Sequential(*layers)
    x = torch.randn(pop, batch, width, generator=g).bfloat16()
    target = torch.randn(batch, width, generator=g)
    prob = VirtualLoRAProblem(model, [(x, target)], nn.MSELoss(reduction="none"), rank, device=cuda, compute_dtype=torch.bfloat16)
    center = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    seeds = torch.randint(0, 2**31, (pop,), generator=g, dtype=torch.int64)
    got = prob.evaluate((center.to(cuda), seeds.to(cuda), sigma))
    torch.cuda.synchronize()
    assert int(lora_layer_bf16.last_error_flag) == 0
    weights = [m.weight.detach() for m in model if isinstance(m, nn.Linear)]
    out = lora.virtual_forward(x.float(), weights, [None] * 3, seeds, prob.counter_offsets, prob.param_shapes, rank, sigma)
    want = ((out - target) ** 2).mean(dim=(1, 2))
    assert got.shape == (pop,)
    assert rel_err(got, want) <= 2e-2


def test_tensor_core_gradient_at_benchmark_block(cuda):
    """One full 4096 x 4096 gradient block at 1,024 individuals — 256 pair tiles walked by 74 CTA pairs over
    several waves, the long K split between two work items per tile — against the fp64 einsum
    (lora_noise.py:188-196) on 320 sampled rows: 1e-5 of the largest entry."""
    from evox_b200.lora_kernels import lora_gradient_from_seeds

    g = torch.Generator().manual_seed(77)
    pop, d, k, counter, sigma = 1024, 4096, 4096, 65536, 0.02
    seeds = torch.randint(0, 2**31, (pop,), generator=g, dtype=torch.int64)
    fit = torch.rand(pop, generator=g) - 0.5
    got = lora_gradient_from_seeds(fit.to(cuda), seeds.to(cuda), (d, k), 8, counter, pop, sigma)
    torch.cuda.synchronize()
    assert int(lora_gradient_from_seeds.last_error_flag) == 0
    assert got.shape == (d, k)
    a, b = lora.generate_lora_factors(seeds, (d, k), 8, counter)
    # rows from every 256-row tile, first and last rows of tiles included
    rows = torch.cat([torch.arange(0, d, 256), torch.arange(255, d, 256), torch.randint(0, d, (288,), generator=g)]).unique()
    fb = (fit.double()[:, None, None] * b[:, rows, :].double()).permute(1, 0, 2).reshape(rows.numel(), pop * 8)
    want = fb @ a.double().reshape(pop * 8, k) / (pop * sigma)
    err = float((got[rows.to(cuda)].double().cpu() - want).abs().max() / want.abs().max())
    assert err <= 1e-5, err


@pytest.mark.parametrize("pop,d,k,parts", [(64, 2048, 2048, 8), (1024, 4096, 4096, 8), (16, 512, 512, 2)])
def test_row_shards_of_a_gradient_block_give_the_whole_block_bit_for_bit(cuda, pop, d, k, parts):
    """A GPU of a sharded VirtualLoRAES computes its rows of every gradient block; the launch then has a
    different number of tiles than the whole block's, and may divide a tile's chunk list between one or two
    work items differently. The chunk sums are always combined as the same two rounded halves, so the rows
    must equal the whole block's rows exactly — which is what lets the sharded centre equal the single-GPU one."""
    from evox_b200.lora_kernels import lora_gradient_from_seeds

    g = torch.Generator().manual_seed(pop + d)
    seeds = torch.randint(0, 2**31, (pop,), generator=g, dtype=torch.int64).to(cuda)
    fit = (torch.rand(pop, generator=g) - 0.5).to(cuda)
    whole = lora_gradient_from_seeds(fit, seeds, (d, k), 8, 40, pop, 0.02).clone()
    step = d // parts
    for i in range(parts):
        part = lora_gradient_from_seeds(fit, seeds, (d, k), 8, 40, pop, 0.02, rows=(i * step, (i + 1) * step))
        assert torch.equal(part, whole[i * step:(i + 1) * step]), i
    torch.cuda.synchronize()
    assert int(lora_gradient_from_seeds.last_error_flag) == 0
