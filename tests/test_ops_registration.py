"""torch.ops.evox_b200.*: registered, traceable with fake tensors on a machine without a GPU,
and (on a GPU) equal to the plain wrappers."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode


def test_ops_are_registered_with_fake_kernels():
    import evox_b200.ops  # noqa: F401

    for name in ("nd_rank", "crowding_distance", "nd_environmental_selection", "ref_vec_guided", "philox_uniform",
                 "philox_normal", "lora_delta_output", "lora_gradient"):
        assert hasattr(torch.ops.evox_b200, name)
    with FakeTensorMode():
        f = torch.empty(100, 3)
        assert torch.ops.evox_b200.nd_rank(f).shape == (100,)
        x = torch.empty(100, 7)
        sx, sf, sr, sc = torch.ops.evox_b200.nd_environmental_selection(x, f, 40)
        assert sx.shape == (40, 7) and sf.shape == (40, 3) and sr.dtype == torch.int32 and sc.shape == (40,)
        nx, nf = torch.ops.evox_b200.ref_vec_guided(x, f, torch.empty(9, 3), torch.empty(()))
        assert nx.shape == (9, 7) and nf.shape == (9, 3)
        seeds = torch.empty(5, dtype=torch.int64)
        assert torch.ops.evox_b200.philox_normal(seeds, 33, 4).shape == (5, 33)


def test_no_cpu_kernel():
    import evox_b200.ops  # noqa: F401

    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.evox_b200.nd_rank(torch.rand(10, 2))


@pytest.mark.gpu
def test_ops_match_wrappers(cuda):
    import evox_b200.ops  # noqa: F401
    from evox_b200.lora_kernels import philox_uniform
    from evox_b200.operators.selection import non_dominate_rank

    f = torch.rand(500, 3, device=cuda)
    assert torch.equal(torch.ops.evox_b200.nd_rank(f), non_dominate_rank(f))
    seeds = torch.arange(7, dtype=torch.int64, device=cuda)
    assert torch.equal(torch.ops.evox_b200.philox_uniform(seeds, 10, 3), philox_uniform(seeds, 10, 3))
    torch.library.opcheck(torch.ops.evox_b200.nd_rank.default, (f,), test_utils=("test_schema", "test_faketensor"))


@pytest.mark.gpu
def test_ops_under_vmap(cuda):
    """torch.vmap over a batch of independent problems: one kernel call per slice, results stacked."""
    import evox_b200.ops  # noqa: F401
    from evox_b200.operators.selection import non_dominate_rank, ref_vec_guided

    g = torch.Generator().manual_seed(0)
    f = torch.rand(4, 300, 3, generator=g).to(cuda)
    ranks = torch.vmap(torch.ops.evox_b200.nd_rank)(f)
    assert ranks.shape == (4, 300)
    for i in range(4):
        assert torch.equal(ranks[i], non_dominate_rank(f[i]))
    # a batched and an unbatched argument together; several outputs
    x = torch.rand(4, 300, 6, generator=g).to(cuda)
    v = torch.rand(10, 3, generator=g).to(cuda)
    theta = torch.tensor(0.3, device=cuda)
    nx, nf = torch.vmap(torch.ops.evox_b200.ref_vec_guided, in_dims=(0, 0, None, None))(x, f, v, theta)
    assert nx.shape == (4, 10, 6) and nf.shape == (4, 10, 3)
    for i in range(4):
        wx, wf = ref_vec_guided(x[i], f[i], v, theta)
        assert torch.equal(torch.nan_to_num(nx[i]), torch.nan_to_num(wx)) and torch.equal(torch.nan_to_num(nf[i]), torch.nan_to_num(wf))
    seeds = torch.arange(12, dtype=torch.int64, device=cuda).view(3, 4)
    u = torch.vmap(lambda s: torch.ops.evox_b200.philox_uniform(s, 8, 2))(seeds)
    assert u.shape == (3, 4, 8)
