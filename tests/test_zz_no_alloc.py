"""evox_nd_rank_static — the rank entry point for callers that cannot allocate device memory
(plug-ins that only own the buffers their host application passed in, loops that must not touch
the allocator while they run). It keeps its scratch in an array inside the library, so it has to
give the same ranks as evox_nd_rank, also when the array still holds a previous call's data.

This file sorts last on purpose: a run that stops at the first failure has then already
exercised every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rank_with_workspace(c, f):
    n, m = f.shape
    rank = torch.empty(n, dtype=torch.int32, device=f.device)
    status = torch.zeros(2, dtype=torch.int32, device=f.device)
    nbytes = c.lib.evox_nds_workspace_bytes(n, m)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=f.device)
    c.check(c.lib.evox_nd_rank(c.ptr(f), n, m, c.ptr(rank), c.ptr(status), c.ptr(ws), nbytes, c.stream_ptr(f.device)))
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    return rank


def _rank_static(c, f):
    n, m = f.shape
    rank = torch.full((n,), -7, dtype=torch.int32, device=f.device)
    status = torch.zeros(2, dtype=torch.int32, device=f.device)
    c.check(c.lib.evox_nd_rank_static(c.ptr(f), n, m, c.ptr(rank), c.ptr(status), c.stream_ptr(f.device)))
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    return rank


def test_static_scratch_rank_matches_workspace_rank(cuda):
    from evox_b200 import _cabi as c

    gen = torch.Generator().manual_seed(11)
    # two calls in a row on different shapes: the second one runs over the first one's leftovers
    first = (torch.round(torch.rand(3000, 3, generator=gen) * 40) / 40).to(cuda)
    second = torch.rand(517, 5, generator=gen).to(cuda)
    for f in (first, second, first):
        got = _rank_static(c, f)
        assert torch.equal(got, _rank_with_workspace(c, f))
        assert int(got.max()) > 0 and int(got.min()) == 0


@pytest.mark.parametrize("m", [16, 3])
def test_static_scratch_at_its_limits(cuda, m):
    """The largest problem the built-in array holds: 4,096 rows, with 16 objectives (the widest layout) and
    with 3 (many fronts, so the peel runs many rounds over the full-size matrix). Two calls in a row each."""
    from evox_b200 import _cabi as c

    gen = torch.Generator().manual_seed(20 + m)
    f = torch.rand(4096, m, generator=gen)
    if m == 16:
        f[:, 8:] = torch.round(f[:, 8:] * 4) / 4  # some ties, some dominance even in 16 dimensions
        f[::7] = f[::7] * 0.5
    f = f.to(cuda)
    want = _rank_with_workspace(c, f)
    for _ in range(2):
        assert torch.equal(_rank_static(c, f), want)
    assert int(want.max()) > 0


def test_static_scratch_calls_leave_the_allocator_alone(cuda):
    """After a first call (which looks the array's address up), further calls must neither take device memory
    from the driver nor from torch's caching allocator: the free memory the driver reports and the allocator's
    reserved bytes stay what they were."""
    from evox_b200 import _cabi as c

    f = torch.rand(2048, 3, generator=torch.Generator().manual_seed(3)).to(cuda)
    n, m = f.shape
    rank = torch.empty(n, dtype=torch.int32, device=cuda)
    status = torch.zeros(2, dtype=torch.int32, device=cuda)

    def call():
        c.check(c.lib.evox_nd_rank_static(c.ptr(f), n, m, c.ptr(rank), c.ptr(status), c.stream_ptr(cuda)))

    call()
    torch.cuda.synchronize()
    free0, reserved0 = torch.cuda.mem_get_info(cuda)[0], torch.cuda.memory_reserved(cuda)
    for _ in range(5):
        call()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(cuda)[0] == free0
    assert torch.cuda.memory_reserved(cuda) == reserved0
    assert int(status[0]) == 0


def test_static_scratch_rejects_oversize(cuda):
    from evox_b200 import _cabi as c

    f = torch.rand(4097, 3, device=cuda)
    rank = torch.empty(4097, dtype=torch.int32, device=cuda)
    rc = c.lib.evox_nd_rank_static(c.ptr(f), 4097, 3, c.ptr(rank), None, c.stream_ptr(cuda))
    assert rc == -1 and b"4096" in c.lib.evox_last_error()
    f = torch.rand(100, 17, device=cuda)
    rc = c.lib.evox_nd_rank_static(c.ptr(f), 100, 17, c.ptr(rank), None, c.stream_ptr(cuda))
    assert rc == -1 and b"16 objectives" in c.lib.evox_last_error()
