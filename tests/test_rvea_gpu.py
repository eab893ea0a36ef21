"""Parity of the CUDA RVEA selection with the reference's recorded outputs and the oracle.

Selected rows are compared as indices. The kernel's cosine, arccos and norm differ from ATen's
CPU routines in the last bits, and association / argmin are discontinuous, so a differing index
is accepted only when it is a genuine near-tie: the reference's own APD of the kernel's choice
is within 1e-5 relative of the reference's minimum for that vector (or the individual sits
within 1e-5 relative of the boundary between two vectors' angles). The number of such cases is
printed; gathered rows must then equal the chosen rows bit for bit.
"""
import pytest
import torch

from oracle import rvea

pytestmark = pytest.mark.gpu


def check_against_oracle(x, f, v, theta, got_x, got_f, got_idx):
    o = rvea.ref_vec_guided(x, f, v, theta)
    got_idx = got_idx.cpu()
    want_idx = o["next_ind"]
    near = 0
    for j in range(v.shape[0]):
        gi, wi = int(got_idx[j]), int(want_idx[j])
        if gi == wi:
            continue
        near += 1
        angle, apd = o["angle"], o["apd"]
        if gi >= 0 and wi >= 0:
            a, b = float(apd[gi, j]), float(apd[wi, j])
            if a != float("inf"):
                assert abs(a - b) <= 1e-5 * abs(b), f"vector {j}: rows {gi} / {wi} have APD {a} / {b}"
                continue
        # association flipped: the row's two best angles must be a near-tie
        rows = [r for r in (gi, wi) if r >= 0]
        for r in rows:
            two = torch.topk(angle[r], 2, largest=False)[0]
            assert float(two[1] - two[0]) <= 1e-5 * float(two[1]), f"vector {j}: row {r} is not a near-tie"
    # gathered rows are exactly the chosen rows
    for j in range(v.shape[0]):
        gi = int(got_idx[j])
        if gi < 0:
            assert torch.isnan(got_x[j]).all() and torch.isnan(got_f[j]).all()
        else:
            assert torch.equal(got_x[j].cpu(), x[gi]) and torch.equal(got_f[j].cpu(), f[gi])
    return near


@pytest.mark.parametrize("case", ["unit", "m10", "m3"])
def test_golden(golden, cuda, case):
    from evox_b200.operators.selection import ref_vec_guided

    g = golden("rvea")
    x, f, v, theta = (torch.from_numpy(g[f"{case}_{k}"]) for k in ("x", "f", "v", "theta"))
    nx, nf, idx = ref_vec_guided(x.to(cuda), f.to(cuda), v.to(cuda), theta.to(cuda), return_index=True)
    near = check_against_oracle(x, f, v, theta, nx, nf, idx)
    want_x = torch.from_numpy(g[f"{case}_next_x"])
    if near == 0:
        assert torch.equal(torch.nan_to_num(nx.cpu(), nan=-1.0), torch.nan_to_num(want_x, nan=-1.0))
    print(f"{case}: {near} near-tie differences")


@pytest.mark.parametrize("n,m,nv_h", [(5000, 10, (3, 2)), (3000, 3, (12, 0)), (257, 5, (4, 3)), (1, 4, (3, 0)), (40, 16, (2, 1))])
def test_vs_oracle(cuda, n, m, nv_h):
    from evox_b200.operators.selection import ref_vec_guided

    g = torch.Generator().manual_seed(n + m)
    f = torch.rand(n, m, generator=g) + 0.05 * torch.randn(n, m, generator=g).abs()
    if n > 100:
        f[11] = float("nan")
        f[50, m - 1] = float("nan")
    x = torch.rand(n, 9, generator=g)
    v = rvea.two_layer_vectors(nv_h[0], nv_h[1], m)
    theta = torch.tensor(0.36)
    nx, nf, idx = ref_vec_guided(x.to(cuda), f.to(cuda), v.to(cuda), theta.to(cuda), return_index=True)
    near = check_against_oracle(x, f, v, theta, nx, nf, idx)
    assert near <= max(1, v.shape[0] // 50)


def test_config2_full_size(cuda):
    """benchmark configuration 2: 50,000 x 10 objectives, 275 vectors, theta = 0.25."""
    from evox_b200.operators.selection import ref_vec_guided

    x, f, v, theta = rvea.config2_inputs()
    nx, nf, idx = ref_vec_guided(x.to(cuda), f.to(cuda), v.to(cuda), theta.to(cuda), return_index=True)
    near = check_against_oracle(x, f, v, theta, nx, nf, idx)
    print(f"configs[2]: {near} near-tie differences of 275 vectors")
    assert near <= 3


def test_float_theta_and_shapes(cuda):
    from evox_b200 import _cabi
    from evox_b200.operators.selection import ref_vec_guided

    x, f, v, _ = rvea.config2_inputs(n=100)
    nx, nf = ref_vec_guided(x.to(cuda), f.to(cuda), v.to(cuda), 0.25)
    assert nx.shape == (275, 19) and nf.shape == (275, 10)
    with pytest.raises(_cabi.EvoxKernelError):
        ref_vec_guided(x.to(cuda), f.to(cuda), v[:, :5].to(cuda), 0.25)


def test_sharded_phases_equal_single_call(cuda):
    """Two row shards emulated on one GPU: ideal point and packed winners merged by minimum, gathered
    rows by sum — exactly what the NCCL reductions do — reproduce the single call bit for bit."""
    from evox_b200 import _cabi as c
    from evox_b200.operators.selection import ref_vec_guided, ref_vec_guided_sharded

    x, f, v, theta = rvea.config2_inputs(n=7001)
    f[5] = float("nan")
    xd, fd, vd, td = x.to(cuda), f.to(cuda), v.to(cuda), theta.to(cuda)
    want_x, want_f, want_i = ref_vec_guided(xd, fd, vd, td, return_index=True)
    # world size 1 through the sharded entry point
    got = ref_vec_guided_sharded(xd, fd, vd, td, 0, return_index=True)
    assert torch.equal(got[2], want_i)
    assert torch.equal(torch.nan_to_num(got[0], nan=-1.0), torch.nan_to_num(want_x, nan=-1.0))
    # two shards by hand
    n, m, nv, dx = 7001, f.shape[1], v.shape[0], x.shape[1]
    bounds = [(0, 3000), (3000, n)]
    parts = []
    for a, b in bounds:
        xs, fs = xd[a:b].contiguous(), fd[a:b].contiguous()
        ws = torch.empty(c.lib.evox_rvea_workspace_bytes(b - a, m, nv), dtype=torch.uint8, device=cuda)
        parts.append(dict(x=xs, f=fs, ws=ws, a=a, n=b - a, ideal=torch.empty(m, device=cuda), keys=torch.empty(nv, dtype=torch.int64, device=cuda),
                          nx=torch.empty(nv, dx, device=cuda), nf=torch.empty(nv, m, device=cuda), ni=torch.empty(nv, dtype=torch.int64, device=cuda)))

    def phase(k, p):
        c.check(c.lib.evox_ref_vec_guided_phase(k, c.ptr(p["x"]), dx, c.ptr(p["f"]), p["n"], m, c.ptr(vd), nv, c.ptr(td), p["a"],
                                                c.ptr(p["ideal"]), c.ptr(p["keys"]), c.ptr(p["nx"]), c.ptr(p["nf"]), c.ptr(p["ni"]),
                                                c.ptr(p["ws"]), p["ws"].numel(), c.stream_ptr(cuda)))

    for p in parts:
        phase(1, p)
    ideal = torch.minimum(parts[0]["ideal"], parts[1]["ideal"])
    for p in parts:
        p["ideal"].copy_(ideal)
        phase(2, p)
    flip = torch.iinfo(torch.int64).min
    keys = torch.minimum(parts[0]["keys"] ^ flip, parts[1]["keys"] ^ flip) ^ flip
    for p in parts:
        p["keys"].copy_(keys)
        phase(3, p)
    torch.cuda.synchronize()
    idx = parts[0]["ni"]
    assert torch.equal(idx, parts[1]["ni"]) and torch.equal(idx, want_i)
    sx, sf = parts[0]["nx"] + parts[1]["nx"], parts[0]["nf"] + parts[1]["nf"]
    live = idx >= 0
    assert torch.equal(sx[live], want_x[live]) and torch.equal(sf[live], want_f[live])


def test_exact_ties_take_the_reference_order(cuda):
    """Individuals that sit exactly between reference vectors (equal cosines, equal angles): the kernel's
    shortcut — associate with the largest cosine when it is clearly the largest — must not apply, and the
    first-minimum rule of torch.argmin decides (rvea_selection.py:82). Also vectors with negative components,
    whose cosines are clamped to 0: every such vector then has the same angle pi / 2."""
    from evox_b200.operators.selection import ref_vec_guided

    v = torch.tensor([[1.0, 0.0, 0.0], [0.0, 1.0, 0.0], [0.0, 0.0, 1.0], [1.0, 1.0, 0.0], [1.0, 0.0, 1.0]])
    f = torch.tensor([[1.0, 1.0, 1.0], [2.0, 2.0, 2.0], [1.0, 1.0, 0.0], [3.0, 3.0, 5.0], [0.5, 0.25, 0.25], [1.0, 0.0, 0.0],
                      [0.0, 1.0, 0.0], [4.0, 4.0, 0.0]]) + 1.0
    x = torch.arange(f.shape[0] * 2, dtype=torch.float32).reshape(-1, 2)
    for theta in (0.0, 0.25):
        nx, nf, idx = ref_vec_guided(x.to(cuda), f.to(cuda), v.to(cuda), torch.tensor(theta).to(cuda), return_index=True)
        o = rvea.ref_vec_guided(x, f, v, torch.tensor(theta))
        assert torch.equal(idx.cpu(), o["next_ind"]), theta
    # reference vectors pointing away from every individual: all cosines negative
    v2 = torch.tensor([[-1.0, -0.5, -0.2], [-0.3, -1.0, -0.1], [-0.2, -0.2, -1.0]])
    nx, nf, idx = ref_vec_guided(x.to(cuda), f.to(cuda), v2.to(cuda), torch.tensor(0.5).to(cuda), return_index=True)
    o = rvea.ref_vec_guided(x, f, v2, torch.tensor(0.5))
    assert torch.equal(idx.cpu(), o["next_ind"])


def test_derived_vectors_are_reused_only_for_the_same_vectors(cuda):
    """The unit vectors and gamma stay in the workspace between calls with the same reference-vector tensor; an
    in-place change of that tensor, or another tensor, must be seen."""
    from evox_b200.operators.selection import ref_vec_guided

    x, f, v, theta = rvea.config2_inputs(n=4000)
    xd, fd, td = x.to(cuda), f.to(cuda), theta.to(cuda)
    vd = v.to(cuda)
    first = ref_vec_guided(xd, fd, vd, td, return_index=True)[2].clone()
    again = ref_vec_guided(xd, fd, vd, td, return_index=True)[2]  # served from the workspace
    assert torch.equal(first, again)
    assert torch.equal(first.cpu(), rvea.ref_vec_guided(x, f, v, theta)["next_ind"])
    v2 = v.flip(0).contiguous()
    vd.copy_(v2)  # same tensor, new contents
    got = ref_vec_guided(xd, fd, vd, td, return_index=True)[2]
    assert torch.equal(got.cpu(), rvea.ref_vec_guided(x, f, v2, theta)["next_ind"])
    v3 = (v * torch.linspace(0.5, 2.0, v.shape[1])).contiguous()
    got = ref_vec_guided(xd, fd, v3.to(cuda), td, return_index=True)[2]  # another tensor
    assert torch.equal(got.cpu(), rvea.ref_vec_guided(x, f, v3, theta)["next_ind"])
