"""Parity of the CUDA particle-swarm path with the reference's recorded states and the oracle.

Tolerances: elementwise state (pop, velocity, personal / global best locations) must be
bit-exact, because the kernel performs the same separately rounded fp32 operations as the
reference. Fitness values differ only by summation order and device libm: relative 1e-5, and
for Rastrigin |diff| <= 1e-5 * max(|ref|, 10 * dim) because 10*d + sum(...) cancels near the optimum.
"""
import math

import numpy as np
import pytest
import torch

from oracle import pso as opso

pytestmark = pytest.mark.gpu

NAMES = ["pop", "velocity", "fit", "local_best_location", "local_best_fit", "global_best_location", "global_best_fit"]
FIT_ID = {"ackley": 0, "rastrigin": 1, "sphere": 2}
PARAMS = {"ackley": (20.0, 0.2, 2 * math.pi), "rastrigin": (0.0, 0.0, 0.0), "sphere": (0.0, 0.0, 0.0)}


def assert_fitness_close(got, ref, prob, dim):
    got, ref = got.double().cpu(), ref.double().cpu()
    scale = ref.abs()
    if prob == "rastrigin":
        scale = torch.maximum(scale, torch.tensor(10.0 * dim, dtype=torch.float64))
    finite = torch.isfinite(ref)
    assert torch.equal(torch.isfinite(got), finite)
    err = ((got - ref).abs() / scale.clamp_min(1e-30))[finite]
    assert err.numel() == 0 or err.max().item() <= 1e-5, f"max rel err {err.max().item():.3e}"


class Swarm:
    """Device copy of a reference-format state + the raw C-ABI calls on it."""

    def __init__(self, state: dict, dev):
        from evox_b200 import _cabi

        self.c = _cabi
        self.dev = dev
        self.t = {k: v.to(dev).contiguous().clone() for k, v in state.items()}
        self.P, self.d = self.t["pop"].shape
        n = _cabi.lib.evox_pso_workspace_bytes(self.P, self.d)
        self.ws = torch.zeros(n, dtype=torch.uint8, device=dev)

    def p(self, k):
        return self.c.ptr(self.t[k], torch.float32, k)

    def step(self, prob, rg=None, rp=None, seed=0, generation=0):
        c = self.c
        rg_d = None if rg is None else rg.to(self.dev).contiguous()
        rp_d = None if rp is None else rp.to(self.dev).contiguous()
        c.check(
            c.lib.evox_pso_step(
                self.p("pop"), self.p("velocity"), self.p("local_best_location"), self.p("local_best_fit"),
                self.p("fit"), self.p("global_best_location"), self.p("global_best_fit"), self.p("lb"), self.p("ub"),
                self.p("w"), self.p("phi_p"), self.p("phi_g"), c.ptr(rg_d), c.ptr(rp_d), self.P, self.d,
                FIT_ID[prob], c.host_floats(PARAMS[prob]), seed, generation, c.ptr(self.ws), self.ws.numel(),
                c.stream_ptr(self.dev),
            )
        )
        torch.cuda.synchronize()

    def local_best(self, record, row_offset=0):
        c = self.c
        c.check(c.lib.evox_pso_local_best(self.p("fit"), self.p("pop"), self.P, self.d, row_offset, c.ptr(record),
                                          c.ptr(self.ws), self.ws.numel(), c.stream_ptr(self.dev)))

    def generation(self, prob, records, n_records, out, rg=None, rp=None, seed=0, generation=0, row_offset=0):
        """evox_pso_generation: fold `records`, move, leave this shard's next record in `out`."""
        c = self.c
        rg_d = None if rg is None else rg.to(self.dev).contiguous()
        rp_d = None if rp is None else rp.to(self.dev).contiguous()
        c.check(
            c.lib.evox_pso_generation(
                self.p("pop"), self.p("velocity"), self.p("local_best_location"), self.p("local_best_fit"),
                self.p("fit"), self.p("global_best_location"), self.p("global_best_fit"), self.p("lb"), self.p("ub"),
                self.p("w"), self.p("phi_p"), self.p("phi_g"), c.ptr(rg_d), c.ptr(rp_d), self.P, self.d,
                FIT_ID[prob], c.host_floats(PARAMS[prob]), seed, generation, row_offset, c.ptr(records), n_records,
                c.ptr(out), c.ptr(self.ws), self.ws.numel(), c.stream_ptr(self.dev),
            )
        )
        torch.cuda.synchronize()

    def generation_peer(self, prob, buffers, rank, tag, status, rg=None, rp=None, seed=0, generation=0, row_offset=0):
        """evox_pso_generation_peer: records come from and go to the ranks' exchange buffers."""
        import ctypes

        c = self.c
        rg_d = None if rg is None else rg.to(self.dev).contiguous()
        rp_d = None if rp is None else rp.to(self.dev).contiguous()
        ptrs = (ctypes.c_uint64 * len(buffers))(*[b.data_ptr() for b in buffers])
        c.check(
            c.lib.evox_pso_generation_peer(
                self.p("pop"), self.p("velocity"), self.p("local_best_location"), self.p("local_best_fit"),
                self.p("fit"), self.p("global_best_location"), self.p("global_best_fit"), self.p("lb"), self.p("ub"),
                self.p("w"), self.p("phi_p"), self.p("phi_g"), c.ptr(rg_d), c.ptr(rp_d), self.P, self.d,
                FIT_ID[prob], c.host_floats(PARAMS[prob]), seed, generation, row_offset, ptrs, len(buffers), rank,
                tag, c.ptr(status), c.ptr(self.ws), self.ws.numel(), c.stream_ptr(self.dev),
            )
        )
        torch.cuda.synchronize()

    def init_step(self, prob):
        c = self.c
        c.check(
            c.lib.evox_pso_init_step(
                self.p("pop"), self.p("fit"), self.p("local_best_fit"), self.p("global_best_location"),
                self.p("global_best_fit"), self.P, self.d, FIT_ID[prob], c.host_floats(PARAMS[prob]),
                c.ptr(self.ws), self.ws.numel(), c.stream_ptr(self.dev),
            )
        )
        torch.cuda.synchronize()


def load_state(g, tag, k):
    s = {n: torch.from_numpy(g[f"{tag}_s{k}_{n}"]) for n in NAMES}
    lo, hi = g[f"{tag}_bounds"]
    dim = s["pop"].shape[1]
    s["lb"] = torch.full((1, dim), float(lo))
    s["ub"] = torch.full((1, dim), float(hi))
    w, pp, pg = g[f"{tag}_hyper"]
    s["w"], s["phi_p"], s["phi_g"] = torch.tensor(w), torch.tensor(pp), torch.tensor(pg)
    return s


def compare_states(got: dict, want: dict, prob: str, exact_fit_inputs=True):
    dim = want["pop"].shape[1]
    for n in ("pop", "velocity", "local_best_location", "global_best_location"):
        assert torch.equal(got[n].cpu(), want[n]), f"{n} differs"
    for n in ("fit", "local_best_fit", "global_best_fit"):
        assert_fitness_close(got[n], want[n], prob, dim)


@pytest.mark.parametrize("prob", ["ackley", "rastrigin"])
@pytest.mark.parametrize("dim", [12, 10])
def test_golden_states(golden, cuda, prob, dim):
    """init_step and three teacher-forced steps against states recorded from the reference."""
    g = golden("pso")
    tag = f"pso_{prob}_d{dim}"
    sw = Swarm(load_state(g, tag, 0), cuda)
    sw.init_step(prob)
    compare_states(sw.t, load_state(g, tag, 1), prob)
    for gen in range(3):
        sw = Swarm(load_state(g, tag, gen + 1), cuda)
        rg = torch.from_numpy(g[f"{tag}_g{gen}_rg"])
        rp = torch.from_numpy(g[f"{tag}_g{gen}_rp"])
        sw.step(prob, rg, rp)
        compare_states(sw.t, load_state(g, tag, gen + 2), prob)


@pytest.mark.parametrize("shape", [(3, 4), (65, 10), (257, 500), (33, 1001), (1, 1)])
@pytest.mark.parametrize("which", [0, 1])
def test_fill_uniform_bit_exact(cuda, shape, which):
    from evox_b200 import _cabi

    P, d = shape
    out = torch.empty(P, d, device=cuda)
    seed, gen, off = 0x1234567890ABCDEF, (5 << 32) + 17, 1000003
    _cabi.check(_cabi.lib.evox_pso_fill_uniform(_cabi.ptr(out), P, d, seed, gen, which, off, _cabi.stream_ptr(cuda)))
    ref = opso.pso_uniform(P, d, seed, gen, which, off)
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("prob", ["ackley", "rastrigin", "sphere"])
@pytest.mark.parametrize("shape", [(1000, 500), (128, 1000), (77, 10), (5, 3)])
def test_eval_fitness(cuda, prob, shape):
    from evox_b200.problems import numerical

    P, d = shape
    lo, hi = (-32.768, 32.768) if prob == "ackley" else (-5.12, 5.12)
    x = lo + (hi - lo) * torch.rand(P, d, generator=torch.Generator().manual_seed(3))
    x[0] = 0.0  # the optimum, where Rastrigin cancels completely
    cls = {"ackley": numerical.Ackley, "rastrigin": numerical.Rastrigin, "sphere": numerical.Sphere}[prob]
    got = cls().evaluate(x.to(cuda))
    assert_fitness_close(got, opso.FITNESS[prob](x), prob, d)


@pytest.mark.parametrize("prob,P,d", [("ackley", 10_000, 500), ("rastrigin", 4096, 1000), ("ackley", 999, 10)])
def test_step_vs_oracle(cuda, prob, P, d):
    """One teacher-forced generation at benchmark shapes: tensor mode, then Philox mode fed
    with the tensors evox_pso_fill_uniform materialises."""
    lo, hi = (-32.768, 32.768) if prob == "ackley" else (-5.12, 5.12)
    hyper = (0.6, 2.5, 0.8) if prob == "ackley" else (0.7, 1.5, 1.5)
    fitness = opso.FITNESS[prob]
    s0 = opso.init_step(opso.make_state(P, d, lo, hi, *hyper, seed=0), fitness)
    rg, rp = opso.draws(P, d, 1000)
    s1 = opso.step(s0, rg, rp, fitness)  # state with a non-trivial personal best
    rg, rp = opso.draws(P, d, 1001)
    want = opso.step(s1, rg, rp, fitness)
    sw = Swarm(s1, cuda)
    sw.step(prob, rg, rp)
    compare_states(sw.t, want, prob)
    # in-kernel Philox == the same draws read from memory
    seed, gen = 42, 7
    rg2 = opso.pso_uniform(P, d, seed, gen, 0)
    rp2 = opso.pso_uniform(P, d, seed, gen, 1)
    a, b = Swarm(s1, cuda), Swarm(s1, cuda)
    a.step(prob, None, None, seed=seed, generation=gen)
    b.step(prob, rg2, rp2)
    for n in NAMES:
        assert torch.equal(a.t[n], b.t[n]), n


def test_global_best_tie_and_nan_rules(cuda):
    """min_by puts the old best first: it wins ties; among particles the lowest index wins;
    NaN counts as the minimum (torch.argmin)."""
    P, d = 300, 8
    s = opso.make_state(P, d, -1.0, 1.0, 0.6, 2.5, 0.8, seed=5)
    s["fit"] = torch.full((P,), 3.0)
    s["fit"][[17, 200]] = 1.0
    s["local_best_fit"] = s["fit"].clone()
    s["global_best_fit"] = torch.tensor(1.0)  # tie with particles 17 and 200 -> old best stays
    s["global_best_location"] = torch.full((d,), 0.25)
    rg, rp = opso.draws(P, d, 1)
    sw = Swarm(s, cuda)
    sw.step("sphere", rg, rp)
    want = opso.step(s, rg, rp, opso.sphere)
    assert torch.equal(sw.t["global_best_location"].cpu(), want["global_best_location"])
    assert torch.equal(sw.t["global_best_location"].cpu(), torch.full((d,), 0.25))
    s["global_best_fit"] = torch.tensor(2.0)  # now particle 17 (the first of the two) wins
    sw = Swarm(s, cuda)
    sw.step("sphere", rg, rp)
    want = opso.step(s, rg, rp, opso.sphere)
    assert torch.equal(sw.t["global_best_location"].cpu(), s["pop"][17])
    assert torch.equal(sw.t["global_best_location"].cpu(), want["global_best_location"])
    s["fit"][250] = float("nan")
    sw = Swarm(s, cuda)
    sw.step("sphere", rg, rp)
    want = opso.step(s, rg, rp, opso.sphere)
    assert torch.equal(sw.t["global_best_location"].cpu(), want["global_best_location"])
    assert math.isnan(sw.t["global_best_fit"].item()) and math.isnan(want["global_best_fit"].item())


def test_sharded_candidates_match_single(cuda):
    """Two shards emulated on one GPU: local_best per shard + merge == the single-GPU result."""
    from evox_b200 import _cabi as c

    P, d = 5001, 40
    s = opso.init_step(opso.make_state(P, d, -5.12, 5.12, 0.7, 1.5, 1.5, seed=9), opso.rastrigin)
    s["global_best_fit"] = torch.tensor(float("inf"))
    single = Swarm(s, cuda)
    rg, rp = opso.draws(P, d, 2)
    single.step("rastrigin", rg, rp)
    words = c.lib.evox_pso_candidate_words(d)
    bounds = [(0, 2501), (2501, P)]
    recs = torch.zeros(2 * words, dtype=torch.int32, device=cuda)
    shards = []
    for r, (a, b) in enumerate(bounds):
        part = {k: (v[a:b] if (v.ndim >= 1 and v.shape[0] == P) else v) for k, v in s.items()}
        sh = Swarm(part, cuda)
        shards.append(sh)
        c.check(c.lib.evox_pso_local_best(sh.p("fit"), sh.p("pop"), b - a, d, a, recs[r * words:].data_ptr(),
                                          c.ptr(sh.ws), sh.ws.numel(), c.stream_ptr(cuda)))
    keep = []  # device slices must outlive the asynchronous launches that read them
    for r, (a, b) in enumerate(bounds):
        sh = shards[r]
        rg_s, rp_s = rg[a:b].to(cuda).contiguous(), rp[a:b].to(cuda).contiguous()
        keep += [rg_s, rp_s]
        c.check(c.lib.evox_pso_merge_best(c.ptr(recs), 2, d, 1, sh.p("global_best_location"), sh.p("global_best_fit"),
                                          c.stream_ptr(cuda)))
        c.check(c.lib.evox_pso_move_eval(sh.p("pop"), sh.p("velocity"), sh.p("local_best_location"),
                                         sh.p("local_best_fit"), sh.p("fit"), sh.p("global_best_location"),
                                         sh.p("lb"), sh.p("ub"), sh.p("w"), sh.p("phi_p"), sh.p("phi_g"),
                                         c.ptr(rg_s), c.ptr(rp_s),
                                         b - a, d, 1, c.host_floats((0, 0, 0)), 0, 0, a, c.stream_ptr(cuda)))
    torch.cuda.synchronize()
    for n in ("pop", "velocity", "fit", "local_best_location", "local_best_fit"):
        assert torch.equal(torch.cat([sh.t[n] for sh in shards]), single.t[n]), n
    for sh in shards:
        assert torch.equal(sh.t["global_best_location"], single.t["global_best_location"])
        assert torch.equal(sh.t["global_best_fit"], single.t["global_best_fit"])


@pytest.mark.parametrize("prob,P,d,philox", [("ackley", 10_000, 500, True), ("rastrigin", 4097, 1000, False),
                                             ("sphere", 77, 10, True), ("ackley", 5, 3, False), ("ackley", 1, 1, True)])
def test_one_launch_generation_equals_two_launch_form(cuda, prob, P, d, philox):
    """evox_pso_generation carries the arg-min of the fitness it produces to the next call; five
    generations of it must leave every state entry, after every generation, bit-identical to the
    two-launch evox_pso_step (same update arithmetic, so the fitness is compared exactly too)."""
    from evox_b200 import _cabi as c

    lo, hi = (-32.768, 32.768) if prob == "ackley" else (-5.12, 5.12)
    s0 = opso.init_step(opso.make_state(P, d, lo, hi, 0.6, 2.5, 0.8, seed=3), opso.FITNESS[prob])
    two, one = Swarm(s0, cuda), Swarm(s0, cuda)
    words = c.lib.evox_pso_candidate_words(d)
    rec = torch.zeros(2, words, dtype=torch.int32, device=cuda)
    one.local_best(rec[0])
    for g in range(5):
        rg, rp = (None, None) if philox else opso.draws(P, d, 50 + g)
        two.step(prob, rg, rp, seed=9, generation=g)
        one.generation(prob, rec[g % 2], 1, rec[(g + 1) % 2], rg, rp, seed=9, generation=g)
        for n in NAMES:
            assert torch.equal(one.t[n], two.t[n]), (g, n)
        # the record left behind describes the new swarm
        want = opso.candidate_record(one.t["fit"].cpu(), one.t["pop"].cpu(), 0)
        assert torch.equal(rec[(g + 1) % 2].cpu(), want), g


def test_one_launch_generation_tie_and_nan_rules(cuda):
    """The head of evox_pso_generation applies min_by's rules: the stored best wins ties, the lowest
    global row wins among records, NaN counts as the minimum."""
    from evox_b200 import _cabi as c

    P, d = 300, 8
    s = opso.make_state(P, d, -1.0, 1.0, 0.6, 2.5, 0.8, seed=5)
    s["fit"] = torch.full((P,), 3.0)
    s["fit"][[17, 200]] = 1.0
    s["local_best_fit"] = s["fit"].clone()
    s["global_best_location"] = torch.full((d,), 0.25)
    rg, rp = opso.draws(P, d, 1)
    words = c.lib.evox_pso_candidate_words(d)
    for old, nan_row in ((1.0, None), (2.0, None), (2.0, 250), (float("nan"), 250)):
        s["global_best_fit"] = torch.tensor(old)
        if nan_row is not None:
            s["fit"][nan_row] = float("nan")
        sw = Swarm(s, cuda)
        rec = torch.zeros(2, words, dtype=torch.int32, device=cuda)
        sw.local_best(rec[0])
        sw.generation("sphere", rec[0], 1, rec[1], rg, rp)
        want = opso.step(s, rg, rp, opso.sphere)
        assert torch.equal(sw.t["global_best_location"].cpu(), want["global_best_location"]), (old, nan_row)
        assert torch.equal(torch.nan_to_num(sw.t["global_best_fit"].cpu(), nan=-7.0), torch.nan_to_num(want["global_best_fit"], nan=-7.0))
        assert torch.equal(sw.t["pop"].cpu(), want["pop"])


def test_one_launch_generation_sharded_matches_single(cuda):
    """Three uneven shards emulated on one GPU: each runs evox_pso_generation over the gathered records of all
    shards (built here by placing every shard's record in one array, which is what the allgather does); after
    four generations the concatenated shards equal the unsharded swarm bit for bit."""
    from evox_b200 import _cabi as c

    P, d = 5001, 40
    s = opso.init_step(opso.make_state(P, d, -5.12, 5.12, 0.7, 1.5, 1.5, seed=9), opso.rastrigin)
    single = Swarm(s, cuda)
    words = c.lib.evox_pso_candidate_words(d)
    bounds = [(0, 1700), (1700, 3401), (3401, P)]
    shards = []
    for a, b in bounds:
        part = {k: (v[a:b] if (v.ndim >= 1 and v.shape[0] == P) else v) for k, v in s.items()}
        shards.append(Swarm(part, cuda))
    gathered = torch.zeros(len(bounds), words, dtype=torch.int32, device=cuda)
    mine = torch.zeros(len(bounds), words, dtype=torch.int32, device=cuda)
    for r, (a, b) in enumerate(bounds):
        shards[r].local_best(gathered[r], row_offset=a)
    rec1 = torch.zeros(2, words, dtype=torch.int32, device=cuda)
    single.local_best(rec1[0])
    for g in range(4):
        single.generation("rastrigin", rec1[g % 2], 1, rec1[(g + 1) % 2], seed=4, generation=g)
        for r, (a, b) in enumerate(bounds):
            shards[r].generation("rastrigin", gathered, len(bounds), mine[r], seed=4, generation=g, row_offset=a)
        gathered.copy_(mine)
        for n in ("pop", "velocity", "fit", "local_best_location", "local_best_fit"):
            assert torch.equal(torch.cat([sh.t[n] for sh in shards]), single.t[n]), (g, n)
        for sh in shards:
            assert torch.equal(sh.t["global_best_location"], single.t["global_best_location"]), g
            assert torch.equal(sh.t["global_best_fit"], single.t["global_best_fit"]), g


@pytest.mark.parametrize("P,d,prob", [(5001, 40, "rastrigin"), (999, 10, "ackley")])
def test_peer_exchange_generation_matches_single(cuda, P, d, prob):
    """evox_pso_generation_peer with three ranks emulated on one GPU: every rank has its own exchange buffer
    and the kernels write their records into all three. The ranks run one after the other within a generation,
    so every wait finds its flag already set. After five generations the concatenated shards equal the
    unsharded swarm bit for bit and no wait gave up."""
    from evox_b200 import _cabi as c

    lo, hi = (-32.768, 32.768) if prob == "ackley" else (-5.12, 5.12)
    s = opso.init_step(opso.make_state(P, d, lo, hi, 0.7, 1.5, 1.5, seed=9), opso.FITNESS[prob])
    single = Swarm(s, cuda)
    words = c.lib.evox_pso_candidate_words(d)
    bounds = [(0, P // 3), (P // 3, 2 * P // 3 + 1), (2 * P // 3 + 1, P)]
    g_ranks = len(bounds)
    shards = []
    for a, b in bounds:
        part = {k: (v[a:b] if (v.ndim >= 1 and v.shape[0] == P) else v) for k, v in s.items()}
        shards.append(Swarm(part, cuda))
    n_words = c.lib.evox_pso_exchange_words(d, g_ranks)
    assert n_words == 2 * g_ranks * words + 2 * g_ranks
    buffers = [torch.zeros((n_words + 3) // 4 * 4, dtype=torch.int32, device=cuda) for _ in bounds]
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    # generation 0 reads tag 1: seed parity slot 1 of every buffer with the gathered records, flags = 1
    first = torch.zeros(g_ranks, words, dtype=torch.int32, device=cuda)
    for r, (a, b) in enumerate(bounds):
        shards[r].local_best(first[r], row_offset=a)
    for buf in buffers:
        buf[g_ranks * words: 2 * g_ranks * words].copy_(first.view(-1))
        buf[2 * g_ranks * words + g_ranks: 2 * g_ranks * words + 2 * g_ranks].fill_(1)
    rec1 = torch.zeros(2, words, dtype=torch.int32, device=cuda)
    single.local_best(rec1[0])
    for g in range(5):
        single.generation(prob, rec1[g % 2], 1, rec1[(g + 1) % 2], seed=4, generation=g)
        for r, (a, b) in enumerate(bounds):
            shards[r].generation_peer(prob, buffers, r, g + 1, status, seed=4, generation=g, row_offset=a)
        for n in ("pop", "velocity", "fit", "local_best_location", "local_best_fit"):
            assert torch.equal(torch.cat([sh.t[n] for sh in shards]), single.t[n]), (g, n)
        for sh in shards:
            assert torch.equal(sh.t["global_best_location"], single.t["global_best_location"]), g
            assert torch.equal(sh.t["global_best_fit"], single.t["global_best_fit"]), g
        assert torch.equal(buffers[0], buffers[1]) and torch.equal(buffers[0], buffers[2])
    assert int(status) == 0


def test_peer_exchange_wait_gives_up(cuda):
    """A flag that nothing sets: the wait ends by itself after its time limit, the kernel reports through the
    status word and returns, the context stays usable, and the next launch does not wait again."""
    import time

    from evox_b200 import _cabi as c

    P, d = 256, 8
    s = opso.init_step(opso.make_state(P, d, -1.0, 1.0, 0.6, 2.5, 0.8, seed=1), opso.sphere)
    sw = Swarm(s, cuda)
    n_words = c.lib.evox_pso_exchange_words(d, 2)
    buffers = [torch.zeros((n_words + 3) // 4 * 4, dtype=torch.int32, device=cuda) for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    t0 = time.perf_counter()
    sw.generation_peer("sphere", buffers, 0, 5, status)  # nobody wrote tag 5
    first = time.perf_counter() - t0
    assert int(status) == 1
    assert first < 30.0
    t0 = time.perf_counter()
    sw.generation_peer("sphere", buffers, 0, 6, status)
    assert time.perf_counter() - t0 < first / 2 + 0.5
    assert torch.isfinite(sw.t["pop"]).all()
    with pytest.raises(c.EvoxKernelError, match="tag 0"):
        sw.generation_peer("sphere", buffers, 0, 0, status)
    with pytest.raises(c.EvoxKernelError, match="rank"):
        sw.generation_peer("sphere", buffers, 2, 1, status)


def test_generation_rejects_overlapping_records(cuda):
    from evox_b200 import _cabi as c

    s = opso.init_step(opso.make_state(64, 8, -1.0, 1.0, 0.6, 2.5, 0.8, seed=1), opso.sphere)
    sw = Swarm(s, cuda)
    rec = torch.zeros(2, c.lib.evox_pso_candidate_words(8), dtype=torch.int32, device=cuda)
    with pytest.raises(c.EvoxKernelError, match="overlap"):
        sw.generation("sphere", rec, 2, rec[1])


def test_step_sees_writes_between_generations(cuda):
    """The record carried from one generation to the next is dropped when something else writes to `fit`
    or `pop`: the next step must find the global best of the swarm as it is then (pso.py:92-95)."""
    from evox_b200.algorithms import PSO
    from evox_b200.problems.numerical import Sphere
    from evox_b200.workflows import StdWorkflow

    d = 16
    algo = PSO(1000, torch.full((d,), -1.0), torch.full((d,), 1.0), device=cuda, seed=2)
    wf = StdWorkflow(algo, Sphere(), device=cuda)
    wf.init_step()
    wf.step()
    wf.step()
    algo = wf.algorithm
    algo.fit[123] = -5.0  # an in-place torch write
    row = algo.pop[123].clone()
    wf.step()
    assert float(algo.global_best_fit) == -5.0
    assert torch.equal(algo.global_best_location, row)
    # a loaded state: the stored bests come from the dict, the record is rebuilt from its fit
    sd = {k: v.clone() for k, v in algo.state_dict().items() if isinstance(v, torch.Tensor)}
    sd["fit"][7] = -9.0
    row = sd["pop"][7].clone()
    algo.load_state_dict(sd)
    wf.step()
    assert float(algo.global_best_fit) == -9.0
    assert torch.equal(algo.global_best_location, row)


def test_workflow_fused_equals_unfused(cuda):
    """StdWorkflow(PSO, Ackley): the fused step and the path through Problem.evaluate agree,
    and the swarm improves."""
    from evox_b200.algorithms import PSO
    from evox_b200.core import Monitor
    from evox_b200.problems.numerical import Ackley
    from evox_b200.workflows import StdWorkflow

    class Count(Monitor):
        def __init__(self):
            super().__init__()
            self.calls = []

        def post_ask(self, x):
            self.calls.append("post_ask")

        def pre_tell(self, f):
            self.calls.append("pre_tell")

    d = 100
    lb, ub = torch.full((d,), -32.768), torch.full((d,), 32.768)
    runs = []
    for fused in (True, False):
        algo = PSO(512, lb, ub, device=cuda, seed=11)
        mon = Count()
        wf = StdWorkflow(algo, Ackley(), monitor=mon, device=cuda,
                         fitness_transform=None if fused else torch.nn.Identity())
        assert (wf._fused_plan() is not None) == fused
        wf.init_step()
        first = wf.algorithm.global_best_fit.item()
        for _ in range(20):
            wf.step()
        assert mon.calls == ["post_ask", "pre_tell"] * 21
        assert wf.algorithm.global_best_fit.item() < first
        runs.append({k: v.clone() for k, v in wf.algorithm.state_dict().items() if isinstance(v, torch.Tensor)})
    for k in runs[0]:
        assert torch.equal(runs[0][k], runs[1][k]), k


def test_reference_state_dict_loads(golden, cuda):
    """A state_dict with the reference's keys loads into the drop-in class, and one step through
    the public API lands on the reference's next state."""
    from evox_b200.algorithms import PSO
    from evox_b200.problems.numerical import Ackley
    from evox_b200.workflows import StdWorkflow

    g = golden("pso")
    tag = "pso_ackley_d12"
    lo, hi = g[f"{tag}_bounds"]
    algo = PSO(37, torch.full((12,), float(lo)), torch.full((12,), float(hi)), device=cuda)
    wf = StdWorkflow(algo, Ackley(), device=cuda)
    sd = {n: torch.from_numpy(g[f"{tag}_s2_{n}"]) for n in NAMES}
    w, pp, pg = g[f"{tag}_hyper"]
    sd.update({"w": torch.tensor(w), "phi_p": torch.tensor(pp), "phi_g": torch.tensor(pg)})
    wf.algorithm.load_state_dict(sd)
    rg = torch.from_numpy(g[f"{tag}_g1_rg"]).to(cuda)
    rp = torch.from_numpy(g[f"{tag}_g1_rp"]).to(cuda)
    wf.algorithm.step(rg=rg, rp=rp)
    got = {k: v for k, v in wf.algorithm.state_dict().items() if isinstance(v, torch.Tensor)}
    compare_states(got, load_state(g, tag, 3), "ackley")


def test_headline_size_properties(cuda):
    """1,000,000 x 1,000 (the headline workload, 12 GB of state): (a) every row's update depends only on that
    row, the global best and its position in the random stream — four row blocks re-run as small swarms with
    `row_offset` must reproduce the big run bit for bit, and the CPU oracle must reproduce them too (a'); (b) the stored fitness is the fitness of the stored positions;
    (c) positions stay inside the bounds; (d) the global best is the smallest fitness seen so far and
    never gets worse."""
    from evox_b200 import _cabi as c
    from evox_b200.algorithms import PSO
    from evox_b200.problems.numerical import Ackley
    from evox_b200.workflows import StdWorkflow

    free, _ = torch.cuda.mem_get_info(cuda)
    if free < 40e9:
        pytest.skip("needs about 30 GB of free device memory")
    P, d = 1_000_000, 1000
    torch.manual_seed(0)
    algo = PSO(P, torch.full((d,), -32.768), torch.full((d,), 32.768), 0.6, 2.5, 0.8, device=cuda, seed=77)
    algo.velocity.mul_(0.2)
    prob = Ackley()
    wf = StdWorkflow(algo, prob, device=cuda)
    wf.init_step()
    wf.step()
    best_before = float(algo.global_best_fit)
    blocks = [(0, 513), (123_456, 124_000), (500_000, 500_257), (P - 300, P)]
    names = ("pop", "velocity", "local_best_location", "local_best_fit", "fit")
    saved = [{n: getattr(algo, n)[a:b].clone() for n in names} for a, b in blocks]
    saved_before = [{n: t.clone() for n, t in part.items()} for part in saved]
    gen = algo.generation
    min_fit_before = float(algo.fit.min())
    wf.step()
    # the step first folded the best of the previous swarm into the global best, then moved
    assert float(algo.global_best_fit) == min(best_before, min_fit_before)
    gbest = algo.global_best_location
    fid, params = prob.fused_fitness()
    for (a, b), part in zip(blocks, saved):
        c.check(c.lib.evox_pso_move_eval(
            c.ptr(part["pop"]), c.ptr(part["velocity"]), c.ptr(part["local_best_location"]), c.ptr(part["local_best_fit"]),
            c.ptr(part["fit"]), c.ptr(gbest), c.ptr(algo.lb), c.ptr(algo.ub), c.ptr(algo.w), c.ptr(algo.phi_p), c.ptr(algo.phi_g),
            None, None, b - a, d, fid, c.host_floats(params), algo.seed, gen, a, c.stream_ptr(cuda)))
        for n in names:
            assert torch.equal(part[n], getattr(algo, n)[a:b]), (a, n)
    # (a') the same four row blocks through the CPU oracle of PSO.step (pso.py:89-106), fed with the draws of the
    # run's random stream at those rows and the run's global best: positions, velocities and personal bests
    # bit for bit, fitness to 1e-5
    hyper = {"lb": algo.lb.cpu(), "ub": algo.ub.cpu(), "w": algo.w.detach().cpu(), "phi_p": algo.phi_p.detach().cpu(),
             "phi_g": algo.phi_g.detach().cpu()}
    for (a, b), before in zip(blocks, saved_before):
        st = {**{n: t.cpu() for n, t in before.items()}, **hyper,
              # min_by over [stored best, block] must keep the run's global best: it is the minimum of the whole swarm
              "global_best_location": gbest.cpu(), "global_best_fit": algo.global_best_fit.cpu()}
        rg = opso.pso_uniform(b - a, d, algo.seed, gen, 0, row_offset=a)
        rp = opso.pso_uniform(b - a, d, algo.seed, gen, 1, row_offset=a)
        want = opso.step(st, rg, rp, opso.ackley)
        for n in ("pop", "velocity", "local_best_location"):
            assert torch.equal(getattr(algo, n)[a:b].cpu(), want[n]), (a, n)
        for n in ("fit", "local_best_fit"):
            assert_fitness_close(getattr(algo, n)[a:b], want[n], "ackley", d)
    # (b) re-evaluation of the stored positions, in slabs to bound memory
    for a in range(0, P, 250_000):
        again = prob.evaluate(algo.pop[a:a + 250_000])
        assert torch.equal(again, algo.fit[a:a + 250_000])
    # (c) bounds
    assert float(algo.pop.min()) >= float(algo.lb.min()) and float(algo.pop.max()) <= float(algo.ub.max())
    assert torch.isfinite(algo.fit).all()
