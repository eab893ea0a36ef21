"""Host-side logic of the sharded swarm on CPU: shard bounds, the record allgather (gloo,
world_size 2) and the merge rule. The kernels themselves are covered by the GPU tests."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import pso as opso


def test_shard_bounds_match_tensor_split():
    from evox_b200.sharding import shard_bounds

    for n in (1, 7, 10, 1000, 1_000_003):
        for world in (1, 2, 3, 4, 8):
            if n < world:
                continue
            pieces = torch.arange(n).tensor_split(world)
            for r in range(world):
                a, b = shard_bounds(n, world, r)
                assert (a, b) == (int(pieces[r][0]), int(pieces[r][-1]) + 1)
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, P, d, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from evox_b200.sharding import allgather_records, group_info, shard_bounds

        assert group_info() == (rank, world)
        state = opso.init_step(opso.make_state(P, d, -5.12, 5.12, 0.7, 1.5, 1.5, seed=4), opso.rastrigin)
        a, b = shard_bounds(P, world, rank)
        rec = opso.candidate_record(state["fit"][a:b], state["pop"][a:b], a)
        records = allgather_records(rec)
        assert records.numel() == world * (4 + d)
        loc, fit = opso.merge_records(records, world, d, state["global_best_location"], torch.tensor(float("inf")))
        want_loc, want_fit = opso.min_by([state["pop"]], [state["fit"]])
        ok = torch.equal(loc, want_loc) and torch.equal(fit, want_fit)
        # a tie with the old best keeps the old best on every rank
        loc2, fit2 = opso.merge_records(records, world, d, torch.zeros(d), want_fit)
        ok = ok and torch.equal(loc2, torch.zeros(d))
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_record_allgather_and_merge_world2():
    world, P, d = 2, 101, 6
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), P, d, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_pso_host_state_without_gpu():
    """Construction, state names and checkpoint round trip work on CPU; stepping does not."""
    from evox_b200 import _cabi
    from evox_b200.algorithms import PSO

    algo = PSO(10, -torch.ones(4), torch.ones(4), device="cpu", seed=3)
    keys = set(algo.state_dict())
    assert {"pop", "velocity", "fit", "local_best_location", "local_best_fit", "global_best_location",
            "global_best_fit", "w", "phi_p", "phi_g"} <= keys
    other = PSO(10, -torch.ones(4), torch.ones(4), device="cpu", seed=4)
    other.generation = 17
    algo.load_state_dict(other.state_dict())
    assert algo.seed == 4 and algo.generation == 17 and torch.equal(algo.pop, other.pop)
    with pytest.raises(_cabi.EvoxKernelError):
        algo.step()


# ---------------------------------------------------------------------------------------------
# Sharded virtual-LoRA ES: host bookkeeping (seed broadcast, fitness allgather, row-sharded
# gradient + allgather of the updated rows) on two gloo ranks, with the kernels replaced by
# the CPU oracle. The kernels themselves are covered by the GPU tests.
# ---------------------------------------------------------------------------------------------
def _oracle_kernels(monkeypatch_target):
    """Replace the two kernel-calling helpers of evox_b200.algorithms.es by oracle arithmetic."""
    from oracle import lora

    def grad_from_seeds(fitness, seeds, shape, rank, counter, pop_size, sigma, out=None, rows=None, passes=3):
        f = lora.generate_lora_factors(seeds, shape, rank, counter)
        if isinstance(f, tuple):
            g = lora.lora_gradient(fitness, f[0], f[1], pop_size, sigma, shape)
            if rows is not None:
                g = g[rows[0] : rows[1]]
        else:
            g = lora.lora_gradient(fitness, f, None, pop_size, sigma, shape)
        out.copy_(g.reshape(-1))
        return out

    def update_center(algo, grad, start=0, count=None):
        count = algo.center.numel() - start if count is None else count
        algo.center[start : start + count] -= algo.learning_rate * grad

    monkeypatch_target.lora_gradient_from_seeds = grad_from_seeds
    monkeypatch_target._update_center = update_center


def _es_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import evox_b200.algorithms.es as es_mod
        from evox_b200 import _cabi
        from evox_b200.core import Problem
        from evox_b200.sharding import shard_bounds
        from evox_b200.workflows import StdWorkflow

        _oracle_kernels(es_mod)
        real_supported = _cabi.lib.evox_lora_gradient_tc_supported
        shapes, pop, rank_r = [(256, 256), (8,)], 16, 8
        dim = 256 * 256 + 8
        center0 = torch.randn(dim, generator=torch.Generator().manual_seed(3)) * 0.1

        class ShardedSphere(Problem):
            """Fitness = f(seed) evaluated for this rank's individuals only, then allgathered."""

            def evaluate(self, payload):
                _, seeds, _ = payload
                a, b = shard_bounds(seeds.shape[0], world, rank)
                local = (seeds[a:b] % 97).float() / 97.0
                full = torch.empty(seeds.shape[0])
                dist.all_gather_into_tensor(full, local.contiguous())
                return full

        torch.manual_seed(100 + rank)  # ranks deliberately disagree: the broadcast must fix the seeds
        algo = es_mod.VirtualLoRAES(shapes, rank_r, pop, center0.clone(), 0.05, 0.1, device="cpu", shard=True)
        assert algo.world_size == world and algo._row_shard((256, 256)) == shard_bounds(256, world, rank)
        assert algo._row_shard((8,)) is None
        wf = StdWorkflow(algo, ShardedSphere(), device="cpu")
        wf.step()
        seeds = wf.algorithm.seeds.clone()
        # single-process expectation from the oracle with the broadcast seeds
        from oracle import lora

        fit = (seeds % 97).float() / 97.0
        parts = []
        for shape, off in zip(shapes, lora.compute_counter_offsets(shapes, rank_r)):
            f = lora.generate_lora_factors(seeds, shape, rank_r, off)
            g = lora.lora_gradient(fit, f[0], f[1], pop, 0.1, shape) if isinstance(f, tuple) else lora.lora_gradient(fit, f, None, pop, 0.1, shape)
            parts.append(g.reshape(-1))
        want = center0 - torch.tensor(0.05) * torch.cat(parts)
        gathered = [torch.empty_like(seeds) for _ in range(world)]
        dist.all_gather(gathered, seeds)
        same_seeds = all(torch.equal(g, gathered[0]) for g in gathered)
        out[rank] = bool(same_seeds and torch.allclose(wf.algorithm.center, want, rtol=1e-6, atol=1e-7))
        assert real_supported is _cabi.lib.evox_lora_gradient_tc_supported
    finally:
        dist.destroy_process_group()


def test_sharded_virtual_lora_es_world2():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_es_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}
