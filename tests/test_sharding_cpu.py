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
