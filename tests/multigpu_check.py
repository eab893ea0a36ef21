"""Multi-GPU consistency check, launched with torch.distributed.run (one rank per GPU, NCCL):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        tests/multigpu_check.py

Every rank runs the sharded algorithm on its GPU and, next to it, the single-GPU algorithm on the same
GPU; after a few generations the gathered sharded state must equal the single-GPU state bit for bit
(PSO), the centre of the sharded virtual-LoRA ES must equal the single-GPU centre, the
row-sharded RVEA selection must pick and gather the same rows as the single call, and the non-dominated
rank with its matrix split over the GPUs must equal the single-GPU rank. Prints
"multigpu ok" from rank 0 and exits non-zero on any mismatch.
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
from torch import nn

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def check_pso(dev, rank, world):
    from evox_b200.algorithms import PSO
    from evox_b200.problems.numerical import Rastrigin
    from evox_b200.workflows import StdWorkflow

    P, d = 20_001, 100  # uneven shards on purpose
    lb, ub = torch.full((d,), -5.12), torch.full((d,), 5.12)
    single = StdWorkflow(PSO(P, lb, ub, 0.7, 1.5, 1.5, device=dev, seed=7), Rastrigin(), device=dev)
    shard = StdWorkflow(PSO(P, lb, ub, 0.7, 1.5, 1.5, device=dev, seed=7, shard=True), Rastrigin(), device=dev)
    a, b = shard.algorithm.row_start, shard.algorithm.row_end
    assert torch.equal(shard.algorithm.pop, single.algorithm.pop[a:b])  # the initial swarm does not depend on the sharding
    # the same sharded swarm with the records exchanged by one NCCL allgather per generation instead
    nccl = StdWorkflow(PSO(P, lb, ub, 0.7, 1.5, 1.5, device=dev, seed=7, shard=True, peer_exchange=False), Rastrigin(), device=dev)
    for wf in (single, shard, nccl):
        wf.init_step()
        for _ in range(5):
            wf.step()
        # the swarm is written between generations: the next step must see it (records rebuilt on every rank)
        wf.algorithm.pop.mul_(0.5)
        for _ in range(4):
            wf.step()
    torch.cuda.synchronize()
    f = single.algorithm
    for s in (shard.algorithm, nccl.algorithm):
        for name in ("pop", "velocity", "fit", "local_best_location", "local_best_fit"):
            assert torch.equal(getattr(s, name), getattr(f, name)[a:b]), f"rank {rank}: {name}"
        assert torch.equal(s.global_best_location, f.global_best_location)
        assert torch.equal(s.global_best_fit, f.global_best_fit)
    assert nccl.algorithm._peer is None
    if shard.algorithm._peer:
        assert shard.algorithm.exchange_status() == 0, f"rank {rank}: a wait for a peer's record gave up"
    if rank == 0:
        how = "kernels over peer memory" if shard.algorithm._peer else f"NCCL ({getattr(shard.algorithm, '_peer_error', '')})"
        print(f"pso records exchanged by: {how}", flush=True)


def check_lora_es(dev, rank, world):
    from evox_b200.algorithms import VirtualLoRAES
    from evox_b200.problems import VirtualLoRAProblem
    from evox_b200.transforms import CenteredRank
    from evox_b200.workflows import StdWorkflow

    gen = torch.Generator().manual_seed(0)
    width, pop, batch = 256 * world, 8 * world, 64
    layers = []
    for i in range(2):
        lin = nn.Linear(width, width, bias=False)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(width, width, generator=gen) / width**0.5)
        layers += [lin] + ([nn.ReLU()] if i == 0 else [])
    model = nn.Sequential(*layers)
    x = torch.randn(pop, batch, width, generator=gen).bfloat16()
    y = torch.randn(batch, width, generator=gen)
    center = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    results = []
    for sharded in (False, True):
        prob = VirtualLoRAProblem(model, [(x, y)], nn.MSELoss(reduction="none"), 8, device=dev, compute_dtype=torch.bfloat16, shard=sharded)
        algo = VirtualLoRAES(prob.param_shapes, 8, pop, center.clone(), 0.01, 0.02, device=dev, shard=sharded)
        wf = StdWorkflow(algo, prob, device=dev, fitness_transform=CenteredRank())
        if sharded:
            assert wf.algorithm._row_shard((width, width)) is not None
        for g in range(3):
            seeds = torch.randint(0, 2**31, (pop,), generator=torch.Generator().manual_seed(50 + g), dtype=torch.int64)
            wf.algorithm.step(seeds=seeds.to(dev))
        torch.cuda.synchronize()
        results.append(wf.algorithm.center.clone())
    assert torch.equal(results[0], results[1]), f"rank {rank}: sharded centre differs by {(results[0] - results[1]).abs().max().item():.3e}"


def check_rvea(dev, rank, world):
    from evox_b200.operators.selection import ref_vec_guided, ref_vec_guided_sharded
    from evox_b200.sharding import shard_bounds
    from oracle import rvea

    x, f, v, theta = rvea.config2_inputs(n=30_001)
    xd, fd, vd, td = x.to(dev), f.to(dev), v.to(dev), theta.to(dev)
    want = ref_vec_guided(xd, fd, vd, td, return_index=True)
    a, b = shard_bounds(x.shape[0], world, rank)
    got = ref_vec_guided_sharded(xd[a:b], fd[a:b], vd, td, a, return_index=True)
    torch.cuda.synchronize()
    assert torch.equal(got[2], want[2]), f"rank {rank}: selected rows differ"
    for g, w in zip(got[:2], want[:2]):
        assert torch.equal(torch.nan_to_num(g, nan=-1.0), torch.nan_to_num(w, nan=-1.0)), f"rank {rank}: gathered rows differ"


def check_nds(dev, rank, world):
    from evox_b200.operators.selection import non_dominate_rank, non_dominate_rank_sharded
    from oracle import nds

    f = nds.dtlz2_objectives(torch.rand(30_001, 12, generator=torch.Generator().manual_seed(4)), 3).to(dev)
    want = non_dominate_rank(f, check=True)
    got = non_dominate_rank_sharded(f)
    torch.cuda.synchronize()
    assert torch.equal(got, want), f"rank {rank}: split-matrix ranks differ"


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    try:
        check_pso(dev, rank, world)
        check_lora_es(dev, rank, world)
        check_rvea(dev, rank, world)
        check_nds(dev, rank, world)
        dist.barrier()
        if rank == 0:
            print("multigpu ok", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
