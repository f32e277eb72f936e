"""Multi-rank host logic on CPU: whole-sequence partitioning and the output gather
(gloo, world size 2)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from raptor_t_b200 import capi, parallel


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, lens, H):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = capi.make_config()
    assignment = parallel.partition_batch(cfg, lens, world)
    # "hidden state" of token t of sequence i: row filled with 1000*i + t (fits fp32 exactly)
    rows = []
    for i in assignment[rank]:
        rows.append((1000.0 * i + torch.arange(lens[i], dtype=torch.float32)[:, None] / 4096).expand(lens[i], H))
    local = torch.cat(rows, 0).contiguous()
    full = parallel.gather_outputs(local, assignment, lens)
    exp = torch.cat([(1000.0 * i + torch.arange(n, dtype=torch.float32)[:, None] / 4096).expand(n, H)
                     for i, n in enumerate(lens)], 0)
    assert torch.equal(full, exp)
    # the set-up-once gatherer: same result through gather() and through start()/finish(), twice
    g = parallel.OutputGatherer(assignment, lens, H, torch.float32, "cpu")
    assert torch.equal(g.gather(local), exp)
    t1 = g.start(local)
    t2 = g.start(local * 2)
    assert torch.equal(g.finish(t1), exp) and torch.equal(g.finish(t2), exp * 2)
    # gather to one rank: grouped send/recv straight into the root's rows, nothing on the others
    for root in (0, world - 1):
        rg = parallel.RootGatherer(assignment, lens, H, torch.float32, "cpu", root=root)
        for scale in (1.0, 3.0):
            got = rg.finish(rg.start(local * scale))
            if rank == root:
                assert torch.equal(got, exp * scale)
            else:
                assert got is None
    dist.destroy_process_group()


def test_partition_covers_all_sequences_and_balances():
    cfg = capi.make_config()
    rng = np.random.default_rng(0)
    lens = [int(x) for x in 64 * rng.integers(16, 65, size=64)]
    for world in (1, 2, 4, 8):
        a = parallel.partition_batch(cfg, lens, world)
        assert sorted(i for r in a for i in r) == list(range(len(lens)))
        costs = parallel.sequence_costs(cfg, lens)
        loads = [sum(costs[i] for i in r) for r in a]
        assert max(loads) / (sum(loads) / world) < 1.05


def test_gather_restores_input_order_gloo_world2():
    lens = [1024, 64, 832, 2048, 1472]
    mp.spawn(_worker, args=(2, _free_port(), lens, 8), nprocs=2, join=True)


def test_gather_restores_input_order_gloo_world3_uneven_shares():
    lens = [4096, 64, 64, 128, 2048, 1472, 704, 64, 3136]
    mp.spawn(_worker, args=(3, _free_port(), lens, 4), nprocs=3, join=True)
