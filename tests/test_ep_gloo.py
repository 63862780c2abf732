"""Expert-parallel dispatch / combine plumbing on CPU: two gloo ranks, a stand-in expert computation.
Checks that every route's row reaches the rank owning its expert and that the returned rows land at token*K+slot."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, T, E, K, C, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tokspur_public_b200 import ep
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn((T, C), generator=g)
        ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
        if rank == 1:
            ids[:, :] = torch.arange(K, dtype=torch.int32)  # a ragged case: every route of rank 1 goes to rank 0
        plan = ep.RoutePlan(ids, E, world)
        rows, lids = ep.dispatch(plan, x)
        per = E // world
        assert rows.shape[0] == plan.received == lids.shape[0]
        assert int(lids.min()) >= 0 and int(lids.max()) < per if plan.received else True
        y = rows * (lids.to(torch.float32) + rank * per + 1).unsqueeze(1)   # stand-in for the expert FFN: scale by (global id + 1)
        routed = torch.zeros((T * K, C))
        ep.combine(plan, y, routed)
        want = (x.unsqueeze(1) * (ids.to(torch.float32) + 1).unsqueeze(2)).reshape(T * K, C)
        result[rank] = bool(torch.equal(routed, want)) and sum(plan.send_splits) == T * K
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T,E,K", [(5, 8, 3), (1, 4, 2), (16, 64, 10)])
def test_dispatch_combine_round_trip_two_ranks(T, E, K):
    world, port = 2, _free_port()
    with mp.Manager() as m:
        result = m.dict()
        mp.spawn(_worker, args=(world, port, T, E, K, 7, result), nprocs=world, join=True)
        assert dict(result) == {0: True, 1: True}
