"""The expert-parallel slab protocol on CPU: two and four gloo ranks exchange the slabs that the numpy statement of the pack
kernels (ep.slab_model) describes, a stand-in expert computation runs on the owners, partial sums travel back and are added
in ascending rank order. Checks that every route reaches the rank holding its expert exactly once, that replicated experts
stay on the token's own rank, and that the returned sums land on the right tokens."""
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


def _worker(rank, world, port, T, E, K, C, rep, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tokspur_public_b200 import ep
        rng = np.random.default_rng(100 + rank)
        x = rng.normal(size=(T, C)).astype(np.float32)
        ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.uint32)
        if rank == 1:
            ids[:, :] = np.arange(K, dtype=np.uint32)   # a ragged case: every route of rank 1 names the first K experts
        w = rng.random((T, K)).astype(np.float32)
        place = ep.placement(E, world, rep)
        local = ep.local_expert_ids(E, world, rank, rep)
        pos, rows = ep.slab_model(ids, w, place, rank, world)
        # dispatch: fixed-size slabs (count, slots, weights, rows), one per destination
        def slab(g):
            toks, slots, ws = rows[g]
            s = np.zeros((T, 1 + 2 * K + C), dtype=np.float64)
            s[:, 0] = len(toks)
            s[:len(toks), 1:1 + K] = slots
            s[:len(toks), 1 + K:1 + 2 * K] = ws
            s[:len(toks), 1 + 2 * K:] = x[toks]
            return torch.from_numpy(s)
        send_all = torch.stack([slab(g) for g in range(world)])
        recv_all = torch.zeros_like(send_all)
        dist.all_to_all_single(recv_all, send_all)   # equal slabs to every rank, as ncclAlltoAll moves them
        recv = [recv_all[p] for p in range(world)]
        # owners: stand-in expert = scale the row by (global expert id + 1); partial sum per received row
        back = []
        seen = 0
        for p in range(world):
            r = recv[p].numpy()
            n = int(r[0, 0])
            part = np.zeros((T, C))
            for j in range(n):
                for k in range(K):
                    slot = int(r[j, 1 + k])
                    if slot == 0xFFFFFFFF:
                        continue
                    assert slot < len(local)
                    seen += 1
                    part[j] += r[j, 1 + K + k] * (local[slot] + 1) * r[j, 1 + 2 * K:]
            back.append(torch.from_numpy(part))
        back_all = torch.stack(back)
        ret_all = torch.zeros_like(back_all)
        dist.all_to_all_single(ret_all, back_all)
        ret = [ret_all[g] for g in range(world)]
        out = np.zeros((T, C))
        for g in range(world):   # ascending rank order
            has = pos[g] >= 0
            out[has] += ret[g].numpy()[pos[g][has]]
        want = (x[:, None, :] * (w * (ids + 1.0))[:, :, None]).sum(axis=1)
        total = torch.tensor([seen])
        dist.all_reduce(total)
        result[rank] = bool(np.allclose(out, want, rtol=1e-12, atol=1e-12)) and int(total.item()) == world * T * K
        # replicated experts never leave the token's rank
        owner = place[ids] >> 16
        for t in range(T):
            for k in range(K):
                if owner[t, k] == ep.REPLICATED:
                    assert pos[rank, t] >= 0
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,T,E,K,rep", [(2, 5, 8, 3, ()), (2, 1, 4, 2, (1,)), (4, 16, 64, 10, (0, 1, 2, 33))])
def test_slab_protocol_round_trip(world, T, E, K, rep):
    port = _free_port()
    with mp.Manager() as m:
        result = m.dict()
        mp.spawn(_worker, args=(world, port, T, E, K, 7, rep, result), nprocs=world, join=True)
        assert dict(result) == {r: True for r in range(world)}
