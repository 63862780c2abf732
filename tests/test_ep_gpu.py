"""Expert parallelism: the slab pack / unpack kernels against their numpy statement on one GPU, and on >= 2 GPUs the layer step
of every rank against the one-GPU layer over the same tokens (same kernels and operands per route; only the FP32 order in
which a token's partial sums are added differs, so equality is to rounding, not bit for bit)."""
import ctypes as C
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("T,E,K,world,rank,rep", [(64, 32, 4, 4, 1, ()), (300, 64, 10, 8, 5, (3, 40)), (5, 8, 2, 2, 0, ()), (1, 16, 3, 4, 3, (1, 2))])
def test_slab_pack_and_unpack_against_numpy_model(T, E, K, world, rank, rep):
    from tokspur_public_b200 import ep, synth
    from tokspur_public_b200 import layer as L
    Cn = 256
    lib = ep.lib()
    place = ep.placement(E, world, rep)
    rng = np.random.default_rng(T + E)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.uint32)
    w = rng.random((T, K)).astype(np.float32)
    x = synth.activations_f16(9, T, Cn)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    d_ids, d_w, d_x, d_place = d(ids.view(np.int32)), d(w), d(x), d(place.view(np.int32))
    S = int(lib.tsp_ep_slab_bytes(T, Cn, K))
    Hr = int(lib.tsp_ep_slab_header_rows(T, Cn, K))
    assert S == (Hr + T) * Cn * 2 and Hr * Cn * 2 >= 256 + T * K * 8
    slabs = torch.full((world * S,), 0x5A, dtype=torch.uint8, device="cuda")
    pos = torch.zeros(world * T, dtype=torch.int32, device="cuda")
    for k_ordered in (0, 1):
        ep.check(lib.tsp_ep_pack(d_ids.data_ptr(), d_w.data_ptr(), d_x.data_ptr(), Cn * 2, d_place.data_ptr(), T, Cn, K, rank, world, k_ordered,
                                 pos.data_ptr(), slabs.data_ptr(), L.stream_ptr()))
        torch.cuda.synchronize()
        want_pos, rows = ep.slab_model(ids, w, place, rank, world)
        assert np.array_equal(pos.cpu().numpy().reshape(world, T), want_pos)
        raw = slabs.cpu().numpy().reshape(world, S)
        order = np.array([0, 2, 1, 3, 4, 6, 5, 7])
        for g in range(world):
            toks, slots, ws = rows[g]
            assert int(raw[g, :4].view(np.uint32)[0]) == len(toks)
            meta_i = raw[g, 256:256 + T * K * 4].view(np.uint32).reshape(T, K)[:len(toks)]
            meta_w = raw[g, 256 + T * K * 4:256 + T * K * 8].view(np.float32).reshape(T, K)[:len(toks)]
            assert np.array_equal(meta_i, slots) and np.array_equal(meta_w, ws)
            got = raw[g, Hr * Cn * 2:].view(np.float16).reshape(T, Cn)[:len(toks)]
            want = x[toks]
            if k_ordered:
                want = want.reshape(len(toks), Cn // 8, 8)[:, :, order].reshape(len(toks), Cn)
            assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
        # unpack: dense routing rows over the row space of all slabs
        R = world * (Hr + T)
        ids_all = torch.zeros(R * K, dtype=torch.int32, device="cuda")
        w_all = torch.zeros(R * K, dtype=torch.float32, device="cuda")
        ep.check(lib.tsp_ep_unpack(slabs.data_ptr(), T, Cn, K, world, ids_all.data_ptr(), w_all.data_ptr(), L.stream_ptr()))
        torch.cuda.synchronize()
        ia = ids_all.cpu().numpy().view(np.uint32).reshape(world, Hr + T, K)
        wa = w_all.cpu().numpy().reshape(world, Hr + T, K)
        for g in range(world):
            n = len(rows[g][0])
            assert np.all(ia[g, :Hr] == 0xFFFFFFFF) and np.all(ia[g, Hr + n:] == 0xFFFFFFFF) and np.all(wa[g, Hr + n:] == 0)
            assert np.array_equal(ia[g, Hr:Hr + n], rows[g][1]) and np.array_equal(wa[g, Hr:Hr + n], rows[g][2])


def _worker(rank, world, port, shape, T, prefill, replicate, result):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from tokspur_public_b200 import ep, synth
        from tokspur_public_b200 import layer as L
        Cn, H, E, K = shape
        dev = torch.device("cuda", rank)
        bias = synth.zipf_bias(5, E) if prefill else None
        x = torch.from_numpy(synth.activations_f16(50 + rank, T, Cn)).to(dev)
        lg = torch.from_numpy(synth.router_logits(60 + rank, T, E, bias)).to(dev)
        out = torch.zeros((T, Cn), dtype=torch.float16, device=dev)
        ctx = ep.EpContext(rank, world, dev)
        rep = ep.hot_experts(synth.router_logits(1999, 256, E, bias), K, replicate)
        layer = ep.EpLayer(ctx, 7, Cn, H, E, K, dev, T, prefill=prefill, replicated=rep)
        for _ in range(2):   # twice: buffers are reused across steps
            layer.step(x, lg, out)
        assert layer.error_word() == 0
        full = L.SynthDeviceLayer(7, Cn, H, E, 12, 1, dev)
        want = torch.zeros_like(out)
        if prefill:
            ps = L.PrefillScratch(Cn, H, E, K, T, dev)
            L.moe_layer_prefill(full, ps, x, lg, want)
            torch.cuda.synchronize()
            assert ps.base.error_word() == 0
        else:
            s = L.Scratch(Cn, H, E, K, T, dev)
            L.moe_layer_decode(full, s, x, lg, want)
            torch.cuda.synchronize()
            assert s.error_word() == 0
        a, b = out.float().cpu().numpy().astype(np.float64), want.float().cpu().numpy().astype(np.float64)
        rel = float(np.linalg.norm(a - b) / np.linalg.norm(b))
        result[rank] = rel <= (1e-3 if prefill else 5e-4)   # prefill: partial sums travel as binary16
        ctx.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("prefill,T,replicate", [(False, 24, 0), (False, 1, 2), (True, 300, 0), (True, 300, 4)])
def test_expert_parallel_layer_equals_single_gpu(world, prefill, T, replicate):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as m:
        result = m.dict()
        mp.spawn(_worker, args=(world, port, (512, 256, 32, 4), T, prefill, replicate, result), nprocs=world, join=True)
        assert dict(result) == {r: True for r in range(world)}
