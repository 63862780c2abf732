"""Expert parallelism on real GPUs (needs >= 2): every rank's layer output must equal the one-GPU layer output for the
same tokens bit for bit, since a route's expert output is computed by the same kernels wherever the expert lives."""
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


def _worker(rank, world, port, shape, T, result):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from tokspur_public_b200 import ep, synth
        from tokspur_public_b200 import layer as L
        Cn, H, E, K = shape
        dev = torch.device("cuda", rank)
        x = torch.from_numpy(synth.activations_f16(50 + rank, T, Cn)).to(dev)
        lg = torch.from_numpy(synth.router_logits(60 + rank, T, E)).to(dev)
        out = torch.zeros((T, Cn), dtype=torch.float16, device=dev)
        layer = ep.EpLayer(7, Cn, H, E, K, rank, world, dev, T)
        for _ in range(2):   # twice: buffers are reused across steps
            layer.step(x, lg, out)
        assert layer.error_word() == 0
        full = L.SynthDeviceLayer(7, Cn, H, E, 12, 1, dev)
        s = L.Scratch(Cn, H, E, K, T, dev)
        want = torch.zeros_like(out)
        L.moe_layer_decode(full, s, x, lg, want)
        torch.cuda.synchronize()
        assert s.error_word() == 0
        ok = bool(torch.equal(out, want))
        out2 = torch.zeros_like(out)
        for _ in range(2):
            layer.step_gathered(x, lg, out2)   # all-gather / reduce-scatter scheme: equal up to FP32 summation order
        assert layer.error_word() == 0
        a, b = out2.float().cpu().numpy().astype(np.float64), want.float().cpu().numpy().astype(np.float64)
        rel = float(np.linalg.norm(a - b) / np.linalg.norm(b))
        result[rank] = ok and rel <= 5e-4 and float(np.max(np.abs(a - b) / np.maximum(1.0, np.abs(b)))) <= 2e-3
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_layer_equals_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as m:
        result = m.dict()
        mp.spawn(_worker, args=(world, port, (512, 256, 32, 4), 24, result), nprocs=world, join=True)
        assert dict(result) == {r: True for r in range(world)}


def _prefill_worker(rank, world, port, shape, T, result):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from tokspur_public_b200 import ep, synth
        from tokspur_public_b200 import layer as L
        Cn, H, E, K = shape
        dev = torch.device("cuda", rank)
        x = torch.from_numpy(synth.activations_f16(70 + rank, T, Cn)).to(dev)
        lg = torch.from_numpy(synth.router_logits(80 + rank, T, E, synth.zipf_bias(5, E))).to(dev)
        out = torch.zeros((T, Cn), dtype=torch.float16, device=dev)
        layer = ep.EpLayer(9, Cn, H, E, K, rank, world, dev, T, prefill=True)
        for _ in range(2):   # twice: buffers are reused across steps
            layer.step_gathered_prefill(x, lg, out)
        assert layer.error_word() == 0
        full = L.SynthDeviceLayer(9, Cn, H, E, 12, 1, dev)
        ps = L.PrefillScratch(Cn, H, E, K, T, dev)
        want = torch.zeros_like(out)
        L.moe_layer_prefill(full, ps, x, lg, want)
        torch.cuda.synchronize()
        assert ps.base.error_word() == 0
        a, b = out.float().cpu().numpy().astype(np.float64), want.float().cpu().numpy().astype(np.float64)
        # same kernels and the same binary16 operands on both sides; only the FP32 order of the mixture differs
        result[rank] = float(np.linalg.norm(a - b) / np.linalg.norm(b)) <= 5e-4
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_prefill_equals_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as m:
        result = m.dict()
        mp.spawn(_prefill_worker, args=(world, port, (512, 256, 32, 4), 300, result), nprocs=world, join=True)
        assert dict(result) == {r: True for r in range(world)}
