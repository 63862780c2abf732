"""Expert parallelism over the GPUs of one node: a thin harness over libtsp_ep.so (include/tsp_ep.h).

The reference is single-GPU; this is the multi-GPU form of its MoE layer. Experts are sharded by contiguous id range, hot
experts may be replicated on every rank, tokens are data-parallel by source rank, and one layer step is sequenced by ONE C
call: route, pack slabs, NCCL all-to-all, the one-GPU kernels on the owners, NCCL exchange of partial sums, local mixture.
`torch.distributed` is used only to hand the communicator id to the other ranks and for the benchmark's barriers.
"""
from __future__ import annotations

import ctypes as C
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from . import build as _build
from . import capi
from .capi import MoeWeights

REPLICATED = 0xFFFF


class EpLayerDesc(C.Structure):
    _fields_ = [("local", MoeWeights), ("local_experts", C.c_uint32), ("d_place", C.c_void_p)]


_vp, _u32, _u64, _i = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int
EP_SIGNATURES = {
    "tsp_ep_last_error": (C.c_char_p, []),
    "tsp_ep_unique_id": (_i, [_vp]),
    "tsp_ep_create": (_i, [_vp, _i, _i, C.POINTER(_vp)]),
    "tsp_ep_destroy": (_i, [_vp]),
    "tsp_ep_scratch_bytes": (_u64, [_u32, _u32, _u32, _u32, _u32, _u32, _u32, _i]),
    "tsp_ep_slab_header_rows": (_u32, [_u32, _u32, _u32]),
    "tsp_ep_slab_bytes": (_u64, [_u32, _u32, _u32]),
    "tsp_ep_pack": (_i, [_vp, _vp, _vp, _u64, _vp, _u32, _u32, _u32, _u32, _u32, _i, _vp, _vp, _vp]),
    "tsp_ep_unpack": (_i, [_vp, _u32, _u32, _u32, _u32, _vp, _vp, _vp]),
    "tsp_ep_moe_layer": (_i, [_vp, C.POINTER(EpLayerDesc), _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u32, _u32, _u32, _u32, _i, _i, _vp, _u64,
                              _vp, _vp]),
}
_lib = None


def lib() -> C.CDLL:
    """Load libtsp_ep.so (built on demand; needs NCCL). Fails loudly when it cannot be built."""
    global _lib
    if _lib is None:
        capi.lib()   # libtsp_moe.so first: the expert-parallel library calls into it
        path = _build.EP_LIB
        if not os.path.exists(path):
            _build.build_ep()
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: NCCL headers / library not found, the expert-parallel library cannot be built")
        L = C.CDLL(path)
        for name, (res, args) in EP_SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise capi.TspError(rc, lib().tsp_ep_last_error().decode())


def placement(experts: int, world: int, replicated=()) -> np.ndarray:
    """Placement words (owner << 16 | slot) of a layer: contiguous ranges of experts/world ids per rank; the experts in `replicated`
    are held by every rank behind its own range."""
    per = experts // world
    place = np.empty(experts, dtype=np.uint32)
    for e in range(experts):
        place[e] = ((e // per) << 16) | (e % per)
    for i, e in enumerate(sorted(replicated)):
        place[e] = (REPLICATED << 16) | (per + i)
    return place


def local_expert_ids(experts: int, world: int, rank: int, replicated=()) -> list[int]:
    per = experts // world
    return list(range(rank * per, (rank + 1) * per)) + sorted(replicated)


def slab_model(ids: np.ndarray, weights: np.ndarray, place: np.ndarray, rank: int, world: int):
    """Plain numpy statement of what the pack kernels put into the slab for every destination: (pos [world, tokens], per
    destination the list of (token, local slots, weights)). The CPU tests compare the protocol against this; the GPU tests compare
    the kernels against it."""
    T, K = ids.shape
    owner = place[ids] >> 16
    dest = np.where(owner == REPLICATED, rank, owner)
    pos = np.full((world, T), -1, dtype=np.int32)
    rows = []
    for g in range(world):
        mine = dest == g
        has = mine.any(axis=1)
        pos[g, has] = np.arange(int(has.sum()), dtype=np.int32)
        slots = np.where(mine, place[ids] & 0xFFFF, 0xFFFFFFFF).astype(np.uint32)
        rows.append((np.nonzero(has)[0], slots[has], np.where(mine, weights, 0.0).astype(np.float32)[has]))
    return pos, rows


class EpContext:
    """This rank's communicator of libtsp_ep.so; the id travels through torch.distributed (any backend)."""

    def __init__(self, rank: int, world: int, device):
        L = lib()
        self.rank, self.world = rank, world
        idbuf = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            raw = (C.c_uint8 * 128)()
            check(L.tsp_ep_unique_id(raw))
            idbuf = torch.tensor(list(raw), dtype=torch.uint8)
        on_device = dist.get_backend() == "nccl"
        t = idbuf.to(device) if on_device else idbuf
        dist.broadcast(t, 0)
        raw = (C.c_uint8 * 128)(*t.cpu().tolist())
        h = C.c_void_p()
        check(L.tsp_ep_create(raw, rank, world, C.byref(h)))
        self.handle = h

    def close(self):
        if self.handle:
            lib().tsp_ep_destroy(self.handle)
            self.handle = None


class EpLayer:
    """One rank's share of a layer: local experts (own range + replicated ones), placement table and step scratch."""

    def __init__(self, ctx: EpContext, seed: int, channels: int, hidden: int, experts: int, selected: int, device, tokens: int,
                 prefill: bool = False, replicated=(), scratch: torch.Tensor | None = None):
        from . import layer as L
        assert experts % ctx.world == 0
        self.ctx, self.C, self.H, self.E, self.K, self.T, self.prefill = ctx, channels, hidden, experts, selected, tokens, prefill
        ids = local_expert_ids(experts, ctx.world, ctx.rank, replicated)
        self.w = L.SynthDeviceLayer(seed, channels, hidden, experts, 12, 1, device, expert_ids=ids)
        self.place = torch.from_numpy(placement(experts, ctx.world, replicated).view(np.int32)).to(device)
        self.desc = EpLayerDesc(self.w.weights, len(ids), self.place.data_ptr())
        need = int(lib().tsp_ep_scratch_bytes(tokens, channels, hidden, experts, len(ids), selected, ctx.world, int(prefill)))
        self.scratch = scratch if scratch is not None and scratch.numel() >= need else torch.zeros(need, dtype=torch.uint8, device=device)
        self.error = torch.zeros(1, dtype=torch.int32, device=device)

    def step(self, x16: torch.Tensor, logits: torch.Tensor, out16: torch.Tensor) -> None:
        from . import layer as L
        T = x16.shape[0]
        assert T == self.T
        check(lib().tsp_ep_moe_layer(self.ctx.handle, C.byref(self.desc), self.scratch.data_ptr(), self.scratch.numel(), x16.data_ptr(),
                                     x16.stride(0) * 2, logits.data_ptr(), logits.stride(0) * 4, T, self.C, self.H, self.E, self.K, 0, 1,
                                     int(self.prefill), out16.data_ptr(), out16.stride(0) * 2, self.error.data_ptr(), L.stream_ptr()))

    def error_word(self) -> int:
        torch.cuda.synchronize()
        return int(self.error.item()) & 0xFFFFFFFF


def hot_experts(logits: np.ndarray, selected: int, count: int) -> list[int]:
    """The `count` experts that receive the most routes of a calibration batch (host side, outside any timed region)."""
    if count <= 0:
        return []
    ids = np.argsort(-logits, axis=1, kind="stable")[:, :selected]
    loads = np.bincount(ids.ravel(), minlength=logits.shape[1])
    return sorted(np.argsort(-loads, kind="stable")[:count].tolist())


# --------------------------------------------------------------------------------------------------
# bench.py --gpus N (N > 1)
# --------------------------------------------------------------------------------------------------
def _timed(fn, steps, warmup, dev):
    """`steps` calls of fn between two barriers, CUDA events on the launching stream, maximum over the ranks (ms per step)."""
    for i in range(warmup):
        fn(i)
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def _phase(ctx, args, rank, world, dev, prefill: bool, T: int, layers_n: int, nb: int, replicate: int, scratch=None):
    """One workload (decode batch or prefill batch per rank) through the expert-parallel layer: resident and end-to-end timing."""
    from . import synth
    from bench import CHANNELS, HIDDEN, EXPERTS, SELECTED
    bias = synth.zipf_bias(5, EXPERTS) if prefill else None
    # the replicated set comes from a calibration batch every rank can generate for itself (same seed everywhere)
    rep = hot_experts(synth.router_logits(1999, min(T, 1024), EXPERTS, bias), SELECTED, replicate) if replicate else []
    layers = [EpLayer(ctx, 100 + i, CHANNELS, HIDDEN, EXPERTS, SELECTED, dev, T, prefill=prefill, replicated=rep, scratch=scratch) for i in range(layers_n)]
    for l in layers[1:]:
        l.scratch = layers[0].scratch
    host_x = [torch.from_numpy(synth.activations_f16(1000 + rank * 64 + b, T, CHANNELS)).pin_memory() for b in range(nb)]
    host_lg = [torch.from_numpy(synth.router_logits(2000 + rank * 64 + b, T, EXPERTS, bias)).pin_memory() for b in range(nb)]
    dev_x, dev_lg = [t.to(dev) for t in host_x], [t.to(dev) for t in host_lg]
    out = torch.zeros((T, CHANNELS), dtype=torch.float16, device=dev)
    host_out = torch.zeros((T, CHANNELS), dtype=torch.float16).pin_memory()
    sx, slg = torch.zeros_like(dev_x[0]), torch.zeros_like(dev_lg[0])
    stream = torch.cuda.current_stream()

    def resident(i):
        layers[i % len(layers)].step(dev_x[i % nb], dev_lg[i % nb], out)

    def e2e(i):
        sx.copy_(host_x[i % nb], non_blocking=True)
        slg.copy_(host_lg[i % nb], non_blocking=True)
        layers[i % len(layers)].step(sx, slg, out)
        host_out.copy_(out, non_blocking=True)
        stream.synchronize()

    steps, warmup = (max(3, args.steps // 4), max(3, args.warmup)) if prefill else (args.steps, max(3, args.warmup))
    ms = _timed(resident, steps, warmup, dev)
    ms_e2e = _timed(e2e, steps, warmup, dev)
    err = torch.tensor([sum(l.error_word() for l in layers)], device=dev)
    dist.all_reduce(err, op=dist.ReduceOp.MAX)
    assert int(err.item()) == 0, "device error word set during the benchmark"
    # parity of this rank's rows of batch 0 against the CPU oracle needs the whole layer's weights: done at N = 1 only
    return {"ms": ms, "ms_e2e": ms_e2e, "tokens_per_rank": T, "replicated_experts": len(rep), "layers": layers, "steps": steps}


def run_bench(args, rank: int, world: int, local: int) -> None:
    """`bench.py --gpus N` for N > 1: every rank brings its own batch (weak scaling), experts are sharded 512/N per GPU, dispatch and
    combine are NCCL all-to-all exchanges inside one C call per layer step; value = all ranks' tokens / max-over-ranks device time."""
    from . import synth
    from bench import CHANNELS, HIDDEN, EXPERTS, SELECTED, ClockSampler, GGUF_EXPERT_GATE_UP, GGUF_EXPERT_DOWN, FLOPS_PER_ROUTE, peaks
    dev = torch.device("cuda", local)
    ctx = EpContext(rank, world, dev)
    T = args.tokens
    nb = 8
    with ClockSampler(local) as clocks:
        dec = _phase(ctx, args, rank, world, dev, False, T, args.layers, nb, 0)
        scratch = dec["layers"][0].scratch
        dec["layers"] = None
        torch.cuda.empty_cache()
        pre = None
        if not getattr(args, "no_prefill", False):
            pre = _phase(ctx, args, rank, world, dev, True, args.prefill_tokens, 1, 2, args.replicate)
            pre["layers"] = None
    if rank == 0:
        hbm_peak, tf_peak, peak_kind = peaks()
        total = T * world
        # algorithmic bytes of a decode step per GPU: the experts its batch of the step hits among the experts it owns, read once
        per = EXPERTS // world
        uniq = []
        for b in range(nb):
            ids = np.concatenate([np.argsort(-synth.router_logits(2000 + r * 64 + b, T, EXPERTS), axis=1, kind="stable")[:, :SELECTED].ravel() for r in range(world)])
            hit = np.unique(ids)
            uniq.append(max(int(((hit // per) == g).sum()) for g in range(world)))
        u_max = float(np.mean(uniq))
        step_bytes = (u_max + 1) * (GGUF_EXPERT_GATE_UP + GGUF_EXPERT_DOWN)
        line = {"metric": "moe_q4k_expert_gemm_tokens_per_s", "value": total / (dec["ms"] * 1e-3), "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": dec["ms"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f16 activations, f32 accumulate", "data": "synthetic",
                "config": {"workload": f"moe_layer_decode_T{T}_per_gpu (BASELINE configs[1] shape, expert-parallel as configs[4])",
                           "hidden": CHANNELS, "experts": EXPERTS, "expert_ffn": HIDDEN, "top_k": SELECTED, "weights": "Q4_K Pack-v3 planar",
                           "parallelism": f"ep{world}", "experts_per_gpu": EXPERTS // world, "tokens_per_gpu": T,
                           "collectives": "NCCL all-to-all dispatch (binary16 token rows, each token once per destination rank, fixed-size slabs with a "
                                          "device-side count) + NCCL all-to-all combine (per-row partial sums); no host synchronisation in a step",
                           "l2_policy": "layers rotate; per step each GPU streams its hit experts once"},
                "e2e": {"value": total / (dec["ms_e2e"] * 1e-3), "unit": "tokens/s", "ms_per_step": dec["ms_e2e"],
                        "h2d_bytes_per_step": world * (T * CHANNELS * 2 + T * EXPERTS * 4), "d2h_bytes_per_step": world * T * CHANNELS * 2},
                "gpu_launches": 17 * args.steps, "clocks": clocks.summary(),
                "roofline": {"bound": "hbm", "kernel": "whole expert-parallel decode step on the busiest GPU (its hit experts + the shared expert, gate-up and down)",
                             "achieved": step_bytes / (dec["ms"] * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                             "frac": step_bytes / (dec["ms"] * 1e-3) / 1e9 / hbm_peak, "peak_kind": peak_kind, "traffic": None,
                             "algorithmic_bytes_per_step": step_bytes, "experts_hit_on_busiest_gpu": u_max},
                "cpu_baseline": {"value": None, "unit": "tokens/s", "cores": 0, "kind": "reference",
                                 "sample": "not timed at N > 1: the CPU arm is measured by the one-GPU run (rank 0, N = 1) and by --impl reference"},
                "extra": {}}
        if pre is not None:
            Tp = pre["tokens_per_rank"]
            flops = world * Tp * (SELECTED + 1) * FLOPS_PER_ROUTE
            line["extra"]["prefill"] = {"tokens_per_s": world * Tp / (pre["ms"] * 1e-3), "ms_per_step": pre["ms"], "tokens_per_gpu": Tp,
                                        "e2e_tokens_per_s": world * Tp / (pre["ms_e2e"] * 1e-3), "tflops": flops / (pre["ms"] * 1e-3) / 1e12,
                                        "frac_of_bf16_peak_all_gpus": flops / (pre["ms"] * 1e-3) / 1e12 / (tf_peak * world),
                                        "replicated_experts": pre["replicated_experts"], "router": "N(0,1) + Zipf(1.1) per-expert bias", "scaling": "weak"}
        print(json.dumps(line), flush=True)
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()
