"""Expert parallelism over the GPUs of one node: experts sharded by contiguous id range, tokens data-parallel by
source rank, one all-to-all each way (dispatch of routed rows, combine of per-route outputs) over NCCL.

The reference is single-GPU; this is the multi-GPU form of its MoE layer with identical per-route arithmetic: a route's
expert output is computed on the rank that owns the expert by the same kernels, returned to the token's rank, and mixed
there in route-rank order with the locally computed shared expert, so the layer output equals the one-GPU output.

`torch.distributed` is the plumbing (process group, all_to_all_single); sort / gather / scatter of route rows use torch
index ops. No TMA multicast and no peer-memory operand is involved: received rows sit in local HBM before any kernel
touches them.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist


class RoutePlan:
    """Where each local route goes and how the returned rows map back. Pure index logic (device-agnostic)."""

    def __init__(self, ids: torch.Tensor, experts: int, world: int, group=None):
        T, K = ids.shape
        per = experts // world
        flat = ids.reshape(-1).to(torch.int64)
        dest = torch.div(flat, per, rounding_mode="floor")
        # stable sort by destination keeps (token, slot) order inside each destination: deterministic layouts
        self.order = torch.sort(dest, stable=True).indices
        self.send_counts = torch.bincount(dest, minlength=world).to(torch.int64)
        self.recv_counts = torch.empty_like(self.send_counts)
        dist.all_to_all_single(self.recv_counts, self.send_counts, group=group)
        both = torch.stack([self.send_counts, self.recv_counts]).cpu()   # the one host synchronisation of a step
        self.send_splits = both[0].tolist()
        self.recv_splits = both[1].tolist()
        self.token_of_route = torch.div(self.order, K, rounding_mode="floor")
        self.local_expert = (flat[self.order] % per).to(torch.int32)
        self.received = int(sum(self.recv_splits))
        self.routes = T * K


def dispatch(plan: RoutePlan, rows: torch.Tensor, group=None):
    """rows: [T, C] on the source. Returns (received rows [R, C], their local expert ids [R])."""
    send_rows = rows.index_select(0, plan.token_of_route)
    recv_rows = rows.new_empty((plan.received, rows.shape[1]))
    dist.all_to_all_single(recv_rows, send_rows, plan.recv_splits, plan.send_splits, group=group)
    recv_ids = plan.local_expert.new_empty(plan.received)
    dist.all_to_all_single(recv_ids, plan.local_expert, plan.recv_splits, plan.send_splits, group=group)
    return recv_rows, recv_ids


def combine(plan: RoutePlan, outputs: torch.Tensor, routed: torch.Tensor, group=None) -> None:
    """outputs: [R, C] per received route. Writes routed[token*K + slot] for every local route."""
    back = outputs.new_empty((plan.routes, outputs.shape[1]))
    dist.all_to_all_single(back, outputs, plan.send_splits, plan.recv_splits, group=group)
    routed.index_copy_(0, plan.order, back)


# --------------------------------------------------------------------------------------------------
# CUDA side: one rank's share of a layer
# --------------------------------------------------------------------------------------------------
class EpLayer:
    def __init__(self, seed: int, channels: int, hidden: int, experts: int, selected: int, rank: int, world: int, device, capacity: int,
                 expert_type: int = 12, layout: int = 1, prefill: bool = False):
        from . import layer as L
        assert experts % world == 0
        self.rank, self.world, self.C, self.H, self.E, self.K = rank, world, channels, hidden, experts, selected
        per = experts // world
        self.per = per
        self.w = L.SynthDeviceLayer(seed, channels, hidden, experts, expert_type, layout, device, expert_range=(rank * per, (rank + 1) * per))
        self.device = device
        self.capacity = capacity   # token rows per rank per step
        max_recv = capacity * selected * world
        f32, i32 = torch.float32, torch.int32
        z = lambda n, dt: torch.zeros(max(int(n), 1), dtype=dt, device=device)
        self.ids = z(capacity * selected, i32)
        self.weights = z(capacity * selected, f32)
        self.routed = torch.zeros((capacity * selected, channels), dtype=f32, device=device)
        self.shared_hidden = z(capacity * hidden, f32)
        self.shared_out = z(capacity * channels, f32)
        self.shared_logit = z(capacity, f32)
        self.x32 = z(capacity * channels, f32)
        self.recv32 = z(max_recv * channels, f32)
        self.hid = z(max_recv * hidden, f32)
        self.y = torch.zeros((max_recv, channels), dtype=f32, device=device)
        self.token_map = z(per * max_recv, i32)
        self.counts = z(per, i32)
        self.tasks = z(max_recv + 2 * per + 2, i32)
        self.error = z(1, i32)
        # buffers of the gathered (all-gather / reduce-scatter) scheme: every rank sees all world*capacity token rows
        G = capacity * world
        self.pack = torch.zeros((capacity, channels * 2 + experts * 4), dtype=torch.uint8, device=device)
        self.gathered = torch.zeros((G, channels * 2 + experts * 4), dtype=torch.uint8, device=device)
        self.g_x32 = z(G * channels, f32)
        self.g_ids = z(G * selected, i32)
        self.g_weights = z(G * selected, f32)
        self.g_hid = z(G * selected * hidden, f32)
        self.g_routed = torch.zeros((G * selected, channels), dtype=f32, device=device)
        self.g_token_map = z(per * G, i32)
        self.g_tasks = z(G * selected + 2 * per + 2, i32)
        self.g_partial = torch.zeros((G, channels), dtype=f32, device=device)
        self.g_zero = torch.zeros((G, channels), dtype=f32, device=device)
        self.rs_out = torch.zeros((capacity, channels), dtype=f32, device=device)
        self.ones = torch.ones(capacity, dtype=f32, device=device)
        if prefill:
            # prefill-size gathered scheme: the local experts' routes of all world*capacity rows through the grouped tensor-core
            # GEMMs (permuted binary16 rows), the shared expert of the local rows through the same kernels
            from . import capi
            f16 = torch.float16
            R = G * selected
            self.p_tasks = z(int(capi.lib().tsp_moe_tasks_words(G, per, selected, 128)), i32)
            self.p_offsets = z(per + 1, i32)
            self.p_pos_route = z(R, i32)
            self.p_xp = torch.zeros((R, channels), dtype=f16, device=device)
            self.p_hp = torch.zeros((R, hidden), dtype=f16, device=device)
            self.s_ids0 = z(capacity, i32)
            self.s_token_map, self.s_counts, self.s_offsets, self.s_pos = z(capacity, i32), z(1, i32), z(2, i32), z(capacity, i32)
            self.s_tasks = z(int(capi.lib().tsp_moe_tasks_words(capacity, 1, 1, 128)), i32)
            self.s_xp = torch.zeros((capacity, channels), dtype=f16, device=device)
            self.s_hp = torch.zeros((capacity, hidden), dtype=f16, device=device)

    def step(self, x16: torch.Tensor, logits: torch.Tensor, out16: torch.Tensor) -> None:
        from . import capi
        from . import layer as L
        lib, st, e = capi.lib(), L.stream_ptr(), self.error.data_ptr()
        T, Cn, H, K = x16.shape[0], self.C, self.H, self.K
        w = self.w.weights
        capi.check(lib.tsp_moe_route(logits.data_ptr(), logits.stride(0) * 4, T, self.E, K, 0, 1, self.ids.data_ptr(), self.weights.data_ptr(), e, st))
        plan = RoutePlan(self.ids[: T * K].view(T, K), self.E, self.world)
        rows, lids = dispatch(plan, x16)
        R = plan.received
        if R:
            capi.check(lib.tsp_rows_f16_to_f32(rows.data_ptr(), Cn * 2, self.recv32.data_ptr(), Cn * 4, R, Cn, st))
            capi.check(lib.tsp_moe_permute(lids.data_ptr(), R, self.per, 1, capi.GEMV_TILE, self.token_map.data_ptr(), self.counts.data_ptr(),
                                           self.tasks.data_ptr(), e, st))
            capi.check(lib.tsp_moe_gate_up_swiglu(C.byref(w.gate), C.byref(w.up), self.recv32.data_ptr(), Cn * 4, R, 1, self.token_map.data_ptr(),
                                                  self.counts.data_ptr(), self.tasks.data_ptr(), self.hid.data_ptr(), H * 4, 1, e, st))
            capi.check(lib.tsp_moe_project(C.byref(w.down), self.hid.data_ptr(), H * 4, 1, R, 1, self.token_map.data_ptr(), self.counts.data_ptr(),
                                           self.tasks.data_ptr(), self.y.data_ptr(), Cn * 4, 0, e, st))
        combine(plan, self.y[:R], self.routed)
        # local: shared expert and the gated mixture in route-rank order
        capi.check(lib.tsp_rows_f16_to_f32(x16.data_ptr(), x16.stride(0) * 2, self.x32.data_ptr(), Cn * 4, T, Cn, st))
        capi.check(lib.tsp_moe_gate_up_swiglu(C.byref(w.shared_gate), C.byref(w.shared_up), self.x32.data_ptr(), Cn * 4, T, 1, None, None, None,
                                              self.shared_hidden.data_ptr(), H * 4, 1, e, st))
        capi.check(lib.tsp_moe_project(C.byref(w.shared_down), self.shared_hidden.data_ptr(), H * 4, 1, T, 1, None, None, None,
                                       self.shared_out.data_ptr(), Cn * 4, 0, e, st))
        capi.check(lib.tsp_moe_combine(self.routed.data_ptr(), Cn * 4, 0, self.weights.data_ptr(), self.shared_out.data_ptr(), Cn * 4,
                                       w.d_shared_router, self.x32.data_ptr(), Cn * 4, 0, self.shared_logit.data_ptr(), T, Cn, K, None, 0,
                                       out16.data_ptr(), out16.stride(0) * 2, e, st))

    def step_gathered(self, x16: torch.Tensor, logits: torch.Tensor, out16: torch.Tensor) -> None:
        """Small-batch scheme without any host synchronisation: all-gather the token rows and router logits (every rank then
        routes all rows itself), compute the routes that hit local experts, mix them per token into partial sums, and
        reduce-scatter the partial sums back to the tokens' ranks. For decode batches the bytes moved equal those of the
        all-to-all form (with top-10 of 8 ranks nearly every row visits most ranks anyway) and both collectives have fixed
        sizes. The mixture adds the ranks' partial sums instead of walking the routes in rank order, so the result agrees with
        the one-GPU layer to FP32 rounding, not bit for bit."""
        from . import capi
        from . import layer as L
        lib, st, e = capi.lib(), L.stream_ptr(), self.error.data_ptr()
        T, Cn, H, K, E, per = x16.shape[0], self.C, self.H, self.K, self.E, self.per
        assert T == self.capacity, "the gathered scheme runs at the capacity it was built for"
        G = T * self.world
        w = self.w.weights
        rowb = Cn * 2 + E * 4
        self.pack[:, : Cn * 2].copy_(x16.view(torch.uint8).view(T, Cn * 2))
        self.pack[:, Cn * 2:].copy_(logits.view(torch.uint8).view(T, E * 4))
        dist.all_gather_into_tensor(self.gathered, self.pack)
        gx, glg = self.gathered.data_ptr(), self.gathered.data_ptr() + Cn * 2
        capi.check(lib.tsp_rows_f16_to_f32(gx, rowb, self.g_x32.data_ptr(), Cn * 4, G, Cn, st))
        capi.check(lib.tsp_moe_route(glg, rowb, G, E, K, 0, 1, self.g_ids.data_ptr(), self.g_weights.data_ptr(), e, st))
        capi.check(lib.tsp_moe_permute_local(self.g_ids.data_ptr(), G, self.rank * per, per, K, capi.GEMV_TILE, self.g_token_map.data_ptr(),
                                             self.counts.data_ptr(), self.g_tasks.data_ptr(), e, st))
        capi.check(lib.tsp_moe_gate_up_swiglu(C.byref(w.gate), C.byref(w.up), self.g_x32.data_ptr(), Cn * 4, G, K, self.g_token_map.data_ptr(),
                                              self.counts.data_ptr(), self.g_tasks.data_ptr(), self.g_hid.data_ptr(), H * 4, 1, e, st))
        capi.check(lib.tsp_moe_project(C.byref(w.down), self.g_hid.data_ptr(), H * 4, 1, G, K, self.g_token_map.data_ptr(), self.counts.data_ptr(),
                                       self.g_tasks.data_ptr(), self.g_routed.data_ptr(), Cn * 4, 0, e, st))
        local = (self.g_ids >= self.rank * per) & (self.g_ids < (self.rank + 1) * per)
        w_local = torch.where(local, self.g_weights, torch.zeros_like(self.g_weights))   # zero weight = route not computed here
        capi.check(lib.tsp_moe_combine(self.g_routed.data_ptr(), Cn * 4, 0, w_local.data_ptr(), self.g_zero.data_ptr(), Cn * 4, None, None, 0, 0, None,
                                       G, Cn, K, self.g_partial.data_ptr(), Cn * 4, None, 0, e, st))
        dist.reduce_scatter_tensor(self.rs_out, self.g_partial)
        x_local = self.g_x32.data_ptr() + self.rank * T * Cn * 4
        capi.check(lib.tsp_moe_gate_up_swiglu(C.byref(w.shared_gate), C.byref(w.shared_up), x_local, Cn * 4, T, 1, None, None, None,
                                              self.shared_hidden.data_ptr(), H * 4, 1, e, st))
        capi.check(lib.tsp_moe_project(C.byref(w.shared_down), self.shared_hidden.data_ptr(), H * 4, 1, T, 1, None, None, None,
                                       self.shared_out.data_ptr(), Cn * 4, 0, e, st))
        capi.check(lib.tsp_moe_combine(self.rs_out.data_ptr(), Cn * 4, 0, self.ones.data_ptr(), self.shared_out.data_ptr(), Cn * 4,
                                       w.d_shared_router, x_local, Cn * 4, 0, self.shared_logit.data_ptr(), T, Cn, 1, None, 0,
                                       out16.data_ptr(), out16.stride(0) * 2, e, st))

    def step_gathered_prefill(self, x16: torch.Tensor, logits: torch.Tensor, out16: torch.Tensor) -> None:
        """The gathered scheme at prefill size: all-gather rows + logits, route everything on every rank, run the routes that hit
        local experts through the grouped tcgen05 GEMMs (tiles of 128 routes), mix them per token into partial sums,
        reduce-scatter the partial sums, then add the local rows' shared expert. No host synchronisation, fixed-size collectives."""
        from . import capi
        from . import layer as L
        lib, st, e = capi.lib(), L.stream_ptr(), self.error.data_ptr()
        T, Cn, H, K, E, per = x16.shape[0], self.C, self.H, self.K, self.E, self.per
        assert T == self.capacity, "the gathered scheme runs at the capacity it was built for"
        G = T * self.world
        R = G * K
        w = self.w.weights
        rowb = Cn * 2 + E * 4
        self.pack[:, : Cn * 2].copy_(x16.view(torch.uint8).view(T, Cn * 2))
        self.pack[:, Cn * 2:].copy_(logits.view(torch.uint8).view(T, E * 4))
        dist.all_gather_into_tensor(self.gathered, self.pack)
        gx, glg = self.gathered.data_ptr(), self.gathered.data_ptr() + Cn * 2
        capi.check(lib.tsp_rows_f16_to_f32(gx, rowb, self.g_x32.data_ptr(), Cn * 4, G, Cn, st))
        capi.check(lib.tsp_moe_route(glg, rowb, G, E, K, 0, 1, self.g_ids.data_ptr(), self.g_weights.data_ptr(), e, st))
        capi.check(lib.tsp_moe_permute_local(self.g_ids.data_ptr(), G, self.rank * per, per, K, 128, self.g_token_map.data_ptr(),
                                             self.counts.data_ptr(), self.p_tasks.data_ptr(), e, st))
        capi.check(lib.tsp_moe_route_offsets(self.counts.data_ptr(), per, self.p_offsets.data_ptr(), st))
        capi.check(lib.tsp_moe_gather_rows(self.g_x32.data_ptr(), Cn * 4, K, self.g_token_map.data_ptr(), self.p_offsets.data_ptr(), per, G, K, Cn,
                                           self.p_xp.data_ptr(), Cn * 2, self.p_pos_route.data_ptr(), e, st))
        capi.check(lib.tsp_moe_grouped_gate_up(C.byref(w.gate), C.byref(w.up), self.p_xp.data_ptr(), Cn * 2, R, self.p_tasks.data_ptr(),
                                               self.counts.data_ptr(), self.p_offsets.data_ptr(), self.p_hp.data_ptr(), H * 2, e, st))
        capi.check(lib.tsp_moe_grouped_down(C.byref(w.down), self.p_hp.data_ptr(), H * 2, R, self.p_tasks.data_ptr(), self.counts.data_ptr(),
                                            self.p_offsets.data_ptr(), self.p_pos_route.data_ptr(), self.g_routed.data_ptr(), Cn * 4, e, st))
        local = (self.g_ids >= self.rank * per) & (self.g_ids < (self.rank + 1) * per)
        w_local = torch.where(local, self.g_weights, torch.zeros_like(self.g_weights))   # zero weight = route not computed here
        capi.check(lib.tsp_moe_combine(self.g_routed.data_ptr(), Cn * 4, 0, w_local.data_ptr(), self.g_zero.data_ptr(), Cn * 4, None, None, 0, 0, None,
                                       G, Cn, K, self.g_partial.data_ptr(), Cn * 4, None, 0, e, st))
        dist.reduce_scatter_tensor(self.rs_out, self.g_partial)
        x_local = self.g_x32.data_ptr() + self.rank * T * Cn * 4
        capi.check(lib.tsp_moe_permute(self.s_ids0.data_ptr(), T, 1, 1, 128, self.s_token_map.data_ptr(), self.s_counts.data_ptr(),
                                       self.s_tasks.data_ptr(), e, st))
        capi.check(lib.tsp_moe_route_offsets(self.s_counts.data_ptr(), 1, self.s_offsets.data_ptr(), st))
        capi.check(lib.tsp_moe_gather_rows(x_local, Cn * 4, 1, self.s_token_map.data_ptr(), self.s_offsets.data_ptr(), 1, T, 1, Cn,
                                           self.s_xp.data_ptr(), Cn * 2, self.s_pos.data_ptr(), e, st))
        capi.check(lib.tsp_moe_grouped_gate_up(C.byref(w.shared_gate), C.byref(w.shared_up), self.s_xp.data_ptr(), Cn * 2, T, self.s_tasks.data_ptr(),
                                               self.s_counts.data_ptr(), self.s_offsets.data_ptr(), self.s_hp.data_ptr(), H * 2, e, st))
        capi.check(lib.tsp_moe_grouped_down(C.byref(w.shared_down), self.s_hp.data_ptr(), H * 2, T, self.s_tasks.data_ptr(), self.s_counts.data_ptr(),
                                            self.s_offsets.data_ptr(), self.s_pos.data_ptr(), self.shared_out.data_ptr(), Cn * 4, e, st))
        capi.check(lib.tsp_moe_combine(self.rs_out.data_ptr(), Cn * 4, 0, self.ones.data_ptr(), self.shared_out.data_ptr(), Cn * 4,
                                       w.d_shared_router, x_local, Cn * 4, 0, self.shared_logit.data_ptr(), T, Cn, 1, None, 0,
                                       out16.data_ptr(), out16.stride(0) * 2, e, st))

    def error_word(self) -> int:
        torch.cuda.synchronize()
        return int(self.error.item()) & 0xFFFFFFFF


def run_bench(args, rank: int, world: int, local: int) -> None:
    """`bench.py --gpus N` for N > 1: every rank brings its own batch of `args.tokens` rows (weak scaling), experts are
    sharded 512/N per GPU; value = all ranks' tokens / max-over-ranks device time."""
    from . import synth
    from bench import CHANNELS, HIDDEN, EXPERTS, SELECTED, ClockSampler
    dev = torch.device("cuda", local)
    prefill = getattr(args, "workload", "decode") == "prefill"
    T = 4096 if prefill and args.tokens == 64 else args.tokens
    layers = [EpLayer(100 + i, CHANNELS, HIDDEN, EXPERTS, SELECTED, rank, world, dev, T, prefill=prefill) for i in range(2 if prefill else args.layers)]
    nb = 2 if prefill else 8
    bias = synth.zipf_bias(5, EXPERTS) if prefill else None
    host_x = [torch.from_numpy(synth.activations_f16(1000 + rank * 64 + b, T, CHANNELS)).pin_memory() for b in range(nb)]
    host_lg = [torch.from_numpy(synth.router_logits(2000 + rank * 64 + b, T, EXPERTS, bias) if prefill else synth.router_logits(2000 + rank * 64 + b, T, EXPERTS)).pin_memory()
               for b in range(nb)]
    dev_x = [t.to(dev) for t in host_x]
    dev_lg = [t.to(dev) for t in host_lg]
    out = torch.zeros((T, CHANNELS), dtype=torch.float16, device=dev)
    host_out = torch.zeros((T, CHANNELS), dtype=torch.float16).pin_memory()
    sx = torch.zeros((T, CHANNELS), dtype=torch.float16, device=dev)
    slg = torch.zeros((T, EXPERTS), dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream()
    step = EpLayer.step if getattr(args, "ep_scheme", "gather") == "alltoall" else EpLayer.step_gathered
    if prefill:
        step = EpLayer.step_gathered_prefill

    def resident(i):
        step(layers[i % len(layers)], dev_x[i % nb], dev_lg[i % nb], out)

    def e2e(i):
        sx.copy_(host_x[i % nb], non_blocking=True)
        slg.copy_(host_lg[i % nb], non_blocking=True)
        step(layers[i % len(layers)], sx, slg, out)
        host_out.copy_(out, non_blocking=True)
        stream.synchronize()

    def timed(fn):
        for i in range(args.warmup):
            fn(i)
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            fn(args.warmup + i)
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    with ClockSampler(local) as clocks:
        ms = timed(resident)
        ms_e2e = timed(e2e)
    err = torch.tensor([sum(l.error_word() for l in layers)], device=dev)
    dist.all_reduce(err, op=dist.ReduceOp.MAX)
    assert int(err.item()) == 0, "device error word set during the benchmark"
    if rank == 0:
        total = T * world
        line = {"metric": "moe_q4k_expert_gemm_tokens_per_s", "value": total / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": (f"moe_layer_prefill_T{T}_per_gpu (BASELINE configs[2] shape and router, expert-parallel as configs[4])" if prefill
                                        else f"moe_layer_decode_T{T}_per_gpu (BASELINE configs[1] shape, expert-parallel as configs[4])"),
                           "hidden": CHANNELS, "experts": EXPERTS, "expert_ffn": HIDDEN, "top_k": SELECTED, "weights": "Q4_K Pack-v3 planar",
                           "parallelism": f"ep{world}", "experts_per_gpu": EXPERTS // world, "tokens_per_gpu": T,
                           "collectives": ("NCCL all-to-all dispatch (binary16 rows) + all-to-all combine (FP32 rows), one count exchange" if step is EpLayer.step
                                           else "NCCL all-gather of token rows + logits, reduce-scatter of per-token partial sums (FP32)"),
                           "l2_policy": "layers rotate; per step each GPU streams its hit experts once"},
                "e2e": {"value": total / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                        "h2d_bytes_per_step": world * (T * CHANNELS * 2 + T * EXPERTS * 4), "d2h_bytes_per_step": world * T * CHANNELS * 2},
                "gpu_launches": (19 if prefill else 10 if step is EpLayer.step else 12) * args.steps, "clocks": clocks.summary(),
                "roofline": None, "cpu_baseline": None}
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
