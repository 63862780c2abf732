#!/usr/bin/env python
"""Benchmark of the routed-MoE FFN hot path (BASELINE metric: MoE Q4_K expert-GEMM tokens/s).

A "step" is one pass of one MoE layer (hidden 2048, 512 routed experts of FFN 512 in Q4_K, top-10, one gated
shared expert) over one fresh batch of synthetic tokens. At N=1 the workload is BASELINE configs[1] at its
largest batch (decode, 64 tokens). Layers rotate over several independently seeded weight sets and every step
takes a different batch, so the bytes a step streams (~650 MB) never sit in the 126 MB L2.

  value     tokens/s with inputs already resident in HBM (CUDA events, max over ranks)
  e2e       tokens/s through the C ABI from pinned HOST buffers: H2D of x and logits and D2H of the
            output rows inside the timed region, one synchronisation per step
  roofline  the dominant kernel (routed gate-up + SwiGLU): algorithmic GGUF bytes / its CUDA-event time
  cpu_baseline  the reference's own CPU composition (oracle/_ref, else the C port) on the host cores

`--impl reference` times that CPU implementation alone (rank 0 only under torchrun).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CHANNELS, HIDDEN, EXPERTS, SELECTED = 2048, 512, 512, 10
GGUF_EXPERT_GATE_UP = 2 * HIDDEN * (CHANNELS // 256) * 144   # 1 179 648 B
GGUF_EXPERT_DOWN = CHANNELS * (HIDDEN // 256) * 144          #   589 824 B
FLOPS_PER_ROUTE = 2 * (2 * HIDDEN * CHANNELS + CHANNELS * HIDDEN)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) every few milliseconds while a timed region runs."""

    def __init__(self, index: int, period_s: float = 0.003):
        self.index, self.period, self.sm, self.reasons, self.max_mhz, self.stop = index, period_s, [], set(), None, False
        self.thread = None

    def __enter__(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            h = nv.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            bits = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                    "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}

            def loop():
                while not self.stop:
                    try:
                        self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                        r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                        for name, bit in bits.items():
                            if r & bit:
                                self.reasons.add(name)
                    except Exception:
                        pass
                    time.sleep(self.period)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        return self

    def __exit__(self, *a):
        self.stop = True
        if self.thread:
            self.thread.join(timeout=2)

    def summary(self):
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.sm)}


# --------------------------------------------------------------------------------------------------
# reference arm: the reference's own CPU implementation, host cores only
# --------------------------------------------------------------------------------------------------
def cpu_layer_inputs(tokens: int, seed: int):
    from tokspur_public_b200 import synth
    x16 = synth.activations_f16(seed * 2 + 1, tokens, CHANNELS)
    logits = synth.router_logits(seed * 2 + 2, tokens, EXPERTS)
    return x16, logits


def host_layer_numpy(seed: int, needed: np.ndarray):
    """GGUF bytes of the experts in `needed` only (all others stay zero and are never touched by the routed tokens)."""
    from tokspur_public_b200 import formats, synth
    from tokspur_public_b200.layer import HostLayer
    gb = formats.gguf_bytes(formats.Q4_K, HIDDEN, CHANNELS)
    rng = np.random.default_rng(seed)
    q = lambda r, c: formats.quantize_q4_k((rng.standard_normal((r, c), dtype=np.float32) * np.float32(0.02))).reshape(-1)
    g = np.zeros((EXPERTS, gb), np.uint8); u = np.zeros((EXPERTS, gb), np.uint8); d = np.zeros((EXPERTS, gb), np.uint8)
    for e in needed:
        g[e], u[e], d[e] = q(HIDDEN, CHANNELS), q(HIDDEN, CHANNELS), q(CHANNELS, HIDDEN)
    return HostLayer(CHANNELS, HIDDEN, EXPERTS, SELECTED, formats.Q4_K, formats.Q4_K, g, u, d, q(HIDDEN, CHANNELS), q(HIDDEN, CHANNELS),
                     q(CHANNELS, HIDDEN), synth.normal(seed + 5, (CHANNELS,), 0.02))


def cpu_oracle():
    from oracle.oracle import Oracle, have_reference
    if have_reference():
        return Oracle(reference=True), "reference"
    return Oracle(), "port"


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    orc, kind = cpu_oracle()
    cores = os.cpu_count() or 1
    sample = min(args.cpu_tokens or cores, 64)
    x16, logits = cpu_layer_inputs(sample, 7)
    ids, _ = __import__("oracle.oracle", fromlist=["Oracle"]).Oracle().route_rows(logits.astype(np.float64), SELECTED)
    host = host_layer_numpy(11, np.unique(ids))
    layer = host.oracle_dict()
    x = x16.astype(np.float32)
    for _ in range(min(args.warmup, 1)):
        orc.moe_layer(layer, x[: max(1, sample // 4)], logits[: max(1, sample // 4)], threads=cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.moe_layer(layer, x, logits, threads=min(cores, sample))
    dt = (time.perf_counter() - t0) / args.steps
    value = sample / dt
    line = {"impl": "reference", "metric": "moe_q4k_expert_gemm_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": "moe_layer_decode_T64 (BASELINE configs[1])", "hidden": CHANNELS, "experts": EXPERTS, "expert_ffn": HIDDEN,
                       "top_k": SELECTED, "weights": "Q4_K GGUF", "sample_tokens_per_step": sample},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": min(cores, sample), "kind": kind,
                             "sample": f"{sample} tokens of the 64-token batch per step, one layer, threads over tokens"},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------------
NCU_GATE_UP_DRAM_BYTES_PER_EXPERT = 457.2e6 / 361   # 360 routed experts + the shared expert in the captured launch


def run_ours(args):
    import torch
    import torch.distributed as dist
    from tokspur_public_b200 import capi, formats
    from tokspur_public_b200 import layer as L

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world > 1:
        from tokspur_public_b200 import ep
        return ep.run_bench(args, rank, world, local)

    if args.workload == "prefill":
        return run_prefill(args, local)
    if args.workload == "head":
        return run_head(args, local)
    dev = torch.device("cuda", local)
    T = args.tokens
    # Q4_K experts default to the Pack-v3 planar layout, Q8_0 experts (the MTP block) stay GGUF blocks
    lname = args.layout or ("gguf" if args.experts == "q8_0" else "planar")
    layout = formats.PLANAR if lname == "planar" else formats.GGUF
    etype = formats.Q8_0 if args.experts == "q8_0" else formats.Q4_K   # q8_0: the MTP block of BASELINE configs[3]
    blk_bytes, blk_cols = (34, 32) if etype == formats.Q8_0 else (144, 256)
    expert_gate_up = 2 * HIDDEN * (CHANNELS // blk_cols) * blk_bytes
    expert_down = CHANNELS * (HIDDEN // blk_cols) * blk_bytes
    layers = [L.SynthDeviceLayer(100 + i, CHANNELS, HIDDEN, EXPERTS, etype, layout, dev, keep_gguf=(i == 0))
              for i in range(args.layers)]
    scratch = L.Scratch(CHANNELS, HIDDEN, EXPERTS, SELECTED, T, dev)
    nb = 8
    from tokspur_public_b200 import synth
    host_x = [torch.from_numpy(synth.activations_f16(1000 + b, T, CHANNELS)).pin_memory() for b in range(nb)]
    host_lg = [torch.from_numpy(synth.router_logits(2000 + b, T, EXPERTS)).pin_memory() for b in range(nb)]
    dev_x = [t.to(dev) for t in host_x]
    dev_lg = [t.to(dev) for t in host_lg]
    out = torch.zeros((T, CHANNELS), dtype=torch.float16, device=dev)
    host_out = torch.zeros((T, CHANNELS), dtype=torch.float16).pin_memory()
    # end-to-end arm: a step's token rows and router logits travel as ONE pinned buffer and one host->device copy
    xb, lb = T * CHANNELS * 2, T * EXPERTS * 4
    host_pack = []
    for b_ in range(nb):
        hp = torch.empty(xb + lb, dtype=torch.uint8).pin_memory()
        hp[:xb].copy_(host_x[b_].view(torch.uint8).view(-1))
        hp[xb:].copy_(host_lg[b_].view(torch.uint8).view(-1))
        host_pack.append(hp)
    stage = torch.zeros(xb + lb, dtype=torch.uint8, device=dev)
    stage_x = stage[:xb].view(torch.float16).view(T, CHANNELS)
    stage_lg = stage[xb:].view(torch.float32).view(T, EXPERTS)
    stream = torch.cuda.current_stream()

    def step_resident(i):
        L.moe_layer_decode(layers[i % len(layers)], scratch, dev_x[i % nb], dev_lg[i % nb], out)

    def step_e2e(i):
        stage.copy_(host_pack[i % nb], non_blocking=True)
        L.moe_layer_decode(layers[i % len(layers)], scratch, stage_x, stage_lg, out)
        host_out.copy_(out, non_blocking=True)
        stream.synchronize()

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps  # ms per step

    with ClockSampler(local) as clocks:
        ms = timed(step_resident, args.steps, args.warmup)
        ms_e2e = timed(step_e2e, args.steps, args.warmup)
        stages = stage_times(L, capi, layers, scratch, dev_x, dev_lg, out, args.steps, args.warmup, T)
    assert scratch.error_word() == 0, "device error word set during the benchmark"
    clk = clocks.summary()

    hbm_peak, _, peak_kind = peaks()
    U = stages["unique_experts"]
    # the launch covers the routed experts that were hit plus the shared expert; activations in (binary16), hidden rows out (FP32)
    gu_bytes = (U + 1) * expert_gate_up + T * CHANNELS * 2 + T * (SELECTED + 1) * HIDDEN * 4
    layer_bytes = (U + 1) * (expert_gate_up + expert_down) + T * (CHANNELS * 2 * 2) + T * EXPERTS * 4
    achieved = gu_bytes / (stages["gate_up_ms"] * 1e-3) / 1e9
    kname = ("gemv3_kernel<planar, gate-up+SwiGLU> (routed experts + shared expert, one launch)" if etype == formats.Q4_K else
             "gemv_kernel<Q8_0, gate-up+SwiGLU> (routed experts, then the shared expert: two launches timed together)")
    roofline = {"bound": "hbm", "kernel": kname, "achieved": achieved, "peak": hbm_peak,
                "unit": "GB/s", "frac": achieved / hbm_peak, "peak_kind": peak_kind,
                # dram__bytes_read.sum + dram__bytes_write.sum of one captured launch (361 experts: 457.2 MB) scaled to the
                # experts this run's batches hit; traffic grows with the experts touched, the activations stay in L2
                "traffic": NCU_GATE_UP_DRAM_BYTES_PER_EXPERT * (U + 1) if etype == formats.Q4_K else None,
                "traffic_source": "ncu capture scaled by experts hit" if etype == formats.Q4_K else None,
                "algorithmic_bytes_per_launch": gu_bytes, "launch_ms": stages["gate_up_ms"]}

    # CPU baseline on the same first layer and batch 0, and an in-run parity figure
    cpu = None
    parity = None
    if args.cpu_tokens != 0:
        orc, kind = cpu_oracle()
        cores = os.cpu_count() or 1
        sample = min(args.cpu_tokens or T, T)
        host = layers[0].host_layer(SELECTED)
        x32 = host_x[0].numpy()[:sample].astype(np.float32)
        lg = host_lg[0].numpy()[:sample]
        t0 = time.perf_counter()
        want = orc.moe_layer(host.oracle_dict(), x32, lg, threads=min(cores, sample))
        dt = time.perf_counter() - t0
        cpu = {"value": sample / dt, "unit": "tokens/s", "cores": min(cores, sample), "kind": kind,
               "sample": f"{sample} of the {T} tokens of one batch, one layer, threads over tokens, {dt:.1f} s"}
        L.moe_layer_decode(layers[0], scratch, dev_x[0], dev_lg[0], out)
        torch.cuda.synchronize()
        got = out.cpu().numpy()[:sample].astype(np.float64)
        parity = float(np.linalg.norm(got - want) / np.linalg.norm(want))

    tokens_s = T / (ms * 1e-3)
    line = {"metric": "moe_q4k_expert_gemm_tokens_per_s", "value": tokens_s, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"moe_layer_decode_T{T} (BASELINE configs[1])" if etype == formats.Q4_K else f"q8_0_mtp_moe_block_T{T} (BASELINE configs[3])", "hidden": CHANNELS, "experts": EXPERTS, "expert_ffn": HIDDEN,
                       "top_k": SELECTED, "weights": ("Q8_0 " if etype == formats.Q8_0 else "Q4_K ") + ("Pack-v3 planar" if layout == formats.PLANAR else "GGUF"),
                       "activations": "binary16 in/out, FP32 accumulate", "layers_rotated": len(layers),
                       "l2_policy": "inputs larger than L2: each step streams ~650 MB of distinct expert weights"},
            "e2e": {"value": T / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": T * CHANNELS * 2 + T * EXPERTS * 4, "d2h_bytes_per_step": T * CHANNELS * 2},
            "gpu_launches": 4 * args.steps, "clocks": clk, "roofline": roofline, "cpu_baseline": cpu,
            "extra": {"layer_hbm_gbs": layer_bytes / (ms * 1e-3) / 1e9, "layer_hbm_frac": layer_bytes / (ms * 1e-3) / 1e9 / hbm_peak,
                      "layer_algorithmic_bytes": layer_bytes, "unique_experts": U, "stage_ms": stages, "parity_rel_l2_vs_cpu": parity,
                      "layer_tflops": T * (SELECTED + 1) * FLOPS_PER_ROUTE / (ms * 1e-3) / 1e12}}
    print(json.dumps(line), flush=True)


def run_prefill(args, local):
    """BASELINE configs[2]: one MoE layer over 4096 tokens, router logits N(0,1) + per-expert Zipf(1.1) bias, through the
    grouped tcgen05 GEMMs. The line's roofline is the tensor bound of the routed gate-up GEMM."""
    import torch
    from tokspur_public_b200 import capi, formats, synth
    from tokspur_public_b200 import layer as L
    dev = torch.device("cuda", local)
    T = args.tokens if args.tokens != 64 else 4096
    layers = [L.SynthDeviceLayer(100 + i, CHANNELS, HIDDEN, EXPERTS, formats.Q4_K, formats.PLANAR, dev, keep_gguf=(i == 0)) for i in range(min(args.layers, 2))]
    ps = L.PrefillScratch(CHANNELS, HIDDEN, EXPERTS, SELECTED, T, dev)
    bias = synth.zipf_bias(5, EXPERTS)
    nb = 4
    host_x = [torch.from_numpy(synth.activations_f16(1000 + b, T, CHANNELS)).pin_memory() for b in range(nb)]
    host_lg = [torch.from_numpy(synth.router_logits(2000 + b, T, EXPERTS, bias)).pin_memory() for b in range(nb)]
    dev_x = [t.to(dev) for t in host_x]
    dev_lg = [t.to(dev) for t in host_lg]
    out = torch.zeros((T, CHANNELS), dtype=torch.float16, device=dev)
    host_out = torch.zeros((T, CHANNELS), dtype=torch.float16).pin_memory()
    sx, slg = torch.zeros_like(dev_x[0]), torch.zeros_like(dev_lg[0])
    lib = capi.lib()
    stream = torch.cuda.current_stream()

    def layer_call(i, x, lg):
        L.moe_layer_prefill(layers[i % len(layers)], ps, x, lg, out)   # tsp_moe_layer_prefill: binary16 rows in and out

    def resident(i):
        layer_call(i, dev_x[i % nb], dev_lg[i % nb])

    def e2e(i):
        sx.copy_(host_x[i % nb], non_blocking=True)
        slg.copy_(host_lg[i % nb], non_blocking=True)
        layer_call(i, sx, slg)
        host_out.copy_(out, non_blocking=True)
        stream.synchronize()

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def stage_pass(steps):
        """CUDA-event time of each launch of the prefill layer, issued exactly as tsp_moe_layer_prefill issues them."""
        s, st = ps.base, L.stream_ptr()
        names = ["rows_f16k", "route", "permute", "offsets", "gather", "gate_up", "down", "combine"]
        acc = dict.fromkeys(names, 0.0)
        C2, C4, H2, E, K = CHANNELS * 2, CHANNELS * 4, HIDDEN * 2, EXPERTS, SELECTED
        for i in range(steps):
            w = layers[i % len(layers)].weights
            x, lg = dev_x[i % nb], dev_lg[i % nb]
            e = s.error.data_ptr()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
            ev[0].record()
            capi.check(lib.tsp_moe_rows_f16k(x.data_ptr(), C2, 1, T, CHANNELS, ps.xk.data_ptr(), C2, e, st)); ev[1].record()
            capi.check(lib.tsp_moe_route(lg.data_ptr(), E * 4, T, E, K, 0, 1, s.ids.data_ptr(), s.weights.data_ptr(), e, st)); ev[2].record()
            capi.check(lib.tsp_moe_permute(s.ids.data_ptr(), T, E, K, ps.tile, s.token_map.data_ptr(), s.counts.data_ptr(), ps.tasks.data_ptr(), e, st)); ev[3].record()
            capi.check(lib.tsp_moe_route_offsets(s.counts.data_ptr(), E, ps.offsets.data_ptr(), st)); ev[4].record()
            capi.check(lib.tsp_moe_gather_rows16(ps.xk.data_ptr(), C2, s.token_map.data_ptr(), ps.offsets.data_ptr(), E, T, K, CHANNELS, ps.xp.data_ptr(), C2, st)); ev[5].record()
            capi.check(lib.tsp_moe_grouped_gate_up(C.byref(w.gate), C.byref(w.up), C.byref(w.shared_gate), C.byref(w.shared_up), ps.xp.data_ptr(), C2,
                                                   ps.xk.data_ptr(), C2, T, T, K, s.token_map.data_ptr(), s.counts.data_ptr(), ps.tasks.data_ptr(),
                                                   ps.offsets.data_ptr(), ps.hp.data_ptr(), H2, ps.s_hp.data_ptr(), H2, e, st)); ev[6].record()
            capi.check(lib.tsp_moe_grouped_down(C.byref(w.down), C.byref(w.shared_down), ps.hp.data_ptr(), H2, T, K, s.token_map.data_ptr(),
                                                s.counts.data_ptr(), ps.tasks.data_ptr(), ps.offsets.data_ptr(), ps.routed16.data_ptr(), C2, 1,
                                                ps.s_hp.data_ptr(), H2, T, s.shared_out.data_ptr(), C4, e, st)); ev[7].record()
            capi.check(lib.tsp_moe_combine(ps.routed16.data_ptr(), C2, 1, s.weights.data_ptr(), s.shared_out.data_ptr(), C4, w.d_shared_router,
                                           x.data_ptr(), C2, 1, s.shared_logit.data_ptr(), T, CHANNELS, K, None, 0, out.data_ptr(), C2, e, st)); ev[8].record()
            torch.cuda.synchronize()
            for k_, n in enumerate(names):
                acc[n] += ev[k_].elapsed_time(ev[k_ + 1])
        return {n + "_ms": acc[n] / steps for n in names}

    with ClockSampler(local) as clocks:
        ms = timed(resident, args.steps, args.warmup)
        ms_e2e = timed(e2e, args.steps, args.warmup)
        stages = stage_pass(max(2, min(args.steps, 5)))
    assert ps.base.error_word() == 0, "device error word set during the benchmark"
    _, tf_peak, peak_kind = peaks()
    gu_flops = T * (SELECTED + 1) * 2 * (2 * HIDDEN * CHANNELS)   # the launch carries the routed experts and the shared expert
    achieved = gu_flops / (stages["gate_up_ms"] * 1e-3) / 1e12
    cpu = parity = None
    if args.cpu_tokens != 0:
        orc, kind = cpu_oracle()
        cores = os.cpu_count() or 1
        sample = min(args.cpu_tokens or 64, T)
        idx = np.unique(np.linspace(0, T - 1, sample).astype(int))
        host = layers[0].host_layer(SELECTED)
        xs, ls = host_x[0].numpy()[idx].astype(np.float32), host_lg[0].numpy()[idx]
        t0 = time.perf_counter()
        want = orc.moe_layer(host.oracle_dict(), xs, ls, threads=min(cores, len(idx)))
        dt = time.perf_counter() - t0
        cpu = {"value": len(idx) / dt, "unit": "tokens/s", "cores": min(cores, len(idx)), "kind": kind,
               "sample": f"{len(idx)} evenly spaced tokens of the {T}-token batch, one layer, threads over tokens, {dt:.1f} s"}
        layer_call(0, dev_x[0], dev_lg[0])
        torch.cuda.synchronize()
        got = out.cpu().numpy()[idx].astype(np.float64)
        parity = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    line = {"metric": "moe_q4k_expert_gemm_tokens_per_s", "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": f"moe_layer_prefill_T{T} (BASELINE configs[2])", "hidden": CHANNELS, "experts": EXPERTS, "expert_ffn": HIDDEN,
                       "top_k": SELECTED, "weights": "Q4_K Pack-v3 planar", "router": "N(0,1) + Zipf(1.1) per-expert bias",
                       "l2_policy": "inputs larger than L2: 0.93 GB of weights and 0.5 GB of intermediates per step"},
            "e2e": {"value": T / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": T * CHANNELS * 2 + T * EXPERTS * 4, "d2h_bytes_per_step": T * CHANNELS * 2},
            "gpu_launches": 9 * args.steps, "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "kernel": "grouped_mma_kernel<gate-up> (routed experts + shared expert, tcgen05)", "achieved": achieved, "peak": tf_peak,
                         "unit": "TFLOP/s", "frac": achieved / tf_peak, "peak_kind": peak_kind, "traffic": None,
                         "algorithmic_flops_per_launch": gu_flops, "launch_ms": stages["gate_up_ms"]},
            "cpu_baseline": cpu,
            "extra": {"layer_tflops": T * (SELECTED + 1) * FLOPS_PER_ROUTE / (ms * 1e-3) / 1e12, "stage_ms": stages, "parity_rel_l2_vs_cpu": parity}}
    print(json.dumps(line), flush=True)


def run_head(args, local):
    """BASELINE configs[3]: the dense Q8_0 vocabulary head [151936 x 2048] on a batch of draft-token hidden states (M <= 16)."""
    import torch
    from tokspur_public_b200 import capi, formats, synth
    from tokspur_public_b200 import layer as L
    dev = torch.device("cuda", local)
    VOCAB, M = 151936, min(max(args.tokens, 1), 16) if args.tokens != 64 else 16
    bpr = CHANNELS // 32                      # Q8_0 blocks per row
    row_bytes = bpr * 34
    lib, st = capi.lib(), L.stream_ptr()
    nw = 2                                     # two independently seeded matrices rotate (each 330 MB, larger than L2)
    mats, sets = [], []
    for i in range(nw):
        t = torch.empty(VOCAB * row_bytes, dtype=torch.uint8, device=dev)
        capi.call("tsp_synth_weights", formats.Q8_0, 900 + i, 0, VOCAB * bpr, 0.02, t.data_ptr(), st)
        mats.append(t)
        sets.append(L.matrix_set(t, formats.Q8_0, formats.GGUF, VOCAB, CHANNELS))
    nb = 4
    host_x = [torch.from_numpy(synth.activations_f16(3000 + b, M, CHANNELS).astype(np.float32)).pin_memory() for b in range(nb)]
    dev_x = [t.to(dev) for t in host_x]
    sx = torch.zeros_like(dev_x[0])
    out = torch.zeros((M, VOCAB), dtype=torch.float32, device=dev)
    host_out = torch.zeros((M, VOCAB), dtype=torch.float32).pin_memory()
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream()

    def project(i, x):
        capi.check(lib.tsp_moe_project(C.byref(sets[i % nw]), x.data_ptr(), CHANNELS * 4, 1, M, 1, None, None, None, out.data_ptr(), VOCAB * 4, 1,
                                       err.data_ptr(), st))

    def resident(i):
        project(i, dev_x[i % nb])

    def e2e(i):
        sx.copy_(host_x[i % nb], non_blocking=True)
        project(i, sx)
        host_out.copy_(out, non_blocking=True)
        stream.synchronize()

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    with ClockSampler(local) as clocks:
        ms = timed(resident, args.steps, args.warmup)
        ms_e2e = timed(e2e, args.steps, args.warmup)
    assert int(err.item()) == 0, "device error word set during the benchmark"
    hbm_peak, _, peak_kind = peaks()
    bytes_launch = VOCAB * row_bytes + M * CHANNELS * 4 + M * VOCAB * 4
    achieved = bytes_launch / (ms * 1e-3) / 1e9
    cpu = parity = None
    if args.cpu_tokens != 0:
        orc, kind = cpu_oracle()
        rows = 4096                                  # the first 4096 vocabulary rows of matrix 0, every token of batch 0
        wbytes = mats[0][: rows * row_bytes].cpu().numpy()
        xs = host_x[0].numpy()
        t0 = time.perf_counter()
        want = np.stack([orc.gemv(formats.Q8_0, wbytes, CHANNELS, rows, xs[m]) for m in range(M)])
        dt = time.perf_counter() - t0
        cpu = {"value": M / (dt * VOCAB / rows), "unit": "tokens/s", "cores": 1, "kind": kind,
               "sample": f"{rows} of the {VOCAB} vocabulary rows for all {M} tokens, one thread, {dt:.1f} s, scaled to the whole matrix"}
        project(0, dev_x[0])
        torch.cuda.synchronize()
        got = out[:, :rows].cpu().numpy().astype(np.float64)
        parity = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    line = {"metric": "moe_q4k_expert_gemm_tokens_per_s", "value": M / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"q8_0_vocabulary_head_M{M} (BASELINE configs[3])", "vocab": VOCAB, "hidden": CHANNELS, "weights": "Q8_0 GGUF blocks",
                       "l2_policy": "inputs larger than L2: two 330 MB matrices rotate"},
            "e2e": {"value": M / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": M * CHANNELS * 4,
                    "d2h_bytes_per_step": M * VOCAB * 4},
            "gpu_launches": args.steps, "clocks": clocks.summary(),
            "roofline": {"bound": "hbm", "kernel": "gemv_kernel<Q8_0> (dense head)", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "peak_kind": peak_kind, "traffic": None, "algorithmic_bytes_per_launch": bytes_launch,
                         "launch_ms": ms},
            "cpu_baseline": cpu, "extra": {"parity_rel_l2_vs_cpu": parity}}
    print(json.dumps(line), flush=True)


def stage_times(L, capi, layers, s, dev_x, dev_lg, out, steps, warmup, T):
    """CUDA-event time of each launch of the layer, averaged over the same rotation as the timed region."""
    import torch
    lib = capi.lib()
    st = L.stream_ptr()
    names = ["convert", "route", "permute", "gate_up", "down", "combine"]
    acc = {n: 0.0 for n in names}
    uniq = 0.0
    C4, H4 = CHANNELS * 4, HIDDEN * 4
    for i in range(warmup + steps):
        w = layers[i % len(layers)].weights
        x, lg = dev_x[i % len(dev_x)], dev_lg[i % len(dev_lg)]
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
        e = s.error.data_ptr()
        ev[0].record()
        capi.check(lib.tsp_rows_f16_to_f32(x.data_ptr(), CHANNELS * 2, s.x32.data_ptr(), C4, T, CHANNELS, st)); ev[1].record()
        capi.check(lib.tsp_moe_route(lg.data_ptr(), EXPERTS * 4, T, EXPERTS, SELECTED, 0, 1, s.ids.data_ptr(), s.weights.data_ptr(), e, st)); ev[2].record()
        capi.check(lib.tsp_moe_permute(s.ids.data_ptr(), T, EXPERTS, SELECTED, capi.GEMV_TILE, s.token_map.data_ptr(), s.counts.data_ptr(),
                                       s.tasks.data_ptr(), e, st)); ev[3].record()
        # the routed experts and the shared expert in one launch each, exactly as tsp_moe_layer_decode issues them
        capi.check(lib.tsp_moe_gate_up_swiglu_shared(C.byref(w.gate), C.byref(w.up), C.byref(w.shared_gate), C.byref(w.shared_up),
                                                     s.x32.data_ptr(), C4, x.data_ptr(), CHANNELS * 2, T, SELECTED, s.token_map.data_ptr(),
                                                     s.counts.data_ptr(), s.tasks.data_ptr(), s.hidden.data_ptr(), H4,
                                                     s.shared_hidden.data_ptr(), H4, 1, e, st)); ev[4].record()
        capi.check(lib.tsp_moe_project_shared(C.byref(w.down), C.byref(w.shared_down), s.hidden.data_ptr(), H4, s.shared_hidden.data_ptr(), H4,
                                              T, SELECTED, s.token_map.data_ptr(), s.counts.data_ptr(), s.tasks.data_ptr(),
                                              s.routed.data_ptr(), C4, s.shared_out.data_ptr(), C4, e, st)); ev[5].record()
        capi.check(lib.tsp_moe_combine(s.routed.data_ptr(), C4, 0, s.weights.data_ptr(), s.shared_out.data_ptr(), C4, w.d_shared_router,
                                       s.x32.data_ptr(), C4, 0, s.shared_logit.data_ptr(), T, CHANNELS, SELECTED, None, 0, out.data_ptr(),
                                       CHANNELS * 2, e, st)); ev[6].record()
        torch.cuda.synchronize()
        if i >= warmup:
            for k, n in enumerate(names):
                acc[n] += ev[k].elapsed_time(ev[k + 1])
            uniq += float((s.counts.cpu().numpy().view(np.uint32) > 0).sum())
    res = {n + "_ms": acc[n] / steps for n in names}
    res["unique_experts"] = uniq / steps
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=64, help="token rows per step (decode batch)")
    ap.add_argument("--layers", type=int, default=4, help="independently seeded weight sets rotated over")
    ap.add_argument("--layout", default=None, choices=["planar", "gguf"], help="weight layout (default: Pack-v3 planar for Q4_K experts, GGUF blocks for Q8_0 experts)")
    ap.add_argument("--experts", default="q4_k", choices=["q4_k", "q8_0"], help="expert encoding of the decode workload (q8_0: the MTP block)")
    ap.add_argument("--cpu-tokens", type=int, default=None, help="tokens of the batch timed on the CPU baseline (0 = skip)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "head"])
    ap.add_argument("--prefill-tokens", type=int, default=4096, help="token rows per GPU of the prefill sub-record")
    ap.add_argument("--replicate", type=int, default=32, help="expert-parallel prefill: hot experts held by every rank (0 = none)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill sub-record")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_ours(args)


if __name__ == "__main__":
    main()
