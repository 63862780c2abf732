#!/usr/bin/env python
"""Benchmark of the routed-MoE FFN hot path (BASELINE metric: MoE Q4_K expert-GEMM tokens/s).

A "step" is one pass of one MoE layer (hidden 2048, 512 routed experts of FFN 512 in Q4_K, top-10, one gated shared expert)
over one fresh batch of synthetic tokens. At N=1 the headline workload is BASELINE configs[1] at its largest batch (decode,
64 tokens). Layers rotate over several independently seeded weight sets and every step takes a different batch, so the bytes
a step streams (~650 MB) never sit in the 126 MB L2.

  value     tokens/s with inputs already resident in HBM (CUDA events, median of repeated timed loops, max over ranks)
  e2e       tokens/s through the C ABI from pinned HOST buffers: H2D of x and logits and D2H of the output rows inside the
            timed region, one synchronisation per step
  roofline  the dominant kernel (routed gate-up + SwiGLU): algorithmic GGUF bytes / its average launch duration in a
            back-to-back loop of that launch alone over the rotating layers (CUDA events around the loop)
  cpu_baseline  the reference's own CPU composition (oracle/_ref, else the C port) on the host cores
  extra     the rest of the metric in the same run: decode at 1 and 8 tokens, the prefill layer (BASELINE configs[2],
            tensor-core bound), the Q8_0 vocabulary head (configs[3]) and the single Q4_K matrix (configs[0]) at M = 1 / 256

`--workload prefill|head|config1` prints the corresponding record as the line itself. `--impl reference` times the CPU
implementation alone (rank 0 only under torchrun). N > 1 runs the expert-parallel layer (tokspur_public_b200/ep.py).
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
VOCAB = 151936


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
    steps = args.steps           # a step = `sample` tokens, ~0.5 core-seconds each, spread over the cores: well under a second
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.moe_layer(layer, x, logits, threads=min(cores, sample))
    dt = (time.perf_counter() - t0) / steps
    value = sample / dt
    line = {"impl": "reference", "metric": "moe_q4k_expert_gemm_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": "moe_layer_decode_T64 (BASELINE configs[1])", "hidden": CHANNELS, "experts": EXPERTS, "expert_ffn": HIDDEN,
                       "top_k": SELECTED, "weights": "Q4_K GGUF", "sample_tokens_per_step": sample},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": min(cores, sample), "kind": kind,
                             "sample": f"{sample} tokens of the 64-token batch per step, one layer, threads over tokens"},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# timing helpers
# --------------------------------------------------------------------------------------------------
def timed(fn, steps, warmup):
    """ms per call of `steps` calls between two CUDA events on the current stream, after `warmup` calls."""
    import torch
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


def timed_median(fn, steps, warmup, min_seconds=0.5, max_repeats=400):
    """Repeats the timed loop of exactly `steps` calls until the timed regions add up to `min_seconds`; returns the median ms per
    call and the number of repeats."""
    vals, total = [], 0.0
    while not vals or (total < min_seconds * 1e3 and len(vals) < max_repeats):
        ms = timed(fn, steps, warmup if not vals else 0)
        vals.append(ms)
        total += ms * steps
    return float(np.median(vals)), len(vals)


# --------------------------------------------------------------------------------------------------
# our arm, one GPU
# --------------------------------------------------------------------------------------------------
def decode_record(args, dev, T, layers, etype, layout, full: bool):
    """One decode batch size: step time (resident and end to end) and, for the headline size, the stage analysis."""
    import torch
    from tokspur_public_b200 import capi, formats, synth
    from tokspur_public_b200 import layer as L
    down_type = getattr(layers[0], "down_type", etype)
    expert_gate_up = 2 * formats.gguf_bytes(etype, HIDDEN, CHANNELS)
    expert_down = formats.gguf_bytes(down_type, CHANNELS, HIDDEN)
    scratch = L.Scratch(CHANNELS, HIDDEN, EXPERTS, SELECTED, T, dev)
    nb = 8
    host_x = [torch.from_numpy(synth.activations_f16(1000 + b, T, CHANNELS)).pin_memory() for b in range(nb)]
    host_lg = [torch.from_numpy(synth.router_logits(2000 + b, T, EXPERTS)).pin_memory() for b in range(nb)]
    dev_x, dev_lg = [t.to(dev) for t in host_x], [t.to(dev) for t in host_lg]
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

    ms, repeats = timed_median(step_resident, args.steps, args.warmup, args.min_seconds)
    ms_e2e, _ = timed_median(step_e2e, args.steps, args.warmup, args.min_seconds / 2)
    assert scratch.error_word() == 0, "device error word set during the benchmark"
    # experts hit per batch (the bytes a step has to stream), from the routing tables of each timed batch
    uniq = []
    for b in range(nb):
        L.moe_layer_decode(layers[0], scratch, dev_x[b], dev_lg[b], out)
        torch.cuda.synchronize()
        uniq.append(float((scratch.counts.cpu().numpy().view(np.uint32) > 0).sum()))
    U = float(np.mean(uniq))
    hbm_peak, _, peak_kind = peaks()
    layer_bytes = (U + 1) * (expert_gate_up + expert_down) + T * (CHANNELS * 2 * 2) + T * EXPERTS * 4
    rec = {"tokens": T, "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "e2e_ms_per_step": ms_e2e, "e2e_tokens_per_s": T / (ms_e2e * 1e-3),
           "timed_repeats": repeats, "unique_experts": U, "layer_algorithmic_bytes": layer_bytes,
           "layer_hbm_gbs": layer_bytes / (ms * 1e-3) / 1e9, "layer_hbm_frac": layer_bytes / (ms * 1e-3) / 1e9 / hbm_peak,
           "layer_tflops": T * (SELECTED + 1) * FLOPS_PER_ROUTE / (ms * 1e-3) / 1e12,
           # routing, tables, gate-up, down, mixture; experts that cannot take the shared expert into their launches (Q8_0, Q5_K) run it
           # in a launch of its own beside each projection
           "launches_per_step": 5 if etype == formats.Q4_K else 7}
    if not full:
        return rec, None
    # ---- the dominant launch alone, back to back over the rotating layers (tables of batch 0; the weights change every launch)
    lib, st, e = capi.lib(), L.stream_ptr(), scratch.error.data_ptr()
    L.moe_layer_decode(layers[0], scratch, dev_x[0], dev_lg[0], out)
    torch.cuda.synchronize()
    U0 = float((scratch.counts.cpu().numpy().view(np.uint32) > 0).sum())
    C4, H4 = CHANNELS * 4, HIDDEN * 4
    x0 = dev_x[0]

    def gate_up_only(i):
        w = layers[i % len(layers)].weights
        capi.check(lib.tsp_moe_gate_up_swiglu_shared(C.byref(w.gate), C.byref(w.up), C.byref(w.shared_gate), C.byref(w.shared_up),
                                                     scratch.x32.data_ptr(), C4, x0.data_ptr(), CHANNELS * 2, T, SELECTED, scratch.token_map.data_ptr(),
                                                     scratch.counts.data_ptr(), scratch.tasks.data_ptr(), scratch.hidden.data_ptr(), H4,
                                                     scratch.shared_hidden.data_ptr(), H4, 1, e, st))

    def down_only(i):
        w = layers[i % len(layers)].weights
        capi.check(lib.tsp_moe_project_shared(C.byref(w.down), C.byref(w.shared_down), scratch.hidden.data_ptr(), H4, scratch.shared_hidden.data_ptr(), H4,
                                              T, SELECTED, scratch.token_map.data_ptr(), scratch.counts.data_ptr(), scratch.tasks.data_ptr(),
                                              scratch.routed.data_ptr(), C4, scratch.shared_out.data_ptr(), C4, e, st))

    gu_ms, _ = timed_median(gate_up_only, args.steps, args.warmup, args.min_seconds / 2)
    dn_ms, _ = timed_median(down_only, args.steps, args.warmup, args.min_seconds / 2)
    assert scratch.error_word() == 0
    # the launch covers the routed experts that were hit plus the shared expert; activations in (binary16), hidden rows out (FP32)
    gu_bytes = (U0 + 1) * expert_gate_up + T * CHANNELS * 2 + T * (SELECTED + 1) * HIDDEN * 4
    dn_bytes = (U0 + 1) * expert_down + T * (SELECTED + 1) * (HIDDEN * 4 + CHANNELS * 4)
    achieved = gu_bytes / (gu_ms * 1e-3) / 1e9
    kname = ("gemv3_kernel<planar, gate-up+SwiGLU> (routed experts + shared expert, one launch)" if etype == formats.Q4_K else
             "gemv_k5_kernel<Q5_K, gate-up+SwiGLU> (routed experts) + gemv_kernel<Q8_0> (shared expert): two launches timed together" if etype == formats.Q5_K else
             "gemv_kernel<Q8_0, gate-up+SwiGLU> (routed experts, then the shared expert: two launches timed together)")
    roofline = {"bound": "hbm", "kernel": kname, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "peak_kind": peak_kind, "timing": "average of a back-to-back loop of this launch alone over the rotating layers (CUDA events)",
                # measured DRAM bytes of one captured launch (profiles/gemv3_gate_up_and_down_decode_T64.md: 457.2 MB for 361 experts),
                # scaled to the experts this launch touches: traffic grows with the experts touched, the activations stay in L2
                "traffic": 463.2e6 / 359 * (U0 + 1) if etype == formats.Q4_K and layout == formats.PLANAR else None,
                "traffic_source": "profiles/gemv3_gate_up_and_down_decode_T64.md (ncu), scaled by experts hit",
                "algorithmic_bytes_per_launch": gu_bytes, "launch_ms": gu_ms, "unique_experts": U0}
    rec["stage_ms"] = {"gate_up_launch_ms": gu_ms, "down_launch_ms": dn_ms, "rest_of_step_ms": ms - gu_ms - dn_ms,
                       "down_hbm_frac": dn_bytes / (dn_ms * 1e-3) / 1e9 / hbm_peak}
    # CPU baseline on the same first layer and batch 0, and an in-run parity figure
    cpu = None
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
        rec["parity_rel_l2_vs_cpu"] = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    return rec, (roofline, cpu)


def prefill_record(args, dev, layers, T):
    """BASELINE configs[2]: one MoE layer over T tokens, router logits N(0,1) + per-expert Zipf(1.1) bias, through the grouped
    tcgen05 GEMMs (tsp_moe_layer_prefill: binary16 rows in and out)."""
    import torch
    from tokspur_public_b200 import capi, synth
    from tokspur_public_b200 import layer as L
    ps = L.PrefillScratch(CHANNELS, HIDDEN, EXPERTS, SELECTED, T, dev)
    bias = synth.zipf_bias(5, EXPERTS)
    nb = 4
    host_x = [torch.from_numpy(synth.activations_f16(1000 + b, T, CHANNELS)).pin_memory() for b in range(nb)]
    host_lg = [torch.from_numpy(synth.router_logits(2000 + b, T, EXPERTS, bias)).pin_memory() for b in range(nb)]
    dev_x, dev_lg = [t.to(dev) for t in host_x], [t.to(dev) for t in host_lg]
    out = torch.zeros((T, CHANNELS), dtype=torch.float16, device=dev)
    host_out = torch.zeros((T, CHANNELS), dtype=torch.float16).pin_memory()
    sx, slg = torch.zeros_like(dev_x[0]), torch.zeros_like(dev_lg[0])
    lib, stream = capi.lib(), torch.cuda.current_stream()

    def resident(i):
        L.moe_layer_prefill(layers[i % len(layers)], ps, dev_x[i % nb], dev_lg[i % nb], out)

    def e2e(i):
        sx.copy_(host_x[i % nb], non_blocking=True)
        slg.copy_(host_lg[i % nb], non_blocking=True)
        L.moe_layer_prefill(layers[i % len(layers)], ps, sx, slg, out)
        host_out.copy_(out, non_blocking=True)
        stream.synchronize()

    steps = max(4, args.steps // 4)
    ms, repeats = timed_median(resident, steps, args.warmup, args.min_seconds)
    ms_e2e, _ = timed_median(e2e, steps, args.warmup, args.min_seconds / 2)

    def stage_pass(n):
        """CUDA-event time of each launch of the layer, issued exactly as tsp_moe_layer_prefill issues them."""
        s, st = ps.base, L.stream_ptr()
        mixed = layers[0].shared_type != layers[0].type   # a shared expert in another encoding: launches of its own
        names = ["rows_f16k", "route", "permute", "offsets", "gather", "gate_up"] + (["shared_gate_up"] if mixed else []) + ["down"] + \
                (["shared_down"] if mixed else []) + ["combine"]
        acc = dict.fromkeys(names, 0.0)
        C2, C4, H2, E, K = CHANNELS * 2, CHANNELS * 4, HIDDEN * 2, EXPERTS, SELECTED
        for i in range(n):
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
            k_ev = 6
            capi.check(lib.tsp_moe_grouped_gate_up(C.byref(w.gate), C.byref(w.up), None if mixed else C.byref(w.shared_gate), None if mixed else C.byref(w.shared_up),
                                                   ps.xp.data_ptr(), C2, ps.xk.data_ptr(), C2, T, T, K, s.token_map.data_ptr(), s.counts.data_ptr(), ps.tasks.data_ptr(),
                                                   ps.offsets.data_ptr(), ps.hp.data_ptr(), H2, ps.s_hp.data_ptr(), H2, e, st)); ev[k_ev].record(); k_ev += 1
            if mixed:
                capi.check(lib.tsp_dense_mm_swiglu(C.byref(w.shared_gate), C.byref(w.shared_up), ps.xk.data_ptr(), C2, T, ps.s_hp.data_ptr(), H2,
                                                   ps.offsets.data_ptr() + 4 * (E + 3), e, st)); ev[k_ev].record(); k_ev += 1
            capi.check(lib.tsp_moe_grouped_down(C.byref(w.down), None if mixed else C.byref(w.shared_down), ps.hp.data_ptr(), H2, T, K, s.token_map.data_ptr(),
                                                s.counts.data_ptr(), ps.tasks.data_ptr(), ps.offsets.data_ptr(), ps.routed16.data_ptr(), C2, 1,
                                                ps.s_hp.data_ptr(), H2, T, s.shared_out.data_ptr(), C4, e, st)); ev[k_ev].record(); k_ev += 1
            if mixed:
                capi.check(lib.tsp_dense_mm(C.byref(w.shared_down), ps.s_hp.data_ptr(), H2, T, s.shared_out.data_ptr(), C4, ps.offsets.data_ptr() + 4 * (E + 4),
                                            e, st)); ev[k_ev].record(); k_ev += 1
            capi.check(lib.tsp_moe_combine(ps.routed16.data_ptr(), C2, 1, s.weights.data_ptr(), s.shared_out.data_ptr(), C4, w.d_shared_router,
                                           x.data_ptr(), C2, 1, s.shared_logit.data_ptr(), T, CHANNELS, K, None, 0, out.data_ptr(), C2, e, st)); ev[k_ev].record()
            torch.cuda.synchronize()
            for k_, nme in enumerate(names):
                acc[nme] += ev[k_].elapsed_time(ev[k_ + 1])
        return {nme + "_ms": acc[nme] / n for nme in names}

    stages = stage_pass(5)
    assert ps.base.error_word() == 0, "device error word set during the benchmark"
    _, tf_peak, peak_kind = peaks()
    gu_flops = T * (SELECTED + 1) * 2 * (2 * HIDDEN * CHANNELS)   # the launch carries the routed experts and the shared expert
    layer_flops = T * (SELECTED + 1) * FLOPS_PER_ROUTE
    rec = {"tokens": T, "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "e2e_ms_per_step": ms_e2e, "e2e_tokens_per_s": T / (ms_e2e * 1e-3),
           "timed_repeats": repeats, "layer_tflops": layer_flops / (ms * 1e-3) / 1e12, "layer_frac_of_bf16_peak": layer_flops / (ms * 1e-3) / 1e12 / tf_peak,
           "gate_up_launch_tflops": gu_flops / (stages["gate_up_ms"] * 1e-3) / 1e12,
           "gate_up_launch_frac_of_bf16_peak": gu_flops / (stages["gate_up_ms"] * 1e-3) / 1e12 / tf_peak, "peak_tflops": tf_peak, "peak_kind": peak_kind,
           "stage_ms": stages, "launches_per_step": 9 + 2 * int(layers[0].shared_type != layers[0].type), "router": "N(0,1) + Zipf(1.1) per-expert bias",
           "h2d_bytes_per_step": T * CHANNELS * 2 + T * EXPERTS * 4, "d2h_bytes_per_step": T * CHANNELS * 2}
    cpu = None
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
        L.moe_layer_prefill(layers[0], ps, dev_x[0], dev_lg[0], out)
        torch.cuda.synchronize()
        got = out.cpu().numpy()[idx].astype(np.float64)
        rec["parity_rel_l2_vs_cpu"] = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    return rec, cpu


def head_record(args, dev, M):
    """BASELINE configs[3]: the dense Q8_0 vocabulary head [151936 x 2048] on M draft-token hidden states."""
    import torch
    from tokspur_public_b200 import capi, formats, synth
    from tokspur_public_b200 import layer as L
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

    ms, repeats = timed_median(resident, args.steps, args.warmup, args.min_seconds / 2)
    ms_e2e, _ = timed_median(e2e, max(4, args.steps // 4), args.warmup, args.min_seconds / 4)
    assert int(err.item()) == 0, "device error word set during the benchmark"
    hbm_peak, _, peak_kind = peaks()
    bytes_launch = VOCAB * row_bytes + M * CHANNELS * 4 + M * VOCAB * 4
    rec = {"rows": M, "ms_per_step": ms, "tokens_per_s": M / (ms * 1e-3), "e2e_ms_per_step": ms_e2e, "timed_repeats": repeats,
           "hbm_gbs": bytes_launch / (ms * 1e-3) / 1e9, "hbm_frac": bytes_launch / (ms * 1e-3) / 1e9 / hbm_peak, "peak_kind": peak_kind,
           "algorithmic_bytes_per_launch": bytes_launch, "h2d_bytes_per_step": M * CHANNELS * 4, "d2h_bytes_per_step": M * VOCAB * 4}
    # the sampler's top-64 rows of the same logits (the step that follows the head in the verify pass): head + top-k per step
    topk_scratch = torch.empty(lib.tsp_logit_topk_scratch_bytes(M, VOCAB), dtype=torch.uint8, device=dev)
    topk_rows = torch.empty(lib.tsp_logit_topk_output_bytes(M), dtype=torch.uint8, device=dev)
    host_rows = torch.empty(topk_rows.numel(), dtype=torch.uint8).pin_memory()

    def topk():
        capi.check(lib.tsp_logit_topk(out.data_ptr(), VOCAB * 4, M, VOCAB, topk_scratch.data_ptr(), topk_scratch.numel(), topk_rows.data_ptr(),
                                      topk_rows.numel(), st))

    def resident_topk(i):
        project(i, dev_x[i % nb])
        topk()

    def e2e_topk(i):   # what the verify pass needs back is the 528-byte rows, not the logits
        sx.copy_(host_x[i % nb], non_blocking=True)
        project(i, sx)
        topk()
        host_rows.copy_(topk_rows, non_blocking=True)
        stream.synchronize()

    ms_tk, _ = timed_median(resident_topk, args.steps, args.warmup, args.min_seconds / 4)
    ms_tk_e2e, _ = timed_median(e2e_topk, max(4, args.steps // 4), args.warmup, args.min_seconds / 4)
    rec["with_logit_topk"] = {"ms_per_step": ms_tk, "e2e_ms_per_step": ms_tk_e2e, "d2h_bytes_per_step": M * 528,
                              "launches_per_step": 4, "note": "head (zeroing pass + kernel) + two top-k launches; only the top-64 rows return to the host"}
    cpu = None
    if args.cpu_tokens != 0:
        orc, kind = cpu_oracle()
        rows = 2048                                  # the first vocabulary rows of matrix 0, every token of batch 0
        wbytes = mats[0][: rows * row_bytes].cpu().numpy()
        xs = host_x[0].numpy()
        t0 = time.perf_counter()
        want = np.stack([orc.gemv(formats.Q8_0, wbytes, CHANNELS, rows, xs[m]) for m in range(min(M, 4))])
        dt = time.perf_counter() - t0
        cpu = {"value": min(M, 4) / (dt * VOCAB / rows), "unit": "tokens/s", "cores": 1, "kind": kind,
               "sample": f"{rows} of the {VOCAB} vocabulary rows for {min(M, 4)} tokens, one thread, {dt:.1f} s, scaled to the whole matrix"}
        project(0, dev_x[0])
        torch.cuda.synchronize()
        got = out[: min(M, 4), :rows].cpu().numpy().astype(np.float64)
        rec["parity_rel_l2_vs_cpu"] = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    del mats
    return rec, cpu


def config1_record(args, dev):
    """BASELINE configs[0]: one Q4_K matrix [1024 x 2048], N(0, 0.02) weights of seed 0, binary16 N(0,1) activations; M = 1 through
    the decode GEMV (HBM bound), M = 256 through the grouped tensor-core kernel as a one-expert set (tensor bound)."""
    import torch
    from tokspur_public_b200 import capi, formats, synth
    from tokspur_public_b200 import layer as L
    rows, cols = 1024, 2048
    lib, st = capi.lib(), L.stream_ptr()
    w = formats.quantize_q4_k(synth.normal(0, (rows, cols), 0.02)).reshape(-1)
    planar = torch.from_numpy(formats.pack_planar(formats.Q4_K, w, rows, cols)).to(dev)
    ms_set = L.matrix_set(planar, formats.Q4_K, formats.PLANAR, rows, cols, 1)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    rec = {}
    # M = 1: GEMV. The matrix is 1.2 MB and sits in L2 after the first call: the figure is a latency, reported as such.
    x1 = torch.from_numpy(synth.activations_f16(1, 1, cols).astype(np.float32)).to(dev)
    o1 = torch.zeros((1, rows), dtype=torch.float32, device=dev)

    def gemv(i):
        capi.check(lib.tsp_moe_project(C.byref(ms_set), x1.data_ptr(), cols * 4, 1, 1, 1, None, None, None, o1.data_ptr(), rows * 4, 1, err.data_ptr(), st))

    ms1, _ = timed_median(gemv, args.steps, args.warmup, args.min_seconds / 8)
    rec["m1"] = {"ms_per_call": ms1, "tokens_per_s": 1 / (ms1 * 1e-3), "note": "1.2 MB matrix: L2-resident after the first call, launch-latency bound"}
    # M = 256: one dense expert through the tensor-core path
    M = 256
    x16 = torch.from_numpy(synth.activations_f16(1, M, cols)).to(dev)
    xk, xp = torch.zeros_like(x16), torch.zeros_like(x16)
    ids = torch.zeros(M, dtype=torch.int32, device=dev)
    tm, counts = torch.zeros(M, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    tasks = torch.zeros(int(lib.tsp_moe_tasks_words(M, 1, 1, 256)), dtype=torch.int32, device=dev)
    offsets = torch.zeros(4, dtype=torch.int32, device=dev)
    o256 = torch.zeros((M, rows), dtype=torch.float32, device=dev)
    e = err.data_ptr()

    def gemm(i):
        capi.check(lib.tsp_moe_rows_f16k(x16.data_ptr(), cols * 2, 1, M, cols, xk.data_ptr(), cols * 2, e, st))
        capi.check(lib.tsp_moe_permute(ids.data_ptr(), M, 1, 1, 256, tm.data_ptr(), counts.data_ptr(), tasks.data_ptr(), e, st))
        capi.check(lib.tsp_moe_route_offsets(counts.data_ptr(), 1, offsets.data_ptr(), st))
        capi.check(lib.tsp_moe_gather_rows16(xk.data_ptr(), cols * 2, tm.data_ptr(), offsets.data_ptr(), 1, M, 1, cols, xp.data_ptr(), cols * 2, st))
        capi.check(lib.tsp_moe_grouped_down(C.byref(ms_set), None, xp.data_ptr(), cols * 2, M, 1, tm.data_ptr(), counts.data_ptr(), tasks.data_ptr(),
                                            offsets.data_ptr(), o256.data_ptr(), rows * 4, 0, None, 0, 0, None, 0, e, st))

    ms256, _ = timed_median(gemm, args.steps, args.warmup, args.min_seconds / 8)
    assert int(err.item()) == 0
    flops = 2 * rows * cols * M
    rec["m256"] = {"ms_per_call": ms256, "tokens_per_s": M / (ms256 * 1e-3), "tflops": flops / (ms256 * 1e-3) / 1e12,
                   "note": "five launches (row preparation, permutation, offsets, routed copy, tcgen05 GEMM) for 1.07 GFLOP: launch-latency bound"}
    if args.cpu_tokens != 0:
        orc, _ = cpu_oracle()
        xs = x16.float().cpu().numpy()
        want = np.stack([orc.gemv(formats.Q4_K, w, cols, rows, xs[m]) for m in (0, 100, 255)])
        got = o256.cpu().numpy()[[0, 100, 255]].astype(np.float64)
        rec["m256"]["parity_rel_l2_vs_cpu"] = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    return rec


def base_line(args, value, ms, workload, weights, dtype, extra_config=None):
    cfg = {"workload": workload, "hidden": CHANNELS, "experts": EXPERTS, "expert_ffn": HIDDEN, "top_k": SELECTED, "weights": weights}
    cfg.update(extra_config or {})
    return {"metric": "moe_q4k_expert_gemm_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": cfg}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from tokspur_public_b200 import formats
    from tokspur_public_b200 import layer as L

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        from tokspur_public_b200 import ep
        return ep.run_bench(args, rank, world, local)
    dev = torch.device("cuda", local)
    T = args.tokens
    # Q4_K experts default to the Pack-v3 planar layout, Q8_0 experts (the MTP block) stay GGUF blocks
    lname = args.layout or ("gguf" if args.experts == "q8_0" else "planar")
    layout = formats.PLANAR if lname == "planar" else formats.GGUF
    # q8_0: the MTP block of BASELINE configs[3]; q5_k: the reference model's other pairing (Q5_K gate / up, Q5_1 down, Q8_0 shared), raw blocks
    etype = {"q8_0": formats.Q8_0, "q5_k": formats.Q5_K}.get(args.experts, formats.Q4_K)
    if etype == formats.Q5_K:
        layout = formats.GGUF
    wname = {formats.Q8_0: "Q8_0 ", formats.Q5_K: "Q5_K gate/up + Q5_1 down + Q8_0 shared ", formats.Q4_K: "Q4_K "}[etype] + \
            ("Pack-v3 planar" if layout == formats.PLANAR else "GGUF")
    with ClockSampler(local) as clocks:
        if args.workload == "head":
            M = min(max(args.tokens, 1), 16) if args.tokens != 64 else 16
            rec, cpu = head_record(args, dev, M)
            line = base_line(args, rec["tokens_per_s"], rec["ms_per_step"], f"q8_0_vocabulary_head_M{M} (BASELINE configs[3])", "Q8_0 GGUF blocks", "f16 activations, f32 accumulate",
                             {"vocab": VOCAB, "l2_policy": "inputs larger than L2: two 330 MB matrices rotate"})
            hbm_peak, _, peak_kind = peaks()
            line.update({"e2e": {"value": M / (rec["e2e_ms_per_step"] * 1e-3), "unit": "tokens/s", "ms_per_step": rec["e2e_ms_per_step"],
                                 "h2d_bytes_per_step": rec["h2d_bytes_per_step"], "d2h_bytes_per_step": rec["d2h_bytes_per_step"]},
                         "gpu_launches": args.steps,
                         "roofline": {"bound": "hbm", "kernel": "gemv_kernel<Q8_0> (dense head)", "achieved": rec["hbm_gbs"], "peak": hbm_peak, "unit": "GB/s",
                                      "frac": rec["hbm_frac"], "peak_kind": peak_kind, "traffic": 348.1e6 if M == 16 else None,
                                      "traffic_source": "profiles/gemv_q8_0_head_M16.md (ncu: DRAM throughput x duration of one launch at 16 rows)",
                                      "algorithmic_bytes_per_launch": rec["algorithmic_bytes_per_launch"]},
                         "cpu_baseline": cpu, "extra": {"head": rec}})
        elif args.workload == "config1":
            rec = config1_record(args, dev)
            line = base_line(args, rec["m256"]["tokens_per_s"], rec["m256"]["ms_per_call"], "single_q4k_matmul_1024x2048_M256 (BASELINE configs[0])", "Q4_K Pack-v3 planar",
                             "f16 operands, f32 accumulate")
            line.update({"e2e": None, "gpu_launches": 5 * args.steps, "roofline": None, "cpu_baseline": None, "extra": {"config1": rec}})
        elif args.workload == "prefill":
            Tp = args.tokens if args.tokens != 64 else args.prefill_tokens
            p_layout = formats.GGUF if args.layout == "gguf" else formats.PLANAR
            sh_type = formats.Q8_0 if args.shared == "q8_0" else None
            layers = [L.SynthDeviceLayer(100 + i, CHANNELS, HIDDEN, EXPERTS, formats.Q4_K, p_layout, dev, keep_gguf=(i == 0), shared_type=sh_type)
                      for i in range(min(args.layers, 2))]
            rec, cpu = prefill_record(args, dev, layers, Tp)
            _, tf_peak, peak_kind = peaks()
            line = base_line(args, rec["tokens_per_s"], rec["ms_per_step"], f"moe_layer_prefill_T{Tp} (BASELINE configs[2])",
                             ("Q4_K GGUF" if p_layout == formats.GGUF else "Q4_K Pack-v3 planar") + (" + dense Q8_0 shared expert" if sh_type else ""),
                             "f16 operands, f32 accumulate", {"router": rec["router"], "l2_policy": "inputs larger than L2: 0.93 GB of weights and 0.4 GB of intermediates per step"})
            line.update({"e2e": {"value": rec["e2e_tokens_per_s"], "unit": "tokens/s", "ms_per_step": rec["e2e_ms_per_step"],
                                 "h2d_bytes_per_step": rec["h2d_bytes_per_step"], "d2h_bytes_per_step": rec["d2h_bytes_per_step"]},
                         "gpu_launches": 9 * max(4, args.steps // 4),
                         "roofline": {"bound": "tensor", "kernel": "grouped_mma_kernel<gate-up> (routed experts + shared expert, tcgen05)", "achieved": rec["gate_up_launch_tflops"],
                                      "peak": tf_peak, "unit": "TFLOP/s", "frac": rec["gate_up_launch_frac_of_bf16_peak"], "peak_kind": peak_kind, "traffic": 478.4e6 if Tp == 4096 else None,
                                      "traffic_source": "profiles/grouped_mma_prefill_T4096.md (ncu: DRAM throughput x duration of the gate-up launch)",
                                      "launch_ms": rec["stage_ms"]["gate_up_ms"]},
                         "cpu_baseline": cpu, "extra": {"prefill": rec}})
        else:
            extra_types = dict(down_type=formats.Q5_1, shared_type=formats.Q8_0) if etype == formats.Q5_K else {}
            layers = [L.SynthDeviceLayer(100 + i, CHANNELS, HIDDEN, EXPERTS, etype, layout, dev, keep_gguf=(i == 0), **extra_types) for i in range(args.layers)]
            rec, (roofline, cpu) = decode_record(args, dev, T, layers, etype, layout, True)
            extra = {"decode": rec}
            headline = etype == formats.Q4_K and layout == formats.PLANAR and T == 64 and not args.decode_only
            if headline:
                # the rest of the metric, measured in the same run on the same GPU
                for t_small in (1, 8):
                    extra[f"decode_T{t_small}"] = decode_record(args, dev, t_small, layers, etype, layout, False)[0]
                extra["prefill"] = prefill_record(args, dev, layers[:2], args.prefill_tokens)[0]
                del layers
                torch.cuda.empty_cache()
                extra["head_M16"] = head_record(args, dev, 16)[0]
                extra["head_M1"] = head_record(args, dev, 1)[0]
                extra["config1"] = config1_record(args, dev)
            line = base_line(args, rec["tokens_per_s"], rec["ms_per_step"],
                             f"moe_layer_decode_T{T} (BASELINE configs[1])" if etype == formats.Q4_K else
                             f"moe_layer_decode_T{T} (reference model encodings at the BASELINE shape)" if etype == formats.Q5_K else
                             f"q8_0_mtp_moe_block_T{T} (BASELINE configs[3])",
                             wname, "f16 activations, f32 accumulate",
                             {"activations": "binary16 in/out, FP32 accumulate", "layers_rotated": args.layers,
                              "l2_policy": "inputs larger than L2: each step streams ~650 MB of distinct expert weights",
                              "timing": f"median of {rec['timed_repeats']} timed loops of {args.steps} steps"})
            line.update({"e2e": {"value": rec["e2e_tokens_per_s"], "unit": "tokens/s", "ms_per_step": rec["e2e_ms_per_step"],
                                 "h2d_bytes_per_step": T * CHANNELS * 2 + T * EXPERTS * 4, "d2h_bytes_per_step": T * CHANNELS * 2},
                         "gpu_launches": rec["launches_per_step"] * args.steps, "roofline": roofline, "cpu_baseline": cpu, "extra": extra})
    line["clocks"] = clocks.summary()
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=64, help="token rows per step (decode batch)")
    ap.add_argument("--layers", type=int, default=4, help="independently seeded weight sets rotated over")
    ap.add_argument("--layout", default=None, choices=["planar", "gguf"], help="weight layout (default: Pack-v3 planar for Q4_K experts, GGUF blocks for Q8_0 experts)")
    ap.add_argument("--experts", default="q4_k", choices=["q4_k", "q8_0", "q5_k"],
                    help="expert encoding of the decode workload (q8_0: the MTP block; q5_k: Q5_K gate/up, Q5_1 down, Q8_0 shared expert)")
    ap.add_argument("--shared", default=None, choices=["q8_0"], help="prefill workload: the shared expert as dense Q8_0 blocks (launches of its own)")
    ap.add_argument("--cpu-tokens", type=int, default=None, help="tokens of the batch timed on the CPU baseline (0 = skip)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "head", "config1"])
    ap.add_argument("--decode-only", action="store_true", help="decode workload without the extra sub-records")
    ap.add_argument("--min-seconds", type=float, default=0.5, help="each headline timed region is repeated until it adds up to this long")
    ap.add_argument("--prefill-tokens", type=int, default=4096, help="token rows (per GPU) of the prefill record")
    ap.add_argument("--replicate", type=int, default=32, help="expert-parallel prefill: hot experts held by every rank (0 = none)")
    ap.add_argument("--no-prefill", action="store_true", help="N > 1: skip the prefill sub-record")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_ours(args)


if __name__ == "__main__":
    main()
