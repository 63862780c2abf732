"""Harness objects over the C ABI: device-resident MoE layer weights, caller-owned scratch and the
operator calls, mirroring the reference's MoeWeights / MoeScratch / encode_moe (moe.hpp:9-45).

torch supplies device memory and streams only; every computation is a libtsp_moe.so kernel.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import capi, formats
from .capi import MatrixSet, MoeScratch, MoeWeights


def _dev(a: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def matrix_set(t: torch.Tensor, type_: int, layout: int, rows: int, cols: int, experts: int = 1, *, base_hi: torch.Tensor | None = None,
               split: int | None = None, expert_stride: int | None = None, offset: int = 0) -> MatrixSet:
    bytes_ = int(capi.lib().tsp_expert_bytes(type_, layout, rows, cols))
    return MatrixSet(t.data_ptr() + offset, (base_hi.data_ptr() + offset) if base_hi is not None else None,
                     expert_stride if expert_stride is not None else bytes_, split if split is not None else experts,
                     experts, rows, cols, type_, layout)


@dataclass
class HostLayer:
    """One MoE layer's weights as GGUF bytes on the host (the oracle's input)."""
    channels: int
    hidden: int
    experts: int
    selected: int
    expert_type: int
    shared_type: int
    gate: np.ndarray         # [E, gguf bytes of hidden x channels]
    up: np.ndarray
    down: np.ndarray         # [E, gguf bytes of channels x hidden]
    shared_gate: np.ndarray
    shared_up: np.ndarray
    shared_down: np.ndarray
    shared_router: np.ndarray  # f32 [channels]
    down_type: int | None = None  # defaults to expert_type

    def oracle_dict(self, mode: int = 0, normalize: bool = True) -> dict:
        return dict(channels=self.channels, hidden=self.hidden, experts=self.experts, selected=self.selected,
                    expert_type=self.expert_type, shared_type=self.shared_type, gate=self.gate, up=self.up, down=self.down,
                    shared_gate=self.shared_gate, shared_up=self.shared_up, shared_down=self.shared_down,
                    shared_router=self.shared_router, router=None, mode=mode, normalize=normalize,
                    down_type=self.down_type if self.down_type not in (None, self.expert_type) else 0)


def synth_host_layer(seed: int, channels: int, hidden: int, experts: int, selected: int, expert_type: int = formats.Q4_K,
                     shared_type: int | None = None, sigma: float = 0.02) -> HostLayer:
    """Seeded N(0, sigma) weights quantised with this build's encoders."""
    from . import synth
    shared_type = expert_type if shared_type is None else shared_type
    q = formats.quantize

    def experts_of(s, rows, cols):
        return np.stack([q(expert_type, synth.normal(s * 100003 + e, (rows, cols), sigma)).reshape(-1) for e in range(experts)])

    return HostLayer(channels, hidden, experts, selected, expert_type, shared_type,
                     experts_of(seed * 4 + 0, hidden, channels), experts_of(seed * 4 + 1, hidden, channels),
                     experts_of(seed * 4 + 2, channels, hidden),
                     q(shared_type, synth.normal(seed * 4 + 3, (hidden, channels), sigma)).reshape(-1),
                     q(shared_type, synth.normal(seed * 4 + 3 + 7777, (hidden, channels), sigma)).reshape(-1),
                     q(shared_type, synth.normal(seed * 4 + 3 + 9999, (channels, hidden), sigma)).reshape(-1),
                     synth.normal(seed * 4 + 3 + 5555, (channels,), sigma))


class DeviceLayer:
    """Device-resident weights of one layer in the chosen layout, plus their matrix-set descriptors."""

    def __init__(self, host: HostLayer, layout: int = formats.PLANAR, device="cuda", shared_layout: int | None = None):
        C_, H, E = host.channels, host.hidden, host.experts
        self.host = host
        self.layout = layout
        shared_layout = layout if shared_layout is None else shared_layout
        et, st = host.expert_type, host.shared_type
        dt = host.down_type or et
        self.tensors = []

        def keep(t):
            self.tensors.append(t)
            return t

        if layout == formats.PLANAR:
            gp = formats.pack_planar_experts(et, host.gate, E, H, C_)
            up = formats.pack_planar_experts(et, host.up, E, H, C_)
            pb = gp.shape[1]
            if E % 2 == 0:
                lo, hi = formats.colocate_gate_up(gp, up)
                tlo, thi = keep(_dev(lo, device)), keep(_dev(hi, device))
                gate = matrix_set(tlo, et, layout, H, C_, E, base_hi=thi, split=E // 2, expert_stride=2 * pb)
                upm = matrix_set(tlo, et, layout, H, C_, E, base_hi=thi, split=E // 2, expert_stride=2 * pb, offset=pb)
            else:
                tg, tu = keep(_dev(gp, device)), keep(_dev(up, device))
                gate, upm = matrix_set(tg, et, layout, H, C_, E), matrix_set(tu, et, layout, H, C_, E)
            td = keep(_dev(formats.pack_planar_experts(dt, host.down, E, C_, H), device))
        else:
            tg, tu, td = keep(_dev(host.gate, device)), keep(_dev(host.up, device)), keep(_dev(host.down, device))
            gate, upm = matrix_set(tg, et, layout, H, C_, E), matrix_set(tu, et, layout, H, C_, E)
        down = matrix_set(td, dt, layout, C_, H, E)

        def dense(b, rows, cols):
            data = formats.pack_planar(st, b, rows, cols) if shared_layout == formats.PLANAR else b
            return matrix_set(keep(_dev(data, device)), st, shared_layout, rows, cols, 1)

        self.shared_router = keep(_dev(host.shared_router.astype(np.float32), device))
        self.weights = MoeWeights(gate, upm, down, dense(host.shared_gate, H, C_), dense(host.shared_up, H, C_),
                                  dense(host.shared_down, C_, H), self.shared_router.data_ptr())


class Scratch:
    """Caller-owned scratch for `capacity` token rows (MoeScratch / MoeMmManyScratch)."""

    def __init__(self, channels: int, hidden: int, experts: int, selected: int, capacity: int, device="cuda", decode_buffers: bool = True):
        f32, u32 = torch.float32, torch.int32  # int32 storage holds uint32 bit patterns
        z = lambda n, dt: torch.zeros(max(int(n), 1), dtype=dt, device=device)
        big = (lambda n, dt: z(n, dt)) if decode_buffers else (lambda n, dt: z(1, dt))   # the prefill path keeps its own forms of these
        self.capacity = capacity
        self.shape = (channels, hidden, experts, selected)
        self.ids = z(capacity * selected, u32)
        self.weights = z(capacity * selected, f32)
        self.hidden = big(capacity * selected * hidden, f32)
        self.routed = big(capacity * selected * channels, f32)
        self.shared_hidden = big(capacity * hidden, f32)
        self.shared_out = z(capacity * channels, f32)
        self.shared_logit = z(capacity, f32)
        self.x32 = big(capacity * channels, f32)
        self.token_map = z(experts * capacity, u32)
        self.counts = z(experts, u32)
        self.tasks = z(capacity * selected + 2 * experts + 2, u32)  # covers every tile size >= 2
        self.error = z(1, u32)
        self.c = MoeScratch(self.ids.data_ptr(), self.weights.data_ptr(), self.hidden.data_ptr(), self.routed.data_ptr(),
                            self.shared_hidden.data_ptr(), self.shared_out.data_ptr(), self.shared_logit.data_ptr(),
                            self.x32.data_ptr(), self.token_map.data_ptr(), self.counts.data_ptr(), self.tasks.data_ptr(), capacity)

    def error_word(self) -> int:
        w = C.c_uint32(0)
        rc = capi.lib().tsp_error_word_read(self.error.data_ptr(), stream_ptr(), C.byref(w))
        if rc not in (0, capi.E_DEVICE):
            capi.check(rc)
        return w.value

    def reset_error(self) -> None:
        capi.call("tsp_error_word_reset", self.error.data_ptr(), stream_ptr())


def moe_layer_decode(dl: DeviceLayer, s: Scratch, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor,
                     mode: int = 0, normalize: bool = True) -> None:
    """Launch one whole layer on the current stream. x/out: [T, channels] float32 or float16; logits [T, E] float32."""
    C_, H, E, K = s.shape
    T = x.shape[0]
    xd = 1 if x.dtype == torch.float16 else 0
    od = 1 if out.dtype == torch.float16 else 0
    capi.call("tsp_moe_layer_decode", C.byref(dl.weights), C.byref(s.c), x.data_ptr(), x.stride(0) * x.element_size(), xd,
              logits.data_ptr(), logits.stride(0) * 4, T, C_, H, E, K, mode, int(normalize), out.data_ptr(),
              out.stride(0) * out.element_size(), od, s.error.data_ptr(), stream_ptr())


class SynthDeviceLayer:
    """One MoE layer of seeded synthetic weights generated and packed on the device (benchmark scale).

    Seeds: gate/up/down/shared streams are `seed*8 + {0,1,2,3..5}`; the shared-router vector `seed*8 + 6`.
    `expert_range` restricts the routed experts held to [lo, hi) of the global id space (expert parallelism):
    the stream position of an expert does not depend on the range, so shards equal slices of the full layer."""

    def __init__(self, seed: int, channels: int, hidden: int, experts: int, expert_type: int = formats.Q4_K,
                 layout: int = formats.PLANAR, device="cuda", sigma: float = 0.02, expert_range: tuple[int, int] | None = None,
                 keep_gguf: bool = False, expert_ids: list[int] | None = None, shared_type: int | None = None, down_type: int | None = None):
        lib = capi.lib()
        lo, hi = expert_range if expert_range else (0, experts)
        # `expert_ids` names the routed experts held one by one (expert parallelism with replicated experts): local slot i holds
        # global expert expert_ids[i]
        ids = list(expert_ids) if expert_ids is not None else list(range(lo, hi))
        n = len(ids)
        self.channels, self.hidden, self.experts_global, self.experts_local, self.first_expert = channels, hidden, experts, n, ids[0]
        self.expert_ids = ids
        self.type, self.layout = expert_type, layout
        epb = formats.block_geometry(expert_type)[0]
        gb = int(lib.tsp_expert_bytes(expert_type, formats.GGUF, hidden, channels))
        pb = int(lib.tsp_expert_bytes(expert_type, formats.PLANAR, hidden, channels))
        blocks_per_expert = hidden * channels // epb
        st = stream_ptr()
        u8 = lambda nbytes: torch.empty(int(nbytes), dtype=torch.uint8, device=device)

        self.down_type = expert_type if down_type is None else down_type
        assert self.down_type == expert_type or layout == formats.GGUF, "a down encoding of its own is kept as raw GGUF blocks"

        def gen(stream_seed, which, type_=expert_type):
            """The experts `which` (global ids) of one weight stream; runs of consecutive ids become one call."""
            if type_ != expert_type:   # tensors in another encoding (a dense shared expert, the down experts): raw blocks
                nb = int(lib.tsp_expert_bytes(type_, formats.GGUF, hidden, channels))
                per = hidden * channels // formats.block_geometry(type_)[0]
                t = u8(len(which) * nb)
                for i, e in enumerate(which):
                    capi.call("tsp_synth_weights", type_, stream_seed, e * per, per, sigma, t.data_ptr() + i * nb, st)
                return t
            t = u8(len(which) * gb)
            at = 0
            while at < len(which):
                run = 1
                while at + run < len(which) and which[at + run] == which[at] + run:
                    run += 1
                capi.call("tsp_synth_weights", expert_type, stream_seed, which[at] * blocks_per_expert, run * blocks_per_expert, sigma,
                          t.data_ptr() + at * gb, st)
                at += run
            return t

        g, u, d = gen(seed * 8 + 0, ids), gen(seed * 8 + 1, ids), gen(seed * 8 + 2, ids, self.down_type)
        self.shared_type = expert_type if shared_type is None else shared_type
        sg, su, sd = (gen(seed * 8 + 3 + i, [0], self.shared_type) for i in range(3))
        self.shared_router = torch.empty(channels, dtype=torch.float32, device=device)
        capi.call("tsp_synth_weights", capi.TYPE_F32, seed * 8 + 6, 0, channels, sigma, self.shared_router.data_ptr(), st)
        self.gguf = dict(gate=g, up=u, down=d, shared_gate=sg, shared_up=su, shared_down=sd) if keep_gguf or layout == formats.GGUF else None
        self.tensors = []
        if layout == formats.PLANAR:
            def pack(src, rows, cols, count, dst, dst_off, stride):
                capi.call("tsp_pack_planar", expert_type, rows, cols, count, src.data_ptr(), gb, dst.data_ptr() + dst_off, stride, st)
            if n % 2 == 0 and n >= 2:
                half = n // 2
                plo, phi = u8(half * 2 * pb), u8(half * 2 * pb)
                pack(g[: half * gb], hidden, channels, half, plo, 0, 2 * pb)
                pack(u[: half * gb], hidden, channels, half, plo, pb, 2 * pb)
                pack(g[half * gb:], hidden, channels, half, phi, 0, 2 * pb)
                pack(u[half * gb:], hidden, channels, half, phi, pb, 2 * pb)
                gate = matrix_set(plo, expert_type, layout, hidden, channels, n, base_hi=phi, split=half, expert_stride=2 * pb)
                up = matrix_set(plo, expert_type, layout, hidden, channels, n, base_hi=phi, split=half, expert_stride=2 * pb, offset=pb)
                self.tensors += [plo, phi]
            else:
                pg, pu = u8(n * pb), u8(n * pb)
                pack(g, hidden, channels, n, pg, 0, pb)
                pack(u, hidden, channels, n, pu, 0, pb)
                gate, up = matrix_set(pg, expert_type, layout, hidden, channels, n), matrix_set(pu, expert_type, layout, hidden, channels, n)
                self.tensors += [pg, pu]
            pd = u8(n * pb)
            pack(d, channels, hidden, n, pd, 0, pb)
            down = matrix_set(pd, expert_type, layout, channels, hidden, n)
            self.tensors.append(pd)
            if self.shared_type != expert_type:   # raw blocks of the other encoding, as generated
                shared = [matrix_set(sg, self.shared_type, formats.GGUF, hidden, channels), matrix_set(su, self.shared_type, formats.GGUF, hidden, channels),
                          matrix_set(sd, self.shared_type, formats.GGUF, channels, hidden)]
                self.tensors += [sg, su, sd]
            else:
                psg, psu, psd = u8(pb), u8(pb), u8(pb)
                pack(sg, hidden, channels, 1, psg, 0, pb)
                pack(su, hidden, channels, 1, psu, 0, pb)
                pack(sd, channels, hidden, 1, psd, 0, pb)
                self.tensors += [psg, psu, psd]
                shared = [matrix_set(psg, expert_type, layout, hidden, channels), matrix_set(psu, expert_type, layout, hidden, channels),
                          matrix_set(psd, expert_type, layout, channels, hidden)]
            torch.cuda.synchronize()
            if not keep_gguf:
                del g, u, d, sg, su, sd
        else:
            gate, up = matrix_set(g, expert_type, layout, hidden, channels, n), matrix_set(u, expert_type, layout, hidden, channels, n)
            down = matrix_set(d, self.down_type, layout, channels, hidden, n)
            shared = [matrix_set(sg, self.shared_type, layout, hidden, channels), matrix_set(su, self.shared_type, layout, hidden, channels),
                      matrix_set(sd, self.shared_type, layout, channels, hidden)]
        self.weights = MoeWeights(gate, up, down, shared[0], shared[1], shared[2], self.shared_router.data_ptr())

    def host_layer(self, selected: int) -> HostLayer:
        """GGUF bytes of this layer on the host (needs keep_gguf=True): the CPU baseline's input."""
        assert self.gguf is not None
        h = {k: v.cpu().numpy() for k, v in self.gguf.items()}
        n = self.experts_local
        return HostLayer(self.channels, self.hidden, n, selected, self.type, self.shared_type, h["gate"].reshape(n, -1), h["up"].reshape(n, -1),
                         h["down"].reshape(n, -1), h["shared_gate"], h["shared_up"], h["shared_down"], self.shared_router.cpu().numpy(),
                         down_type=self.down_type)


class PrefillScratch:
    """Extra caller-owned buffers of the prefill-size path (grouped tensor-core GEMMs) for `capacity` token rows."""

    def __init__(self, channels: int, hidden: int, experts: int, selected: int, capacity: int, device="cuda"):
        i32, f16 = torch.int32, torch.float16
        z = lambda n, dt: torch.zeros(max(int(n), 1), dtype=dt, device=device)
        routes = capacity * selected
        self.tile = 256   # routes per task of the table the layer call builds (TSP_GROUPED_TILE)
        self.base = Scratch(channels, hidden, experts, selected, capacity, device, decode_buffers=False)
        self.routed16 = torch.zeros((routes, channels), dtype=f16, device=device)   # per-route expert outputs, binary16
        self.xk = torch.zeros((capacity, channels), dtype=f16, device=device)       # input rows, tile K order
        self.xp = torch.zeros((routes, channels), dtype=f16, device=device)         # their routed copy, permuted position order
        self.hp = torch.zeros((routes, hidden), dtype=f16, device=device)           # hidden rows, permuted position order
        self.offsets = z(experts + 5, i32)   # first position of every expert, total, and the four item counters
        self.tasks = z(int(capi.lib().tsp_moe_tasks_words(capacity, experts, selected, self.tile)), i32)
        self.s_hp = torch.zeros((capacity, hidden), dtype=f16, device=device)       # the shared expert's hidden rows
        base = capi.MoeScratch.from_buffer_copy(self.base.c)
        base.d_tasks = self.tasks.data_ptr()
        base.d_routed = self.routed16.data_ptr()
        self.c = capi.MoePrefillScratch(base, self.xk.data_ptr(), self.xp.data_ptr(), self.hp.data_ptr(), self.offsets.data_ptr(), self.s_hp.data_ptr())

    def routed_rows(self, tokens: int):
        """Per-route expert outputs [tokens*selected, channels] of the last layer call (binary16 on this path) as float32."""
        K = self.base.shape[3]
        return self.routed16[: tokens * K].float().cpu().numpy()

    def shared_out_rows(self, tokens: int):
        """The shared expert's output rows [tokens, channels] of the last layer call as float32."""
        Cn = self.base.shape[0]
        return self.base.shared_out.cpu().numpy()[: tokens * Cn].reshape(tokens, Cn)


def moe_layer_prefill(dl, ps: PrefillScratch, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor, mode: int = 0, normalize: bool = True) -> None:
    """One MoE layer for a prefill-size batch through the grouped tcgen05 GEMMs (tsp_moe_layer_prefill).
    x: [T, channels] float32 or float16 rows; out float32 or float16."""
    s = ps.base
    C_, H, E, K = s.shape
    T = x.shape[0]
    xd = 1 if x.dtype == torch.float16 else 0
    od = 1 if out.dtype == torch.float16 else 0
    capi.call("tsp_moe_layer_prefill", C.byref(dl.weights), C.byref(ps.c), x.data_ptr(), x.stride(0) * x.element_size(), xd, logits.data_ptr(),
              logits.stride(0) * 4, T, C_, H, E, K, mode, int(normalize), out.data_ptr(), out.stride(0) * out.element_size(), od,
              s.error.data_ptr(), stream_ptr())
