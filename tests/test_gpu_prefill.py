"""Prefill-size path (grouped tcgen05 GEMMs) against the CPU oracle: hidden rows and routed rows per stage, then whole layers
with skewed expert loads, empty experts, partial tiles and experts with more than one tile of 128 routes.
Bar: rel-L2 <= 2e-3 (binary16 operands, FP32 accumulate); the reference's own bound for this path is NMSE 2e-3."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tokspur_public_b200 import capi, formats, synth  # noqa: E402
from tokspur_public_b200 import layer as L  # noqa: E402


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize("T,E,K,skew", [(3, 4, 2, False), (40, 4, 2, False), (200, 8, 3, True), (700, 8, 2, True), (1300, 4, 1, True)])
def test_prefill_layer_against_oracle(oracle, T, E, K, skew):
    Cn, H = 256, 256
    host = L.synth_host_layer(5, Cn, H, E, K, expert_type=formats.Q4_K)
    dl = L.DeviceLayer(host, formats.PLANAR, "cuda")
    ps = L.PrefillScratch(Cn, H, E, K, T, "cuda")
    x16 = synth.activations_f16(7, T, Cn)
    logits = synth.router_logits(8, T, E, synth.zipf_bias(9, E) * 3 if skew else None)
    x32 = torch.from_numpy(x16.astype(np.float32)).cuda()
    out = torch.zeros((T, Cn), dtype=torch.float32, device="cuda")
    L.moe_layer_prefill(dl, ps, x32, torch.from_numpy(logits).cuda(), out)
    torch.cuda.synchronize()
    assert ps.base.error_word() == 0
    n = min(T, 24)
    sample = np.unique(np.linspace(0, T - 1, n).astype(int))
    want, st = oracle.moe_layer(host.oracle_dict(), x16[sample].astype(np.float32), logits[sample], threads=4, stages=True)
    ids = ps.base.ids.cpu().numpy().view(np.uint32)[:T * K].reshape(T, K)
    assert np.array_equal(ids[sample], st["indices"])
    routed = ps.routed_rows(T).reshape(T, K, Cn)
    assert rel_l2(routed[sample], st["routed"]) <= 2e-3
    shared = ps.shared_out_rows(T)
    assert rel_l2(shared[sample], st["shared_out"]) <= 2e-3
    assert rel_l2(out.cpu().numpy()[sample], want) <= 2e-3


@pytest.mark.parametrize("T,E,K,Cn,H,order", [(40, 4, 2, 256, 256, "separate"), (700, 8, 2, 512, 256, "gate_first"), (300, 3, 2, 256, 512, "up_first")])
def test_prefill_layer_gguf_blocks_against_oracle(oracle, T, E, K, Cn, H, order):
    """The same layer with the expert and shared tensors left as plain GGUF super-blocks (no planar copy): the code and header
    maps walk the 144-byte blocks. `order` puts gate and up in one allocation (one copy brings both when up follows gate at a
    constant distance) or the other way round (two copies), or leaves them as separate allocations."""
    host = L.synth_host_layer(11, Cn, H, E, K, expert_type=formats.Q4_K)
    dl = L.DeviceLayer(host, formats.GGUF, "cuda")
    if order != "separate":
        pair = np.concatenate([host.gate.reshape(-1), host.up.reshape(-1)] if order == "gate_first" else [host.up.reshape(-1), host.gate.reshape(-1)])
        both = torch.from_numpy(pair).cuda()
        dl.tensors.append(both)
        n = host.gate.size
        g_off, u_off = (0, n) if order == "gate_first" else (n, 0)
        dl.weights.gate = L.matrix_set(both, formats.Q4_K, formats.GGUF, H, Cn, E, offset=g_off)
        dl.weights.up = L.matrix_set(both, formats.Q4_K, formats.GGUF, H, Cn, E, offset=u_off)
    ps = L.PrefillScratch(Cn, H, E, K, T, "cuda")
    x16 = synth.activations_f16(12, T, Cn)
    logits = synth.router_logits(13, T, E, synth.zipf_bias(14, E) * 2)
    x32 = torch.from_numpy(x16.astype(np.float32)).cuda()
    out = torch.zeros((T, Cn), dtype=torch.float32, device="cuda")
    L.moe_layer_prefill(dl, ps, x32, torch.from_numpy(logits).cuda(), out)
    torch.cuda.synchronize()
    assert ps.base.error_word() == 0
    sample = np.unique(np.linspace(0, T - 1, 24).astype(int))
    want, st = oracle.moe_layer(host.oracle_dict(), x16[sample].astype(np.float32), logits[sample], threads=4, stages=True)
    routed = ps.routed_rows(T).reshape(T, K, Cn)
    assert rel_l2(routed[sample], st["routed"]) <= 2e-3
    assert rel_l2(ps.shared_out_rows(T)[sample], st["shared_out"]) <= 2e-3
    assert rel_l2(out.cpu().numpy()[sample], want) <= 2e-3
    # the planar copy of the same weights gives the same bits: both layouts stage identical binary16 operands
    dp = L.DeviceLayer(host, formats.PLANAR, "cuda")
    out_p = torch.zeros_like(out)
    L.moe_layer_prefill(dp, ps, x32, torch.from_numpy(logits).cuda(), out_p)
    torch.cuda.synchronize()
    assert torch.equal(out, out_p)


def test_staged_weight_values_against_rounded_reference(oracle):
    """The binary16 weight values the tensor-core kernels multiply, against RN16 of the reference's dequantised value.
    The kernels stage RN16((q - 8) * RN16(d*sc) + RN16(8*d*sc - dmin*mn)): three roundings of small quantities instead of one
    rounding of the exact value. Bound checked here: relative L2 deviation from the exact values <= 4e-4 (one rounding alone
    gives about 2.1e-4), no value further than 2^-10 of its group's largest magnitude from the once-rounded value."""
    rows, cols = 128, 2048
    w = formats.quantize_q4_k(synth.normal(17, (rows, cols), 0.02)).reshape(-1)
    planar = formats.pack_planar(formats.Q4_K, w, rows, cols)
    t = torch.from_numpy(planar).cuda()
    ms = L.matrix_set(t, formats.Q4_K, formats.PLANAR, rows, cols, 1)
    out = torch.zeros((rows, cols), dtype=torch.float16, device="cuda")
    capi.call("tsp_moe_staged_f16", C.byref(ms), 0, out.data_ptr(), L.stream_ptr())
    torch.cuda.synchronize()
    got = out.cpu().numpy().astype(np.float64)
    exact = oracle.dequantize(formats.Q4_K, w, rows * cols).reshape(rows, cols).astype(np.float64)
    once = exact.astype(np.float16).astype(np.float64)
    rel = np.linalg.norm(got - exact) / np.linalg.norm(exact)
    rel_once = np.linalg.norm(once - exact) / np.linalg.norm(exact)
    group_max = np.abs(exact).reshape(rows, cols // 32, 32).max(axis=2, keepdims=True)
    dev = (np.abs(got - once).reshape(rows, cols // 32, 32) / np.maximum(group_max, 1e-30)).max()
    print(f"staged weights: rel-L2 vs exact {rel:.3e} (one rounding: {rel_once:.3e}), worst deviation from RN16 {dev:.3e} of the group maximum")
    assert rel <= 4e-4 and dev <= 2.0 ** -10
