"""Dense Q8_0 row batches on the tensor cores (tsp_dense_mm_swiglu / tsp_dense_mm) and the prefill layer with the reference's
mix of encodings: Q4_K routed experts beside a dense Q8_0 shared expert (moe_mm_many.cpp:236-259), and the all-Q8_0 MTP block.
Bar: rel-L2 <= 2e-3 against the CPU oracle (binary16 operands, FP32 accumulate); the staged Q8_0 operand is RN16(d * q), one
rounding of the exact weight."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tokspur_public_b200 import capi, formats, synth  # noqa: E402
from tokspur_public_b200 import layer as L  # noqa: E402


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def silu(v):
    return v / (1.0 + np.exp(-v))


@pytest.mark.parametrize("T,Cn,H", [(1, 256, 256), (77, 256, 512), (300, 2048, 512), (513, 512, 256)])
def test_dense_q8_gate_up_swiglu_then_down(oracle, T, Cn, H):
    """x [T x Cn] -> h = silu(Wg x) * (Wu x) [T x H] -> y = Wd h [T x Cn], all three matrices dense Q8_0 GGUF blocks. Odd and even
    128-column spans, rows that are not a multiple of the 256-row task, one row."""
    q = lambda seed, r, c: formats.quantize(formats.Q8_0, synth.normal(seed, (r, c), 0.02)).reshape(-1)
    wg, wu, wd = q(31, H, Cn), q(32, H, Cn), q(33, Cn, H)
    dev = lambda a: torch.from_numpy(a).cuda()
    tg, tu, td = dev(wg), dev(wu), dev(wd)
    mg, mu = L.matrix_set(tg, formats.Q8_0, formats.GGUF, H, Cn, 1), L.matrix_set(tu, formats.Q8_0, formats.GGUF, H, Cn, 1)
    md = L.matrix_set(td, formats.Q8_0, formats.GGUF, Cn, H, 1)
    x16 = synth.activations_f16(34, T, Cn)
    x = dev(x16)
    xk = torch.zeros((T, Cn), dtype=torch.float16, device="cuda")
    hk = torch.zeros((T, H), dtype=torch.float16, device="cuda")
    y = torch.zeros((T, Cn), dtype=torch.float32, device="cuda")
    counters = torch.zeros(2, dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    st, e = L.stream_ptr(), err.data_ptr()
    capi.call("tsp_moe_rows_f16k", x.data_ptr(), Cn * 2, 1, T, Cn, xk.data_ptr(), Cn * 2, e, st)
    capi.call("tsp_dense_mm_swiglu", C.byref(mg), C.byref(mu), xk.data_ptr(), Cn * 2, T, hk.data_ptr(), H * 2, counters.data_ptr(), e, st)
    capi.call("tsp_dense_mm", C.byref(md), hk.data_ptr(), H * 2, T, y.data_ptr(), Cn * 4, counters.data_ptr() + 4, e, st)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    xs = x16.astype(np.float64)
    deq = lambda w, r, c: oracle.dequantize(formats.Q8_0, w, r * c).reshape(r, c).astype(np.float64)
    Wg, Wu, Wd = deq(wg, H, Cn), deq(wu, H, Cn), deq(wd, Cn, H)
    spot = oracle.gemv(formats.Q8_0, wg, Cn, H, x16[T // 2].astype(np.float32))
    assert np.allclose((xs @ Wg.T)[T // 2], spot, rtol=1e-12, atol=1e-12)      # the matrix product is the oracle's GEMV row for row
    h = silu(xs @ Wg.T) * (xs @ Wu.T)
    want = h @ Wd.T
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    assert rel_l2(got, want) <= 2e-3
    # the hidden rows come back in the K order of the tiles (positions 1 <-> 2 and 5 <-> 6 of every run of 8 swapped)
    hk_host = hk.cpu().numpy().astype(np.float64).reshape(T, H // 8, 8)[:, :, [0, 2, 1, 3, 4, 6, 5, 7]].reshape(T, H)
    assert rel_l2(hk_host, h) <= 2e-3


def test_dense_refusals():
    t = torch.zeros(128 * 272, dtype=torch.uint8, device="cuda")
    ms = L.matrix_set(t, formats.Q8_0, formats.GGUF, 128, 256, 1)
    two = L.matrix_set(torch.zeros(2 * 128 * 272, dtype=torch.uint8, device="cuda"), formats.Q8_0, formats.GGUF, 128, 256, 2)
    xk = torch.zeros((4, 256), dtype=torch.float16, device="cuda")
    y = torch.zeros((4, 128), dtype=torch.float32, device="cuda")
    c = torch.zeros(1, dtype=torch.int32, device="cuda")
    e = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib, st = capi.lib(), L.stream_ptr()
    assert lib.tsp_dense_mm(C.byref(two), xk.data_ptr(), 512, 4, y.data_ptr(), 512, c.data_ptr(), e.data_ptr(), st) != 0      # an expert set
    assert lib.tsp_dense_mm(C.byref(ms), xk.data_ptr(), 512, 0, y.data_ptr(), 512, c.data_ptr(), e.data_ptr(), st) != 0       # no rows
    assert lib.tsp_dense_mm(C.byref(ms), xk.data_ptr(), 512, 4, y.data_ptr(), 512, None, e.data_ptr(), st) != 0               # no counter
    assert lib.tsp_dense_mm(C.byref(ms), xk.data_ptr(), 500, 4, y.data_ptr(), 512, c.data_ptr(), e.data_ptr(), st) != 0       # short stride
    torch.cuda.synchronize()


@pytest.mark.parametrize("expert_type,layout,T,E,K,Cn,H", [
    (formats.Q4_K, formats.PLANAR, 300, 8, 2, 512, 256),     # the reference's mix: Q4_K planar experts, dense Q8_0 shared expert
    (formats.Q4_K, formats.GGUF, 150, 4, 2, 256, 256),       # raw Q4_K blocks beside the Q8_0 shared expert
    (formats.Q8_0, formats.GGUF, 260, 4, 2, 256, 256),       # the MTP block: Q8_0 experts and shared expert (rides in the launches)
])
def test_prefill_layer_with_q8_shared_expert(oracle, expert_type, layout, T, E, K, Cn, H):
    host = L.synth_host_layer(21, Cn, H, E, K, expert_type=expert_type, shared_type=formats.Q8_0)
    dl = L.DeviceLayer(host, layout, "cuda", shared_layout=formats.GGUF)
    ps = L.PrefillScratch(Cn, H, E, K, T, "cuda")
    x16 = synth.activations_f16(22, T, Cn)
    logits = synth.router_logits(23, T, E, synth.zipf_bias(24, E) * 2)
    x32 = torch.from_numpy(x16.astype(np.float32)).cuda()
    out = torch.zeros((T, Cn), dtype=torch.float32, device="cuda")
    for _ in range(2):   # twice: the item counters are cleared by every call
        out.zero_()
        L.moe_layer_prefill(dl, ps, x32, torch.from_numpy(logits).cuda(), out)
        torch.cuda.synchronize()
        assert ps.base.error_word() == 0
        sample = np.unique(np.linspace(0, T - 1, 24).astype(int))
        want, st = oracle.moe_layer(host.oracle_dict(), x16[sample].astype(np.float32), logits[sample], threads=4, stages=True)
        assert rel_l2(ps.routed_rows(T).reshape(T, K, Cn)[sample], st["routed"]) <= 2e-3
        assert rel_l2(ps.shared_out_rows(T)[sample], st["shared_out"]) <= 2e-3
        assert rel_l2(out.cpu().numpy()[sample], want) <= 2e-3
