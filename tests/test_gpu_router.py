"""Router projection (FP32 GEMM for batches, GEMV for a few rows, shared-router row fused) and the top-k margin audit, against
double-precision logits. The reference's forced-route fixture (native/tests/test_moe_mm_many_gpu.cpp:96-104) pins the ids."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tokspur_public_b200 import capi, synth  # noqa: E402
from tokspur_public_b200 import layer as L  # noqa: E402


def project(w, x, extra=None, x_pad=0):
    rows, cols = w.shape
    T = x.shape[0]
    dw = torch.from_numpy(w).cuda()
    xs = torch.full((T, cols + x_pad), -7654.25, dtype=torch.float32, device="cuda")
    xs[:, :cols] = torch.from_numpy(x).cuda()
    out = torch.full((T, rows + 4), -7654.25, dtype=torch.float32, device="cuda")
    de = torch.from_numpy(extra).cuda() if extra is not None else None
    eo = torch.zeros(T, dtype=torch.float32, device="cuda") if extra is not None else None
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.call("tsp_router_project", dw.data_ptr(), rows, cols, de.data_ptr() if de is not None else None, xs.data_ptr(), (cols + x_pad) * 4, T,
              out.data_ptr(), (rows + 4) * 4, eo.data_ptr() if eo is not None else None, err.data_ptr(), L.stream_ptr())
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    o = out.cpu().numpy()
    assert np.all(o[:, rows:] == np.float32(-7654.25))   # padding canaries untouched
    return o[:, :rows], (eo.cpu().numpy() if eo is not None else None)


@pytest.mark.parametrize("T", [1, 5, 40, 300, 1000])
@pytest.mark.parametrize("rows,cols", [(512, 2048), (130, 100)])
def test_router_projection_against_double(T, rows, cols):
    w = synth.normal(7 + rows, (rows, cols), 0.05)
    extra = synth.normal(9 + rows, (cols,), 0.05)
    x = synth.normal(11 + T, (T, cols))
    got, gex = project(w, x, extra, x_pad=4)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    wex = x.astype(np.float64) @ extra.astype(np.float64)
    scale = np.maximum(1.0, np.abs(want))
    assert np.max(np.abs(got - want) / scale) <= 5e-5
    assert np.max(np.abs(gex - wex) / np.maximum(1.0, np.abs(wex))) <= 5e-5


def test_forced_route_fixture_ids_and_margins(oracle):
    E, Cn, K = 512, 64, 10
    w = np.zeros((E, Cn), np.float32)
    e = np.arange(E)
    w[:, 0] = (e - 8) / 32.0
    w[:, 1] = ((7 * e) % 17 - 8) / 16.0
    for T in (4, 130):   # the GEMV and the GEMM path
        x = np.zeros((T, Cn), np.float32)
        x[:, 0] = 1.0
        x[:, 1] = np.array([0.5, -0.5, 0.25, -0.25] * ((T + 3) // 4), np.float32)[:T]
        logits, _ = project(w, x)
        exact = x.astype(np.float64) @ w.astype(np.float64).T
        assert np.array_equal(logits.astype(np.float64), exact)   # every product and sum here is exact in binary32
        lg = torch.from_numpy(logits).cuda()
        ids = torch.zeros(T * K, dtype=torch.int32, device="cuda")
        wt = torch.zeros(T * K, dtype=torch.float32, device="cuda")
        mg = torch.zeros(T, dtype=torch.float32, device="cuda")
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        for mode in (0, 1):
            capi.call("tsp_moe_route_audit", lg.data_ptr(), E * 4, T, E, K, mode, 1, ids.data_ptr(), wt.data_ptr(), mg.data_ptr(), err.data_ptr(), L.stream_ptr())
            torch.cuda.synchronize()
            oi, ow = oracle.route_rows(exact, K, mode, True)
            assert np.array_equal(ids.cpu().numpy().view(np.uint32).reshape(T, K), oi)
            assert np.max(np.abs(wt.cpu().numpy().reshape(T, K) - ow)) <= 1e-6
            srt = np.sort(logits, axis=1)[:, ::-1]
            assert np.array_equal(mg.cpu().numpy(), (srt[:, K - 1] - srt[:, K]).astype(np.float32))
        assert int(err.item()) == 0
        tel = capi.RouterMarginTelemetry()
        fb = C.c_int(-1)
        capi.call("tsp_router_margin_evaluate", mg.data_ptr(), T, 1e-4, L.stream_ptr(), C.byref(tel), C.byref(fb))
        m = mg.cpu().numpy()
        assert tel.total_tokens == T and tel.total_layers == 1 and tel.violation_count == int((m <= 2e-4).sum())
        assert abs(tel.min_margin - float(m.min())) == 0 and abs(tel.sum_margin - float(m.astype(np.float64).sum())) <= 1e-9
        assert fb.value == int(tel.violation_count > 0) and tel.fallback_layers == fb.value
