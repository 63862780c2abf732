"""BASELINE configs[0]: ONE Q4_K matrix [1024 x 2048] (N(0, 0.02) weights of seed 0, binary16 N(0,1) activations) through both
paths of the library: M = 1 through the decode GEMV (5e-5 scaled error against the oracle) and M = 256 through the tcgen05
grouped kernel as a one-expert set (binary16 operands, FP32 accumulate: relative L2 <= 2e-3, all 256 rows checked)."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tokspur_public_b200 import capi, formats, synth  # noqa: E402
from tokspur_public_b200 import layer as L  # noqa: E402

ROWS, COLS = 1024, 2048


def matrix():
    w = formats.quantize_q4_k(synth.normal(0, (ROWS, COLS), 0.02)).reshape(-1)
    planar = torch.from_numpy(formats.pack_planar(formats.Q4_K, w, ROWS, COLS)).cuda()
    return w, planar, L.matrix_set(planar, formats.Q4_K, formats.PLANAR, ROWS, COLS, 1)


def test_single_matrix_m1_decode_gemv(oracle):
    w, planar, ms = matrix()
    x = synth.activations_f16(1, 1, COLS).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    out = torch.zeros((1, ROWS), dtype=torch.float32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.call("tsp_moe_project", C.byref(ms), dx.data_ptr(), COLS * 4, 1, 1, 1, None, None, None, out.data_ptr(), ROWS * 4, 1, err.data_ptr(),
              L.stream_ptr())
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    want = oracle.gemv(formats.Q4_K, w, COLS, ROWS, x[0])
    got = out.cpu().numpy()[0].astype(np.float64)
    assert float(np.max(np.abs(got - want) / np.maximum(1.0, np.abs(want)))) <= 5e-5


def test_single_matrix_m256_tensor_core_path(oracle):
    w, planar, ms = matrix()
    M = 256
    lib, st = capi.lib(), L.stream_ptr()
    x16 = torch.from_numpy(synth.activations_f16(1, M, COLS)).cuda()
    xk, xp = torch.zeros_like(x16), torch.zeros_like(x16)
    ids = torch.zeros(M, dtype=torch.int32, device="cuda")
    tm, counts = torch.zeros(M, dtype=torch.int32, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda")
    tasks = torch.zeros(int(lib.tsp_moe_tasks_words(M, 1, 1, 256)), dtype=torch.int32, device="cuda")
    offsets = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.zeros((M, ROWS), dtype=torch.float32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    e = err.data_ptr()
    capi.call("tsp_moe_rows_f16k", x16.data_ptr(), COLS * 2, 1, M, COLS, xk.data_ptr(), COLS * 2, e, st)
    capi.call("tsp_moe_permute", ids.data_ptr(), M, 1, 1, 256, tm.data_ptr(), counts.data_ptr(), tasks.data_ptr(), e, st)
    capi.call("tsp_moe_route_offsets", counts.data_ptr(), 1, offsets.data_ptr(), st)
    capi.call("tsp_moe_gather_rows16", xk.data_ptr(), COLS * 2, tm.data_ptr(), offsets.data_ptr(), 1, M, 1, COLS, xp.data_ptr(), COLS * 2, st)
    capi.call("tsp_moe_grouped_down", C.byref(ms), None, xp.data_ptr(), COLS * 2, M, 1, tm.data_ptr(), counts.data_ptr(), tasks.data_ptr(),
              offsets.data_ptr(), out.data_ptr(), ROWS * 4, 0, None, 0, 0, None, 0, e, st)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    xs = x16.float().cpu().numpy()
    dense = oracle.dequantize(formats.Q4_K, w, ROWS * COLS).reshape(ROWS, COLS).astype(np.float64)
    want = xs.astype(np.float64) @ dense.T          # exact weights x exact binary16 activations in double
    spot = oracle.gemv(formats.Q4_K, w, COLS, ROWS, xs[100])
    assert np.allclose(want[100], spot, rtol=1e-12, atol=1e-12)   # the matrix product above is the oracle's GEMV row for row
    got = out.cpu().numpy().astype(np.float64)
    rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    assert rel <= 2e-3, f"M = 256 through the tensor cores: relative L2 {rel:.3e}"
    assert rel <= 1e-3, f"regression guard: relative L2 {rel:.3e} (measured 3e-4)"


def test_bounded_wait_gives_up_and_reports():
    """A wait on a barrier that nothing arrives on runs out after its poll limit, the kernel sets TSP_ERR_TIMEOUT in the sticky
    error word and returns; the device stays usable (the next launch works). No fault, trap or endless loop is involved."""
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.call("tsp_selftest_bounded_wait", 1000, err.data_ptr(), L.stream_ptr())
    torch.cuda.synchronize()
    assert int(err.item()) == 8    # TSP_ERR_TIMEOUT
    err.zero_()
    x = torch.ones(4, device="cuda") * 2
    assert float(x.sum().item()) == 8.0 and int(err.item()) == 0
    lib = capi.lib()
    assert lib.tsp_selftest_bounded_wait(0, err.data_ptr(), None) == capi.E_ARG
    assert lib.tsp_selftest_bounded_wait(1 << 20, err.data_ptr(), None) == capi.E_ARG
