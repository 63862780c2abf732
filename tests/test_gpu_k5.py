"""The five-bit encodings of the reference's model on the decode-size path: Q5_K gate / up tensors and Q5_1 down tensors
(model.cpp:50-57; decoders numeric.cpp:38-50), plain GGUF rows. Dequantised weights bit-exact against the CPU oracle (which is
pinned to the reference's decoder and its fixture blocks); projections and whole layers within the reference's 5e-5 scaled
error (ffn_check.cpp:48-55)."""
import ctypes as C

import numpy as np
import pytest

import fixtures

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tokspur_public_b200 import capi, formats, synth  # noqa: E402
from tokspur_public_b200 import layer as L  # noqa: E402

DEV = "cuda"


def scaled_error(actual, expected):
    return float(np.max(np.abs(actual.astype(np.float64) - expected) / np.maximum(1.0, np.abs(expected))))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.mark.parametrize("type_", [formats.Q5_K, formats.Q5_1])
def test_dequant_bit_exact(oracle, type_):
    cols, rows, E = 512, 16, 2
    for w in (fixtures.lcg_weights(type_, cols, rows, E),      # every bit pattern of codes and factors, extreme scales
              np.stack([formats.quantize(type_, synth.normal(40 + e, (rows, cols), 0.02)).reshape(-1) for e in range(E)])):
        t = dev(w)
        ms = L.matrix_set(t, type_, formats.GGUF, rows, cols, E)
        out = torch.empty(rows * cols, dtype=torch.float32, device=DEV)
        e = torch.zeros(1, dtype=torch.int32, device=DEV)
        for ex in range(E):
            capi.call("tsp_dequant_f32", C.byref(ms), ex, out.data_ptr(), e.data_ptr(), L.stream_ptr())
            got = out.cpu().numpy()
            assert np.array_equal(got.view(np.uint32), oracle.dequantize(type_, w[ex], rows * cols).view(np.uint32))
        torch.cuda.synchronize()
        assert int(e.item()) == 0


def test_planar_layout_is_refused():
    t = torch.zeros(16 * 2 * 176, dtype=torch.uint8, device=DEV)
    ms = L.matrix_set(t, formats.Q5_K, formats.GGUF, 16, 512, 1)
    ms.layout = formats.PLANAR
    out = torch.empty(16 * 512, dtype=torch.float32, device=DEV)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert capi.lib().tsp_dequant_f32(C.byref(ms), 0, out.data_ptr(), e.data_ptr(), L.stream_ptr()) != 0
    assert capi.lib().tsp_expert_bytes(formats.Q5_K, formats.PLANAR, 16, 512) == 0


@pytest.mark.parametrize("type_,rows,cols,T", [(formats.Q5_K, 64, 512, 5), (formats.Q5_1, 96, 256, 16), (formats.Q5_K, 32, 2048, 11), (formats.Q5_1, 16, 64, 1)])
def test_dense_projection_against_oracle(oracle, type_, rows, cols, T):
    w = formats.quantize(type_, synth.normal(51, (rows, cols), 0.02)).reshape(-1)
    t = dev(w)
    ms = L.matrix_set(t, type_, formats.GGUF, rows, cols, 1)
    x = synth.normal(52, (T, cols), 1.0)
    dx = dev(x)
    out = torch.zeros((T, rows), dtype=torch.float32, device=DEV)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    capi.call("tsp_moe_project", C.byref(ms), dx.data_ptr(), cols * 4, 1, T, 1, None, None, None, out.data_ptr(), rows * 4, 0, e.data_ptr(), L.stream_ptr())
    torch.cuda.synchronize()
    assert int(e.item()) == 0
    want = np.stack([oracle.gemv(type_, w, cols, rows, x[i]) for i in range(T)])
    assert scaled_error(out.cpu().numpy(), want) <= 5e-5


@pytest.mark.parametrize("T", [1, 8, 29, 64])
@pytest.mark.parametrize("shared_type", [formats.Q8_0, formats.Q5_K])
def test_layer_q5k_gate_up_q51_down(oracle, T, shared_type):
    """The reference model's pairing: Q5_K gate / up, Q5_1 down, Q8_0 shared expert (and, as a second case, a Q5_K shared
    expert through the same plain kernel), top-4 of 16 experts so that tiles of more than 8 routes occur."""
    Cn, H, E, K = 512, 256, 16, 4
    q = formats.quantize
    ex = lambda s, t, r, c: np.stack([q(t, synth.normal(s * 1000 + e, (r, c), 0.02)).reshape(-1) for e in range(E)])
    host = L.HostLayer(Cn, H, E, K, formats.Q5_K, shared_type, ex(1, formats.Q5_K, H, Cn), ex(2, formats.Q5_K, H, Cn), ex(3, formats.Q5_1, Cn, H),
                       q(shared_type, synth.normal(7001, (H, Cn), 0.02)).reshape(-1), q(shared_type, synth.normal(7002, (H, Cn), 0.02)).reshape(-1),
                       q(shared_type, synth.normal(7003, (Cn, H), 0.02)).reshape(-1), synth.normal(7004, (Cn,), 0.02), down_type=formats.Q5_1)
    x16 = synth.activations_f16(5, T, Cn)
    logits = synth.router_logits(6, T, E)
    dl = L.DeviceLayer(host, formats.GGUF, DEV)
    s = L.Scratch(Cn, H, E, K, T, DEV)
    out = torch.zeros((T, Cn), dtype=torch.float32, device=DEV)
    L.moe_layer_decode(dl, s, dev(x16.astype(np.float32)), dev(logits), out)
    torch.cuda.synchronize()
    assert s.error_word() == 0
    want, st = oracle.moe_layer(host.oracle_dict(), x16.astype(np.float32), logits, threads=4, stages=True)
    assert np.array_equal(s.ids.cpu().numpy().view(np.uint32)[:T * K].reshape(T, K), st["indices"])
    assert scaled_error(s.hidden.cpu().numpy()[:T * K * H].reshape(T, K, H), st["activated"]) <= 5e-5
    assert scaled_error(s.routed.cpu().numpy()[:T * K * Cn].reshape(T, K, Cn), st["routed"]) <= 5e-5
    assert scaled_error(s.shared_out.cpu().numpy()[:T * Cn].reshape(T, Cn), st["shared_out"]) <= 5e-5
    assert scaled_error(out.cpu().numpy(), want) <= 5e-5


def test_nonfinite_scale_sets_the_error_word():
    w = formats.quantize(formats.Q5_1, synth.normal(61, (16, 64), 0.02)).reshape(-1).copy()
    w[0:2] = [0x00, 0x7c]   # d = +inf in the first block
    t = dev(w)
    ms = L.matrix_set(t, formats.Q5_1, formats.GGUF, 16, 64, 1)
    dx = dev(synth.normal(62, (1, 64), 1.0))
    out = torch.zeros((1, 16), dtype=torch.float32, device=DEV)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    capi.call("tsp_moe_project", C.byref(ms), dx.data_ptr(), 256, 1, 1, 1, None, None, None, out.data_ptr(), 64, 0, e.data_ptr(), L.stream_ptr())
    torch.cuda.synchronize()
    assert int(e.item()) & capi.ERR_NONFINITE
