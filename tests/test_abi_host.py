"""CPU-only checks: the C-ABI library loads and exports every symbol the header declares, refuses
contract violations before touching a device, and the host-side format helpers agree with the oracle."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import fixtures
from tokspur_public_b200 import capi, formats, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "tsp_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tsp_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = capi.lib()
    names = header_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/tsp_moe.h but not exported"
        assert name in capi.SIGNATURES, f"{name} has no ctypes signature"


def test_prefill_entries_refuse_bad_arguments():
    lib = capi.lib()
    buf = (C.c_uint8 * 64)()
    p = C.addressof(buf) & ~15
    g = capi.MatrixSet(p + 16, None, 0, 1, 1, 64, 256, 8, 1)      # Q8_0: the tensor-core path takes Q4_K planar only
    assert lib.tsp_moe_staged_f16(C.byref(g), 0, p, None) == capi.E_TYPE
    assert lib.tsp_moe_rows_f16k(p, 8, 0, 1, 12, p, 32, p, None) == capi.E_ARG                      # columns not a multiple of 8
    assert lib.tsp_moe_rows_f16k(p, 64, 2, 1, 16, p, 32, p, None) == capi.E_ARG                     # unknown dtype
    q = capi.MatrixSet(p + 16, None, 0, 1, 1, 64, 256, 12, 1)
    assert lib.tsp_moe_grouped_gate_up(C.byref(q), C.byref(q), C.byref(q), None, p, 512, p, 512, 1, 1, 1, p, p, p, p, p, 128, None, 0, p, None) == capi.E_ARG
    assert "go together" in capi.last_error()
    assert lib.tsp_moe_grouped_down(C.byref(q), None, p, 512, 1, 1, p, p, p, p, p, 128, 3, None, 0, 0, None, 0, p, None) == capi.E_ARG   # row dtype 3


def test_expert_byte_constants():
    lib = capi.lib()
    assert lib.tsp_expert_bytes(12, 0, 1024, 2048) == 1179648
    assert lib.tsp_expert_bytes(12, 1, 1024, 2048) == 1212416
    assert lib.tsp_expert_bytes(12, 0, 2048, 512) == 589824
    assert lib.tsp_expert_bytes(8, 0, 151936, 2048) == 330612736
    assert lib.tsp_expert_bytes(12, 1, 1024, 300) == 0 and lib.tsp_expert_bytes(8, 1, 4, 32) == 0
    assert lib.tsp_moe_tasks_words(64, 512, 10, 8) == 2 + 2 * (80 + 512)


def test_contract_violations_are_refused_before_any_launch():
    lib = capi.lib()
    buf = (C.c_uint8 * 64)()
    p = C.addressof(buf) & ~15
    assert lib.tsp_moe_route(p, 16, 1, 8, 9, 0, 1, p, p, p, None) == capi.E_ARG          # selected > experts
    assert "invalid router" in capi.last_error()
    assert lib.tsp_moe_route(p, 16, 1, 8, 2, 7, 1, p, p, p, None) == capi.E_ARG          # unknown mode
    assert lib.tsp_moe_route(None, 16, 1, 8, 2, 0, 1, p, p, p, None) == capi.E_ARG
    assert lib.tsp_moe_permute(p, 4, 8, 2, 0, p, p, p, p, None) == capi.E_ARG            # tile 0
    m = capi.MatrixSet(p + 16, None, 0, 1, 1, 64, 256, 5, 0)
    assert lib.tsp_dequant_f32(C.byref(m), 0, p, p, None) == capi.E_TYPE                 # encoding without a kernel
    m = capi.MatrixSet(p + 16, None, 0, 1, 1, 64, 300, 12, 0)
    assert lib.tsp_dequant_f32(C.byref(m), 0, p, p, None) == capi.E_ARG                  # columns not block aligned
    m = capi.MatrixSet(p + 17, None, 0, 1, 1, 64, 256, 12, 0)
    assert lib.tsp_dequant_f32(C.byref(m), 0, p, p, None) == capi.E_ARG                  # misaligned base
    g = capi.MatrixSet(p + 16, None, 0, 1, 1, 64, 256, 12, 0)
    u = capi.MatrixSet(p + 16, None, 0, 1, 1, 32, 256, 12, 0)
    assert lib.tsp_moe_gate_up_swiglu(C.byref(g), C.byref(u), p, 1024, 1, 1, None, None, None, p + 4096, 256, 0, p, None) == capi.E_ARG
    with pytest.raises(capi.TspError):
        capi.call("tsp_moe_combine", None, 0, 0, None, None, 0, None, None, 0, 0, None, 1, 8, 2, None, 0, None, 0, None, None)


@pytest.mark.parametrize("type_", [8, 12, 13, 7])
def test_numpy_formats_agree_with_oracle(oracle, type_):
    rows, cols = 32, 512
    w = synth.normal(3, (rows, cols), 0.02)
    g = formats.quantize(type_, w).reshape(-1)
    assert g.size == formats.gguf_bytes(type_, rows, cols)
    dec = oracle.dequantize(type_, g, rows * cols).reshape(rows, cols)
    assert np.array_equal(dec, formats.dequantize_gguf(type_, g, rows, cols))
    err = np.abs(dec - w).max()
    assert err < {12: 0.006, 8: 0.0006, 13: 0.003, 7: 0.003}[type_]  # the encoder is sane: within a code step of the source
    lcg5 = fixtures.lcg_weights(type_, cols, rows, 1)[0]   # every code / factor bit pattern
    assert np.array_equal(oracle.dequantize(type_, lcg5, rows * cols).reshape(rows, cols).view(np.uint32),
                          formats.dequantize_gguf(type_, lcg5, rows, cols).view(np.uint32))
    if type_ in (13, 7):   # no planar form of the five-bit encodings in this build
        assert capi.lib().tsp_expert_bytes(type_, formats.PLANAR, rows, cols) == 0
        assert capi.lib().tsp_expert_bytes(type_, formats.GGUF, rows, cols) == g.size
        return
    spec = oracle.spec(type_, cols, rows)
    assert np.array_equal(formats.pack_planar(type_, g, rows, cols), oracle.pack_expert(spec, g))
    lcg = fixtures.lcg_weights(type_, cols, rows, 1)[0]
    assert np.array_equal(formats.pack_planar(type_, lcg, rows, cols), oracle.pack_expert(spec, lcg))


def test_colocated_pairs_layout(oracle):
    E, rows, cols = 4, 8, 256
    g = fixtures.lcg_weights(12, cols, rows, E, seed=5)
    u = fixtures.lcg_weights(12, cols, rows, E, seed=6)
    gp, up = formats.pack_planar_experts(12, g, E, rows, cols), formats.pack_planar_experts(12, u, E, rows, cols)
    lo, hi = formats.colocate_gate_up(gp, up)
    pb = gp.shape[1]
    for e in range(E):
        base = (lo if e < E // 2 else hi)[2 * (e % (E // 2)) * pb:]
        assert np.array_equal(base[:pb], gp[e]) and np.array_equal(base[pb:2 * pb], up[e])


def test_synthetic_generator_is_counter_based():
    a = synth.normal(7, (4, 100))
    b = synth.normal(7, (2, 100), offset=200)
    assert np.array_equal(a[2:], b)
    assert abs(float(synth.normal(1, (200000,)).std()) - 1) < 0.01
    bias = synth.zipf_bias(3, 512)
    p = np.exp(bias) / 512
    assert abs(p.sum() - 1) < 1e-5 and p.max() / p.min() > 500
