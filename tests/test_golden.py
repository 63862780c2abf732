"""Replays the committed outputs of the reference's own CPU code (tests/golden/reference_outputs.npz,
made by tests/golden/make_golden.py) against the CPU oracle. Inputs are regenerated from integer recipes."""
import os

import numpy as np
import pytest

import fixtures
import golden_cases

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz"))


@pytest.mark.parametrize("type_", [8, 12, 13, 7])
def test_decode_and_gemv_match_reference_outputs(oracle, type_):
    cols, rows = 512, 16
    w = fixtures.lcg_weights(type_, cols, rows, 2)
    for e in range(2):
        got = oracle.dequantize(type_, w[e], rows * cols)
        assert np.array_equal(got.view(np.uint32), GOLD[f"dequant_{type_}"][e].view(np.uint32))
    x = fixtures.lcg_activations(3, cols)
    assert np.array_equal(oracle.gemv(type_, w[1], cols, rows, x), GOLD[f"gemv_{type_}"])


def test_routes_match_reference_outputs(oracle):
    lg = (fixtures.lcg_activations(9, 8 * 64).reshape(8, 64) * np.float32(5)).astype(np.float64)  # binary32-exact values
    lg[3, 10:20] = lg[3, 5]
    for mode in (0, 1):
        for norm in (0, 1):
            ids, w = oracle.route_rows(lg, 10, mode, bool(norm))
            assert np.array_equal(ids, GOLD[f"route_ids_{mode}{norm}"])
            assert np.array_equal(w, GOLD[f"route_w_{mode}{norm}"])


@pytest.mark.parametrize("type_", [8, 12])
def test_layer_matches_reference_outputs(oracle, type_):
    layer, x, logits = golden_cases.small_layer(type_)
    y, st = oracle.moe_layer(layer, x, logits, threads=3, stages=True)
    assert np.array_equal(st["indices"], GOLD[f"layer_ids_{type_}"])
    assert list(st["indices"][1]) == [0, 1, 2]
    assert np.array_equal(y, GOLD[f"layer_out_{type_}"])


def test_five_bit_layer_matches_reference_outputs(oracle):
    """Q5_K gate / up, Q5_1 down, Q8_0 shared expert: the layer the reference's CPU code computed from the same bytes."""
    layer, x, logits = golden_cases.five_bit_layer()
    y, st = oracle.moe_layer(layer, x, logits, threads=2, stages=True)
    assert np.array_equal(st["indices"], GOLD["layer_ids_five_bit"])
    assert np.array_equal(y, GOLD["layer_out_five_bit"])
    assert np.isfinite(y).all() and float(np.abs(y).max()) > 0
