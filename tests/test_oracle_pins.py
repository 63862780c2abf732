"""Pins the CPU oracle (oracle/tsp_oracle.c) to the reference's own known-answer tests, restated here
from native/tests/test_numeric.cpp, test_routing.cpp, test_operators.cpp and test_planar_pack_v3.cpp,
and, where oracle/_ref was built from the reference's sources, to those sources on random inputs."""
import math
import random

import numpy as np
import pytest

import fixtures


def test_binary16_every_pattern(oracle):
    # native/tests/test_numeric.cpp:40-54: independent formula for all 65536 patterns
    for bits in range(65536):
        got = oracle.binary16(bits)
        e, f = (bits >> 10) & 31, bits & 1023
        sign = -1.0 if bits & 0x8000 else 1.0
        if e == 31:
            assert (math.isnan(got) if f else (math.isinf(got) and (got < 0) == (sign < 0)))
        else:
            want = sign * (math.ldexp(1 + f / 1024.0, e - 15) if e else math.ldexp(f, -24))
            assert got == want and math.copysign(1, got) == sign


def _q4k_fixture_block():
    # native/tests/test_numeric.cpp:81-103: logical values and bit ownership, no decoder involved
    block = np.zeros(144, dtype=np.uint8)
    block[0:2] = [0x00, 0x30]  # 0.125
    block[2:4] = [0x00, 0x34]  # 0.25
    expected = np.zeros(256, dtype=np.float32)
    for group in range(8):
        scale, minimum = (group * 11 + 3) % 64, (group * 7 + 5) % 64
        for bit in range(6):
            scale_byte = 4 + group if group < 4 else (8 + group if bit < 4 else group)
            min_byte = 8 + group if group < 4 else (8 + group if bit < 4 else 4 + group)
            scale_bit = bit if (group < 4 or bit < 4) else bit + 2
            min_bit = bit if group < 4 else (bit + 4 if bit < 4 else bit + 2)
            block[scale_byte] |= ((scale >> bit) & 1) << scale_bit
            block[min_byte] |= ((minimum >> bit) & 1) << min_bit
        for lane in range(32):
            code = (lane * 3 + group * 5) % 16
            block[16 + (group // 2) * 32 + lane] |= code << ((group % 2) * 4)
            expected[group * 32 + lane] = np.float32(0.125) * scale * code - np.float32(0.25) * minimum
    return block, expected


def _q5k_fixture_block():
    # native/tests/test_numeric.cpp:81-103 for type 13: the Q4_K header, 32 bytes of fifth bits (bit g of byte lane), nibbles at 48
    block = np.zeros(176, dtype=np.uint8)
    block[0:2] = [0x00, 0x30]
    block[2:4] = [0x00, 0x34]
    expected = np.zeros(256, dtype=np.float32)
    for group in range(8):
        scale, minimum = (group * 11 + 3) % 64, (group * 7 + 5) % 64
        for bit in range(6):
            scale_byte = 4 + group if group < 4 else (8 + group if bit < 4 else group)
            min_byte = 8 + group if group < 4 else (8 + group if bit < 4 else 4 + group)
            scale_bit = bit if (group < 4 or bit < 4) else bit + 2
            min_bit = bit if group < 4 else (bit + 4 if bit < 4 else bit + 2)
            block[scale_byte] |= ((scale >> bit) & 1) << scale_bit
            block[min_byte] |= ((minimum >> bit) & 1) << min_bit
        for lane in range(32):
            code = (lane * 3 + group * 5) % 32
            block[48 + (group // 2) * 32 + lane] |= (code % 16) << ((group % 2) * 4)
            block[16 + lane] |= (code // 16) << group
            expected[group * 32 + lane] = np.float32(0.125) * scale * code - np.float32(0.25) * minimum
    return block, expected


def _q51_fixture_block():
    # native/tests/test_numeric.cpp:62-73: d = 0.5, m = -2, code = (13 i + 7) % 32, fifth bits in the word at byte 4
    block = np.zeros(24, dtype=np.uint8)
    block[0:2] = [0x00, 0x38]
    block[2:4] = [0x00, 0xc0]
    expected = np.zeros(32, dtype=np.float32)
    high = 0
    for i in range(32):
        code = (i * 13 + 7) % 32
        high |= (code // 16) << i
        block[8 + i % 16] |= (code % 16) << ((i // 16) * 4)
        expected[i] = 0.5 * code - 2
    block[4:8] = np.frombuffer(int(high).to_bytes(4, "little"), dtype=np.uint8)
    return block, expected


def _q6k_fixture_block():
    # native/tests/test_numeric.cpp:104-114: d = 0.03125, code = (7 i + 1) % 64, group scale = 15 (i / 16) - 120
    block = np.zeros(210, dtype=np.uint8)
    block[208:210] = [0x00, 0x28]
    expected = np.zeros(256, dtype=np.float32)
    for i in range(256):
        code = (i * 7 + 1) % 64
        block[(i // 128) * 64 + (i % 64)] |= (code % 16) << ((i % 128 // 64) * 4)
        block[128 + (i // 128) * 32 + i % 32] |= (code // 16) << ((i % 128 // 32) * 2)
        scale = (i // 16) * 15 - 120
        block[192 + i // 16] = scale & 255
        expected[i] = np.float32(0.03125) * scale * (code - 32)
    return block, expected


def _iq4nl_fixture_block():
    # native/tests/test_numeric.cpp:115-123: d = 0.5, code = 7 i % 16 into the encoding's fixed value alphabet
    alphabet = [-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113]
    block = np.zeros(18, dtype=np.uint8)
    block[0:2] = [0x00, 0x38]
    expected = np.zeros(32, dtype=np.float32)
    for i in range(32):
        code = (i * 7) % 16
        block[2 + i % 16] |= code << ((i // 16) * 4)
        expected[i] = 0.5 * alphabet[code]
    return block, expected


def _q8_fixture_block():
    block = np.zeros(34, dtype=np.uint8)
    block[0:2] = [0x00, 0x34]  # 0.25
    expected = np.zeros(32, dtype=np.float32)
    for i in range(32):
        code = i * 8 - 128
        block[2 + i] = code & 255
        expected[i] = 0.25 * code
    return block, expected


@pytest.mark.parametrize("type_,maker", [(12, _q4k_fixture_block), (8, _q8_fixture_block), (13, _q5k_fixture_block), (7, _q51_fixture_block),
                                         (14, _q6k_fixture_block), (20, _iq4nl_fixture_block)])
def test_format_fixture_blocks(oracle, type_, maker):
    block, expected = maker()
    got = oracle.dequantize(type_, block, expected.size)
    assert np.array_equal(got, expected)
    x = np.array([(i % 13 - 6) * 0.25 for i in range(expected.size)], dtype=np.float32)
    dot = 0.0
    for i in range(expected.size):
        dot += float(expected[i]) * float(x[i])
    assert oracle.gemv(type_, block, expected.size, 1, x)[0] == dot            # float input
    assert oracle.gemv(type_, block, expected.size, 1, x.astype(np.float64))[0] == dot  # double input
    with pytest.raises(Exception):
        oracle.dequantize(type_, block[:-1], expected.size)


def test_q8_multiblock_extreme_scales(oracle):
    # native/tests/test_numeric.cpp:164-191: subnormal / extreme scales, bit-compared
    scales = [0x0000, 0x8000, 0x0001, 0x03ff, 0x0400, 0x3555, 0xb555, 0x7bff, 0xfbff]
    enc = np.zeros(len(scales) * 34, dtype=np.uint8)
    expected = np.zeros(len(scales) * 32, dtype=np.float32)
    for b, bits in enumerate(scales):
        enc[b * 34] = bits & 255
        enc[b * 34 + 1] = bits >> 8
        e, f = (bits >> 10) & 31, bits & 1023
        scale = (-1.0 if bits & 0x8000 else 1.0) * (math.ldexp(1 + f / 1024.0, e - 15) if e else math.ldexp(f, -24))
        for i in range(32):
            code = (b * 37 + i * 19) & 255
            enc[b * 34 + 2 + i] = code
            expected[b * 32 + i] = np.float32(scale * (code if code < 128 else code - 256))
    got = oracle.dequantize(8, enc, expected.size)
    assert np.array_equal(got.view(np.uint32), expected.view(np.uint32))
    for bad in (0x7c00, 0xfc00, 0x7e01):
        enc[8 * 34] = bad & 255
        enc[8 * 34 + 1] = bad >> 8
        with pytest.raises(Exception):
            oracle.dequantize(8, enc, expected.size)


def test_float_decoders_and_refusals(oracle):
    f32 = np.array([1, -2, 0.25], dtype=np.float32)
    assert np.array_equal(oracle.dequantize(0, f32.view(np.uint8), 3), f32)
    assert np.array_equal(oracle.dequantize(1, f32.astype(np.float16).view(np.uint8), 3), f32)
    bf = (f32.view(np.uint32) >> 16).astype(np.uint16)
    assert np.array_equal(oracle.dequantize(30, bf.view(np.uint8), 3), f32)
    inf = np.array([np.inf], dtype=np.float32)
    with pytest.raises(Exception):
        oracle.dequantize(0, inf.view(np.uint8), 1)
    with pytest.raises(Exception):
        oracle.dequantize(999, np.zeros(4, np.uint8), 1)
    two = np.array([2.0], dtype=np.float32).view(np.uint8)
    with pytest.raises(Exception):
        oracle.gemv(0, two, 1, 1, np.array([np.nan], dtype=np.float32))
    assert oracle.gemv(0, two, 1, 1, np.array([1 + 1e-12]))[0] == (1 + 1e-12) * 2  # double input is not rounded to float
    with pytest.raises(Exception):
        oracle.gemv(0, two, 1, 1, np.array([np.finfo(np.float64).max]))


def test_routing_against_independent_ordering(oracle):
    # native/tests/test_routing.cpp:24-49: ids equal a stable sort by probability; weights within 1e-13
    rnd = random.Random(0x726F7574)
    for _ in range(300):
        count = 1 + rnd.randrange(1024)
        selected = 1 + rnd.randrange(min(64, count))
        logits = np.array([(rnd.randrange(2001) - 1000) / 100.0 for _ in range(count)])
        for mode in (0, 1):
            prob = np.exp(logits) if mode == 0 else 1 / (1 + np.exp(-logits))
            if mode == 0:
                prob = prob / prob.sum()
            order = sorted(range(count), key=lambda i: -prob[i])[:selected]  # sorted() is stable
            for normalize in (False, True):
                ids, w = oracle.route(logits, selected, mode, normalize)
                assert list(ids) == order
                den = prob[order].sum() if normalize else 1.0
                assert np.max(np.abs(w - prob[order] / den)) < 1e-13


def test_routing_ties_underflow_and_refusals(oracle):
    ids, _ = oracle.route(np.array([3, 3, 2, 1, 3.0]), 3, 0, True)
    assert list(ids) == [0, 1, 4]
    assert list(oracle.route(np.array([-1000.0]), 1, 1, True)[1]) == [1.0]
    ids, w = oracle.route(np.array([-1000.0]), 1, 0, True)
    assert list(ids) == [0] and list(w) == [1.0]
    ties = np.array([3, 3, 2, 1, 3.0])
    for bad in (lambda: oracle.route(ties, 0), lambda: oracle.route(ties, 6), lambda: oracle.route(ties, 1, 99),
                lambda: oracle.route(np.array([np.nan]), 1)):
        with pytest.raises(Exception):
            bad()


def test_mixture_golden(oracle):
    # native/tests/test_routing.cpp:53-56
    out = oracle.mixture(np.array([1, 2, 3, 4.0]), np.array([0.25, 0.75]), np.array([5, 6.0]), 0.0)
    assert list(out) == [5, 6.5]
    with pytest.raises(Exception):
        oracle.mixture(np.array([1, 2, 3, 4.0]), np.array([np.nan, 1.0]), np.array([5, 6.0]), 0.0)


def test_activation_functions(oracle):
    for v in (-50.0, -3.5, -1e-9, 0.0, 0.25, 7.0, 40.0):
        s = 1 / (1 + math.exp(-v)) if v >= 0 else math.exp(v) / (1 + math.exp(v))
        assert oracle.sigmoid(v) == s
        assert oracle.silu(v) == v * s
        assert abs(oracle.softplus(v) - math.log1p(math.exp(-abs(v))) - max(v, 0)) < 1e-15
    assert oracle.sigmoid(-800.0) == 0.0 and oracle.sigmoid(800.0) == 1.0


def test_sm16_bijection_and_refusal(oracle):
    # native/tests/test_planar_pack_v3.cpp:194-234: pack_sm16 equals the GGUF factor unpack, round-trips, refuses >= 64
    rng = np.random.default_rng(5)
    for _ in range(4096):
        s12 = rng.integers(0, 256, 12, dtype=np.uint8)
        block = np.zeros(144, dtype=np.uint8)
        block[4:16] = s12
        block[0:2] = [0x00, 0x3c]  # d = 1
        block[2:4] = [0x00, 0x3c]  # dmin = 1
        sm = oracle.pack_sm16(s12)
        for g in range(8):
            # with q = 0 the decoded value is -mn; with d = 1, value(q=1) + mn = sc
            assert oracle.lib.tso_value(12, block.ctypes.data_as(oracle.lib.tso_value.argtypes[1]), g * 32) == -float(sm[8 + g])
        assert np.array_equal(oracle.unpack_sm16(sm), s12)
        assert np.all(sm < 64)
    bad = np.zeros(16, dtype=np.uint8)
    bad[7] = 64
    with pytest.raises(Exception):
        oracle.unpack_sm16(bad)


@pytest.mark.parametrize("type_,cols,rows", [(12, 512, 64), (8, 512, 64), (8, 64, 16), (13, 512, 64), (7, 512, 64), (7, 64, 16)])
def test_planar_round_trip_and_zero_difference(oracle, type_, cols, rows):
    # native/tests/test_planar_pack_v3.cpp:236-281: byte-exact round trip, identical FP32 operands
    g = fixtures.lcg_weights(type_, cols, rows, 1)[0]
    spec = oracle.spec(type_, cols, rows)
    p = oracle.pack_expert(spec, g)
    assert np.array_equal(oracle.unpack_expert(spec, p), g)
    a = oracle.dequantize(type_, g, rows * cols)
    b = oracle.dequantize_planar(spec, p)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_planar_spec_byte_constants(oracle):
    s = oracle.spec(12, 2048, 1024)
    assert (s.planar_expert_bytes, s.source_expert_bytes, s.sm_offset, s.dm_offset) == (1212416, 1179648, 1048576, 1179648)
    s = oracle.spec(12, 512, 2048)
    assert (s.planar_expert_bytes, s.source_expert_bytes) == (606208, 589824)
    s = oracle.spec(13, 512, 64)     # Q5_K: 128 + 32 + 16 + 4 bytes per super-block, plane after plane
    assert (s.planar_row_bytes, s.source_row_bytes, s.qh_offset, s.sm_offset, s.dm_offset) == (360, 352, 128 * 128, 128 * 160, 128 * 176)
    s = oracle.spec(7, 64, 16)       # Q5_1: 16 + 4 + 4 bytes per block
    assert (s.planar_row_bytes, s.source_row_bytes, s.qh_offset, s.dm_offset) == (48, 48, 32 * 16, 32 * 20)
    for bad in ((12, 2048, 6), (12, 300, 8), (8, 48, 8), (8, 32, 4), (5, 256, 8), (13, 300, 8), (7, 48, 8)):
        with pytest.raises(Exception):
            oracle.spec(*bad)


def test_permutation_tables(oracle):
    # grouped_mpp.metal:12-66 semantics: ascending token order per expert; tiles in ascending expert order
    ids = np.array([[2, 0], [1, 2], [2, 3], [0, 1]], dtype=np.uint32)
    tm, counts = oracle.grouped_routes(ids, 4)
    assert list(counts) == [2, 2, 3, 1]
    assert list(tm[0, :2]) == [1, 6] and list(tm[1, :2]) == [2, 7] and list(tm[2, :3]) == [0, 3, 4] and list(tm[3, :1]) == [5]
    tasks = oracle.grouped_tasks(counts, 4, 2, tile=2)
    assert list(tasks[:2]) == [5, 8]
    assert [tuple(tasks[2 + 2 * i: 4 + 2 * i]) for i in range(5)] == [(0, 0), (1, 0), (2, 0), (2, 2), (3, 0)]
    assert np.all(tasks[12:] == 0xFFFFFFFF)
    with pytest.raises(Exception):
        oracle.grouped_routes(np.array([[1, 1]], dtype=np.uint32), 4)   # an expert named twice by one token
    with pytest.raises(Exception):
        oracle.grouped_routes(np.array([[1, 9]], dtype=np.uint32), 4)   # id out of range


# ---- the restatement against the reference's own compiled sources, on random inputs ----

@pytest.mark.parametrize("type_", [8, 12, 13, 7, 14, 20])
def test_port_equals_reference_decode_and_gemv(oracle, ref_oracle, type_):
    cols, rows = 512, 24
    w = fixtures.lcg_weights(type_, cols, rows, 1)[0]
    a, b = oracle.dequantize(type_, w, rows * cols), ref_oracle.dequantize(type_, w, rows * cols)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    x = fixtures.lcg_activations(7, cols)
    assert np.array_equal(oracle.gemv(type_, w, cols, rows, x), ref_oracle.gemv(type_, w, cols, rows, x))
    xd = x.astype(np.float64) * 1.000000001
    assert np.array_equal(oracle.gemv(type_, w, cols, rows, xd), ref_oracle.gemv(type_, w, cols, rows, xd))
    assert np.array_equal(oracle.binary16_all().view(np.uint32), ref_oracle.binary16_all().view(np.uint32))


def test_port_equals_reference_routing(oracle, ref_oracle):
    rng = np.random.default_rng(11)
    for trial in range(200):
        E = int(rng.integers(1, 600))
        k = int(rng.integers(1, min(64, E) + 1))
        lg = np.round(rng.normal(size=E) * 4, 1)  # coarse values: many exact ties
        for mode in (0, 1):
            for norm in (False, True):
                ia, wa = oracle.route(lg, k, mode, norm)
                ib, wb = ref_oracle.route(lg, k, mode, norm)
                assert np.array_equal(ia, ib) and np.array_equal(wa, wb)
    y = rng.normal(size=(5, 33))
    w = np.abs(rng.normal(size=5))
    sh = rng.normal(size=33)
    assert np.array_equal(oracle.mixture(y, w, sh, 0.3), ref_oracle.mixture(y, w, sh, 0.3))
    for v in rng.normal(size=50) * 20:
        assert oracle.silu(v) == ref_oracle.silu(v) and oracle.softplus(v) == ref_oracle.softplus(v)


def test_port_equals_reference_layer(oracle, ref_oracle):
    import golden_cases
    layer, x, logits = golden_cases.small_layer(12)
    a, st = oracle.moe_layer(layer, x, logits, threads=2, stages=True)
    b, sb = ref_oracle.moe_layer(layer, x, logits, threads=2, stages=True)
    assert np.array_equal(a, b) and np.array_equal(st["indices"], sb["indices"])


def test_residual_read_write_port_equals_reference(oracle, ref_oracle):
    """operators.cpp:60-96: the port's gated residual read and residual write against the reference's own functions, bit for bit."""
    rng = np.random.default_rng(5)
    for B, Cn, R in ((4, 96, 8), (1, 7, 1), (3, 256, 16)):
        st, g = rng.normal(size=(B, Cn)), rng.normal(size=(B, Cn))
        dn, up, inj = rng.normal(size=(R, B * Cn)) * 0.1, rng.normal(size=(B * Cn, R)), rng.normal(size=(B, B * Cn)) * 0.1
        a, b = oracle.gated_residual(st, g, dn, up, inj, R, 1e-6), ref_oracle.gated_residual(st, g, dn, up, inj, R, 1e-6)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
        out = rng.normal(size=Cn)
        assert np.array_equal(oracle.residual_write(st, out, a[1]), ref_oracle.residual_write(st, out, a[1]))


def _topk_brute(row):
    """Independent statement of the order: finite values, -0 as +0, value descending, column ascending."""
    row = np.asarray(row, dtype=np.float32)
    finite = np.isfinite(row)
    cols = np.nonzero(finite)[0]
    canon = np.where(row[cols] == 0, np.float32(0), row[cols])
    order = np.lexsort((cols, -canon.astype(np.float64)))[:64]
    return cols[order], row[cols[order]]


def test_logit_topk_known_answers_of_the_reference_test(oracle):
    """The rows native/tests/test_logit_topk.cpp:104-155 and :197-222 build, with the answers that test states: ties at 17.5 to
    the lower column, -0 before +0 by column with its sign bit kept, bad-value columns recorded. (The reference's sampling.cpp
    includes arm_neon.h and cannot be compiled here: this pin is by known answers and by an independent ordering.)"""
    for vocab in (32, 64, 5000, 248320):
        rows = 4 if vocab == 248320 else 3
        rng = np.random.default_rng(0x51A70000 ^ vocab)
        logits = (rng.standard_normal((rows, vocab)) * 3.25).astype(np.float32)
        logits[0, [3, 19, 31]] = 17.5
        if vocab >= 64:
            logits[0, vocab - 2], logits[0, vocab - 1] = -0.0, 0.0
            c = np.arange(vocab - 2)
            keep = np.isin(c, [3, 19, 31])
            logits[0, :vocab - 2] = np.where(keep, logits[0, :vocab - 2], -100.0 - (c % 11))
        for r in range(rows):
            got = oracle.logit_topk_row(logits[r])
            assert got["vocabulary"] == vocab and got["count"] == min(vocab, 64)
            assert got["first_nonfinite_col"] == 0xFFFFFFFF and got["first_subnormal_col"] == 0xFFFFFFFF
            ids, vals = _topk_brute(logits[r])
            assert np.array_equal(got["ids"][:got["count"]], ids)
            assert np.array_equal(got["logits"][:got["count"]].view(np.uint32), vals.view(np.uint32))
        first = oracle.logit_topk_row(logits[0])
        assert list(first["ids"][:3]) == [3, 19, 31]
        if vocab >= 64:
            assert first["ids"][3] == vocab - 2 and first["logits"][3:4].view(np.uint32)[0] == 0x80000000
            assert first["ids"][4] == vocab - 1 and first["logits"][4:5].view(np.uint32)[0] == 0
    vocab = 8192
    bad = np.full((2, vocab), -1.0, dtype=np.float32)
    bad.view(np.uint32)[0, 5] = 1
    bad[0, 5000] = np.nan
    bad[1, 17] = -np.inf
    bad.view(np.uint32)[1, 99] = 0x80000001
    a, b = oracle.logit_topk_row(bad[0]), oracle.logit_topk_row(bad[1])
    assert (a["first_subnormal_col"], a["first_nonfinite_col"]) == (5, 5000)
    assert (b["first_nonfinite_col"], b["first_subnormal_col"]) == (17, 99)
    assert a["ids"][0] == 5 and a["count"] == 64   # the positive subnormal beats every -1 and still competes
    short = oracle.logit_topk_row(np.array([np.nan, 2.0, np.inf, 1.0], dtype=np.float32))
    assert short["count"] == 2 and list(short["ids"][:3]) == [1, 3, 0] and np.isneginf(short["logits"][2])
    with pytest.raises(Exception):
        oracle.logit_topk_row(np.zeros(0, dtype=np.float32))


@pytest.mark.parametrize("type_,columns", [(8, 2048), (8, 2560), (8, 32), (8, 32 * 19), (8, 32 * 33), (12, 2048), (12, 256), (12, 256 * 5), (12, 256 * 7)])
def test_lane_layout_port_equals_reference(oracle, ref_oracle, type_, columns):
    """`q8_lanes_v1` (and the Q4_K lane rows) against the reference's own pack_rows / unpack_rows (expert_lanes.cpp:92-130) on
    random bytes, including rows whose last run is short; lossless both ways."""
    bpb, epb = (34, 32) if type_ == 8 else (144, 256)
    rows = 5
    rng = np.random.default_rng(columns * 31 + type_)
    original = rng.integers(0, 256, rows * (columns // epb) * bpb, dtype=np.uint8)
    packed = oracle.lanes_pack_rows(type_, columns, original)
    assert np.array_equal(packed, ref_oracle.lanes_pack_rows(type_, columns, original))
    assert np.array_equal(oracle.lanes_pack_rows(type_, columns, packed, unpack=True), original)
    assert np.array_equal(ref_oracle.lanes_pack_rows(type_, columns, packed, unpack=True), original)
    if columns // epb > 1:
        assert not np.array_equal(packed, original)
    with pytest.raises(Exception):
        oracle.lanes_pack_rows(type_, columns, original[:-1])
    with pytest.raises(Exception):
        oracle.lanes_pack_rows(type_, columns + 1, original)
