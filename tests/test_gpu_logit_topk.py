"""`tsp_logit_topk` (the sampler's top-64 rows behind the vocabulary head) against the oracle's `logit_topk_row`, bit for bit:
the rows the reference's own test builds (native/tests/test_logit_topk.cpp:104-155: ties, signed zeros; :197-222: NaN, -Inf and
subnormal columns) at its vocabularies and at the benchmark's, strided rows, fewer finite values than slots, and the rows the
Q8_0 head itself produces."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tokspur_public_b200 import capi, formats, synth  # noqa: E402
from tokspur_public_b200 import layer as L  # noqa: E402


def run_topk(logits_dev, rows, vocab, stride_elems):
    lib = capi.lib()
    scratch = torch.empty(lib.tsp_logit_topk_scratch_bytes(rows, vocab), dtype=torch.uint8, device="cuda")
    out = torch.empty(lib.tsp_logit_topk_output_bytes(rows), dtype=torch.uint8, device="cuda")
    capi.call("tsp_logit_topk", logits_dev.data_ptr(), stride_elems * 4, rows, vocab, scratch.data_ptr(), scratch.numel(), out.data_ptr(),
              out.numel(), L.stream_ptr())
    torch.cuda.synchronize()
    return out.cpu().numpy().view(np.uint32).reshape(rows, 132)


def check_rows(oracle, got, logits):
    for r in range(logits.shape[0]):
        want = oracle.logit_topk_row(logits[r])
        g = got[r]
        assert (int(g[0]), int(g[1]), int(g[2]), int(g[3])) == (want["vocabulary"], want["count"], want["first_nonfinite_col"], want["first_subnormal_col"])
        assert np.array_equal(g[4:68], want["ids"])
        assert np.array_equal(g[68:132], want["logits"].view(np.uint32))


@pytest.mark.parametrize("vocab", [32, 64, 5000, 151936, 248320])
def test_reference_test_rows(oracle, vocab):
    rows = 4 if vocab >= 151936 else 3
    rng = np.random.default_rng(0x51A70000 ^ vocab)
    logits = (rng.standard_normal((rows, vocab)) * 3.25).astype(np.float32)
    logits[0, [3, 19, 31]] = 17.5
    if vocab >= 64:
        logits[0, vocab - 2], logits[0, vocab - 1] = -0.0, 0.0
        c = np.arange(vocab - 2)
        logits[0, :vocab - 2] = np.where(np.isin(c, [3, 19, 31]), logits[0, :vocab - 2], -100.0 - (c % 11))
        logits[1, :] = 0.25          # one value everywhere: the 64 lowest columns win
        logits[1, 7::2] = -0.0       # and a field of signed zeros below it
    got = run_topk(torch.from_numpy(logits).cuda(), rows, vocab, vocab)
    check_rows(oracle, got, logits)
    assert list(got[0, 4:7]) == [3, 19, 31]


def test_bad_value_columns_and_short_rows(oracle):
    vocab = 8192
    bad = np.full((3, vocab), -1.0, dtype=np.float32)
    bad.view(np.uint32)[0, 5] = 1
    bad[0, 5000] = np.nan
    bad[1, 17] = -np.inf
    bad.view(np.uint32)[1, 99] = 0x80000001
    bad[2, :] = np.nan
    bad[2, [4100, 77, 8191]] = [1.0, 1.0, -3.0]   # three finite values in two tiles: count 3, the rest -inf / id 0
    got = run_topk(torch.from_numpy(bad).cuda(), 3, vocab, vocab)
    check_rows(oracle, got, bad)
    assert (int(got[0, 3]), int(got[0, 2])) == (5, 5000) and (int(got[1, 2]), int(got[1, 3])) == (17, 99)
    assert int(got[2, 1]) == 3 and list(got[2, 4:8]) == [77, 4100, 8191, 0]


def test_strided_rows_and_refusals(oracle):
    vocab, rows, stride = 4097, 5, 4104
    rng = np.random.default_rng(9)
    buf = rng.standard_normal((rows, stride)).astype(np.float32)
    got = run_topk(torch.from_numpy(buf).cuda(), rows, vocab, stride)
    check_rows(oracle, got, np.ascontiguousarray(buf[:, :vocab]))
    lib = capi.lib()
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    assert lib.tsp_logit_topk(t.data_ptr(), 16, 1, 8, t.data_ptr() + 4096, 528, t.data_ptr() + 8192, 528, None) == capi.E_ARG          # stride < row
    assert lib.tsp_logit_topk(t.data_ptr(), 32, 1, 8, t.data_ptr() + 4096, 527, t.data_ptr() + 8192, 528, None) == capi.E_ARG          # short scratch
    assert lib.tsp_logit_topk(t.data_ptr(), 32, 1, 8, t.data_ptr() + 16, 528, t.data_ptr() + 8192, 528, None) == capi.E_ARG            # overlap
    assert lib.tsp_logit_topk(t.data_ptr(), 32, 2049, 8, t.data_ptr() + 4096, 1 << 14, t.data_ptr() + 8192, 1 << 14, None) == capi.E_ARG
    assert lib.tsp_logit_topk_scratch_bytes(16, 151936) == 16 * 38 * 528 and lib.tsp_logit_topk_output_bytes(16) == 16 * 528


def test_rows_of_the_q8_head(oracle):
    """Head -> top-k as the verify step runs them: Q8_0 [8192 x 2048] on 5 rows, top-64 of each logits row."""
    vocab, cols, M = 8192, 2048, 5
    bpr = cols // 32
    w = torch.empty(vocab * bpr * 34, dtype=torch.uint8, device="cuda")
    capi.call("tsp_synth_weights", formats.Q8_0, 77, 0, vocab * bpr, 0.02, w.data_ptr(), L.stream_ptr())
    ms = L.matrix_set(w, formats.Q8_0, formats.GGUF, vocab, cols)
    x = torch.from_numpy(synth.activations_f16(31, M, cols).astype(np.float32)).cuda()
    logits = torch.zeros((M, vocab), dtype=torch.float32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.call("tsp_moe_project", C.byref(ms), x.data_ptr(), cols * 4, 1, M, 1, None, None, None, logits.data_ptr(), vocab * 4, 1, err.data_ptr(),
              L.stream_ptr())
    got = run_topk(logits, M, vocab, vocab)
    assert int(err.item()) == 0
    check_rows(oracle, got, logits.cpu().numpy())
