"""Hyper-connection residual read / write around the FFN sub-layer against the CPU oracle (operators.cpp:60-96); the oracle's
own functions are pinned to the reference's in test_oracle_pins.py."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tokspur_public_b200 import capi  # noqa: E402
from tokspur_public_b200 import layer as L  # noqa: E402


@pytest.mark.parametrize("tokens,branches,channels,rank", [(1, 4, 2560, 16), (5, 4, 2048, 8), (3, 2, 100, 4), (2, 64, 33, 3)])
def test_residual_read_write_rows(oracle, tokens, branches, channels, rank):
    rng = np.random.default_rng(tokens * 7 + branches)
    width = branches * channels
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    norm, scores, logits, want_in, want_sc, streams = [], [], [], [], [], []
    for t in range(tokens):
        st = rng.normal(size=(branches, channels)).astype(np.float32)
        gains = rng.normal(size=(branches, channels)).astype(np.float32)
        down = (rng.normal(size=(rank, width)) * 0.05).astype(np.float32)
        up = rng.normal(size=(width, rank)).astype(np.float32)
        inject = (rng.normal(size=(branches, width)) * 0.05).astype(np.float32)
        i, s, n, sc, lg = oracle.gated_residual(st, gains, down, up, inject, rank, 1e-6, intermediates=True)
        streams.append(st); norm.append(n); scores.append(sc); logits.append(lg); want_in.append(i); want_sc.append(s)
    dn = torch.from_numpy(np.stack(norm).astype(np.float32)).cuda()
    ds = torch.from_numpy(np.stack(scores).astype(np.float32)).cuda()
    dl = torch.from_numpy(np.stack(logits).astype(np.float32)).cuda()
    out = torch.zeros((tokens, channels), dtype=torch.float32, device="cuda")
    scales = torch.zeros((tokens, branches), dtype=torch.float32, device="cuda")
    capi.call("tsp_residual_read", dn.data_ptr(), ds.data_ptr(), dl.data_ptr(), branches, channels, tokens, out.data_ptr(), scales.data_ptr(),
              err.data_ptr(), L.stream_ptr())
    torch.cuda.synchronize()
    wi, ws = np.stack(want_in), np.stack(want_sc)
    assert np.max(np.abs(out.cpu().numpy() - wi) / np.maximum(1.0, np.abs(wi))) <= 5e-6
    assert np.max(np.abs(scales.cpu().numpy() - ws)) <= 5e-6
    # write: the FFN output back onto the streams, in place
    ffn = rng.normal(size=(tokens, channels)).astype(np.float32)
    dst = torch.from_numpy(np.stack(streams)).cuda()
    dffn = torch.from_numpy(ffn).cuda()
    capi.call("tsp_residual_write", dst.data_ptr(), dffn.data_ptr(), scales.data_ptr(), branches, channels, tokens, dst.data_ptr(), err.data_ptr(),
              L.stream_ptr())
    torch.cuda.synchronize()
    sc32 = scales.cpu().numpy()
    for t in range(tokens):
        want = oracle.residual_write(streams[t], ffn[t], sc32[t])
        assert np.max(np.abs(dst[t].cpu().numpy() - want) / np.maximum(1.0, np.abs(want))) <= 1e-6
    assert int(err.item()) == 0
