"""`q8_lanes_v1` rows (the layout the Pack v3 container keeps dense Q8_0 matrices in) to GGUF rows and back on the device,
bit for bit against the oracle's pack_rows / unpack_rows (which is pinned to the reference's expert_lanes.cpp), and the
vocabulary-head projection on a matrix that arrived in the lane layout."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tokspur_public_b200 import capi, formats, synth  # noqa: E402
from tokspur_public_b200 import layer as L  # noqa: E402


@pytest.mark.parametrize("rows,cols", [(7, 32), (5, 32 * 19), (130, 2048), (3, 2560), (2, 32 * 33)])
def test_unpack_and_pack_match_the_oracle(oracle, rows, cols):
    rng = np.random.default_rng(rows * 1000 + cols)
    gguf = rng.integers(0, 256, rows * (cols // 32) * 34, dtype=np.uint8)
    lanes = oracle.lanes_pack_rows(formats.Q8_0, cols, gguf)
    d_lanes, d_gguf = torch.from_numpy(lanes).cuda(), torch.from_numpy(gguf).cuda()
    out = torch.zeros_like(d_gguf)
    capi.call("tsp_q8_lanes_unpack", d_lanes.data_ptr(), out.data_ptr(), rows, cols, L.stream_ptr())
    assert np.array_equal(out.cpu().numpy(), gguf)
    out.zero_()
    capi.call("tsp_q8_lanes_pack", d_gguf.data_ptr(), out.data_ptr(), rows, cols, L.stream_ptr())
    assert np.array_equal(out.cpu().numpy(), lanes)
    lib = capi.lib()
    assert lib.tsp_q8_lanes_unpack(d_lanes.data_ptr(), d_lanes.data_ptr(), rows, cols, None) == capi.E_ARG     # in place
    assert lib.tsp_q8_lanes_unpack(d_lanes.data_ptr(), out.data_ptr(), rows, cols + 1, None) == capi.E_ARG


def test_head_projection_on_a_matrix_loaded_from_lane_rows(oracle):
    vocab, cols, M = 4096, 2048, 3
    bpr = cols // 32
    w = torch.empty(vocab * bpr * 34, dtype=torch.uint8, device="cuda")
    capi.call("tsp_synth_weights", formats.Q8_0, 55, 0, vocab * bpr, 0.02, w.data_ptr(), L.stream_ptr())
    gguf = w.cpu().numpy()
    lanes = torch.from_numpy(oracle.lanes_pack_rows(formats.Q8_0, cols, gguf)).cuda()   # what the container holds
    loaded = torch.zeros_like(w)
    capi.call("tsp_q8_lanes_unpack", lanes.data_ptr(), loaded.data_ptr(), vocab, cols, L.stream_ptr())
    ms = L.matrix_set(loaded, formats.Q8_0, formats.GGUF, vocab, cols)
    x = synth.activations_f16(9, M, cols).astype(np.float32)
    out = torch.zeros((M, vocab), dtype=torch.float32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.call("tsp_moe_project", C.byref(ms), torch.from_numpy(x).cuda().data_ptr(), cols * 4, 1, M, 1, None, None, None, out.data_ptr(), vocab * 4, 1,
              err.data_ptr(), L.stream_ptr())
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    got = out.cpu().numpy()
    for m in range(M):
        want = oracle.gemv(formats.Q8_0, gguf, cols, vocab, x[m])
        assert float(np.max(np.abs(got[m] - want) / np.maximum(1.0, np.abs(want)))) <= 5e-5
