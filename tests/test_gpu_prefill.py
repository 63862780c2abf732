"""Prefill-size path (grouped tcgen05 GEMMs) against the CPU oracle: hidden rows and routed rows per stage, then whole layers
with skewed expert loads, empty experts, partial tiles and experts with more than one tile of 128 routes.
Bar: rel-L2 <= 2e-3 (binary16 operands, FP32 accumulate); the reference's own bound for this path is NMSE 2e-3."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tokspur_public_b200 import capi, formats, synth  # noqa: E402
from tokspur_public_b200 import layer as L  # noqa: E402


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize("T,E,K,skew", [(3, 4, 2, False), (40, 4, 2, False), (200, 8, 3, True), (700, 8, 2, True)])
def test_prefill_layer_against_oracle(oracle, T, E, K, skew):
    Cn, H = 256, 256
    host = L.synth_host_layer(5, Cn, H, E, K, expert_type=formats.Q4_K)
    dl = L.DeviceLayer(host, formats.PLANAR, "cuda")
    ps = L.PrefillScratch(Cn, H, E, K, T, "cuda")
    x16 = synth.activations_f16(7, T, Cn)
    logits = synth.router_logits(8, T, E, synth.zipf_bias(9, E) * 3 if skew else None)
    x32 = torch.from_numpy(x16.astype(np.float32)).cuda()
    out = torch.zeros((T, Cn), dtype=torch.float32, device="cuda")
    L.moe_layer_prefill(dl, ps, x32, torch.from_numpy(logits).cuda(), out)
    torch.cuda.synchronize()
    assert ps.base.error_word() == 0
    n = min(T, 24)
    sample = np.unique(np.linspace(0, T - 1, n).astype(int))
    want, st = oracle.moe_layer(host.oracle_dict(), x16[sample].astype(np.float32), logits[sample], threads=4, stages=True)
    ids = ps.base.ids.cpu().numpy().view(np.uint32)[:T * K].reshape(T, K)
    assert np.array_equal(ids[sample], st["indices"])
    routed = ps.base.routed.cpu().numpy()[:T * K * Cn].reshape(T, K, Cn)
    assert rel_l2(routed[sample], st["routed"]) <= 2e-3
    shared = ps.base.shared_out.cpu().numpy()[:T * Cn].reshape(T, Cn)
    assert rel_l2(shared[sample], st["shared_out"]) <= 2e-3
    assert rel_l2(out.cpu().numpy()[sample], want) <= 2e-3
