"""Gate and up tensors in either address order: when the up tensor lies below the gate tensor the kernels cannot fetch both
with one tensor copy and take one copy per matrix instead; the results must be bit-identical to the one-copy path."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _sets(host, order, dev):
    """gate / up matrix sets over ONE device buffer holding the two planar tensors in the given order."""
    from tokspur_public_b200 import formats
    from tokspur_public_b200 import layer as L
    Cn, H, E = host.channels, host.hidden, host.experts
    gp = formats.pack_planar_experts(host.expert_type, host.gate, E, H, Cn)
    up = formats.pack_planar_experts(host.expert_type, host.up, E, H, Cn)
    nbytes = gp.size
    first, second = (gp, up) if order == "gate_first" else (up, gp)
    buf = torch.from_numpy(np.concatenate([first.reshape(-1), second.reshape(-1)])).to(dev)
    g_off, u_off = (0, nbytes) if order == "gate_first" else (nbytes, 0)
    gate = L.matrix_set(buf, host.expert_type, formats.PLANAR, H, Cn, E, offset=g_off)
    upm = L.matrix_set(buf, host.expert_type, formats.PLANAR, H, Cn, E, offset=u_off)
    return buf, gate, upm


@pytest.mark.parametrize("tokens", [5, 150])
def test_gate_up_address_order(tokens):
    from tokspur_public_b200 import capi, formats, synth
    from tokspur_public_b200 import layer as L
    Cn, H, E, K = 512, 256, 6, 2
    dev = torch.device("cuda")
    host = L.synth_host_layer(21, Cn, H, E, K, expert_type=formats.Q4_K)
    lib, st = capi.lib(), L.stream_ptr()
    x16 = torch.from_numpy(synth.activations_f16(3, tokens, Cn)).to(dev)
    x32 = x16.float().contiguous()
    lg = torch.from_numpy(synth.router_logits(4, tokens, E)).to(dev)
    results = {}
    for order in ("gate_first", "up_first"):
        buf, gate, upm = _sets(host, order, dev)
        sc = L.Scratch(Cn, H, E, K, tokens, dev)
        ps = L.PrefillScratch(Cn, H, E, K, tokens, dev)
        e = sc.error.data_ptr()
        capi.check(lib.tsp_moe_route(lg.data_ptr(), E * 4, tokens, E, K, 0, 1, sc.ids.data_ptr(), sc.weights.data_ptr(), e, st))
        # decode-size kernel (tiles of 8 routes)
        capi.check(lib.tsp_moe_permute(sc.ids.data_ptr(), tokens, E, K, capi.GEMV_TILE, sc.token_map.data_ptr(), sc.counts.data_ptr(),
                                       sc.tasks.data_ptr(), e, st))
        h = torch.zeros((tokens * K, H), dtype=torch.float32, device=dev)
        capi.check(lib.tsp_moe_gate_up_swiglu(C.byref(gate), C.byref(upm), x32.data_ptr(), Cn * 4, tokens, K, sc.token_map.data_ptr(),
                                              sc.counts.data_ptr(), sc.tasks.data_ptr(), h.data_ptr(), H * 4, 1, e, st))
        # prefill-size kernel (tasks of 256 routes), fed from the routed copy of the K-ordered input rows
        capi.check(lib.tsp_moe_permute(sc.ids.data_ptr(), tokens, E, K, ps.tile, sc.token_map.data_ptr(), sc.counts.data_ptr(), ps.tasks.data_ptr(), e, st))
        capi.check(lib.tsp_moe_route_offsets(sc.counts.data_ptr(), E, ps.offsets.data_ptr(), st))
        capi.check(lib.tsp_moe_rows_f16k(x16.data_ptr(), Cn * 2, 1, tokens, Cn, ps.xk.data_ptr(), Cn * 2, e, st))
        capi.check(lib.tsp_moe_gather_rows16(ps.xk.data_ptr(), Cn * 2, sc.token_map.data_ptr(), ps.offsets.data_ptr(), E, tokens, K, Cn, ps.xp.data_ptr(), Cn * 2, st))
        capi.check(lib.tsp_moe_grouped_gate_up(C.byref(gate), C.byref(upm), None, None, ps.xp.data_ptr(), Cn * 2, None, 0, 0, tokens, K, sc.token_map.data_ptr(),
                                               sc.counts.data_ptr(), ps.tasks.data_ptr(), ps.offsets.data_ptr(), ps.hp.data_ptr(), H * 2, None, 0, e, st))
        torch.cuda.synchronize()
        assert sc.error_word() == 0
        results[order] = (h.clone(), ps.hp.clone())
        del buf
    assert torch.equal(results["gate_first"][0], results["up_first"][0])
    assert torch.equal(results["gate_first"][1], results["up_first"][1])
