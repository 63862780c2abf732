"""The routed + shared expert entries (one launch each) against the separate entries: bit-identical rows."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens", [1, 5, 64])
def test_fused_entries_match_separate_launches(tokens):
    from tokspur_public_b200 import capi, formats, synth
    from tokspur_public_b200 import layer as L
    Cn, H, E, K = 1024, 256, 32, 4
    dev = torch.device("cuda")
    sl = L.SynthDeviceLayer(7, Cn, H, E, formats.Q4_K, formats.PLANAR, dev)
    sc = L.Scratch(Cn, H, E, K, tokens, dev)
    w = sl.weights
    lib = capi.lib()
    st = L.stream_ptr()
    x16 = torch.from_numpy(synth.activations_f16(3, tokens, Cn)).to(dev)
    x32 = x16.float().contiguous()
    lg = torch.from_numpy(synth.router_logits(4, tokens, E)).to(dev)
    e = sc.error.data_ptr()
    capi.check(lib.tsp_moe_route(lg.data_ptr(), E * 4, tokens, E, K, 0, 1, sc.ids.data_ptr(), sc.weights.data_ptr(), e, st))
    capi.check(lib.tsp_moe_permute(sc.ids.data_ptr(), tokens, E, K, capi.GEMV_TILE, sc.token_map.data_ptr(), sc.counts.data_ptr(),
                                   sc.tasks.data_ptr(), e, st))
    tm, cn, tk = sc.token_map.data_ptr(), sc.counts.data_ptr(), sc.tasks.data_ptr()

    def zeros(*shape):
        return torch.zeros(shape, dtype=torch.float32, device=dev)

    h_a, sh_a, out_a, so_a = zeros(tokens * K, H), zeros(tokens, H), zeros(tokens * K, Cn), zeros(tokens, Cn)
    capi.check(lib.tsp_moe_gate_up_swiglu(C.byref(w.gate), C.byref(w.up), x32.data_ptr(), Cn * 4, tokens, K, tm, cn, tk, h_a.data_ptr(), H * 4, 1, e, st))
    capi.check(lib.tsp_moe_gate_up_swiglu(C.byref(w.shared_gate), C.byref(w.shared_up), x32.data_ptr(), Cn * 4, tokens, 1, None, None, None,
                                          sh_a.data_ptr(), H * 4, 1, e, st))
    capi.check(lib.tsp_moe_project(C.byref(w.down), h_a.data_ptr(), H * 4, 1, tokens, K, tm, cn, tk, out_a.data_ptr(), Cn * 4, 0, e, st))
    capi.check(lib.tsp_moe_project(C.byref(w.shared_down), sh_a.data_ptr(), H * 4, 1, tokens, 1, None, None, None, so_a.data_ptr(), Cn * 4, 0, e, st))
    for use_x16 in (False, True):
        h_b, sh_b, out_b, so_b = zeros(tokens * K, H), zeros(tokens, H), zeros(tokens * K, Cn), zeros(tokens, Cn)
        capi.check(lib.tsp_moe_gate_up_swiglu_shared(C.byref(w.gate), C.byref(w.up), C.byref(w.shared_gate), C.byref(w.shared_up), x32.data_ptr(),
                                                     Cn * 4, x16.data_ptr() if use_x16 else None, Cn * 2, tokens, K, tm, cn, tk,
                                                     h_b.data_ptr(), H * 4, sh_b.data_ptr(), H * 4, 1, e, st))
        capi.check(lib.tsp_moe_project_shared(C.byref(w.down), C.byref(w.shared_down), h_b.data_ptr(), H * 4, sh_b.data_ptr(), H * 4, tokens, K,
                                              tm, cn, tk, out_b.data_ptr(), Cn * 4, so_b.data_ptr(), Cn * 4, e, st))
        torch.cuda.synchronize()
        assert sc.error_word() == 0
        for a, b in ((h_a, h_b), (sh_a, sh_b), (out_a, out_b), (so_a, so_b)):
            assert torch.equal(a, b)


@pytest.mark.parametrize("tokens,shared_tokens", [(20, 7), (5, 33), (64, 64)])
def test_shared_expert_on_other_rows_matches_separate_launches(tokens, shared_tokens):
    """The `_shared_rows` entries: routed experts over one set of rows, the dense shared expert over ANOTHER set (what the
    expert-parallel layer does with received rows and the rank's own rows), against the separate launches: bit-identical."""
    from tokspur_public_b200 import capi, formats, synth
    from tokspur_public_b200 import layer as L
    Cn, H, E, K = 1024, 256, 32, 4
    dev = torch.device("cuda")
    sl = L.SynthDeviceLayer(9, Cn, H, E, formats.Q4_K, formats.PLANAR, dev)
    sc = L.Scratch(Cn, H, E, K, tokens, dev)
    w = sl.weights
    lib = capi.lib()
    st = L.stream_ptr()
    x32 = torch.from_numpy(synth.activations_f16(3, tokens, Cn)).to(dev).float().contiguous()
    xs32 = torch.from_numpy(synth.activations_f16(5, shared_tokens, Cn)).to(dev).float().contiguous()
    lg = torch.from_numpy(synth.router_logits(4, tokens, E)).to(dev)
    e = sc.error.data_ptr()
    capi.check(lib.tsp_moe_route(lg.data_ptr(), E * 4, tokens, E, K, 0, 1, sc.ids.data_ptr(), sc.weights.data_ptr(), e, st))
    capi.check(lib.tsp_moe_permute(sc.ids.data_ptr(), tokens, E, K, capi.GEMV_TILE, sc.token_map.data_ptr(), sc.counts.data_ptr(),
                                   sc.tasks.data_ptr(), e, st))
    tm, cn, tk = sc.token_map.data_ptr(), sc.counts.data_ptr(), sc.tasks.data_ptr()

    def zeros(*shape):
        return torch.zeros(shape, dtype=torch.float32, device=dev)

    h_a, sh_a, out_a, so_a = zeros(tokens * K, H), zeros(shared_tokens, H), zeros(tokens * K, Cn), zeros(shared_tokens, Cn)
    capi.check(lib.tsp_moe_gate_up_swiglu(C.byref(w.gate), C.byref(w.up), x32.data_ptr(), Cn * 4, tokens, K, tm, cn, tk, h_a.data_ptr(), H * 4, 1, e, st))
    capi.check(lib.tsp_moe_gate_up_swiglu(C.byref(w.shared_gate), C.byref(w.shared_up), xs32.data_ptr(), Cn * 4, shared_tokens, 1, None, None, None,
                                          sh_a.data_ptr(), H * 4, 1, e, st))
    capi.check(lib.tsp_moe_project(C.byref(w.down), h_a.data_ptr(), H * 4, 1, tokens, K, tm, cn, tk, out_a.data_ptr(), Cn * 4, 0, e, st))
    capi.check(lib.tsp_moe_project(C.byref(w.shared_down), sh_a.data_ptr(), H * 4, 1, shared_tokens, 1, None, None, None, so_a.data_ptr(), Cn * 4, 0, e, st))
    h_b, sh_b, out_b, so_b = zeros(tokens * K, H), zeros(shared_tokens, H), zeros(tokens * K, Cn), zeros(shared_tokens, Cn)
    capi.check(lib.tsp_moe_gate_up_swiglu_shared_rows(C.byref(w.gate), C.byref(w.up), C.byref(w.shared_gate), C.byref(w.shared_up), x32.data_ptr(), Cn * 4,
                                                      None, 0, tokens, K, tm, cn, tk, h_b.data_ptr(), H * 4, xs32.data_ptr(), Cn * 4, shared_tokens,
                                                      sh_b.data_ptr(), H * 4, 1, e, st))
    capi.check(lib.tsp_moe_project_shared_rows(C.byref(w.down), C.byref(w.shared_down), h_b.data_ptr(), H * 4, sh_b.data_ptr(), H * 4, shared_tokens, tokens, K,
                                               tm, cn, tk, out_b.data_ptr(), Cn * 4, so_b.data_ptr(), Cn * 4, e, st))
    torch.cuda.synchronize()
    assert sc.error_word() == 0
    for a, b in ((h_a, h_b), (sh_a, sh_b), (out_a, out_b), (so_a, so_b)):
        assert torch.equal(a, b)
    # binary16 rows can serve both row sets only when they are the same rows
    x16 = torch.zeros((tokens, Cn), dtype=torch.float16, device=dev)
    rc = lib.tsp_moe_gate_up_swiglu_shared_rows(C.byref(w.gate), C.byref(w.up), C.byref(w.shared_gate), C.byref(w.shared_up), x32.data_ptr(), Cn * 4,
                                                x16.data_ptr(), Cn * 2, tokens, K, tm, cn, tk, h_b.data_ptr(), H * 4, xs32.data_ptr(), Cn * 4, shared_tokens,
                                                sh_b.data_ptr(), H * 4, 1, e, st)
    assert rc == capi.E_ARG
