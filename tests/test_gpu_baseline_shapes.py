"""The benchmark's own shapes under `-m gpu`: the prefill layer at hidden 2048 / FFN 512 / 512 experts / top-10 with the
Zipf-skewed router (4096 tokens, K = 2048: eight super-blocks per row, 32 K chunks per item), a cheap K = 2048 case that
runs the same rings on every pass, and the Q8_0 vocabulary head at its full [151 936 x 2048] size.

Weights are generated and packed on the device (`SynthDeviceLayer`, GGUF bytes kept for the oracle); the oracle runs on a
spread sample of token rows because one row costs it about half a core-second.

Error budget of the prefill path: bar 2e-3 relative L2 (binary16 operands, FP32 accumulate). The guard below is tighter
than the bar on purpose, so that a change which eats into the margin is seen before it reaches the bar."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tokspur_public_b200 import capi, formats, synth  # noqa: E402
from tokspur_public_b200 import layer as L  # noqa: E402

CHANNELS, HIDDEN, EXPERTS, SELECTED = 2048, 512, 512, 10
PREFILL_BAR = 2e-3      # the stated tolerance of the path
PREFILL_GUARD = 1.5e-3  # regression guard: the measured figure has to stay well inside the bar


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def scaled_error(actual, expected):
    return float(np.max(np.abs(actual.astype(np.float64) - expected) / np.maximum(1.0, np.abs(expected))))


def prefill_case(oracle, seed, Cn, H, E, K, T, sample_n, bias_seed, guard):
    dl = L.SynthDeviceLayer(seed, Cn, H, E, formats.Q4_K, formats.PLANAR, "cuda", keep_gguf=True)
    ps = L.PrefillScratch(Cn, H, E, K, T, "cuda")
    x16 = synth.activations_f16(seed + 1, T, Cn)
    logits = synth.router_logits(seed + 2, T, E, synth.zipf_bias(bias_seed, E))
    out = torch.zeros((T, Cn), dtype=torch.float16, device="cuda")
    L.moe_layer_prefill(dl, ps, torch.from_numpy(x16).cuda(), torch.from_numpy(logits).cuda(), out)
    torch.cuda.synchronize()
    assert ps.base.error_word() == 0

    # integer results for ALL rows: ids, per-expert token order, counts, tile table
    ids = ps.base.ids.cpu().numpy().view(np.uint32)[:T * K].reshape(T, K)
    oi, ow = oracle.route_rows(logits.astype(np.float64), K, 0, True)
    assert np.array_equal(ids, oi)
    weights = ps.base.weights.cpu().numpy()[:T * K].reshape(T, K)
    assert np.max(np.abs(weights - ow)) <= 1e-6
    otm, ocounts = oracle.grouped_routes(oi, E)
    counts = ps.base.counts.cpu().numpy().view(np.uint32)[:E]
    assert np.array_equal(counts, ocounts)
    tm = ps.base.token_map.cpu().numpy().view(np.uint32)[:E * T].reshape(E, T)
    for e in range(E):
        assert np.array_equal(tm[e, :counts[e]], otm[e, :counts[e]])
    tile = int(ps.tile)
    tasks = ps.tasks.cpu().numpy().view(np.uint32)
    assert np.array_equal(tasks[:len(oracle.grouped_tasks(ocounts, T, K, tile))], oracle.grouped_tasks(ocounts, T, K, tile))

    # floating-point results on a spread sample of rows
    sample = np.unique(np.linspace(0, T - 1, sample_n).astype(int))
    host = dl.host_layer(K)
    want, st = oracle.moe_layer(host.oracle_dict(), x16[sample].astype(np.float32), logits[sample], threads=16, stages=True)
    got = out.cpu().numpy()[sample]
    r = rel_l2(got, want)
    assert r <= PREFILL_BAR, f"layer output rel-L2 {r:.3e} above the bar"
    assert r <= guard, f"layer output rel-L2 {r:.3e} above the regression guard {guard:.1e}"
    shared = ps.shared_out_rows(T)
    if shared is not None:
        assert rel_l2(shared[sample], st["shared_out"]) <= guard
    routed = ps.routed_rows(T)
    if routed is not None:
        assert rel_l2(routed.reshape(T, K, Cn)[sample], st["routed"]) <= guard
    return r


def test_prefill_layer_benchmark_shape_4096_tokens(oracle):
    """BASELINE configs[2]: 4096 tokens, Zipf(1.1) bias: one expert with ~4000 routes, hundreds with none."""
    prefill_case(oracle, 100, CHANNELS, HIDDEN, EXPERTS, SELECTED, 4096, 64, 5, PREFILL_GUARD)


def test_prefill_layer_k2048_small(oracle):
    """K = 2048 (eight super-blocks per row) with few experts and rows: the deep rings in every test pass."""
    prefill_case(oracle, 7, CHANNELS, HIDDEN, 8, 3, 300, 24, 9, PREFILL_GUARD)


@pytest.mark.parametrize("M", [1, 8, 16])
def test_vocabulary_head_full_size(oracle, M):
    """BASELINE configs[3]: dense Q8_0 [151 936 x 2048] on M draft-token rows; 4096 sampled vocabulary rows incl. the last item."""
    VOCAB = 151936
    bpr = CHANNELS // 32
    row_bytes = bpr * 34
    t = torch.empty(VOCAB * row_bytes, dtype=torch.uint8, device="cuda")
    capi.call("tsp_synth_weights", formats.Q8_0, 900, 0, VOCAB * bpr, 0.02, t.data_ptr(), L.stream_ptr())
    ms = L.matrix_set(t, formats.Q8_0, formats.GGUF, VOCAB, CHANNELS)
    x = synth.activations_f16(3000 + M, M, CHANNELS).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    out = torch.zeros((M, VOCAB), dtype=torch.float32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.call("tsp_moe_project", C.byref(ms), dx.data_ptr(), CHANNELS * 4, 1, M, 1, None, None, None, out.data_ptr(), VOCAB * 4, 1,
              err.data_ptr(), L.stream_ptr())
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    rng = np.random.default_rng(M)
    rows = np.unique(np.concatenate([rng.integers(0, VOCAB, 3968), np.arange(VOCAB - 128, VOCAB)]))   # the last 128-row item included
    w = t.view(VOCAB, row_bytes)[torch.from_numpy(rows).cuda()].cpu().numpy()
    got = out[:, torch.from_numpy(rows).cuda()].cpu().numpy()
    for m in range(M):
        want = oracle.gemv(formats.Q8_0, w.reshape(-1), CHANNELS, len(rows), x[m])
        assert scaled_error(got[m], want) <= 5e-5
