"""The allocation-free layer entry point against the ordinary one.

`tsp_moe_layer_decode_static` is for callers that cannot obtain device scratch themselves (code running under
somebody else's allocator or inside a hook where device allocation is off limits): it keeps every intermediate
buffer in an array built into the library. This test drives it through the C ABI twice in a row, with different
inputs, so that the second call runs over whatever the first one left in that array, and requires the same output
rows as the caller-scratch entry point produces. It is collected last on purpose: a run that stops at the first
failure has then already exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tokspur_public_b200 import capi, formats, synth  # noqa: E402
from tokspur_public_b200 import layer as L  # noqa: E402


def scaled_error(actual, expected):
    return float(np.max(np.abs(actual.astype(np.float64) - expected) / np.maximum(1.0, np.abs(expected))))


def run_static(dl, x, logits, shape):
    Cn, H, E, K = shape
    T = x.shape[0]
    out = torch.zeros((T, Cn), dtype=x.dtype, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    dt = 1 if x.dtype == torch.float16 else 0
    capi.call("tsp_moe_layer_decode_static", C.byref(dl.weights), x.data_ptr(), x.stride(0) * x.element_size(), dt, logits.data_ptr(),
              logits.stride(0) * 4, T, Cn, H, E, K, 0, 1, out.data_ptr(), out.stride(0) * out.element_size(), dt, err.data_ptr(),
              L.stream_ptr())
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    return out.cpu().numpy()


def run_ordinary(dl, x, logits, shape):
    Cn, H, E, K = shape
    s = L.Scratch(Cn, H, E, K, x.shape[0], "cuda")
    out = torch.zeros((x.shape[0], Cn), dtype=x.dtype, device="cuda")
    L.moe_layer_decode(dl, s, x, logits, out)
    torch.cuda.synchronize()
    assert s.error_word() == 0
    return out.cpu().numpy()


def test_static_scratch_entry_matches_caller_scratch_entry_twice_in_a_row(oracle):
    shape = (512, 256, 16, 4)
    Cn, H, E, K = shape
    host = L.synth_host_layer(21, Cn, H, E, K, expert_type=formats.Q4_K)
    dl = L.DeviceLayer(host, formats.PLANAR, "cuda")
    for call, (T, dtype) in enumerate([(8, torch.float16), (5, torch.float32)]):   # second call: fewer rows, other dtype, stale array
        x = torch.from_numpy(synth.activations_f16(30 + call, T, Cn)).cuda().to(dtype)
        logits = torch.from_numpy(synth.router_logits(40 + call, T, E)).cuda()
        got = run_static(dl, x, logits, shape)
        want = run_ordinary(dl, x, logits, shape)
        assert scaled_error(got.astype(np.float32), want.astype(np.float64)) <= 5e-5
        assert np.array_equal(got, want)   # same kernels, same order of operations: the rows agree bit for bit
        if dtype == torch.float32:         # and against the CPU oracle directly, not only through the other entry point
            truth, _ = oracle.moe_layer(host.oracle_dict(), x.cpu().numpy(), logits.cpu().numpy(), threads=4, stages=True)
            assert scaled_error(got, truth) <= 5e-5


def test_static_scratch_entry_leaves_device_memory_alone():
    """Free device memory as the driver reports it (cudaMemGetInfo) is the same before and after calls of the entry point.
    Inputs and outputs are allocated up front. One call is made before the first reading: with lazy module loading the CUDA
    driver places a library's kernel image, of which the built-in array is a part, on the device when the first kernel of the
    image launches; that is the cost of loading the library, paid once, and not an allocation the entry point makes."""
    shape = (512, 256, 16, 4)
    Cn, H, E, K = shape
    host = L.synth_host_layer(22, Cn, H, E, K, expert_type=formats.Q4_K)
    dl = L.DeviceLayer(host, formats.PLANAR, "cuda")
    T = 8
    x = torch.from_numpy(synth.activations_f16(50, T, Cn)).cuda().float()
    logits = torch.from_numpy(synth.router_logits(51, T, E)).cuda()
    out = torch.zeros((T, Cn), dtype=torch.float32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = (C.byref(dl.weights), x.data_ptr(), Cn * 4, 0, logits.data_ptr(), E * 4, T, Cn, H, E, K, 0, 1, out.data_ptr(), Cn * 4, 0,
            err.data_ptr(), L.stream_ptr())
    capi.call("tsp_moe_layer_decode_static", *args)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        capi.call("tsp_moe_layer_decode_static", *args)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, f"free device memory moved by {free_before - free_after} bytes across the call"
    assert int(err.item()) == 0


def test_static_scratch_entry_refuses_what_does_not_fit():
    lib = capi.lib()
    limit = 4 << 20
    # the benchmark layer shape: 34 token rows are the most the array holds
    assert lib.tsp_moe_layer_decode_static_bytes(34, 2048, 512, 512, 10) == 4187904 <= limit
    assert lib.tsp_moe_layer_decode_static_bytes(35, 2048, 512, 512, 10) == 4310784 > limit
    shape = (512, 256, 16, 4)
    host = L.synth_host_layer(21, *shape, expert_type=formats.Q4_K)
    dl = L.DeviceLayer(host, formats.PLANAR, "cuda")
    T = 600   # 600 rows of this small layer need more than the built-in array holds
    x = torch.zeros((T, 512), dtype=torch.float32, device="cuda")
    logits = torch.zeros((T, 16), dtype=torch.float32, device="cuda")
    out = torch.zeros_like(x)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.tsp_moe_layer_decode_static(C.byref(dl.weights), x.data_ptr(), 2048, 0, logits.data_ptr(), 64, T, 512, 256, 16, 4, 0, 1,
                                         out.data_ptr(), 2048, 0, err.data_ptr(), L.stream_ptr())
    assert rc == capi.E_ARG and "built-in array" in capi.last_error()
