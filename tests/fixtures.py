"""Deterministic, integer-only test inputs restating the reference's own fixture recipes.

  lcg_weights      every block byte from the 32-bit LCG x <- x*1664525 + 1013904223 (byte = x >> 24), seed 44, then
                   the binary16 scale fields overwritten from a fixed table (native/tests/grouped_mm_fixture.hpp:10-19).
  bounded_weights  the "bounded nonzero quant domain" matrices (native/tests/test_moe_mm_many_gpu.cpp:30-47):
                   d = 0x0c01, Q8 codes in -15..15, Q4_K dmin = 0x0401, factors 1 / 0x11, nibbles masked 0x77.
  lcg_activations  float(int(x % 1993) - 996) / 997 (native/tests/test_planar_pack_v3.cpp:476-480).
"""
import numpy as np

A, Cc = 1664525, 1013904223


def lcg_stream(seed: int, n: int) -> np.ndarray:
    """The next n LCG states after `seed` as uint32, vectorised with wrap-around arithmetic."""
    with np.errstate(over="ignore"):
        a_pow = np.cumprod(np.full(n, A, dtype=np.uint32), dtype=np.uint32)            # a^1 .. a^n
        geo = np.cumsum(np.concatenate([[np.uint32(1)], a_pow[:-1]]), dtype=np.uint32)  # 1 + a + ... + a^(k-1)
        return a_pow * np.uint32(seed) + geo * np.uint32(Cc)


def block_bytes(type_: int) -> int:
    return {7: 24, 8: 34, 12: 144, 13: 176, 14: 210, 20: 18}[type_]


def lcg_weights(type_: int, cols: int, rows: int, experts: int, seed: int = 44) -> np.ndarray:
    bpb = block_bytes(type_)
    epb = 32 if type_ in (7, 8, 20) else 256
    nblocks = cols // epb * rows * experts
    out = (lcg_stream(seed, nblocks * bpb) >> np.uint32(24)).astype(np.uint8).reshape(nblocks, bpb)
    ds = np.array([0x0401, 0x0568, 0x068e, 0x0ac2, 0x2401, 0x2803, 0xa401, 0x1801], dtype=np.uint16)
    d = ds[np.arange(nblocks) % 8]
    out[:, 0] = d & 255
    out[:, 1] = d >> 8
    if type_ == 14:        # Q6_K keeps its scale at the end of the block
        out[:, 208] = d & 255
        out[:, 209] = d >> 8
    if type_ != 8:
        out[:, 2] = 0x03
        out[:, 3] = 0x1c
    return out.reshape(experts, -1)


def bounded_weights(type_: int, cols: int, rows: int, experts: int, seed: int) -> np.ndarray:
    bpb = block_bytes(type_)
    epb = 32 if type_ == 8 else 256
    nblocks = cols // epb * rows * experts
    draws = bpb + (32 if type_ == 8 else 0)
    s = lcg_stream(seed, nblocks * draws).reshape(nblocks, draws)
    out = (s[:, :bpb] >> np.uint32(24)).astype(np.uint8)
    out[:, 0] = 1
    out[:, 1] = 0x0c
    if type_ == 8:
        out[:, 2:34] = ((s[:, bpb:] % np.uint32(31)).astype(np.int64) - 15).astype(np.int8).view(np.uint8)
    else:
        out[:, 2] = 1
        out[:, 3] = 4
        out[:, 4:12] = 1
        out[:, 12:16] = 0x11
        out[:, 16:] &= 0x77
    return out.reshape(experts, -1)


def lcg_activations(seed: int, n: int) -> np.ndarray:
    s = lcg_stream(seed, n)
    return ((s % np.uint32(1993)).astype(np.int64) - 996).astype(np.float32) / np.float32(997)
