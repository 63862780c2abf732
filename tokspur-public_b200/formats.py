"""Weight byte formats on the MoE path: GGUF Q4_K / Q8_0 blocks and the Pack v3 planar expert layout.

The encoders here are this build's own deterministic quantizers (the reference ships decoders only);
their output is defined by the reference *decoder*, which is what every parity check runs on.
Layout facts restated from the reference: Q4_K block (numeric.cpp:25-31,44-50), Q8_0 block (numeric.cpp:43),
planar planes and `sm16` scale bytes (planar_pack_v3.cpp:601-716), co-located gate/up pairs
(planar_pack_v3.cpp:1076-1093).
"""
from __future__ import annotations

import numpy as np

Q8_0, Q4_K = 8, 12
Q5_1, Q5_K = 7, 13   # the reference model's down / gate-up encodings beside Q4_K and Q8_0 (decode-size kernels, GGUF rows)
GGUF, PLANAR = 0, 1


def block_geometry(type_: int) -> tuple[int, int]:
    """(elements per block, bytes per block) of a GGUF encoding."""
    return {Q8_0: (32, 34), Q4_K: (256, 144), Q5_1: (32, 24), Q5_K: (256, 176)}[type_]


def gguf_bytes(type_: int, rows: int, cols: int) -> int:
    e, b = block_geometry(type_)
    assert cols % e == 0
    return rows * (cols // e) * b


def planar_bytes(type_: int, rows: int, cols: int) -> int:
    e, _ = block_geometry(type_)
    return rows * (cols // e) * (148 if type_ == Q4_K else 34)


# --------------------------------------------------------------------------------------------
# encoders
# --------------------------------------------------------------------------------------------
def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    """[rows, cols] float32 -> uint8 [rows, cols/32*34]: d = amax/127 as binary16, q = round(w/d)."""
    rows, cols = w.shape
    blk = w.reshape(rows, cols // 32, 32).astype(np.float32)
    amax = np.abs(blk).max(axis=2)
    d = (amax / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df > 0, 1.0 / np.where(df > 0, df, 1), 0).astype(np.float32)
    q = np.clip(np.rint(blk * inv[..., None]), -127, 127).astype(np.int8)
    out = np.empty((rows, cols // 32, 34), dtype=np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, cols // 32, 2)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(rows, -1)


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    """[rows, cols] float32 -> uint8 [rows, cols/256*144].

    Per 32-wide group an affine code: min_g = max(0, -min), scale_g = (max + min_g)/15; the super-block keeps
    d = max(scale_g)/63 and dmin = max(min_g)/63 as binary16 and 6-bit integer factors sc_g, mn_g;
    q = clamp(round((w + dmin*mn_g) / (d*sc_g)), 0, 15)."""
    rows, cols = w.shape
    nb = cols // 256
    x = w.reshape(rows, nb, 8, 32).astype(np.float32)
    lo = np.minimum(x.min(axis=3), 0)
    hi = x.max(axis=3)
    min_g = -lo
    scale_g = (hi + min_g) / 15.0
    d = (scale_g.max(axis=2) / 63.0).astype(np.float16)
    dmin = (min_g.max(axis=2) / 63.0).astype(np.float16)
    df, mf = d.astype(np.float32), dmin.astype(np.float32)
    sc = np.where(df[..., None] > 0, np.rint(scale_g / np.where(df > 0, df, 1)[..., None]), 0)
    mn = np.where(mf[..., None] > 0, np.rint(min_g / np.where(mf > 0, mf, 1)[..., None]), 0)
    sc = np.clip(sc, 0, 63).astype(np.uint8)
    mn = np.clip(mn, 0, 63).astype(np.uint8)
    dl = df[..., None] * sc
    ml = mf[..., None] * mn
    q = np.where(dl[..., None] > 0, np.rint((x + ml[..., None]) / np.where(dl > 0, dl, 1)[..., None]), 0)
    q = np.clip(q, 0, 15).astype(np.uint8)
    out = np.zeros((rows, nb, 144), dtype=np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, nb, 2)
    out[..., 2:4] = dmin.view(np.uint8).reshape(rows, nb, 2)
    out[..., 4:8] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    out[..., 8:12] = mn[..., 0:4] | ((mn[..., 4:8] >> 4) << 6)
    out[..., 12:16] = (sc[..., 4:8] & 15) | ((mn[..., 4:8] & 15) << 4)
    qp = q.reshape(rows, nb, 4, 2, 32)  # pair j holds groups 2j (low nibble) and 2j+1 (high nibble)
    out[..., 16:] = (qp[:, :, :, 0, :] | (qp[:, :, :, 1, :] << 4)).reshape(rows, nb, 128)
    return out.reshape(rows, -1)


def quantize_q5_k(w: np.ndarray) -> np.ndarray:
    """[rows, cols] float32 -> uint8 [rows, cols/256*176]: the Q4_K scheme with 32 levels. Block: d, dmin, the twelve factor
    bytes, 32 bytes of fifth bits (bit g of byte i = weight i of group g), 128 bytes of low nibbles (numeric.cpp:44-50)."""
    rows, cols = w.shape
    nb = cols // 256
    x = w.reshape(rows, nb, 8, 32).astype(np.float32)
    lo = np.minimum(x.min(axis=3), 0)
    hi = x.max(axis=3)
    min_g = -lo
    scale_g = (hi + min_g) / 31.0
    d = (scale_g.max(axis=2) / 63.0).astype(np.float16)
    dmin = (min_g.max(axis=2) / 63.0).astype(np.float16)
    df, mf = d.astype(np.float32), dmin.astype(np.float32)
    sc = np.where(df[..., None] > 0, np.rint(scale_g / np.where(df > 0, df, 1)[..., None]), 0)
    mn = np.where(mf[..., None] > 0, np.rint(min_g / np.where(mf > 0, mf, 1)[..., None]), 0)
    sc = np.clip(sc, 0, 63).astype(np.uint8)
    mn = np.clip(mn, 0, 63).astype(np.uint8)
    dl = df[..., None] * sc
    ml = mf[..., None] * mn
    q = np.where(dl[..., None] > 0, np.rint((x + ml[..., None]) / np.where(dl > 0, dl, 1)[..., None]), 0)
    q = np.clip(q, 0, 31).astype(np.uint8)
    out = np.zeros((rows, nb, 176), dtype=np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, nb, 2)
    out[..., 2:4] = dmin.view(np.uint8).reshape(rows, nb, 2)
    out[..., 4:8] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    out[..., 8:12] = mn[..., 0:4] | ((mn[..., 4:8] >> 4) << 6)
    out[..., 12:16] = (sc[..., 4:8] & 15) | ((mn[..., 4:8] & 15) << 4)
    high = np.zeros((rows, nb, 32), dtype=np.uint8)
    for g in range(8):
        high |= (q[:, :, g, :] >> 4) << g
    out[..., 16:48] = high
    qp = (q & 15).reshape(rows, nb, 4, 2, 32)
    out[..., 48:] = (qp[:, :, :, 0, :] | (qp[:, :, :, 1, :] << 4)).reshape(rows, nb, 128)
    return out.reshape(rows, -1)


def quantize_q5_1(w: np.ndarray) -> np.ndarray:
    """[rows, cols] float32 -> uint8 [rows, cols/32*24]: d = (max - min)/31 and m = min as binary16, q = round((w - m)/d);
    block: d, m, 32 fifth bits (bit i = weight i), 16 bytes of nibbles (weight i in nibble i/16 of byte i%16; numeric.cpp:38-42)."""
    rows, cols = w.shape
    nb = cols // 32
    x = w.reshape(rows, nb, 32).astype(np.float32)
    mn, mx = x.min(axis=2), x.max(axis=2)
    d = ((mx - mn) / 31.0).astype(np.float16)
    m = mn.astype(np.float16)
    df, mf = d.astype(np.float32), m.astype(np.float32)
    q = np.where(df[..., None] > 0, np.rint((x - mf[..., None]) / np.where(df > 0, df, 1)[..., None]), 0)
    q = np.clip(q, 0, 31).astype(np.uint32)
    out = np.zeros((rows, nb, 24), dtype=np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, nb, 2)
    out[..., 2:4] = m.view(np.uint8).reshape(rows, nb, 2)
    high = np.zeros((rows, nb), dtype=np.uint32)
    for i in range(32):
        high |= (q[..., i] >> 4) << np.uint32(i)
    out[..., 4:8] = high.view(np.uint8).reshape(rows, nb, 4)
    out[..., 8:24] = ((q[..., 0:16] & 15) | ((q[..., 16:32] & 15) << 4)).astype(np.uint8)
    return out.reshape(rows, -1)


def quantize(type_: int, w: np.ndarray) -> np.ndarray:
    return {Q4_K: quantize_q4_k, Q8_0: quantize_q8_0, Q5_K: quantize_q5_k, Q5_1: quantize_q5_1}[type_](w)


# --------------------------------------------------------------------------------------------
# decoders (vectorised; used for data preparation and cross-checks, never on the product path)
# --------------------------------------------------------------------------------------------
def sm16_from_scales12(s12: np.ndarray) -> np.ndarray:
    """[..., 12] GGUF packed 6-bit factors -> [..., 16] planar bytes sc[0..7], mn[0..7] (planar_pack_v3.cpp:652-661)."""
    s12 = s12.astype(np.uint8)
    out = np.empty(s12.shape[:-1] + (16,), dtype=np.uint8)
    out[..., 0:4] = s12[..., 0:4] & 0x3F
    out[..., 4:8] = (s12[..., 8:12] & 0x0F) | ((s12[..., 0:4] >> 6) << 4)
    out[..., 8:12] = s12[..., 4:8] & 0x3F
    out[..., 12:16] = (s12[..., 8:12] >> 4) | ((s12[..., 4:8] >> 6) << 4)
    return out


def dequantize_gguf(type_: int, data: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """GGUF bytes -> float32 [rows, cols], the exact value rounded once (float64 arithmetic is exact here)."""
    if type_ == Q8_0:
        b = data.reshape(rows, cols // 32, 34)
        d = b[..., 0:2].copy().view(np.float16).astype(np.float64)
        q = b[..., 2:].view(np.int8).astype(np.float64)
        return (d * q).reshape(rows, cols).astype(np.float32)
    if type_ == Q5_1:
        b = data.reshape(rows, cols // 32, 24)
        d = b[..., 0:2].copy().view(np.float16).astype(np.float64)
        m = b[..., 2:4].copy().view(np.float16).astype(np.float64)
        high = b[..., 4:8].copy().view(np.uint32)
        i = np.arange(32)
        q = ((b[..., 8 + i % 16] >> (4 * (i // 16))) & 15) | (((high >> i.astype(np.uint32)) & 1) << 4)
        return (d * q + m).reshape(rows, cols).astype(np.float32)
    if type_ == Q5_K:
        b = data.reshape(rows, cols // 256, 176)
        d = b[..., 0:2].copy().view(np.float16).astype(np.float64)[..., 0]
        dmin = b[..., 2:4].copy().view(np.float16).astype(np.float64)[..., 0]
        sm = sm16_from_scales12(b[..., 4:16]).astype(np.float64)
        qs = b[..., 48:].reshape(rows, cols // 256, 4, 32)
        q = np.stack([qs & 15, qs >> 4], axis=3).reshape(rows, cols // 256, 8, 32).astype(np.uint32)
        q |= ((b[..., None, 16:48].astype(np.uint32) >> np.arange(8, dtype=np.uint32)[:, None]) & 1) << 4
        v = (d[..., None] * sm[..., 0:8])[..., None] * q - (dmin[..., None] * sm[..., 8:16])[..., None]
        return v.reshape(rows, cols).astype(np.float32)
    b = data.reshape(rows, cols // 256, 144)
    d = b[..., 0:2].copy().view(np.float16).astype(np.float64)[..., 0]
    dmin = b[..., 2:4].copy().view(np.float16).astype(np.float64)[..., 0]
    sm = sm16_from_scales12(b[..., 4:16]).astype(np.float64)
    qs = b[..., 16:].reshape(rows, cols // 256, 4, 32)
    q = np.stack([qs & 15, qs >> 4], axis=3).reshape(rows, cols // 256, 8, 32).astype(np.float64)
    v = (d[..., None] * sm[..., 0:8])[..., None] * q - (dmin[..., None] * sm[..., 8:16])[..., None]
    return v.reshape(rows, cols).astype(np.float32)


# --------------------------------------------------------------------------------------------
# Pack v3 planar layout
# --------------------------------------------------------------------------------------------
def pack_planar(type_: int, gguf: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """One expert, GGUF rows -> planar planes qs | sm | dm (Q4_K) or qs | dm (Q8_0)."""
    if type_ == Q4_K:
        assert rows % 4 == 0 and cols % 256 == 0
        b = gguf.reshape(rows * (cols // 256), 144)
        return np.concatenate([b[:, 16:].reshape(-1), sm16_from_scales12(b[:, 4:16]).reshape(-1), b[:, 0:4].reshape(-1)])
    assert rows % 4 == 0 and cols % 32 == 0 and (rows * (cols // 32)) % 8 == 0
    b = gguf.reshape(rows * (cols // 32), 34)
    return np.concatenate([b[:, 2:].reshape(-1), b[:, 0:2].reshape(-1)])


def pack_planar_experts(type_: int, gguf: np.ndarray, experts: int, rows: int, cols: int) -> np.ndarray:
    """[experts, gguf_bytes] -> [experts, planar_bytes]."""
    g = gguf.reshape(experts, -1)
    return np.stack([pack_planar(type_, g[e], rows, cols) for e in range(experts)])


def colocate_gate_up(gate_planar: np.ndarray, up_planar: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Planar gate/up experts -> the two co-located tensors: pair_lo holds experts [0, E/2) as
    [gate_e, up_e] pairs, pair_hi holds experts [E/2, E)."""
    E = gate_planar.shape[0]
    assert E % 2 == 0 and up_planar.shape == gate_planar.shape
    pairs = np.stack([gate_planar, up_planar], axis=1)  # [E, 2, bytes]
    return np.ascontiguousarray(pairs[: E // 2]).reshape(-1), np.ascontiguousarray(pairs[E // 2:]).reshape(-1)
