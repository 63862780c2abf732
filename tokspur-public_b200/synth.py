"""Seeded synthetic tensors with the shapes and value distributions the benchmark configurations name.

A counter-based generator (splitmix64 of seed and element index, then Box-Muller) so that any slice of a
tensor can be produced independently and identically by every rank. Stands in for the real model's
weights and activations, which are not available.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def uniform(seed: int, n: int, offset: int = 0) -> np.ndarray:
    """n doubles in (0, 1): element i depends only on (seed, offset + i)."""
    with np.errstate(over="ignore"):
        idx = np.arange(offset, offset + n, dtype=np.uint64)
        key = splitmix64(np.full(1, seed, dtype=np.uint64))[0]
        bits = splitmix64(idx * np.uint64(0xD1342543DE82EF95) + key)
    return ((bits >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)


def normal(seed: int, shape, sigma: float = 1.0, offset: int = 0) -> np.ndarray:
    n = int(np.prod(shape))
    u = uniform(seed, 2 * n, 2 * offset)
    r = np.sqrt(-2.0 * np.log(u[0::2]))
    return (sigma * r * np.cos(2.0 * np.pi * u[1::2])).astype(np.float32).reshape(shape)


def activations_f16(seed: int, tokens: int, channels: int) -> np.ndarray:
    """N(0,1) rounded to binary16."""
    return normal(seed, (tokens, channels)).astype(np.float16)


def zipf_bias(seed: int, experts: int, exponent: float = 1.1) -> np.ndarray:
    """Per-expert additive logit bias ln(p_e * E), p_e proportional to rank_e^-exponent over a seeded permutation."""
    order = np.argsort(uniform(seed, experts))
    rank = np.empty(experts, dtype=np.int64)
    rank[order] = np.arange(1, experts + 1)
    p = rank.astype(np.float64) ** (-exponent)
    p /= p.sum()
    return np.log(p * experts).astype(np.float32)


def router_logits(seed: int, tokens: int, experts: int, bias: np.ndarray | None = None) -> np.ndarray:
    lg = normal(seed, (tokens, experts))
    if bias is not None:
        lg = lg + bias[None, :]
    return lg.astype(np.float32)
