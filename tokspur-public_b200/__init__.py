"""B200-native (sm_100a) routed-MoE FFN hot path behind tokspur's operator entry points.

The product is the CUDA library `libtsp_moe.so` (C ABI in include/tsp_moe.h) and the C++ host layer
under native/ that mirrors the reference's `encode_moe*` functions. This Python package is the
harness around them: build, ctypes binding, weight-format helpers and synthetic data.
There is no CPU fallback: importing `capi` without a built library raises.
"""
from . import build as _build  # noqa: F401

__all__ = ["capi", "formats", "synth", "layer"]
