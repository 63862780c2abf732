"""ctypes binding of the C ABI declared in include/tsp_moe.h.

Device memory is passed as raw pointers (`tensor.data_ptr()` of torch CUDA tensors); torch is used
only for allocation, streams and copies. Every call raises `TspError` on a non-zero status, with the
library's own message. Loading fails loudly when the library has not been built.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

LIB_PATH = _build.LIB

TYPE_F32, TYPE_Q8_0, TYPE_Q4_K = 0, 8, 12
TYPE_Q5_1, TYPE_Q5_K = 7, 13
LAYOUT_GGUF, LAYOUT_PLANAR = 0, 1
ROUTER_SOFTMAX, ROUTER_SIGMOID = 0, 1
ERR_NONFINITE, ERR_INDEX, ERR_TIMEOUT = 2, 4, 8
GEMV_TILE = 8
E_ARG, E_TYPE, E_CUDA, E_DEVICE = -1, -2, -3, -4


class TspError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"tsp status {code}: {message}")
        self.code = code
        self.message = message


class MatrixSet(C.Structure):
    _fields_ = [("base", C.c_void_p), ("base_hi", C.c_void_p), ("expert_stride", C.c_uint64), ("split", C.c_uint32),
                ("experts", C.c_uint32), ("rows", C.c_uint32), ("cols", C.c_uint32), ("type", C.c_uint32), ("layout", C.c_uint32)]


class MoeScratch(C.Structure):
    _fields_ = [("d_ids", C.c_void_p), ("d_weights", C.c_void_p), ("d_hidden", C.c_void_p), ("d_routed", C.c_void_p),
                ("d_shared_hidden", C.c_void_p), ("d_shared_out", C.c_void_p), ("d_shared_logit", C.c_void_p),
                ("d_x32", C.c_void_p), ("d_token_map", C.c_void_p), ("d_counts", C.c_void_p), ("d_tasks", C.c_void_p),
                ("capacity", C.c_uint32)]


class MoePrefillScratch(C.Structure):
    _fields_ = [("base", MoeScratch), ("d_xk", C.c_void_p), ("d_xp", C.c_void_p), ("d_hp", C.c_void_p), ("d_offsets", C.c_void_p),
                ("d_s_hp", C.c_void_p)]


class RouterMarginTelemetry(C.Structure):
    _fields_ = [("min_margin", C.c_float), ("sum_margin", C.c_double), ("total_tokens", C.c_uint64), ("violation_count", C.c_uint64),
                ("fallback_layers", C.c_uint64), ("total_layers", C.c_uint64)]


class MoeWeights(C.Structure):
    _fields_ = [("gate", MatrixSet), ("up", MatrixSet), ("down", MatrixSet), ("shared_gate", MatrixSet),
                ("shared_up", MatrixSet), ("shared_down", MatrixSet), ("d_shared_router", C.c_void_p)]


# name -> (restype, argtypes); the list is also what the symbol-export test checks against the header
_vp, _u32, _u64, _i = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int
_MS = C.POINTER(MatrixSet)
SIGNATURES = {
    "tsp_last_error": (C.c_char_p, []),
    "tsp_device_info": (_i, [C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "tsp_error_word_read": (_i, [_vp, _vp, C.POINTER(_u32)]),
    "tsp_error_word_reset": (_i, [_vp, _vp]),
    "tsp_expert_bytes": (_u64, [_u32, _u32, _u32, _u32]),
    "tsp_dequant_f32": (_i, [_MS, _u32, _vp, _vp, _vp]),
    "tsp_moe_route": (_i, [_vp, _u64, _u32, _u32, _u32, _u32, _i, _vp, _vp, _vp, _vp]),
    "tsp_moe_permute": (_i, [_vp, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp]),
    "tsp_moe_permute_local": (_i, [_vp, _u32, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp]),
    "tsp_moe_tasks_words": (_u64, [_u32, _u32, _u32, _u32]),
    "tsp_moe_gate_up_swiglu": (_i, [_MS, _MS, _vp, _u64, _u32, _u32, _vp, _vp, _vp, _vp, _u64, _i, _vp, _vp]),
    "tsp_moe_project": (_i, [_MS, _vp, _u64, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _u64, _i, _vp, _vp]),
    "tsp_moe_gate_up_swiglu_shared": (_i, [_MS, _MS, _MS, _MS, _vp, _u64, _vp, _u64, _u32, _u32, _vp, _vp, _vp, _vp, _u64, _vp, _u64, _i, _vp, _vp]),
    "tsp_moe_project_shared": (_i, [_MS, _MS, _vp, _u64, _vp, _u64, _u32, _u32, _vp, _vp, _vp, _vp, _u64, _vp, _u64, _vp, _vp]),
    "tsp_moe_gate_up_swiglu_shared_rows": (_i, [_MS, _MS, _MS, _MS, _vp, _u64, _vp, _u64, _u32, _u32, _vp, _vp, _vp, _vp, _u64, _vp, _u64, _u32, _vp, _u64, _i, _vp, _vp]),
    "tsp_moe_project_shared_rows": (_i, [_MS, _MS, _vp, _u64, _vp, _u64, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _u64, _vp, _u64, _vp, _vp]),
    "tsp_moe_combine": (_i, [_vp, _u64, _u32, _vp, _vp, _u64, _vp, _vp, _u64, _u32, _vp, _u32, _u32, _u32, _vp, _u64, _vp, _u64, _vp, _vp]),
    "tsp_synth_weights": (_i, [_u32, _u64, _u64, _u64, C.c_float, _vp, _vp]),
    "tsp_pack_planar": (_i, [_u32, _u32, _u32, _u32, _vp, _u64, _vp, _u64, _vp]),
    "tsp_gemv_f32": (_i, [_vp, _u32, _u32, _vp, _u64, _u32, _vp, _u64, _vp, _vp]),
    "tsp_router_project": (_i, [_vp, _u32, _u32, _vp, _vp, _u64, _u32, _vp, _u64, _vp, _vp, _vp]),
    "tsp_moe_route_audit": (_i, [_vp, _u64, _u32, _u32, _u32, _u32, _i, _vp, _vp, _vp, _vp, _vp]),
    "tsp_router_margin_evaluate": (_i, [_vp, _u32, C.c_float, _vp, C.POINTER(RouterMarginTelemetry), C.POINTER(_i)]),
    "tsp_residual_read": (_i, [_vp, _vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp, _vp]),
    "tsp_residual_write": (_i, [_vp, _vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp]),
    "tsp_rows_f16_to_f32": (_i, [_vp, _u64, _vp, _u64, _u32, _u32, _vp]),
    "tsp_moe_layer_decode": (_i, [C.POINTER(MoeWeights), C.POINTER(MoeScratch), _vp, _u64, _u32, _vp, _u64, _u32, _u32, _u32,
                                  _u32, _u32, _u32, _i, _vp, _u64, _u32, _vp, _vp]),
    "tsp_moe_layer_prefill": (_i, [C.POINTER(MoeWeights), C.POINTER(MoePrefillScratch), _vp, _u64, _u32, _vp, _u64, _u32, _u32, _u32,
                                   _u32, _u32, _u32, _i, _vp, _u64, _u32, _vp, _vp]),
    "tsp_moe_route_offsets": (_i, [_vp, _u32, _vp, _vp]),
    "tsp_moe_rows_f16k": (_i, [_vp, _u64, _u32, _u32, _u32, _vp, _u64, _vp, _vp]),
    "tsp_moe_gather_rows16": (_i, [_vp, _u64, _vp, _vp, _u32, _u32, _u32, _u32, _vp, _u64, _vp]),
    "tsp_moe_grouped_gate_up": (_i, [_MS, _MS, _MS, _MS, _vp, _u64, _vp, _u64, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _u64, _vp, _u64, _vp, _vp]),
    "tsp_moe_grouped_down": (_i, [_MS, _MS, _vp, _u64, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _u64, _u32, _vp, _u64, _u32, _vp, _u64, _vp, _vp]),
    "tsp_dense_mm_swiglu": (_i, [_MS, _MS, _vp, _u64, _u32, _vp, _u64, _vp, _vp, _vp]),
    "tsp_dense_mm": (_i, [_MS, _vp, _u64, _u32, _vp, _u64, _vp, _vp, _vp]),
    "tsp_moe_staged_f16": (_i, [_MS, _u32, _vp, _vp]),
    "tsp_moe_layer_decode_static_bytes": (_u64, [_u32, _u32, _u32, _u32, _u32]),
    "tsp_q8_lanes_unpack": (_i, [_vp, _vp, _u64, _u32, _vp]),
    "tsp_q8_lanes_pack": (_i, [_vp, _vp, _u64, _u32, _vp]),
    "tsp_selftest_bounded_wait": (_i, [_u32, _vp, _vp]),
    "tsp_logit_topk_scratch_bytes": (_u64, [_u32, _u32]),
    "tsp_logit_topk_output_bytes": (_u64, [_u32]),
    "tsp_logit_topk": (_i, [_vp, _u64, _u32, _u32, _vp, _u64, _vp, _u64, _vp]),
    "tsp_moe_layer_decode_static": (_i, [C.POINTER(MoeWeights), _vp, _u64, _u32, _vp, _u64, _u32, _u32, _u32, _u32, _u32, _u32, _i,
                                         _vp, _u64, _u32, _vp, _vp]),
}

_lib = None


def lib() -> C.CDLL:
    """Load libtsp_moe.so (building it first if the sources changed and nvcc is present)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            _build.build()
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build the CUDA library first (python -m tokspur_public_b200.build)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError here = symbol missing from the library
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().tsp_last_error().decode()


def check(rc: int) -> None:
    if rc != 0:
        raise TspError(rc, last_error())


def call(name: str, *args) -> None:
    check(getattr(lib(), name)(*args))
