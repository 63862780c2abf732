"""ctypes bindings for the CPU checkers. TEST INFRASTRUCTURE ONLY.

`Oracle()` binds the plain-C restatement (liboracle.so, built from tsp_oracle.c);
`Oracle(reference=True)` binds the reference's own CPU sources compiled into
_ref/libtokspur_ref.so (same call signatures, `ref_` prefix). Only the test-suite, the
smoke check and the benchmark's CPU-baseline / reference arms import this module; the
product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libtokspur_ref.so")

u8p = C.POINTER(C.c_uint8)
u32p = C.POINTER(C.c_uint32)
f32p = C.POINTER(C.c_float)
f64p = C.POINTER(C.c_double)


def build(reference_root: str = "/root/reference") -> None:
    """Compile liboracle.so, and _ref/ when the reference tree is present."""
    subprocess.run(["make", "-s", "-C", HERE, f"REF={reference_root}"], check=True)


def have_reference() -> bool:
    return os.path.exists(REF_SO)


def _ptr(a, t):
    return a.ctypes.data_as(t) if a is not None else None


class _Layer(C.Structure):
    _fields_ = [("channels", C.c_uint32), ("hidden", C.c_uint32), ("experts", C.c_uint32), ("selected", C.c_uint32),
                ("expert_type", C.c_uint32), ("shared_type", C.c_uint32),
                ("gate", u8p), ("up", u8p), ("down", u8p), ("shared_gate", u8p), ("shared_up", u8p), ("shared_down", u8p),
                ("shared_router", f32p), ("router", f32p), ("mode", C.c_uint32), ("normalize_selected", C.c_int),
                ("down_type", C.c_uint32)]


class _Stages(C.Structure):
    _fields_ = [("indices", u32p), ("weights", f64p), ("activated", f64p), ("routed", f64p),
                ("shared_act", f64p), ("shared_out", f64p), ("shared_logit", f64p)]


class _Spec(C.Structure):
    _fields_ = [("source_type", C.c_uint32), ("columns", C.c_uint32), ("rows", C.c_uint32), ("blocks_per_row", C.c_uint32),
                ("source_row_bytes", C.c_uint64), ("planar_row_bytes", C.c_uint64),
                ("source_expert_bytes", C.c_uint64), ("planar_expert_bytes", C.c_uint64),
                ("qs_offset", C.c_uint64), ("sm_offset", C.c_uint64), ("dm_offset", C.c_uint64), ("qh_offset", C.c_uint64)]


class OracleError(RuntimeError):
    def __init__(self, code):
        super().__init__(f"oracle refused the input (code {code})")
        self.code = code


class Oracle:
    def __init__(self, reference: bool = False):
        self.reference = reference
        path = REF_SO if reference else PORT_SO
        if not os.path.exists(path):
            if reference:
                raise FileNotFoundError(path)
            build()
        self.lib = C.CDLL(path)
        self.p = "ref_" if reference else "tso_"
        L = self.lib
        f = lambda name: getattr(L, self.p + name)
        f("binary16").restype = C.c_float
        f("binary16").argtypes = [C.c_uint16]
        for n in ("sigmoid", "silu", "softplus"):
            f(n).restype = C.c_double
            f(n).argtypes = [C.c_double]
        f("dequantize").argtypes = [C.c_uint32, u8p, C.c_size_t, f32p, C.c_size_t]
        f("gemv_f64").argtypes = [C.c_uint32, u8p, C.c_size_t, C.c_uint32, C.c_uint32, f64p, f64p]
        f("gemv_f32").argtypes = [C.c_uint32, u8p, C.c_size_t, C.c_uint32, C.c_uint32, f32p, f64p]
        f("route").argtypes = [f64p, C.c_size_t, C.c_size_t, C.c_uint32, C.c_int, u32p, f64p]
        f("mixture").argtypes = [f64p, f64p, C.c_size_t, f64p, C.c_size_t, C.c_double, f64p]
        f("gated_residual").argtypes = [f64p, f64p, f64p, f64p, f64p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_double, f64p, f64p, f64p, f64p, f64p]
        f("residual_write").argtypes = [f64p, f64p, f64p, C.c_size_t, C.c_size_t, f64p]
        if reference:
            L.ref_moe_layer.argtypes = [C.POINTER(_Layer), f32p, f32p, C.c_uint32, f64p, u32p, C.c_uint32]
        else:
            L.tso_moe_layer.argtypes = [C.POINTER(_Layer), f32p, f32p, C.c_uint32, f64p, C.POINTER(_Stages), C.c_uint32]
            L.tso_make_expert_spec.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(_Spec)]
            L.tso_pack_sm16.argtypes = [u8p, u8p]
            L.tso_pack_sm16.restype = None
            L.tso_unpack_sm16.argtypes = [u8p, u8p]
            L.tso_pack_expert_planar.argtypes = [C.POINTER(_Spec), u8p, u8p]
            L.tso_unpack_expert_planar.argtypes = [C.POINTER(_Spec), u8p, u8p]
            L.tso_dequantize_expert_planar.argtypes = [C.POINTER(_Spec), u8p, f32p]
            L.tso_grouped_routes.argtypes = [u32p, C.c_uint32, C.c_uint32, C.c_uint32, u32p, u32p]
            L.tso_grouped_tasks.argtypes = [u32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, u32p]
            L.tso_value.restype = C.c_double
            L.tso_value.argtypes = [C.c_uint32, u8p, C.c_uint32]

    def _f(self, name):
        return getattr(self.lib, self.p + name)

    @staticmethod
    def _ok(rc):
        if rc:
            raise OracleError(rc)

    # ---- numeric ----
    def binary16(self, bits: int) -> float:
        return self._f("binary16")(bits)

    def binary16_all(self) -> np.ndarray:
        return np.array([self.binary16(b) for b in range(65536)], dtype=np.float32)

    def sigmoid(self, v): return self._f("sigmoid")(v)
    def silu(self, v): return self._f("silu")(v)
    def softplus(self, v): return self._f("softplus")(v)

    def dequantize(self, type_: int, data: np.ndarray, elements: int) -> np.ndarray:
        data = np.ascontiguousarray(data, dtype=np.uint8)
        out = np.empty(elements, dtype=np.float32)
        self._ok(self._f("dequantize")(type_, _ptr(data, u8p), data.size, _ptr(out, f32p), elements))
        return out

    def gemv(self, type_: int, matrix: np.ndarray, columns: int, rows: int, x: np.ndarray) -> np.ndarray:
        matrix = np.ascontiguousarray(matrix, dtype=np.uint8)
        out = np.empty(rows, dtype=np.float64)
        if x.dtype == np.float32:
            x = np.ascontiguousarray(x)
            self._ok(self._f("gemv_f32")(type_, _ptr(matrix, u8p), matrix.size, columns, rows, _ptr(x, f32p), _ptr(out, f64p)))
        else:
            x = np.ascontiguousarray(x, dtype=np.float64)
            self._ok(self._f("gemv_f64")(type_, _ptr(matrix, u8p), matrix.size, columns, rows, _ptr(x, f64p), _ptr(out, f64p)))
        return out

    # ---- routing ----
    def route(self, logits: np.ndarray, selected: int, mode: int = 0, normalize: bool = True):
        logits = np.ascontiguousarray(logits, dtype=np.float64)
        ids = np.empty(selected, dtype=np.uint32)
        w = np.empty(selected, dtype=np.float64)
        self._ok(self._f("route")(_ptr(logits, f64p), logits.size, selected, mode, int(normalize), _ptr(ids, u32p), _ptr(w, f64p)))
        return ids, w

    def route_rows(self, logits: np.ndarray, selected: int, mode: int = 0, normalize: bool = True):
        ids = np.empty((logits.shape[0], selected), dtype=np.uint32)
        w = np.empty((logits.shape[0], selected), dtype=np.float64)
        for t in range(logits.shape[0]):
            ids[t], w[t] = self.route(logits[t], selected, mode, normalize)
        return ids, w

    def lanes_pack_rows(self, type_: int, columns: int, original: np.ndarray, unpack: bool = False) -> np.ndarray:
        """Whole rows of GGUF blocks -> lane layout (`q8_lanes_v1` for Q8_0), or back with unpack=True. Lossless."""
        src = np.ascontiguousarray(original, dtype=np.uint8).reshape(-1)
        out = np.empty_like(src)
        fn = self._f("lanes_unpack_rows" if unpack else "lanes_pack_rows")
        fn.argtypes = [C.c_uint32, C.c_uint32, u8p, u8p, C.c_size_t]
        self._ok(fn(type_, columns, _ptr(src, u8p), _ptr(out, u8p), src.size))
        return out

    def logit_topk_row(self, logits: np.ndarray):
        """Top-64 row of the sampler (port only: the reference's sampling.cpp needs arm_neon.h and does not build here).
        Returns a dict: vocabulary, count, first_nonfinite_col, first_subnormal_col, ids [64] uint32, logits [64] float32."""
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        raw = np.zeros(132, dtype=np.uint32)   # 528 bytes
        self.lib.tso_logit_topk_row.argtypes = [f32p, C.c_size_t, u32p]
        self._ok(self.lib.tso_logit_topk_row(_ptr(logits, f32p), logits.size, _ptr(raw, u32p)))
        return {"vocabulary": int(raw[0]), "count": int(raw[1]), "first_nonfinite_col": int(raw[2]), "first_subnormal_col": int(raw[3]),
                "ids": raw[4:68].copy(), "logits": raw[68:132].view(np.float32).copy()}

    def mixture(self, experts: np.ndarray, weights: np.ndarray, shared: np.ndarray, shared_logit: float) -> np.ndarray:
        experts = np.ascontiguousarray(experts, dtype=np.float64)
        weights = np.ascontiguousarray(weights, dtype=np.float64)
        shared = np.ascontiguousarray(shared, dtype=np.float64)
        out = np.empty(shared.size, dtype=np.float64)
        self._ok(self._f("mixture")(_ptr(experts, f64p), _ptr(weights, f64p), weights.size, _ptr(shared, f64p), shared.size,
                                    float(shared_logit), _ptr(out, f64p)))
        return out

    def gated_residual(self, streams, gains, down, up, inject, rank: int, epsilon: float, intermediates: bool = False):
        """Hyper-connection residual read: streams/gains [branches, channels], down [rank, branches*channels],
        up [branches*channels, rank], inject [branches, branches*channels] -> (input [channels], write_scales [branches])."""
        streams = np.ascontiguousarray(streams, dtype=np.float64)
        branches, channels = streams.shape
        a = [np.ascontiguousarray(v, dtype=np.float64) for v in (gains, down, up, inject)]
        inp, scales = np.empty(channels), np.empty(branches)
        norm, scores, logits = (np.empty((branches, channels)), np.empty((branches, channels)), np.empty(branches)) if intermediates and not self.reference else (None, None, None)
        self._ok(self._f("gated_residual")(_ptr(streams, f64p), _ptr(a[0], f64p), _ptr(a[1], f64p), _ptr(a[2], f64p), _ptr(a[3], f64p), branches,
                                           channels, rank, float(epsilon), _ptr(inp, f64p), _ptr(scales, f64p), _ptr(norm, f64p),
                                           _ptr(scores, f64p), _ptr(logits, f64p)))
        return (inp, scales, norm, scores, logits) if intermediates else (inp, scales)

    def residual_write(self, streams, output, scales):
        streams = np.ascontiguousarray(streams, dtype=np.float64)
        branches, channels = streams.shape
        out = np.empty_like(streams)
        self._ok(self._f("residual_write")(_ptr(streams, f64p), _ptr(np.ascontiguousarray(output, dtype=np.float64), f64p),
                                           _ptr(np.ascontiguousarray(scales, dtype=np.float64), f64p), branches, channels, _ptr(out, f64p)))
        return out

    # ---- planar (port only) ----
    def spec(self, type_: int, columns: int, rows: int) -> _Spec:
        s = _Spec()
        self._ok(self.lib.tso_make_expert_spec(type_, columns, rows, C.byref(s)))
        return s

    def pack_sm16(self, s12: np.ndarray) -> np.ndarray:
        s12 = np.ascontiguousarray(s12, dtype=np.uint8)
        out = np.empty(16, dtype=np.uint8)
        self.lib.tso_pack_sm16(_ptr(s12, u8p), _ptr(out, u8p))
        return out

    def unpack_sm16(self, sm: np.ndarray) -> np.ndarray:
        sm = np.ascontiguousarray(sm, dtype=np.uint8)
        out = np.empty(12, dtype=np.uint8)
        self._ok(self.lib.tso_unpack_sm16(_ptr(sm, u8p), _ptr(out, u8p)))
        return out

    def pack_expert(self, spec: _Spec, gguf: np.ndarray) -> np.ndarray:
        gguf = np.ascontiguousarray(gguf, dtype=np.uint8)
        assert gguf.size == spec.source_expert_bytes
        out = np.empty(spec.planar_expert_bytes, dtype=np.uint8)
        self._ok(self.lib.tso_pack_expert_planar(C.byref(spec), _ptr(gguf, u8p), _ptr(out, u8p)))
        return out

    def unpack_expert(self, spec: _Spec, planar: np.ndarray) -> np.ndarray:
        planar = np.ascontiguousarray(planar, dtype=np.uint8)
        assert planar.size == spec.planar_expert_bytes
        out = np.empty(spec.source_expert_bytes, dtype=np.uint8)
        self._ok(self.lib.tso_unpack_expert_planar(C.byref(spec), _ptr(planar, u8p), _ptr(out, u8p)))
        return out

    def dequantize_planar(self, spec: _Spec, planar: np.ndarray) -> np.ndarray:
        planar = np.ascontiguousarray(planar, dtype=np.uint8)
        assert planar.size == spec.planar_expert_bytes
        out = np.empty(spec.rows * spec.columns, dtype=np.float32)
        self._ok(self.lib.tso_dequantize_expert_planar(C.byref(spec), _ptr(planar, u8p), _ptr(out, f32p)))
        return out

    # ---- permutation (port only) ----
    def grouped_routes(self, indices: np.ndarray, experts: int):
        indices = np.ascontiguousarray(indices, dtype=np.uint32)
        tokens, selected = indices.shape
        token_map = np.full((experts, tokens), 0xFFFFFFFF, dtype=np.uint32)
        counts = np.zeros(experts, dtype=np.uint32)
        self._ok(self.lib.tso_grouped_routes(_ptr(indices, u32p), tokens, experts, selected, _ptr(token_map, u32p), _ptr(counts, u32p)))
        return token_map, counts

    def grouped_tasks(self, counts: np.ndarray, tokens: int, selected: int, tile: int = 32):
        counts = np.ascontiguousarray(counts, dtype=np.uint32)
        experts = counts.size
        tasks = np.zeros(2 + 2 * (tokens * selected // tile + experts), dtype=np.uint32)
        self._ok(self.lib.tso_grouped_tasks(_ptr(counts, u32p), tokens, experts, selected, tile, _ptr(tasks, u32p)))
        return tasks

    # ---- whole layer ----
    def moe_layer(self, layer: dict, x: np.ndarray, logits: np.ndarray | None, threads: int = 1, stages: bool = False):
        """layer: dict with channels, hidden, experts, selected, expert_type, shared_type (and optionally down_type), gate, up, down,
        shared_gate, shared_up, shared_down (uint8 arrays, GGUF layout), shared_router (f32 or None),
        router (f32 or None), mode, normalize. Returns out [T,C] float64 (and a dict of stages)."""
        keep = []

        def b(name):
            a = np.ascontiguousarray(layer[name], dtype=np.uint8)
            keep.append(a)
            return _ptr(a, u8p)

        def fl(name):
            if layer.get(name) is None:
                return None
            a = np.ascontiguousarray(layer[name], dtype=np.float32)
            keep.append(a)
            return _ptr(a, f32p)

        Ls = _Layer(layer["channels"], layer["hidden"], layer["experts"], layer["selected"],
                    layer["expert_type"], layer["shared_type"], b("gate"), b("up"), b("down"),
                    b("shared_gate"), b("shared_up"), b("shared_down"), fl("shared_router"), fl("router"),
                    layer.get("mode", 0), int(layer.get("normalize", True)), int(layer.get("down_type") or 0))
        x = np.ascontiguousarray(x, dtype=np.float32)
        T, Cn = x.shape
        lg = np.ascontiguousarray(logits, dtype=np.float32) if logits is not None else None
        out = np.empty((T, Cn), dtype=np.float64)
        K, H = layer["selected"], layer["hidden"]
        if self.reference:
            ids = np.empty((T, K), dtype=np.uint32)
            self._ok(self.lib.ref_moe_layer(C.byref(Ls), _ptr(x, f32p), _ptr(lg, f32p), T, _ptr(out, f64p), _ptr(ids, u32p), threads))
            return (out, {"indices": ids}) if stages else out
        st = None
        sd = {}
        if stages:
            sd = {"indices": np.empty((T, K), np.uint32), "weights": np.empty((T, K)), "activated": np.empty((T, K, H)),
                  "routed": np.empty((T, K, Cn)), "shared_act": np.empty((T, H)), "shared_out": np.empty((T, Cn)),
                  "shared_logit": np.empty(T)}
            st = _Stages(_ptr(sd["indices"], u32p), *[_ptr(sd[k], f64p) for k in
                         ("weights", "activated", "routed", "shared_act", "shared_out", "shared_logit")])
        self._ok(self.lib.tso_moe_layer(C.byref(Ls), _ptr(x, f32p), _ptr(lg, f32p), T, _ptr(out, f64p),
                                        C.byref(st) if st is not None else None, threads))
        return (out, sd) if stages else out
