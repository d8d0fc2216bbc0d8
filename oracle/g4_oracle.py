"""ctypes/numpy front end of the CPU oracle. TEST INFRASTRUCTURE ONLY.

Two interchangeable back ends with the same function set:

* ``load("port")``      -> ``oracle/libg4oracle.so``, the plain-C restatement
  (``g4_oracle.c``), symbols ``g4o_*``;
* ``load("reference")`` -> ``oracle/_ref/libg4ref.so``, the reference engine's own
  host sources behind ``ref_shim.cc``, symbols ``g4ref_*`` (present only where it
  was built next to a reference checkout, or shipped prebuilt).

Only the tests, the smoke check and the CPU-baseline leg of the benchmark import
this module; the product path never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_P = C.c_void_p


def _ptr(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(_P)


def reference_root() -> str | None:
    """Where a checkout of the reference engine lies, if anywhere: $G4_REFERENCE_ROOT, else a
    directory named `reference` beside this repository."""
    for cand in (os.environ.get("G4_REFERENCE_ROOT"),
                 os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "engine", "src", "kernel_math.h")):
            return os.path.abspath(cand)
    return None


def build(ref_root: str | None = None) -> None:
    """(Re)build the port, and the reference-backed library when a reference tree is there."""
    subprocess.run(["make", "-s", "-C", _HERE, "all"], check=True)
    ref_root = ref_root or reference_root()
    if ref_root is not None:
        subprocess.run(["make", "-s", "-C", _HERE, "_ref", f"REF={ref_root}"], check=True)


class Oracle:
    def __init__(self, path: str, prefix: str, kind: str):
        self.kind = kind
        self.path = path
        self._lib = C.CDLL(path)
        self._p = prefix
        f = self._fn
        f("bf16_to_f32", C.c_float, [C.c_uint16])
        f("f32_to_bf16", C.c_uint16, [C.c_float])
        f("fp8_e4m3_encode", C.c_uint8, [C.c_double])
        f("fp8_e4m3_decode", C.c_float, [C.c_uint8])
        f("kv8_scale", C.c_float, [C.c_float])
        f("kv8_quant", C.c_int8, [C.c_float, C.c_float])
        f("kv8_dequant", C.c_float, [C.c_int8, C.c_float])
        f("silu", C.c_float, [C.c_float])
        f("fill_bf16", None, [C.c_uint64, C.c_double, C.c_long, _P])
        f("embed_rows", None, [_P, C.c_long, C.c_long, _P, C.c_float, _P, C.c_int])
        f("add_rmsnorm", None, [_P, C.c_int, _P, C.c_int, _P, C.c_float, C.c_float, C.c_long,
                                C.c_int, _P, _P])
        f("amax_bf16", None, [_P, C.c_long, C.POINTER(C.c_float)])
        f("fp8_scale_from_amax", C.c_float, [C.c_float])
        f("quant_fp8_with_scale", None, [_P, C.c_long, C.c_float, _P])
        f("rope_tables", None, [C.c_double, C.c_int, C.c_long, _P, _P])
        f("rope_rows", None, [_P, _P, _P, C.c_long, C.c_int, _P])
        f("rope_kv_int8", None, [_P, _P, _P, _P, _P, C.c_long, C.c_int, C.c_int, C.c_int,
                                 C.c_long, C.c_int, _P, _P, _P, _P, _P])
        f("kv_append_int8", None, [_P, _P, _P, C.c_long, C.c_int, C.c_int, C.c_long, _P, _P, _P,
                                   _P])
        f("swiglu", None, [_P, _P, C.c_int, C.c_long, C.c_long, C.c_int, _P])
        f("argmax_rows", None, [_P, C.c_long, C.c_int, _P])
        f("attn_decode_int8", None, [_P, _P, _P, _P, _P, _P, _P, C.c_long, C.c_int, C.c_int, C.c_int,
                                     C.c_long, C.c_float, _P])
        f("gemm_fp8", None, [_P, C.c_long, _P, C.c_long, C.c_long, C.c_long, C.c_float, C.c_float, C.c_float,
                             C.c_float, C.c_long, C.c_long, C.c_int, _P, C.c_float, C.c_long, _P, _P])

    def _fn(self, name, res, args):
        fn = getattr(self._lib, self._p + name)
        fn.restype = res
        fn.argtypes = args
        setattr(self, "_c_" + name, fn)

    # ---- scalars -----------------------------------------------------------
    def bf16_to_f32(self, b):
        return float(self._c_bf16_to_f32(int(b)))

    def f32_to_bf16(self, f):
        return int(self._c_f32_to_bf16(float(f)))

    def fp8_encode(self, v):
        return int(self._c_fp8_e4m3_encode(float(v)))

    def fp8_decode(self, c):
        return float(self._c_fp8_e4m3_decode(int(c)))

    def kv8_scale(self, amax):
        return np.float32(self._c_kv8_scale(float(amax)))

    def kv8_quant(self, x, s):
        return int(self._c_kv8_quant(float(x), float(s)))

    def kv8_dequant(self, q, s):
        return np.float32(self._c_kv8_dequant(int(q), float(s)))

    def silu(self, x):
        return np.float32(self._c_silu(float(x)))

    def fill_bf16(self, seed, a, n):
        out = np.empty(n, np.uint16)
        self._c_fill_bf16(seed, a, n, _ptr(out))
        return out

    # ---- ops (numpy in, numpy out) ----------------------------------------------
    def embed_rows(self, tokens, start, rows, emb, mult):
        H = emb.shape[1]
        out = np.empty((rows, H), np.uint16)
        self._c_embed_rows(_ptr(tokens), start, rows, _ptr(emb), mult, _ptr(out), H)
        return out

    def add_rmsnorm(self, y, res, w, eps, rm, want_h=True, want_n=True):
        """y: uint16 (bf16 bits) or float32 [rows][cols]; res: same kinds or None."""
        rows, cols = y.shape
        h = np.empty((rows, cols), np.uint16) if want_h else None
        n = np.empty((rows, cols), np.uint16) if want_n else None
        self._c_add_rmsnorm(_ptr(y), int(y.dtype == np.float32), _ptr(res),
                            int(res is not None and res.dtype == np.float32), _ptr(w), eps, rm,
                            rows, cols, _ptr(h), _ptr(n))
        return h, n

    def amax_bf16(self, v):
        out = C.c_float(0.0)
        self._c_amax_bf16(_ptr(v), v.size, C.byref(out))
        return np.float32(out.value)

    def fp8_scale_from_amax(self, amax):
        return np.float32(self._c_fp8_scale_from_amax(float(amax)))

    def quant_fp8_with_scale(self, v, scale):
        codes = np.empty(v.shape, np.uint8)
        self._c_quant_fp8_with_scale(_ptr(v), v.size, float(scale), _ptr(codes))
        return codes

    def quant_fp8(self, v):
        """Per-tensor quantisation: returns (codes, scale, amax)."""
        amax = self.amax_bf16(v)
        scale = self.fp8_scale_from_amax(amax)
        return self.quant_fp8_with_scale(v, scale), scale, amax

    def rope_tables(self, theta, d, max_pos):
        c = np.empty((max_pos, d // 2), np.float32)
        s = np.empty((max_pos, d // 2), np.float32)
        self._c_rope_tables(theta, d, max_pos, _ptr(c), _ptr(s))
        return c, s

    def rope_rows(self, x, cos_tbl, sin_tbl):
        rows, d = x.shape
        out = np.empty_like(x)
        self._c_rope_rows(_ptr(x), _ptr(cos_tbl), _ptr(sin_tbl), rows, d, _ptr(out))
        return out

    def rope_kv_int8(self, qkv, cos_tbl, sin_tbl, pos_rows, kv_rows, Hq, Hk, d, stride,
                     k_from_bf16, caches=None):
        """Returns (q_rot, cache_k, cache_v, k_scale, v_scale); caches are created zeroed
        ([Hk][stride][d] int8, [Hk][stride] f32) unless passed in."""
        rows = qkv.shape[0]
        q_rot = np.empty((rows, Hq * d), np.uint16)
        if caches is None:
            ck = np.zeros((Hk, stride, d), np.int8)
            cv = np.zeros((Hk, stride, d), np.int8)
            ks = np.zeros((Hk, stride), np.float32)
            vs = np.zeros((Hk, stride), np.float32)
        else:
            ck, cv, ks, vs = caches
        self._c_rope_kv_int8(_ptr(qkv), _ptr(cos_tbl), _ptr(sin_tbl),
                             _ptr(np.ascontiguousarray(pos_rows, np.int32)),
                             _ptr(np.ascontiguousarray(kv_rows, np.int32)), rows, Hq, Hk, d,
                             stride, int(k_from_bf16), _ptr(q_rot), _ptr(ck), _ptr(cv), _ptr(ks),
                             _ptr(vs))
        return q_rot, ck, cv, ks, vs

    def kv_append_int8(self, src_k, src_v, kv_rows, Hk, d, stride):
        rows = src_k.shape[0]
        ck = np.zeros((Hk, stride, d), np.int8)
        cv = np.zeros((Hk, stride, d), np.int8)
        ks = np.zeros((Hk, stride), np.float32)
        vs = np.zeros((Hk, stride), np.float32)
        self._c_kv_append_int8(_ptr(src_k), _ptr(src_v),
                               _ptr(np.ascontiguousarray(kv_rows, np.int32)), rows, Hk, d, stride,
                               _ptr(ck), _ptr(cv), _ptr(ks), _ptr(vs))
        return ck, cv, ks, vs

    def swiglu(self, gate, up):
        """gate, up: uint16 (bf16 bits) or float32, [rows][I] views of equal row pitch."""
        rows, I = gate.shape
        assert gate.strides == up.strides and gate.strides[1] == gate.itemsize
        ld = gate.strides[0] // gate.itemsize
        act = np.empty((rows, I), np.uint16)
        self._c_swiglu(C.c_void_p(gate.ctypes.data), C.c_void_p(up.ctypes.data),
                       int(gate.dtype == np.float32), ld, rows, I, _ptr(act))
        return act

    def argmax_rows(self, logits):
        """bf16 logits [rows][V] (no NaN) -> int32 [rows], first index of each row's maximum."""
        rows, V = logits.shape
        out = np.empty(rows, np.int32)
        self._c_argmax_rows(_ptr(np.ascontiguousarray(logits)), rows, V, _ptr(out))
        return out

    def attn_decode_int8(self, q, ck, cv, ks, vs, row_pos, row_tables, Hq, Hk, d, scale):
        """q [rows][Hq d] bf16 bits; pool codes [Hk][stride][d] int8 + scales [Hk][stride];
        row_tables: None (identity) or a list of int32 arrays, one position -> pool row table
        per query row. Returns out [rows][Hq d] bf16 bits (golden bf16 pipeline)."""
        rows = q.shape[0]
        stride = ck.shape[1]
        out = np.empty((rows, Hq * d), np.uint16)
        pos = np.ascontiguousarray(row_pos, np.int32)
        if row_tables is None:
            tables = None
        else:
            keep = [np.ascontiguousarray(t, np.int32) for t in row_tables]
            tables = (C.c_void_p * rows)(*[t.ctypes.data for t in keep])
        self._c_attn_decode_int8(_ptr(q), _ptr(ck), _ptr(cv), _ptr(ks), _ptr(vs), _ptr(pos), tables,
                                 rows, Hq, Hk, d, stride, scale, _ptr(out))
        return out

    def gemm_fp8(self, a, w, a_scale=1.0, w_scales=(1.0,), segs=(), kind="bf16", residual=None,
                 resid_scale=1.0):
        """a [M][K], w [N][K] e4m3 codes (uint8). kind "bf16" / "f32"; a bf16-bits residual [M][N]
        selects bf16(residual + resid_scale * y). Returns [M][N] bf16 bits or float32."""
        a, w = np.ascontiguousarray(a, np.uint8), np.ascontiguousarray(w, np.uint8)
        (M, K), N = a.shape, w.shape[0]
        ws = list(w_scales) + [w_scales[-1]] * (3 - len(w_scales))
        sg = list(segs) + [2 ** 31 - 1] * (2 - len(segs))
        out_kind = 1 if kind == "f32" else (0 if residual is None else 2)
        out = np.empty((M, N), np.float32 if kind == "f32" else np.uint16)
        res = None if residual is None else np.ascontiguousarray(residual, np.uint16)
        self._c_gemm_fp8(_ptr(a), K, _ptr(w), M, N, K, a_scale, ws[0], ws[1], ws[2], sg[0], sg[1], out_kind,
                         None if res is None else _ptr(res), resid_scale, N,
                         _ptr(out) if kind != "f32" else None, _ptr(out) if kind == "f32" else None)
        return out

    # ---- the whole per-layer glue sequence over a slice of rows, for timing ---------
    def layer_glue(self, y_attn, y_mlp, res, w1, w2, qkv, gate, up, cos_tbl, sin_tbl, pos_rows,
                   kv_rows, caches, eps, rm, Hq, Hk, d, stride):
        """One layer: add+norm(+fp8), rope+KV, add+norm(+fp8), SwiGLU(+fp8). Returns the
        per-shard outputs; used by the CPU baseline (rows split over threads)."""
        h1, n1 = self.add_rmsnorm(y_attn, res, w1, eps, rm)
        c1 = self.quant_fp8(n1)
        rk = self.rope_kv_int8(qkv, cos_tbl, sin_tbl, pos_rows, kv_rows, Hq, Hk, d, stride, 0,
                               caches)
        h2, n2 = self.add_rmsnorm(y_mlp, h1, w2, eps, rm)
        c2 = self.quant_fp8(n2)
        act = self.swiglu(gate, up)
        c3 = self.quant_fp8(act)
        return h2, c1, c2, c3, rk[0]


def parallel_rows(fn, rows: int, threads: int):
    """Run fn(lo, hi) over `threads` contiguous row ranges concurrently (ctypes drops the GIL)."""
    threads = max(1, min(threads, rows))
    bounds = [(rows * t // threads, rows * (t + 1) // threads) for t in range(threads)]
    with ThreadPoolExecutor(max_workers=threads) as ex:
        return list(ex.map(lambda b: fn(*b), bounds))


_PATHS = {
    "port": (os.path.join(_HERE, "libg4oracle.so"), "g4o_"),
    "reference": (os.path.join(_HERE, "_ref", "libg4ref.so"), "g4ref_"),
}


def available(kind: str) -> bool:
    return os.path.isfile(_PATHS[kind][0])


def load(kind: str = "port") -> Oracle:
    path, prefix = _PATHS[kind]
    if kind == "port" and not os.path.isfile(path):
        build()
    if not os.path.isfile(path):
        raise FileNotFoundError(f"oracle library missing: {path} (run make -C oracle)")
    return Oracle(path, prefix, kind)
