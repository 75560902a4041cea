"""ctypes bindings for the CPU oracle and for the in-place build of the reference helpers.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by the CPU-baseline leg of
bench.py.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libnihilus_ref.so")

QK = 32
BLOCK_BYTES = 34

# enum orc_mode
Q8ACT_LANES, Q8ACT_SCALAR, Q8ACT_CHUNK16, F32ACT_EVAL, F32ACT_PROMPT, Q8ACT_F64, F32ACT_F64 = range(7)

_c_f32p = C.POINTER(C.c_float)
_c_u8p = C.POINTER(C.c_uint8)


def reference_root() -> str:
    """Where the reference's source tree lies: $NIHILUS_REFERENCE, else `reference_path` of BASELINE.json beside this
    package, else nowhere (the prebuilt oracle/_ref is then used as it is)."""
    env = os.environ.get("NIHILUS_REFERENCE")
    if env:
        return env
    try:
        import json

        with open(os.path.join(HERE, "..", "BASELINE.json")) as f:
            return str(json.load(f).get("reference_path") or "")
    except (OSError, ValueError):
        return ""


def build(force: bool = False) -> None:
    """Compile liboracle.so (and oracle/_ref when the reference tree is present)."""
    src_m = max(os.path.getmtime(os.path.join(HERE, f)) for f in ("q8_oracle.c", "q8_oracle.h"))
    if force or not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < src_m:
        subprocess.run(["make", "-C", HERE, "liboracle.so"], check=True, capture_output=True)
    ref = reference_root()
    if ref and os.path.isdir(os.path.join(ref, "include", "nihilus-incl")):
        shim_m = max(os.path.getmtime(os.path.join(HERE, f)) for f in ("ref_prelude.hpp", "ref_postlude.cpp", "build_ref.sh"))
        if force or not os.path.exists(REF_SO) or os.path.getmtime(REF_SO) < shim_m:
            subprocess.run(["make", "-C", HERE, "ref", "REF=" + ref], check=True, capture_output=True)


def _ptr(a: np.ndarray, typ):
    return a.ctypes.data_as(typ)


class Oracle:
    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build()
        self.lib = L = C.CDLL(path)
        L.orc_fp32_to_fp16.restype = C.c_uint16
        L.orc_fp32_to_fp16.argtypes = [C.c_float]
        L.orc_fp32_to_fp16_bittrick.restype = C.c_uint16
        L.orc_fp32_to_fp16_bittrick.argtypes = [C.c_float]
        L.orc_fp16_to_fp32.restype = C.c_float
        L.orc_fp16_to_fp32.argtypes = [C.c_uint16]
        L.orc_quantize_row_q8_0.restype = None
        L.orc_quantize_row_q8_0.argtypes = [_c_f32p, _c_u8p, C.c_int64]
        L.orc_vec_dot_q8_0_q8_0.restype = C.c_float
        L.orc_vec_dot_q8_0_q8_0.argtypes = [C.c_int, _c_u8p, _c_u8p, C.c_int64]
        L.orc_vec_dot_q8_f32.restype = C.c_float
        L.orc_vec_dot_q8_f32.argtypes = [C.c_int, _c_u8p, _c_f32p, C.c_int64]
        L.orc_mul_mat_q8_0.restype = C.c_int
        L.orc_mul_mat_q8_0.argtypes = [C.c_int, _c_u8p, C.c_int64, C.c_int64, _c_f32p, C.c_int64, C.c_int64, _c_f32p, C.c_int64,
                                       C.c_int64, C.c_int64, C.c_int]
        L.orc_mul_mat_block_dots.restype = C.c_int
        L.orc_mul_mat_block_dots.argtypes = [_c_u8p, C.c_int64, C.c_int64, _c_f32p, C.c_int64, C.c_int64, C.POINTER(C.c_int32), C.c_int]
        L.orc_repack_planes.restype = None
        L.orc_repack_planes.argtypes = [_c_u8p, C.c_int64, C.c_int64, C.c_int64, C.POINTER(C.c_int8), C.POINTER(C.c_uint16)]
        L.orc_unpack_planes.restype = None
        L.orc_unpack_planes.argtypes = [C.POINTER(C.c_int8), C.POINTER(C.c_uint16), C.c_int64, C.c_int64, _c_u8p]
        L.orc_quantize_matrix_q8_0.restype = None
        L.orc_quantize_matrix_q8_0.argtypes = [_c_f32p, C.c_int64, C.c_int64, _c_u8p, C.c_int]
        for name in ("orc_swiglu", "orc_swiglu_f64", "orc_add"):
            getattr(L, name).restype = None
            getattr(L, name).argtypes = [_c_f32p, _c_f32p, _c_f32p, C.c_int64]
        L.orc_get_rows_q8_0.restype = C.c_int
        L.orc_get_rows_q8_0.argtypes = [_c_u8p, C.c_int64, C.c_int64, C.POINTER(C.c_int32), C.c_int64, _c_f32p, C.c_int64]
        L.orc_sum_squares.restype = C.c_float
        L.orc_sum_squares.argtypes = [_c_f32p, C.c_int64]
        L.orc_sqrtf_fast.restype = C.c_float
        L.orc_sqrtf_fast.argtypes = [C.c_float]
        L.orc_rms_norm_mul.restype = C.c_int
        L.orc_rms_norm_mul.argtypes = [_c_f32p, C.c_int64, _c_f32p, C.c_float, C.c_int, _c_f32p, C.c_int64, C.c_int64, C.c_int64]
        L.orc_rms_norm_mul_q8_0.restype = C.c_int
        L.orc_rms_norm_mul_q8_0.argtypes = [_c_f32p, C.c_int64, _c_f32p, C.c_float, C.c_int, _c_u8p, C.c_int64, C.c_int64]

    # scalars
    def fp32_to_fp16(self, f: float) -> int:
        return int(self.lib.orc_fp32_to_fp16(f))

    # element-wise neighbours of the mul_mats
    def swiglu(self, g: np.ndarray, u: np.ndarray, f64: bool = False) -> np.ndarray:
        g = np.ascontiguousarray(g, dtype=np.float32)
        u = np.ascontiguousarray(u, dtype=np.float32)
        h = np.empty_like(g)
        fn = self.lib.orc_swiglu_f64 if f64 else self.lib.orc_swiglu
        fn(_ptr(g, _c_f32p), _ptr(u, _c_f32p), _ptr(h, _c_f32p), g.size)
        return h

    def get_rows(self, table: np.ndarray, ids: np.ndarray) -> np.ndarray:
        """table: uint8 [N, K/32, 34]; ids: int32 [M] -> f32 [M, K]."""
        table = np.ascontiguousarray(table, dtype=np.uint8)
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        N, nb, _ = table.shape
        y = np.zeros((ids.size, nb * QK), dtype=np.float32)
        rc = self.lib.orc_get_rows_q8_0(_ptr(table, _c_u8p), N, nb * QK, _ptr(ids, C.POINTER(C.c_int32)), ids.size, _ptr(y, _c_f32p), nb * QK)
        if rc != 0:
            raise ValueError("orc_get_rows_q8_0: token id outside the table")
        return y

    def add(self, a: np.ndarray, b: np.ndarray) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        y = np.empty_like(a)
        self.lib.orc_add(_ptr(a, _c_f32p), _ptr(b, _c_f32p), _ptr(y, _c_f32p), a.size)
        return y

    def fp32_to_fp16_bittrick(self, f: float) -> int:
        return int(self.lib.orc_fp32_to_fp16_bittrick(f))

    def fp16_to_fp32(self, h: int) -> float:
        return float(self.lib.orc_fp16_to_fp32(h))

    def quantize_rows(self, x: np.ndarray, threads: int = 1) -> np.ndarray:
        """f32 [rows, K] -> uint8 [rows, K/32, 34] Q8_0 blocks."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        rows, K = x.shape
        assert K % QK == 0
        out = np.empty((rows, K // QK, BLOCK_BYTES), dtype=np.uint8)
        self.lib.orc_quantize_matrix_q8_0(_ptr(x, _c_f32p), rows, K, _ptr(out, _c_u8p), threads)
        return out

    def vec_dot_q8q8(self, mode: int, w: np.ndarray, a: np.ndarray) -> float:
        nb = w.size // BLOCK_BYTES
        return float(self.lib.orc_vec_dot_q8_0_q8_0(mode, _ptr(w, _c_u8p), _ptr(a, _c_u8p), nb))

    def vec_dot_q8f32(self, mode: int, w: np.ndarray, x: np.ndarray) -> float:
        nb = w.size // BLOCK_BYTES
        return float(self.lib.orc_vec_dot_q8_f32(mode, _ptr(w, _c_u8p), _ptr(x, _c_f32p), nb))

    def mul_mat(self, mode: int, w: np.ndarray, x: np.ndarray, n0: int = 0, n1: int | None = None, threads: int = 0) -> np.ndarray:
        """w: uint8 [N, K/32, 34]; x: f32 [M, K] -> y f32 [M, N] (rows outside [n0, n1) stay 0)."""
        w = np.ascontiguousarray(w, dtype=np.uint8)
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        N, nb, _ = w.shape
        M, K = x.shape
        assert K == nb * QK
        y = np.zeros((M, N), dtype=np.float32)
        n1 = N if n1 is None else n1
        rc = self.lib.orc_mul_mat_q8_0(mode, _ptr(w, _c_u8p), N, K, _ptr(x, _c_f32p), K, M, _ptr(y, _c_f32p), max(N, 1), n0, n1,
                                       threads or (os.cpu_count() or 1))
        if rc != 0:
            raise ValueError("orc_mul_mat_q8_0: bad arguments")
        return y

    def block_dots(self, w: np.ndarray, x: np.ndarray, threads: int = 0) -> np.ndarray:
        w = np.ascontiguousarray(w, dtype=np.uint8)
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        N, nb, _ = w.shape
        M, K = x.shape
        out = np.zeros((M, N, nb), dtype=np.int32)
        rc = self.lib.orc_mul_mat_block_dots(_ptr(w, _c_u8p), N, K, _ptr(x, _c_f32p), K, M, _ptr(out, C.POINTER(C.c_int32)),
                                             threads or (os.cpu_count() or 1))
        if rc != 0:
            raise ValueError("orc_mul_mat_block_dots: bad arguments")
        return out

    def repack(self, w: np.ndarray, n0: int = 0, n1: int | None = None):
        w = np.ascontiguousarray(w, dtype=np.uint8)
        N, nb, _ = w.shape
        n1 = N if n1 is None else n1
        q = np.empty((n1 - n0, nb * QK), dtype=np.int8)
        d = np.empty((n1 - n0, nb), dtype=np.uint16)
        self.lib.orc_repack_planes(_ptr(w, _c_u8p), nb * QK, n0, n1, _ptr(q, C.POINTER(C.c_int8)), _ptr(d, C.POINTER(C.c_uint16)))
        return q, d

    def unpack(self, q: np.ndarray, d: np.ndarray) -> np.ndarray:
        rows, K = q.shape
        out = np.empty((rows, K // QK, BLOCK_BYTES), dtype=np.uint8)
        self.lib.orc_unpack_planes(_ptr(np.ascontiguousarray(q), C.POINTER(C.c_int8)), _ptr(np.ascontiguousarray(d), C.POINTER(C.c_uint16)),
                                   K, rows, _ptr(out, _c_u8p))
        return out

    # rms_norm x norm-weight
    def sum_squares(self, x: np.ndarray) -> float:
        x = np.ascontiguousarray(x, dtype=np.float32)
        return float(self.lib.orc_sum_squares(_ptr(x, _c_f32p), x.size))

    def sqrtf_fast(self, v: float) -> float:
        return float(self.lib.orc_sqrtf_fast(v))

    def rms_norm_mul(self, x: np.ndarray, w: np.ndarray, eps: float, sqrt_mode: int = 0) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        M, K = x.shape
        y = np.empty((M, K), dtype=np.float32)
        rc = self.lib.orc_rms_norm_mul(_ptr(x, _c_f32p), K, _ptr(w, _c_f32p), eps, sqrt_mode, _ptr(y, _c_f32p), K, M, K)
        if rc != 0:
            raise ValueError(f"orc_rms_norm_mul rc={rc}")
        return y

    def rms_norm_mul_q8_0(self, x: np.ndarray, w: np.ndarray, eps: float, sqrt_mode: int = 0) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        M, K = x.shape
        out = np.empty((M, K // QK, BLOCK_BYTES), dtype=np.uint8)
        rc = self.lib.orc_rms_norm_mul_q8_0(_ptr(x, _c_f32p), K, _ptr(w, _c_f32p), eps, sqrt_mode, _ptr(out, _c_u8p), M, K)
        if rc != 0:
            raise ValueError(f"orc_rms_norm_mul_q8_0 rc={rc}")
        return out


class Reference:
    """The reference's own helper functions, compiled in place into oracle/_ref/ (may be absent)."""

    def __init__(self, path: str = REF_SO):
        self.lib = L = C.CDLL(path)
        L.ref_fp32_to_fp16.restype = C.c_uint16
        L.ref_fp32_to_fp16.argtypes = [C.c_float]
        L.ref_fp32_to_fp16_bittrick.restype = C.c_uint16
        L.ref_fp32_to_fp16_bittrick.argtypes = [C.c_float]
        L.ref_fp16_to_fp32.restype = C.c_float
        L.ref_fp16_to_fp32.argtypes = [C.c_uint16]
        L.ref_quantize_row_q8_0.restype = None
        L.ref_quantize_row_q8_0.argtypes = [_c_f32p, C.c_void_p, C.c_int64]
        for name in ("ref_vec_dot_q8_0_q8_0", "ref_vec_dot_q8_0_q8_0_chunk16"):
            fn = getattr(L, name)
            fn.restype = C.c_float
            fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        for name in ("ref_vec_dot_q8_f32_eval", "ref_scalar_dot_product_q8_f32"):
            fn = getattr(L, name)
            fn.restype = C.c_float
            fn.argtypes = [_c_f32p, C.c_void_p, C.c_int64]
        L.ref_mul_mat_q8_0.restype = C.c_int
        L.ref_mul_mat_q8_0.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int64, _c_f32p, C.c_int64, C.c_int64, _c_f32p, C.c_int64, C.c_int]
        self.has_rms_norm = hasattr(L, "ref_rms_norm_mul")  # absent from a library built before these were added
        if self.has_rms_norm:
            L.ref_sum_squares.restype = C.c_float
            L.ref_sum_squares.argtypes = [_c_f32p, C.c_int64]
            L.ref_sqrtf_fast.restype = C.c_float
            L.ref_sqrtf_fast.argtypes = [C.c_float]
            L.ref_rms_norm_mul.restype = C.c_int
            L.ref_rms_norm_mul.argtypes = [_c_f32p, C.c_int64, _c_f32p, C.c_float, C.c_int, _c_f32p, C.c_int64, C.c_int64, C.c_int64]
            L.ref_rms_norm_mul_q8_0.restype = C.c_int
            L.ref_rms_norm_mul_q8_0.argtypes = [_c_f32p, C.c_int64, _c_f32p, C.c_float, C.c_int, C.c_void_p, C.c_int64, C.c_int64]

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def fp32_to_fp16(self, f: float) -> int:
        return int(self.lib.ref_fp32_to_fp16(f))

    def fp32_to_fp16_bittrick(self, f: float) -> int:
        return int(self.lib.ref_fp32_to_fp16_bittrick(f))

    def fp16_to_fp32(self, h: int) -> float:
        return float(self.lib.ref_fp16_to_fp32(h))

    def quantize_rows(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        rows, K = x.shape
        out = np.empty((rows, K // QK, BLOCK_BYTES), dtype=np.uint8)
        for r in range(rows):
            self.lib.ref_quantize_row_q8_0(_ptr(x[r], _c_f32p), out[r].ctypes.data, K)
        return out

    def vec_dot_q8q8(self, w: np.ndarray, a: np.ndarray, chunk16: bool = False) -> float:
        nb = w.size // BLOCK_BYTES
        fn = self.lib.ref_vec_dot_q8_0_q8_0_chunk16 if chunk16 else self.lib.ref_vec_dot_q8_0_q8_0
        return float(fn(w.ctypes.data, a.ctypes.data, nb))

    def vec_dot_q8f32(self, w: np.ndarray, x: np.ndarray, prompt: bool = False) -> float:
        K = (w.size // BLOCK_BYTES) * QK
        fn = self.lib.ref_scalar_dot_product_q8_f32 if prompt else self.lib.ref_vec_dot_q8_f32_eval
        return float(fn(_ptr(np.ascontiguousarray(x, dtype=np.float32), _c_f32p), w.ctypes.data, K))

    def mul_mat(self, mode: int, w: np.ndarray, x: np.ndarray, threads: int = 0) -> np.ndarray:
        w = np.ascontiguousarray(w, dtype=np.uint8)
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        N, nb, _ = w.shape
        M, K = x.shape
        y = np.zeros((M, N), dtype=np.float32)
        rc = self.lib.ref_mul_mat_q8_0(mode, w.ctypes.data, N, K, _ptr(x, _c_f32p), K, M, _ptr(y, _c_f32p), max(N, 1),
                                       threads or (os.cpu_count() or 1))
        if rc != 0:
            raise ValueError(f"ref_mul_mat_q8_0 rc={rc}")
        return y

    def sum_squares(self, x: np.ndarray) -> float:
        x = np.ascontiguousarray(x, dtype=np.float32)
        return float(self.lib.ref_sum_squares(_ptr(x, _c_f32p), x.size))

    def sqrtf_fast(self, v: float) -> float:
        return float(self.lib.ref_sqrtf_fast(v))

    def rms_norm_mul(self, x: np.ndarray, w: np.ndarray, eps: float, sqrt_mode: int = 0) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        M, K = x.shape
        y = np.empty((M, K), dtype=np.float32)
        rc = self.lib.ref_rms_norm_mul(_ptr(x, _c_f32p), K, _ptr(w, _c_f32p), eps, sqrt_mode, _ptr(y, _c_f32p), K, M, K)
        if rc != 0:
            raise ValueError(f"ref_rms_norm_mul rc={rc}")
        return y

    def rms_norm_mul_q8_0(self, x: np.ndarray, w: np.ndarray, eps: float, sqrt_mode: int = 0) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        M, K = x.shape
        out = np.empty((M, K // QK, BLOCK_BYTES), dtype=np.uint8)
        rc = self.lib.ref_rms_norm_mul_q8_0(_ptr(x, _c_f32p), K, _ptr(w, _c_f32p), eps, sqrt_mode, out.ctypes.data, M, K)
        if rc != 0:
            raise ValueError(f"ref_rms_norm_mul_q8_0 rc={rc}")
        return out
