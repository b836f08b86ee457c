"""ctypes doorway to the two CPU checkers (test infrastructure only).

``zo``  -- liboracle.so, the plain-C restatement in zen_oracle.c.
``zr``  -- _ref/libzenref.so, the unmodified reference compiled from its own
           sources (present only where ``make -C oracle ref`` could run or a
           prebuilt copy travelled with the tree).

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module.  The product package never does: it has no CPU path.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
Q8_0, Q4_0, Q6_K, Q4_K, Q5_K = 8, 2, 14, 12, 13  # GGML type ids, as in the GGUF tensor directory

_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)
_f32p = C.POINTER(C.c_float)
_sz = C.c_size_t


def build(with_reference: bool = True) -> None:
    """Compile liboracle.so and, when the reference tree is present, _ref/libzenref.so."""
    targets = ["oracle"] + (["ref"] if with_reference else [])
    subprocess.run(["make", "-C", _HERE, "-j8", *targets], check=True, stdout=subprocess.DEVNULL)


def _ptr(a: np.ndarray, ty):
    return a.ctypes.data_as(ty)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


class Oracle:
    """The plain-C restatement (zen_oracle.c)."""

    def __init__(self) -> None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build(with_reference=False)
        self.lib = L = C.CDLL(path)
        L.zo_half_to_float.restype = C.c_float
        L.zo_half_to_float.argtypes = [C.c_uint16]
        L.zo_float_to_half.restype = C.c_uint16
        L.zo_float_to_half.argtypes = [C.c_float]
        L.zo_row_bytes.restype = _sz
        L.zo_row_bytes.argtypes = [C.c_int, _sz]
        L.zo_dequantize.argtypes = [C.c_int, _u8p, _sz, _f32p]
        L.zo_quantise_acts_q8_0.restype = None
        L.zo_quantise_acts_q8_0.argtypes = [_f32p, _sz, _i8p, _f32p]
        L.zo_gemv_q8_0_i8_prequant.argtypes = [_u8p, _i8p, _f32p, _f32p, _sz, _sz]
        L.zo_gemv.argtypes = [C.c_int, _u8p, _f32p, _f32p, _sz, _sz, C.c_int]
        L.zo_gemm.argtypes = [C.c_int, _u8p, _f32p, _f32p, _sz, _sz, _sz, C.c_int]
        L.zo_gemm_q8_0_f32.argtypes = [_u8p, _f32p, _f32p, _sz, _sz, _sz]
        L.zo_gemm_q8_0_f32_kblk.argtypes = [_u8p, _f32p, _f32p, _sz, _sz, _sz]
        L.zo_argmax.restype = C.c_int64
        L.zo_argmax.argtypes = [_f32p, _sz]
        L.zo_row_slice.restype = None
        L.zo_row_slice.argtypes = [_sz, C.c_uint, C.c_uint, C.POINTER(_sz), C.POINTER(_sz)]

    def half_to_float(self, h: int) -> float:
        return float(self.lib.zo_half_to_float(h))

    def float_to_half(self, v: float) -> int:
        return int(self.lib.zo_float_to_half(C.c_float(v)))

    def row_bytes(self, fmt: int, columns: int) -> int:
        return int(self.lib.zo_row_bytes(fmt, columns))

    def dequantize(self, fmt: int, blocks, n: int) -> np.ndarray:
        src = _u8(blocks)
        out = np.empty(n, np.float32)
        if not self.lib.zo_dequantize(fmt, _ptr(src, _u8p), n, _ptr(out, _f32p)):
            raise ValueError("oracle declined dequantize")
        return out

    def quantise_acts(self, x) -> tuple[np.ndarray, np.ndarray]:
        """x: [..., K] fp32 -> (int8 codes [..., K], fp32 scales [..., K/32])."""
        x = _f32(x)
        k = x.shape[-1]
        flat = x.reshape(-1, k)
        q = np.empty(flat.shape, np.int8)
        sc = np.empty((flat.shape[0], k // 32), np.float32)
        for t in range(flat.shape[0]):
            self.lib.zo_quantise_acts_q8_0(_ptr(flat[t], _f32p), k, _ptr(q[t], _i8p), _ptr(sc[t], _f32p))
        return q.reshape(x.shape), sc.reshape(x.shape[:-1] + (k // 32,))

    def gemv_q8_0_i8_prequant(self, w, xq, xsc, rows: int, cols: int) -> np.ndarray:
        w, xq, xsc = _u8(w), np.ascontiguousarray(xq, np.int8), _f32(xsc)
        y = np.empty(rows, np.float32)
        if not self.lib.zo_gemv_q8_0_i8_prequant(_ptr(w, _u8p), _ptr(xq, _i8p), _ptr(xsc, _f32p), _ptr(y, _f32p), rows, cols):
            raise ValueError("oracle declined gemv_q8_0_i8_prequant")
        return y

    def gemv(self, fmt: int, w, x, rows: int, cols: int, int8_acts: bool = False) -> np.ndarray:
        w, x = _u8(w), _f32(x)
        y = np.empty(rows, np.float32)
        if not self.lib.zo_gemv(fmt, _ptr(w, _u8p), _ptr(x, _f32p), _ptr(y, _f32p), rows, cols, int(int8_acts)):
            raise ValueError("oracle declined gemv")
        return y

    def gemm(self, fmt: int, w, x, tokens: int, rows: int, cols: int, int8_acts: bool = False) -> np.ndarray:
        w, x = _u8(w), _f32(x)
        out = np.empty((tokens, rows), np.float32)
        if not self.lib.zo_gemm(fmt, _ptr(w, _u8p), _ptr(x, _f32p), _ptr(out, _f32p), tokens, rows, cols, int(int8_acts)):
            raise ValueError("oracle declined gemm")
        return out

    def gemm_q8_0_f32(self, w, x, tokens: int, rows: int, cols: int, kblk: bool) -> np.ndarray:
        w, x = _u8(w), _f32(x)
        out = np.empty((tokens, rows), np.float32)
        fn = self.lib.zo_gemm_q8_0_f32_kblk if kblk else self.lib.zo_gemm_q8_0_f32
        if not fn(_ptr(w, _u8p), _ptr(x, _f32p), _ptr(out, _f32p), tokens, rows, cols):
            raise ValueError("oracle declined gemm_q8_0_f32")
        return out

    def argmax(self, logits) -> int:
        v = _f32(logits)
        return int(self.lib.zo_argmax(_ptr(v, _f32p), v.size))

    def row_slice(self, count: int, workers: int, i: int) -> tuple[int, int]:
        a, b = _sz(), _sz()
        self.lib.zo_row_slice(count, workers, i, C.byref(a), C.byref(b))
        return int(a.value), int(b.value)


class Reference:
    """The unmodified reference behind ref_shim.cpp.  Raises FileNotFoundError when not built.

    The reference latches ZEN_CPU_Q8_ACT on its first Q8_0 call, so one process
    sees one activation mode through ``gemv``/``gemm``; ``gemv_q8_0_i8_prequant``
    is mode-independent.
    """

    def __init__(self) -> None:
        path = os.path.join(_HERE, "_ref", "libzenref.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = L = C.CDLL(path)
        L.zr_row_bytes.restype = _sz
        L.zr_row_bytes.argtypes = [C.c_int, _sz]
        L.zr_dequantize.argtypes = [C.c_int, _u8p, _sz, _f32p]
        L.zr_encode_fp16.argtypes = [_f32p, C.POINTER(C.c_uint16), _sz]
        L.zr_decode_fp16.argtypes = [C.POINTER(C.c_uint16), _f32p, _sz]
        L.zr_gemv.argtypes = [C.c_int, _u8p, _f32p, _f32p, _sz, _sz, C.c_uint]
        L.zr_gemm.argtypes = [C.c_int, _u8p, _f32p, _f32p, _sz, _sz, _sz, C.c_uint]
        L.zr_gemv_batch.argtypes = [C.c_int, C.POINTER(C.c_void_p), _f32p, C.POINTER(C.c_void_p), C.POINTER(_sz), _sz, _sz, C.c_uint]
        L.zr_gemv_q8_0_i8_prequant.argtypes = [_u8p, _i8p, _f32p, _f32p, _sz, _sz]
        L.zr_gemv_q6k_avx2.argtypes = [_u8p, _f32p, _f32p, _sz, _sz]
        for name in ("zr_gemm_q8_0_avx2", "zr_gemm_q8_0_kblk_avx2", "zr_gemm_q6k_kblk_avx2"):
            getattr(L, name).argtypes = [_u8p, _f32p, _f32p, _sz, _sz, _sz]
        L.zr_pool_workers.restype = C.c_uint

    def row_bytes(self, fmt: int, columns: int) -> int:
        return int(self.lib.zr_row_bytes(fmt, columns))

    def dequantize(self, fmt: int, blocks, n: int) -> np.ndarray:
        src = _u8(blocks)
        out = np.empty(n, np.float32)
        if not self.lib.zr_dequantize(fmt, _ptr(src, _u8p), n, _ptr(out, _f32p)):
            raise ValueError("reference declined dequantize")
        return out

    def encode_fp16(self, values) -> np.ndarray:
        v = _f32(values)
        out = np.empty(v.size, np.uint16)
        self.lib.zr_encode_fp16(_ptr(v, _f32p), _ptr(out, C.POINTER(C.c_uint16)), v.size)
        return out

    def decode_fp16(self, halves) -> np.ndarray:
        h = np.ascontiguousarray(halves, np.uint16)
        out = np.empty(h.size, np.float32)
        self.lib.zr_decode_fp16(_ptr(h, C.POINTER(C.c_uint16)), _ptr(out, _f32p), h.size)
        return out

    def gemv(self, fmt: int, w, x, rows: int, cols: int, workers: int = 1) -> np.ndarray:
        w, x = _u8(w), _f32(x)
        y = np.empty(rows, np.float32)
        if not self.lib.zr_gemv(fmt, _ptr(w, _u8p), _ptr(x, _f32p), _ptr(y, _f32p), rows, cols, workers):
            raise ValueError("reference declined gemv")
        return y

    def gemv_batch(self, fmt: int, ws, x, rows, cols: int, workers: int = 1, outs=None) -> list[np.ndarray]:
        """zen::quant::gemv_batch: several matvecs sharing x in one submission (one parallel_for over the concatenated rows)."""
        ws, x = [_u8(w) for w in ws], _f32(x)
        n = len(ws)
        ys = outs if outs is not None else [np.empty(r, np.float32) for r in rows]
        wp = (C.c_void_p * n)(*[w.ctypes.data for w in ws])
        yp = (C.c_void_p * n)(*[y.ctypes.data for y in ys])
        rs = (_sz * n)(*rows)
        if not self.lib.zr_gemv_batch(fmt, wp, _ptr(x, _f32p), yp, rs, cols, n, workers):
            raise ValueError("reference declined gemv_batch")
        return ys

    def gemm(self, fmt: int, w, x, tokens: int, rows: int, cols: int, workers: int = 1) -> np.ndarray:
        w, x = _u8(w), _f32(x)
        out = np.empty((tokens, rows), np.float32)
        if not self.lib.zr_gemm(fmt, _ptr(w, _u8p), _ptr(x, _f32p), _ptr(out, _f32p), tokens, rows, cols, workers):
            raise ValueError("reference declined gemm")
        return out

    def gemv_q8_0_i8_prequant(self, w, xq, xsc, rows: int, cols: int) -> np.ndarray:
        w, xq, xsc = _u8(w), np.ascontiguousarray(xq, np.int8), _f32(xsc)
        y = np.empty(rows, np.float32)
        if not self.lib.zr_gemv_q8_0_i8_prequant(_ptr(w, _u8p), _ptr(xq, _i8p), _ptr(xsc, _f32p), _ptr(y, _f32p), rows, cols):
            raise ValueError("reference declined gemv_q8_0_i8_prequant")
        return y

    def gemm_direct(self, kind: str, w, x, tokens: int, rows: int, cols: int) -> np.ndarray:
        """kind: 'q8_0' (row-pair kernel), 'q8_0_kblk', 'q6k_kblk' -- single-thread direct kernels."""
        fn = {"q8_0": self.lib.zr_gemm_q8_0_avx2, "q8_0_kblk": self.lib.zr_gemm_q8_0_kblk_avx2,
              "q6k_kblk": self.lib.zr_gemm_q6k_kblk_avx2}[kind]
        w, x = _u8(w), _f32(x)
        out = np.empty((tokens, rows), np.float32)
        if not fn(_ptr(w, _u8p), _ptr(x, _f32p), _ptr(out, _f32p), tokens, rows, cols):
            raise ValueError("reference declined " + kind)
        return out

    def pool_workers(self) -> int:
        return int(self.lib.zr_pool_workers())


def reference_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libzenref.so"))
