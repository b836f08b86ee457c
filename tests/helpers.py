"""Shared test helpers: seeded inputs, vectorised float64 references, the parity gate."""
from __future__ import annotations

import numpy as np

from zeninfer_b200 import blocks


def seeded_weights(fmt: int, rows: int, cols: int, seed: int) -> np.ndarray:
    """N(0, 0.02) fp32 weights packed to `fmt`; uint8 [rows, row_bytes]."""
    w = np.random.default_rng(seed).standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
    return np.ascontiguousarray(blocks.quantize(fmt, w))


def seeded_acts(tokens: int, cols: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((tokens, cols), dtype=np.float32)


def ref_int8_f64(packed_q8_0: np.ndarray, xq: np.ndarray, xsc: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """Float64 restatement of the int8-activation product (tools/d3d12_gemm_parity.cpp:130-147 shape):
    y[t, r] = sum_b d_w[r, b] * d_x[t, b] * sum_k q_w[r, b, k] * q_x[t, b, k].  xq: [T, K] int8, xsc: [T, K/32]."""
    nb = cols // 32
    b = packed_q8_0.reshape(rows, nb, 34)
    dw = b[..., :2].copy().view(np.float16).astype(np.float64)[..., 0]            # [rows, nb]
    qw = b[..., 2:].view(np.int8).astype(np.int32)                                 # [rows, nb, 32]
    qx = xq.reshape(-1, nb, 32).astype(np.int32)                                   # [T, nb, 32]
    out = np.empty((qx.shape[0], rows), np.float64)
    for t in range(qx.shape[0]):
        isum = np.einsum("rbk,bk->rb", qw, qx[t]).astype(np.float64)
        out[t] = (isum * dw * xsc[t].astype(np.float64)[None, :]).sum(axis=1)
    return out


def ref_fp32_f64(fmt: int, packed: np.ndarray, x: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """Float64 dequantise-then-dot, the gate every reference sweep uses (tests/core_tests.cpp:360-367)."""
    w = blocks.dequantize(fmt, packed, rows, cols).astype(np.float64)
    return np.asarray(x, np.float64).reshape(-1, cols) @ w.T


def assert_parity(got, ref, tol: float = 1e-3, what: str = "") -> float:
    """The parity gate: max|got-ref| / max|ref| <= tol  (tools/hip_parity.cpp:126-134) AND, per element,
    |got-ref| <= tol * max(1, |ref|)  (tests/core_tests.cpp:367).  Returns the first figure."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    max_ref = np.abs(ref).max()
    err = np.abs(got - ref)
    rel = float(err.max() / max_ref) if max_ref > 0 else float(err.max())
    assert rel <= tol, f"{what}: max_abs/max_ref = {rel:.3e} > {tol}"
    assert np.all(err <= tol * np.maximum(1.0, np.abs(ref))), f"{what}: per-element gate failed, worst {err.max():.3e}"
    return rel


class Q6KFixture:
    """tests/q6k_gemm_tests.cpp:11-45: Q6_K blocks built from known codes and scales, one shared LCG."""

    def __init__(self):
        self.state = 0x7136A95B

    def u32(self):
        self.state = (self.state * 1664525 + 1013904223) & 0xFFFFFFFF
        return self.state

    def weights(self, rows, cols):
        halves = [0x3400, 0xB800, 0x0001, 0x3C00]
        factors = [np.float32(0.25), np.float32(-0.5), np.float32(2.0 ** -24), np.float32(1.0)]
        nb = cols // 256
        packed = np.zeros((rows, nb, 210), np.uint8)
        expected = np.zeros((rows, cols), np.float32)
        for r in range(rows):
            for b in range(nb):
                p = packed[r, b]
                di = (r + b) % 4
                p[208], p[209] = halves[di] & 255, halves[di] >> 8
                scales = []
                for i in range(16):
                    s = (self.u32() >> 24) % 31 - 15
                    scales.append(s)
                    p[192 + i] = np.int8(s).view(np.uint8)
                for half in range(2):
                    for l in range(32):
                        q = []
                        for group in range(4):
                            q.append(self.u32() >> 26)
                            col = b * 256 + half * 128 + group * 32 + l
                            expected[r, col] = factors[di] * np.float32(scales[half * 8 + group * 2 + l // 16]) * np.float32(q[group] - 32)
                        p[half * 64 + l] = (q[0] & 15) | ((q[2] & 15) << 4)
                        p[half * 64 + 32 + l] = (q[1] & 15) | ((q[3] & 15) << 4)
                        p[128 + half * 32 + l] = (q[0] >> 4) | ((q[1] >> 4) << 2) | ((q[2] >> 4) << 4) | ((q[3] >> 4) << 6)
        return packed, expected


# ---- the group-scale product, restated (zeninfer_b200/csrc/gemm_groups.cuh) -------------------------------------------

GROUP = 256
FULL_SCALE = np.float32(32639.0)        # 256 * 127 + 127


def group_digits(v: np.ndarray) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """v [n, K] fp32, K a multiple of 256 -> (hi, lo) int32 [n, K] and unit fp32 [n, K / 256] with
    v ~= unit * (256 * hi + lo): unit = max|v| of the group / 32639 (fp32 division), the fixed-point value is
    rint(v * (1 / unit)) clamped to +-32639, hi = floor((V + 128) / 256), lo = V - 256 hi in -128..127.  fp32 throughout, as
    group_digits8 computes it."""
    v = np.asarray(v, np.float32)
    n, K = v.shape
    g = v.reshape(n, K // GROUP, GROUP)
    amax = np.abs(g).max(axis=2)
    with np.errstate(divide="ignore", invalid="ignore"):
        unit = np.where(amax > 0, amax / FULL_SCALE, np.float32(0)).astype(np.float32)
        inv = np.where(unit > 0, np.float32(1) / unit, np.float32(0)).astype(np.float32)
    V = np.clip(np.rint(g * inv[..., None]).astype(np.int32), -32639, 32639)
    hi = (V + 128) >> 8
    lo = V - 256 * hi
    return hi.reshape(n, K), lo.reshape(n, K), unit


def group_product(w_values: np.ndarray, x_values: np.ndarray) -> np.ndarray:
    """The kernel's arithmetic on dequantised weights [rows, K] and activation values [T, K]: per group the integer sums
    A = sum wh xh and B = sum wh xl + sum wl xh (the wl xl term is dropped), then out += (256 u_w u_x) * (256 A + B) group by
    group in fp32 (each step one fused multiply-add, emulated in float64).  Returns [T, rows] fp32."""
    wh, wl, uw = group_digits(w_values)
    xh, xl, ux = group_digits(x_values)
    rows, K = wh.shape
    T = xh.shape[0]
    out = np.zeros((T, rows), np.float32)
    for g in range(K // GROUP):
        s = slice(g * GROUP, (g + 1) * GROUP)
        A = xh[:, s].astype(np.int64) @ wh[:, s].astype(np.int64).T
        B = xl[:, s].astype(np.int64) @ wh[:, s].astype(np.int64).T + xh[:, s].astype(np.int64) @ wl[:, s].astype(np.int64).T
        f = (256.0 * A.astype(np.float32).astype(np.float64) + B.astype(np.float32).astype(np.float64)).astype(np.float32)
        scale = (ux[:, g][:, None] * (uw[:, g] * np.float32(256.0))[None, :]).astype(np.float32)
        out = (f.astype(np.float64) * scale.astype(np.float64) + out.astype(np.float64)).astype(np.float32)
    return out
