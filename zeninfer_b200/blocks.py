"""GGUF block formats on the path: byte sizes, NumPy packers and decoders.

The reference ships decoders only (``zen::quant::dequantize``,
src/quant.cpp:391-397 Q4_0, :410-416 Q8_0, :500-517 Q6_K); model files arrive
already quantised.  The packers here exist to synthesise weights for tests and
benchmarks.  Any valid block content is acceptable because parity is defined on
the packed bytes, not on how they were produced.

Block layouts (little endian):
  Q8_0  34 B / 32 el : f16 d | 32 x int8                         w = q * d
  Q4_0  18 B / 32 el : f16 d | 16 B, low nibble = el j, high = el j+16
                                                                 w = (q - 8) * d
  Q6_K 210 B / 256 el: ql[128] | qh[64] | int8 sc[16] | f16 d    w = d * sc * (q - 32)
  Q4_K 144 B / 256 el: f16 d | f16 dmin | 12 B of 6-bit (scale, min) x 8 | 128 B nibbles
                                                                 w = (d * sc_j) * q - dmin * m_j, j = element / 32
  Q5_K 176 B / 256 el: Q4_K with a 32-byte plane of fifth bits between the scales and the nibbles (src/quant.cpp:439-476)

Q4_K and Q5_K have no quantiser here (the reference has none either): random_k_blocks draws valid rows for tests and benchmarks.
"""
from __future__ import annotations

import numpy as np

Q8_0, Q4_0, Q6_K, Q4_K, Q5_K = 8, 2, 14, 12, 13  # GGML type ids
BLOCK_ELEMENTS = {Q8_0: 32, Q4_0: 32, Q6_K: 256, Q4_K: 256, Q5_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18, Q6_K: 210, Q4_K: 144, Q5_K: 176}
NAMES = {Q8_0: "Q8_0", Q4_0: "Q4_0", Q6_K: "Q6_K", Q4_K: "Q4_K", Q5_K: "Q5_K"}


def row_bytes(fmt: int, columns: int) -> int:
    """Bytes of one weight row; 0 when ``columns`` is not block aligned (src/quant.cpp:894-943)."""
    be = BLOCK_ELEMENTS[fmt]
    return 0 if columns % be else (columns // be) * BLOCK_BYTES[fmt]


def _round_half_away(v: np.ndarray) -> np.ndarray:
    """C ``lround`` on float32 input, evaluated exactly: truncation and the fractional part are exact in
    float32, so no step re-rounds (v +/- 0.5 computed in float32 would, just below a tie)."""
    v = np.asarray(v, np.float32)
    t = np.trunc(v)
    return t + np.where(np.abs(v - t) >= np.float32(0.5), np.sign(v), np.float32(0)).astype(np.float32)


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    """fp32 [rows, K] -> uint8 [rows, K/32*34].

    Same arithmetic as the reference's only Q8_0 encoder (src/quant.cpp:1265-1276):
    scale = amax/127 in fp32, stored as binary16 (round to nearest even), codes
    from the UNROUNDED fp32 scale, round half away from zero, clamp to +-127.
    """
    w = np.ascontiguousarray(w, np.float32)
    rows, k = w.shape
    assert k % 32 == 0
    blk = w.reshape(rows, k // 32, 32)
    amax = np.abs(blk).max(axis=2)
    scale = (amax / np.float32(127.0)).astype(np.float32)
    scale = np.where(amax > 0, scale, np.float32(0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(scale > 0, np.float32(1.0) / scale, np.float32(0)).astype(np.float32)
    q = _round_half_away((blk * inv[..., None]).astype(np.float32))
    q = np.clip(q, -127, 127).astype(np.int8)
    out = np.empty((rows, k // 32, 34), np.uint8)
    out[..., 0:2] = scale.astype(np.float16).view(np.uint8).reshape(rows, k // 32, 2)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(rows, -1)


def quantize_q4_0(w: np.ndarray) -> np.ndarray:
    """fp32 [rows, K] -> uint8 [rows, K/32*18]; the published GGML Q4_0 rule.

    d = (signed value of largest magnitude) / -8, q = min(15, trunc(x/d + 8.5)).
    """
    w = np.ascontiguousarray(w, np.float32)
    rows, k = w.shape
    assert k % 32 == 0
    blk = w.reshape(rows, k // 32, 32)
    idx = np.abs(blk).argmax(axis=2)
    mx = np.take_along_axis(blk, idx[..., None], axis=2)[..., 0]
    d = (mx / np.float32(-8.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0)).astype(np.float32)
    q = np.minimum(15, ((blk * inv[..., None]).astype(np.float32) + np.float32(8.5)).astype(np.int32)).astype(np.uint8)
    q = np.maximum(q, 0).astype(np.uint8)
    out = np.empty((rows, k // 32, 18), np.uint8)
    out[..., 0:2] = d.astype(np.float16).view(np.uint8).reshape(rows, k // 32, 2)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(rows, -1)


def pack_q6_k(q: np.ndarray, sc: np.ndarray, d_half: np.ndarray) -> np.ndarray:
    """Pack known Q6_K fields.  q: uint8 [n, 256] in 0..63, sc: int8 [n, 16], d_half: uint16 [n] -> uint8 [n, 210].

    Element c = half*128 + group*32 + l lives in ql[half*64 + (group%2)*32 + l]
    (low nibble for group < 2, high nibble otherwise) and in bits 2*group..2*group+1
    of qh[half*32 + l]; its scale is sc[half*8 + group*2 + l/16]
    (src/quant.cpp:500-517).
    """
    n = q.shape[0]
    q = q.reshape(n, 2, 4, 32).astype(np.uint8)
    out = np.zeros((n, 210), np.uint8)
    ql = out[:, :128].reshape(n, 2, 2, 32)
    qh = out[:, 128:192].reshape(n, 2, 32)
    ql[:, :, 0, :] = (q[:, :, 0, :] & 15) | ((q[:, :, 2, :] & 15) << 4)
    ql[:, :, 1, :] = (q[:, :, 1, :] & 15) | ((q[:, :, 3, :] & 15) << 4)
    qh[:] = (q[:, :, 0, :] >> 4) | ((q[:, :, 1, :] >> 4) << 2) | ((q[:, :, 2, :] >> 4) << 4) | ((q[:, :, 3, :] >> 4) << 6)
    out[:, 192:208] = sc.astype(np.int8).view(np.uint8).reshape(n, 16)
    out[:, 208:210] = np.ascontiguousarray(d_half, np.uint16).view(np.uint8).reshape(n, 2)
    return out


def quantize_q6_k(w: np.ndarray) -> np.ndarray:
    """fp32 [rows, K] -> uint8 [rows, K/256*210].

    A plain valid encoder (not GGML's error-minimising search): each 16-element
    group gets scale amax/31, the super-block d maps the largest group scale to
    int8 127, and codes are round(x / (d*sc)) + 32 clamped to 0..63.
    """
    w = np.ascontiguousarray(w, np.float32)
    rows, k = w.shape
    assert k % 256 == 0
    n = rows * (k // 256)
    grp = w.reshape(n, 16, 16)
    gscale = np.abs(grp).max(axis=2) / np.float32(31.0)
    d = (gscale.max(axis=1) / np.float32(127.0)).astype(np.float16)
    d32 = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(d32[:, None] > 0, np.rint(gscale / d32[:, None]), 0)
    sc = np.clip(sc, 1, 127).astype(np.int8)
    eff = d32[:, None] * sc.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(eff[..., None] > 0, np.rint(grp / eff[..., None]), 0)
    q = (np.clip(q, -32, 31) + 32).astype(np.uint8)
    return pack_q6_k(q.reshape(n, 256), sc, d.view(np.uint16)).reshape(rows, -1)


def quantize(fmt: int, w: np.ndarray) -> np.ndarray:
    return {Q8_0: quantize_q8_0, Q4_0: quantize_q4_0, Q6_K: quantize_q6_k}[fmt](w)


def random_k_blocks(fmt: int, rows: int, columns: int, seed: int) -> np.ndarray:
    """Valid Q4_K / Q5_K rows with random content (uint8 [rows, row_bytes]): every code, 6-bit scale and minimum is
    uniform, d and dmin are small positive normal halves, so decoded weights are of the order of 0.02."""
    if fmt not in (Q4_K, Q5_K) or columns % 256:
        raise ValueError("Q4_K / Q5_K rows of whole super-blocks")
    rng = np.random.default_rng(seed)
    n = rows * (columns // 256)
    b = rng.integers(0, 256, size=(n, BLOCK_BYTES[fmt]), dtype=np.uint8)
    b[:, 0:2] = (rng.uniform(6.2e-5, 1.5e-4, size=n).astype(np.float16)).view(np.uint8).reshape(n, 2)
    b[:, 2:4] = (rng.uniform(6.2e-5, 1.5e-4, size=n).astype(np.float16)).view(np.uint8).reshape(n, 2)
    return np.ascontiguousarray(b.reshape(rows, -1))


def _k_scales_mins(s: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """The eight 6-bit (scale, minimum) pairs of a super-block from its 12 packed bytes [n, 12] (src/quant.cpp:133-141)."""
    s = s.astype(np.uint32)
    sc = np.concatenate([s[:, 0:4] & 63, (s[:, 8:12] & 15) | ((s[:, 0:4] >> 6) << 4)], axis=1)
    mn = np.concatenate([s[:, 4:8] & 63, (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)], axis=1)
    return sc.astype(np.float32), mn.astype(np.float32)


def dequantize(fmt: int, packed: np.ndarray, rows: int, columns: int) -> np.ndarray:
    """Vectorised decoder with the reference's operation order; uint8 [rows, row_bytes] -> fp32 [rows, K]."""
    p = np.ascontiguousarray(packed, np.uint8).reshape(rows, -1)
    if fmt == Q8_0:
        b = p.reshape(rows, columns // 32, 34)
        d = b[..., 0:2].copy().view(np.float16).astype(np.float32)
        return (b[..., 2:].view(np.int8).astype(np.float32) * d).reshape(rows, columns)
    if fmt == Q4_0:
        b = p.reshape(rows, columns // 32, 18)
        d = b[..., 0:2].copy().view(np.float16).astype(np.float32)
        lo = (b[..., 2:] & 15).astype(np.int32) - 8
        hi = (b[..., 2:] >> 4).astype(np.int32) - 8
        return (np.concatenate([lo, hi], axis=2).astype(np.float32) * d).reshape(rows, columns)
    if fmt == Q6_K:
        n = rows * (columns // 256)
        b = p.reshape(n, 210)
        ql = b[:, :128].reshape(n, 2, 2, 32)
        qh = b[:, 128:192].reshape(n, 2, 1, 32)
        lo = np.concatenate([ql & 15, ql >> 4], axis=2)  # groups 0,1 then 2,3
        hi = (qh >> (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 4, 1)) & 3
        q = (lo | (hi << 4)).astype(np.int32) - 32  # [n, half, group, l]
        sc = b[:, 192:208].view(np.int8).astype(np.float32).reshape(n, 2, 4, 2)
        d = b[:, 208:210].copy().view(np.float16).astype(np.float32).reshape(n, 1, 1, 1)
        ds = (d * sc)[..., None]  # [n, half, group, 2, 1]
        return (ds * q.reshape(n, 2, 4, 2, 16).astype(np.float32)).reshape(rows, columns)
    if fmt in (Q4_K, Q5_K):
        n = rows * (columns // 256)
        b = p.reshape(n, BLOCK_BYTES[fmt])
        d = b[:, 0:2].copy().view(np.float16).astype(np.float32)            # [n, 1]
        dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)
        sc, mn = _k_scales_mins(b[:, 4:16])                                 # [n, 8]
        ql = b[:, (48 if fmt == Q5_K else 16):].reshape(n, 4, 32)           # 32 bytes serve sub-blocks 2p (low nibbles) and 2p + 1 (high)
        q = np.stack([ql & 15, ql >> 4], axis=2).reshape(n, 8, 32).astype(np.uint32)
        if fmt == Q5_K:
            qh = b[:, 16:48].astype(np.uint32)                              # bit j of byte l: the fifth bit of element l of sub-block j
            q = q | (((qh[:, None, :] >> np.arange(8, dtype=np.uint32).reshape(1, 8, 1)) & 1) << 4)
        ds = (d * sc)[..., None]
        ms = (dmin * mn)[..., None]
        return (ds * q.astype(np.float32) - ms).reshape(rows, columns)
    raise ValueError(fmt)
