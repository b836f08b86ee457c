"""Q4_K and Q5_K on the host side: the C restatement (oracle/zen_oracle.c) and the numpy decoder (zeninfer_b200/blocks.py)
against vectors the unmodified reference produced (tests/golden/kquant_vectors.npz) and, where the compiled reference is
present, against it directly on more shapes.  Bit-exact: the decoder is two roundings per value, the product kernel a
fixed lane order."""
import os

import numpy as np
import pytest

import oracle
from zeninfer_b200 import blocks

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "kquant_vectors.npz")
FORMATS = [(blocks.Q4_K, "q4_k"), (blocks.Q5_K, "q5_k")]


def _golden(key: str) -> np.ndarray:
    with np.load(GOLDEN) as g:
        return g[key]


@pytest.mark.parametrize("fmt,tag", FORMATS)
def test_against_the_reference_vectors(zo, fmt, tag):
    with np.load(GOLDEN) as g:
        w, x, y, deq = g[tag + "_w"], g[tag + "_x"], g[tag + "_y"], g[tag + "_dequant"]
    rows, cols = w.shape[0], x.size
    assert w.shape[1] == blocks.row_bytes(fmt, cols) == zo.row_bytes(fmt, cols)
    assert np.array_equal(zo.dequantize(fmt, w[:3], 3 * cols), deq)
    assert np.array_equal(blocks.dequantize(fmt, w[:3], 3, cols).reshape(-1), deq)
    assert np.array_equal(zo.gemv(fmt, w, x, rows, cols), y)
    assert np.array_equal(zo.gemm(fmt, w, g_xb := _golden(tag + "_xb"), 3, rows, cols), _golden(tag + "_yb"))
    assert np.abs(_golden(tag + "_yb")[0] - blocks.dequantize(fmt, w, rows, cols).astype(np.float64) @ g_xb[0].astype(np.float64)).max() <= 1e-4
    # the product is the decoded row times x up to the order of the sums
    full = blocks.dequantize(fmt, w, rows, cols).astype(np.float64) @ x.astype(np.float64)
    assert np.abs(y - full).max() <= 1e-5 * np.abs(full).max()


@pytest.mark.parametrize("fmt,tag", FORMATS)
def test_against_the_compiled_reference(zo, fmt, tag):
    if not oracle.reference_available():
        pytest.skip("compiled reference not present")
    zr = oracle.Reference()
    for rows, cols, seed in ((1, 256, 1), (9, 512, 2), (130, 2048, 3)):
        w = blocks.random_k_blocks(fmt, rows, cols, seed)
        x = np.random.default_rng(seed + 10).standard_normal(cols, dtype=np.float32)
        assert np.array_equal(zo.dequantize(fmt, w, rows * cols), zr.dequantize(fmt, w, rows * cols))
        for workers in (1, 3):
            assert np.array_equal(zo.gemv(fmt, w, x, rows, cols), zr.gemv(fmt, w, x, rows, cols, workers=workers))
        for tokens in (1, 2, 5):     # one token: the generic route; more: the K-blocked kernel, row tails through dot_f32
            xb = np.random.default_rng(seed + 20 + tokens).standard_normal((tokens, cols), dtype=np.float32)
            assert np.array_equal(zo.gemm(fmt, w, xb, tokens, rows, cols), zr.gemm(fmt, w, xb, tokens, rows, cols, workers=1))


def test_row_geometry():
    assert blocks.row_bytes(blocks.Q4_K, 4096) == 16 * 144 and blocks.row_bytes(blocks.Q5_K, 4096) == 16 * 176
    assert blocks.row_bytes(blocks.Q4_K, 100) == 0
    with pytest.raises(ValueError):
        blocks.random_k_blocks(blocks.Q4_K, 2, 100, 0)
