"""Writes tests/golden/kquant_vectors.npz: outputs of the UNMODIFIED reference (oracle/_ref/libzenref.so, built by
`make -C oracle ref` where the reference tree is mounted) for Q4_K and Q5_K rows with random valid content: the decoded
weights (zen::quant::dequantize), the fp32-activation product (zen::quant::gemv, one worker and four) and the batched
product of three tokens (zen::quant::gemm, one worker: with several, the rows that fall into a worker's last partial
group of four go through another kernel, so the result depends on the worker count in the last bit).

    python tests/golden/make_kquant_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from zeninfer_b200 import blocks  # noqa: E402

ROWS, COLS = 70, 768     # 70 rows: above the reference's 64-row threshold for splitting rows over workers


def main() -> None:
    zr = oracle.Reference()
    out = {}
    for fmt, tag in ((blocks.Q4_K, "q4_k"), (blocks.Q5_K, "q5_k")):
        w = blocks.random_k_blocks(fmt, ROWS, COLS, 1729 + fmt)
        x = np.random.default_rng(2 * fmt).standard_normal(COLS, dtype=np.float32)
        y1 = zr.gemv(fmt, w, x, ROWS, COLS, workers=1)
        y4 = zr.gemv(fmt, w, x, ROWS, COLS, workers=4)
        assert np.array_equal(y1, y4), "the row split must not change a row's sum"
        out[tag + "_w"], out[tag + "_x"], out[tag + "_y"] = w, x, y1
        out[tag + "_dequant"] = zr.dequantize(fmt, w[:3], 3 * COLS)
        xb = np.random.default_rng(3 * fmt).standard_normal((3, COLS), dtype=np.float32)
        out[tag + "_xb"], out[tag + "_yb"] = xb, zr.gemm(fmt, w, xb, 3, ROWS, COLS, workers=1)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "kquant_vectors.npz"), **out)
    print("wrote kquant_vectors.npz")


if __name__ == "__main__":
    main()
