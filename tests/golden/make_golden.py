"""Generate tests/golden/ref_vectors.npz from the UNMODIFIED reference.

Run where the reference tree is mounted and oracle/_ref/libzenref.so has been
built (``make -C oracle ref``):

    python tests/golden/make_golden.py

The reference latches its activation mode (ZEN_CPU_Q8_ACT) on the first Q8_0
call of a process, so the int8-activation vectors come from a child process
started with ZEN_CPU_Q8_ACT=1.  Inputs are stored next to the outputs, so the
tests that replay them need neither the reference nor this script.
"""
from __future__ import annotations

import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from zeninfer_b200 import blocks  # noqa: E402

OUT = os.path.join(HERE, "ref_vectors.npz")
TMP_I8 = os.path.join(HERE, "_int8_part.npz")


def weights(fmt: int, rows: int, cols: int, seed: int) -> np.ndarray:
    w = np.random.default_rng(seed).standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
    return blocks.quantize(fmt, w)


def acts(tokens: int, cols: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((tokens, cols), dtype=np.float32)


def formula_acts(tokens: int, cols: int) -> np.ndarray:
    """Closed-form activations in the style of the reference's GEMM sweeps (tests/core_tests.cpp:430)."""
    t = np.arange(tokens, dtype=np.int64)[:, None]
    c = np.arange(cols, dtype=np.int64)[None, :]
    a = ((t * 7 + c) % 15 - 7).astype(np.float32) * np.float32(0.017)
    b = ((t * 13 + c * 3) % 7 - 3).astype(np.float32) * np.float32(0.001)
    return (a + b).astype(np.float32)


def identity_q8_0(cols: int) -> np.ndarray:
    """cols x cols Q8_0 matrix: row r has code 1 at column r, block scale 1.0; y = dequantised activation."""
    m = np.zeros((cols, cols // 32, 34), np.uint8)
    m[:, :, 1] = 0x3C  # f16 1.0, little endian
    r = np.arange(cols)
    m[r, r // 32, 2 + r % 32] = 1
    return m.reshape(cols, -1)


def edge_acts(cols: int) -> np.ndarray:
    """Activation rows that stress the quantiser: zero block, exact .5 ties, huge, tiny, negative amax."""
    rng = np.random.default_rng(77)
    x = rng.standard_normal((6, cols), dtype=np.float32)
    x[0, :32] = 0.0
    x[1, :32] = np.arange(32, dtype=np.float32) * 0.5 - 7.75  # amax 7.75: x*inv lands on many .5 ties
    x[1, 31] = 127.0 / 2
    x[2, :32] *= np.float32(1e30)
    x[3, :32] *= np.float32(1e-30)
    x[4, :32] = -np.abs(x[4, :32])
    x[5, :64] = np.repeat(np.float32([3.0, -3.0]), 32)
    return x


def int8_part() -> None:
    assert os.environ.get("ZEN_CPU_Q8_ACT") == "1"
    zr = oracle.Reference()
    out = {}
    cols = 256
    ident = identity_q8_0(cols)
    xs = np.concatenate([acts(4, cols, 11), edge_acts(cols)])
    out["i8_ident_x"] = xs
    out["i8_ident_y"] = np.stack([zr.gemv(oracle.Q8_0, ident, x, cols, cols, workers=1) for x in xs])
    w = weights(oracle.Q8_0, 67, 544, 21)
    x = acts(3, 544, 22)
    out["i8_gemv_w"], out["i8_gemv_x"] = w, x
    out["i8_gemv_y"] = np.stack([zr.gemv(oracle.Q8_0, w, xi, 67, 544, workers=1) for xi in x])
    out["i8_gemv_y_w4"] = np.stack([zr.gemv(oracle.Q8_0, w, xi, 67, 544, workers=4) for xi in x])
    np.savez(TMP_I8, **out)


def main() -> None:
    zr = oracle.Reference()
    out = {}
    for name, fmt in (("q8_0", oracle.Q8_0), ("q4_0", oracle.Q4_0), ("q6_k", oracle.Q6_K)):
        rows, cols, tokens = 37, 768, 5
        w = weights(fmt, rows, cols, 100 + fmt)
        x = acts(tokens, cols, 200 + fmt)
        out[f"{name}_w"], out[f"{name}_x"] = w, x
        out[f"{name}_gemv_y"] = zr.gemv(fmt, w, x[0], rows, cols, workers=1)
        out[f"{name}_gemm_y"] = zr.gemm(fmt, w, x, tokens, rows, cols, workers=1)
    # K-blocked Q8_0 route: tokens*cols >= 131072 (src/quant.cpp:1188-1192)
    w = weights(oracle.Q8_0, 10, 2048, 31)
    x = formula_acts(64, 2048)  # rebuilt by the test from the same formula, not stored
    out["q8_0_kblk_w"] = w
    out["q8_0_kblk_y"] = zr.gemm(oracle.Q8_0, w, x, 64, 10, 2048, workers=1)

    env = dict(os.environ, ZEN_CPU_Q8_ACT="1")
    subprocess.run([sys.executable, os.path.abspath(__file__), "--int8-part"], check=True, env=env)
    with np.load(TMP_I8) as part:
        out.update({k: part[k] for k in part.files})
    os.remove(TMP_I8)
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, os.path.getsize(OUT), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    if "--int8-part" in sys.argv:
        int8_part()
    else:
        main()
