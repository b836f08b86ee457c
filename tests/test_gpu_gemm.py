"""GPU parity for the Q8_0 prefill GEMM (tcgen05 kind::i8), through the C-ABI host-pointer call.

Oracle: the int8-activation arithmetic (per token, kernels/avx2.cpp:562-585).  At sizes the C oracle finishes in
seconds it is used directly; at the full prefill size the check is a float64 restatement: with exact codes and
scales, sum_b d_x d_w sum_k q_x q_w equals (q_x * d_x) @ (q_w * d_w)^T evaluated in float64.
"""
import numpy as np
import pytest

from helpers import assert_parity, seeded_acts, seeded_weights
from zeninfer_b200 import blocks
from zeninfer_b200.backend import ACT_INT8

pytestmark = pytest.mark.gpu
Q8_0 = blocks.Q8_0


@pytest.fixture(scope="module")
def be():
    from zeninfer_b200 import Backend
    b = Backend()
    b.set_q8_act_mode(ACT_INT8)
    return b


def dequant_f64(packed, rows, cols):
    b = packed.reshape(rows, cols // 32, 34)
    d = b[..., :2].copy().view(np.float16).astype(np.float64)
    return (b[..., 2:].view(np.int8).astype(np.float64) * d).reshape(rows, cols)


def ref_f64(zo, packed, x, rows, cols):
    xq, xsc = zo.quantise_acts(x)
    xd = (xq.astype(np.float64).reshape(x.shape[0], -1, 32) * xsc.astype(np.float64)[..., None]).reshape(x.shape)
    return xd @ dequant_f64(packed, rows, cols).T


@pytest.mark.parametrize("tokens,rows,cols", [
    (9, 128, 128), (16, 100, 544), (17, 300, 96), (33, 67, 32), (64, 256, 4096), (65, 130, 2048),
    (128, 512, 1024), (129, 129, 4096), (171, 2048, 2048), (256, 1000, 14336), (300, 4096, 4096)])
def test_gemm_vs_int8_oracle(be, zo, tokens, rows, cols):
    w = seeded_weights(Q8_0, rows, cols, 200 + rows)
    x = seeded_acts(tokens, cols, 300 + tokens)
    got = be.gemm("Q8_0", w, x, tokens, rows, cols)
    if tokens * rows * cols <= 64 * 256 * 4096:
        assert_parity(got, zo.gemm(Q8_0, w, x, tokens, rows, cols, int8_acts=True), what=f"gemm {tokens}x{rows}x{cols} vs oracle")
    assert_parity(got, ref_f64(zo, w, x, rows, cols), tol=1e-5, what=f"gemm {tokens}x{rows}x{cols} vs float64")
    be.release_weights(w)


def test_token_ladder_from_reference(be, zo):
    # tests/core_tests.cpp:345-372: rows = 100, cols = 544 (17 blocks), closed-form bytes and activations
    rows, cols = 100, 544
    r = np.arange(rows)[:, None, None]
    blk = np.arange(17)[None, :, None]
    j = np.arange(2, 34)[None, None, :]
    packed = np.zeros((rows, 17, 34), np.uint8)
    packed[..., 1] = 0x3C
    packed[..., 2:] = (r * 5 + blk * 11 + j * 3) & 255
    packed = np.ascontiguousarray(packed.reshape(rows, -1))
    for T in (9, 16, 32, 171):
        t = np.arange(T)[:, None]
        c = np.arange(cols)[None, :]
        xin = (((t * 7 + c) % 15 - 7).astype(np.float32) * np.float32(0.017)).astype(np.float32)
        got = be.gemm("Q8_0", packed, xin, T, rows, cols)
        assert_parity(got, zo.gemm(Q8_0, packed, xin, T, rows, cols, int8_acts=True), what=f"ladder T={T}")
    be.release_weights(packed)


def test_gemm_batch_shares_input(be, zo):
    cols, rows, tokens = 1024, [512, 128, 128], 40
    ws = [seeded_weights(Q8_0, r, cols, 400 + i) for i, r in enumerate(rows)]
    x = seeded_acts(tokens, cols, 410)
    outs = be.gemm_batch("Q8_0", ws, x, rows, tokens, cols)
    for w, r, o in zip(ws, rows, outs):
        assert_parity(o, zo.gemm(Q8_0, w, x, tokens, r, cols, int8_acts=True), what=f"batched gemm rows={r}")
        assert np.array_equal(o, be.gemm("Q8_0", w, x, tokens, r, cols))
        be.release_weights(w)


def test_gemm_batch_numbers_row_tiles_through_the_tensors(be, zo):
    # 100 + 25 + 25 = 150 row tiles in one launch on 148 SMs: the K tiles are shared evenly and the cuts fall inside tiles of
    # different tensors; the second tensor ends in a ragged tile; the fourth tensor goes into a second launch
    cols, rows, tokens = 1024, [12800, 3190, 3200, 130], 40
    ws = [seeded_weights(Q8_0, r, cols, 430 + i) for i, r in enumerate(rows)]
    x = seeded_acts(tokens, cols, 440)
    outs = be.gemm_batch("Q8_0", ws, x, rows, tokens, cols)
    for w, r, o in zip(ws, rows, outs):
        assert_parity(o, zo.gemm(Q8_0, w, x, tokens, r, cols, int8_acts=True), what=f"batched gemm rows={r}")
        be.release_weights(w)


def test_config1_full_size(be, zo):
    # BASELINE config 1: activations 512 x 4096 N(0,1) seed 2, W 14336 x 4096 N(0,.02) seed 3 -> Q8_0
    tokens, rows, cols = 512, 14336, 4096
    w = seeded_weights(Q8_0, rows, cols, 3)
    x = seeded_acts(tokens, cols, 2)
    got = be.gemm("Q8_0", w, x, tokens, rows, cols)
    assert_parity(got, ref_f64(zo, w, x, rows, cols), tol=1e-5, what="config 1 vs float64 int8 restatement")
    # a sample of rows through the C oracle itself
    sel = np.arange(0, rows, 997)
    sub = np.ascontiguousarray(w[sel])
    ref = zo.gemm(Q8_0, sub, x[:32], 32, len(sel), cols, int8_acts=True)
    assert_parity(got[:32][:, sel], ref, what="config 1 sampled rows vs oracle")
    be.release_weights(w)
