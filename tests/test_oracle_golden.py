"""Pins the CPU oracle (oracle/zen_oracle.c) before anything trusts it.

Three sources of truth, none of them the code under test:
  1. the reference's own known-answer tests, replayed from their definitions
     (tests/core_tests.cpp, tests/q6k_gemm_tests.cpp, tests/support/quant_fixture.h);
  2. tests/golden/ref_vectors.npz -- outputs of the unmodified reference,
     produced by tests/golden/make_golden.py;
  3. the compiled reference itself (oracle/_ref), bit for bit, where present.
"""
import os

import numpy as np
import pytest

from conftest import lcg_bytes
from helpers import Q6KFixture as _Q6KFixture
from zeninfer_b200 import blocks

Q8_0, Q4_0, Q6_K = blocks.Q8_0, blocks.Q4_0, blocks.Q6_K
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz")


# ---- 1. known-answer tests of the reference ---------------------------------

def test_fp16_rounding_golden(zo):
    # tests/core_tests.cpp:263-270: ties-to-even around 1.0, the subnormal boundary, overflow, -0, inf
    inputs = [1.0, 1.00048828125, 1.00146484375, 5.960464477539063e-8, 2.9802322387695312e-8, 65520.0, -0.0, float("inf")]
    expected = [0x3C00, 0x3C00, 0x3C02, 0x0001, 0x0000, 0x7C00, 0x8000, 0x7C00]
    assert [zo.float_to_half(v) for v in inputs] == expected


def test_fp16_roundtrip_every_code(zo):
    # tests/core_tests.cpp:253-262: decode then encode returns the same bits for every non-NaN code
    codes = np.arange(65536, dtype=np.uint16)
    as_np = codes.view(np.float16).astype(np.float32)
    for h in range(0, 65536, 7):  # every 7th code through the C implementation, all codes against NumPy below
        v = zo.half_to_float(h)
        if (h & 0x7C00) == 0x7C00 and (h & 0x3FF):
            assert np.isnan(v)
            e = zo.float_to_half(v)
            assert (e & 0x7C00) == 0x7C00 and (e & 0x3FF) != 0
        else:
            assert v == as_np[h] and np.signbit(np.float32(v)) == np.signbit(as_np[h])
            assert zo.float_to_half(v) == h


def test_q8_0_unit_row_is_exactly_32(zo):
    # tests/core_tests.cpp:272-277
    blk = np.array([0x00, 0x3C] + [1] * 32, np.uint8)
    ones = np.ones(32, np.float32)
    assert zo.gemv(Q8_0, blk, ones, 1, 32)[0] == np.float32(32.0)
    assert zo.gemv(Q8_0, blk, ones, 1, 32, int8_acts=True)[0] == np.float32(32.0)


def test_q8_0_two_rows_vs_dequant_dot(zo):
    # tests/core_tests.cpp:279-292
    m = np.zeros((2, 2, 34), np.uint8)
    for r in range(2):
        for b in range(2):
            m[r, b, 0], m[r, b, 1] = 0x00, 0x34  # f16 0.25
            for i in range(32):
                m[r, b, 2 + i] = np.int8(((b * 32 + i) * 7 + r * 11) % 31 - 15).view(np.uint8)
    x = ((np.arange(64) % 13 - 6) * 0.125).astype(np.float32)
    y = zo.gemv(Q8_0, m, x, 2, 64)
    for r in range(2):
        row = zo.dequantize(Q8_0, m[r], 64)
        ref = float(np.dot(row.astype(np.float64), x.astype(np.float64)))
        assert abs(y[r] - np.float32(ref)) < 2.0e-4


def test_q6_k_dequant_known_answer(zo):
    # tests/core_tests.cpp:304-309
    blk = np.zeros(210, np.uint8)
    blk[208], blk[209] = 0x00, 0x3C
    blk[192:208] = 1
    blk[0] = 1
    out = zo.dequantize(Q6_K, blk, 256)
    assert out[0] == -31.0
    assert np.all(np.delete(out, 0) == -32.0)


def test_q6_k_single_block_gemv(zo):
    # tests/core_tests.cpp:326-333 (check_quant_gemv on a Q6_K block of bytes i*11)
    blk = np.zeros(210, np.uint8)
    blk[:208] = (np.arange(208) * 11) & 255
    blk[208], blk[209] = 0x00, 0x3C
    x = ((np.arange(256) % 17 - 8) * 0.03125).astype(np.float32)
    got = zo.gemv(Q6_K, blk, x, 1, 256)[0]
    ref = float(np.dot(zo.dequantize(Q6_K, blk, 256).astype(np.float64), x.astype(np.float64)))
    assert abs(got - ref) < 1.0e-3 * max(1.0, abs(ref))


def test_q8_0_gemm_token_ladder(zo):
    # tests/core_tests.cpp:345-372: rows=100, cols=544 (17 blocks), T in {5,7,8,9,16}, rel 1e-3
    rows, cols = 100, 544
    r = np.arange(rows)[:, None, None]
    blk = np.arange(17)[None, :, None]
    j = np.arange(2, 34)[None, None, :]
    packed = np.zeros((rows, 17, 34), np.uint8)
    packed[..., 1] = 0x3C
    packed[..., 2:] = (r * 5 + blk * 11 + j * 3) & 255
    ref_w = zo.dequantize(Q8_0, packed, rows * cols).reshape(rows, cols).astype(np.float64)
    for T in (5, 7, 8, 9, 16):
        t = np.arange(T)[:, None]
        c = np.arange(cols)[None, :]
        xin = (((t * 7 + c) % 15 - 7).astype(np.float32) * np.float32(0.017)).astype(np.float32)
        out = zo.gemm(Q8_0, packed, xin, T, rows, cols)
        expect = xin.astype(np.float64) @ ref_w.T
        assert np.all(np.abs(out - expect.astype(np.float32)) <= 1.0e-3 * np.maximum(1.0, np.abs(expect)))


@pytest.mark.parametrize("cols,rows", [(96, 1), (96, 3), (2048, 2), (2048, 100), (8192, 3)])
def test_q8_0_kblk_sweep(zo, cols, rows):
    # tests/core_tests.cpp:411-447 (a subset of its shape grid; same LCG fixture, same tolerance)
    nblk = cols // 32
    stream = lcg_bytes(12345 + ((rows * 1000003 + cols) & 0xFFFFFFFF), rows * nblk * 32).reshape(rows, nblk, 32)
    packed = np.zeros((rows, nblk, 34), np.uint8)
    packed[..., 1] = 0x3C
    packed[..., 2:] = stream
    ref_w = zo.dequantize(Q8_0, packed, rows * cols).reshape(rows, cols).astype(np.float64)
    for T in (2, 3, 5, 8, 171):
        t = np.arange(T)[:, None]
        c = np.arange(cols)[None, :]
        xin = (((t * 7 + c) % 15 - 7).astype(np.float32) * np.float32(0.017)
               + ((t * 13 + c * 3) % 7 - 3).astype(np.float32) * np.float32(0.001)).astype(np.float32)
        expect = xin.astype(np.float64) @ ref_w.T
        for kblk in (False, True):
            out = zo.gemm_q8_0_f32(packed, xin, T, rows, cols, kblk=kblk)
            err = np.abs(out.astype(np.float64) - expect)
            i = np.unravel_index(err.argmax(), err.shape)
            assert err[i] <= 1.5e-3 * max(1.0, abs(expect[i]))


def test_q6_k_constructed_blocks(zo):
    fx = _Q6KFixture()
    for cols in (256, 512, 768):
        for rows in (1, 3, 4, 5, 35):
            packed, expected = fx.weights(rows, cols)
            assert np.array_equal(zo.dequantize(Q6_K, packed, rows * cols).reshape(rows, cols), expected)
            assert np.array_equal(blocks.dequantize(Q6_K, packed, rows, cols), expected)
            for tokens in (1, 2, 3, 5):
                x = np.array([(float((fx.u32() >> 24) - 128) / 128.0) for _ in range(tokens * cols)], np.float32).reshape(tokens, cols)
                terms = expected.astype(np.float64)[None, :, :] * x.astype(np.float64)[:, None, :]
                ref, mag = terms.sum(axis=2), np.abs(terms).sum(axis=2)
                tol = 2e-5 * np.maximum(1.0, mag)
                if tokens == 1:
                    assert np.all(np.abs(zo.gemv(Q6_K, packed, x[0], rows, cols) - ref[0]) <= tol[0])
                assert np.all(np.abs(zo.gemm(Q6_K, packed, x, tokens, rows, cols) - ref) <= tol)


@pytest.mark.parametrize("fmt", [Q4_0, Q8_0, Q6_K])
def test_all_format_sweep_fixture(zo, fmt):
    # tests/cpu_quant_sweep_tests.cpp:12-50 over tests/support/quant_fixture.h (LCG seed 1729,
    # block scale forced to f16 0x3000): |out - sum| <= 2e-5 * max(1, sum|terms|)
    for cols in (256, 768):
        for rows in (1, 5, 67):
            rb = blocks.row_bytes(fmt, cols)
            w = lcg_bytes(1729, rows * rb).reshape(rows, cols // blocks.BLOCK_ELEMENTS[fmt], blocks.BLOCK_BYTES[fmt]).copy()
            at = 208 if fmt == Q6_K else 0
            w[..., at], w[..., at + 1] = 0, 0x30
            decoded = zo.dequantize(fmt, w, rows * cols).reshape(rows, cols)
            assert np.all(np.isfinite(decoded))
            assert np.array_equal(decoded, blocks.dequantize(fmt, w, rows, cols))
            x = (((np.arange(8 * cols) * 37 + 11) % 101 - 50) / 64.0).astype(np.float32).reshape(8, cols)
            for tokens in (1, 2, 3, 8):
                terms = decoded.astype(np.float64)[None] * x[:tokens].astype(np.float64)[:, None, :]
                ref, mag = terms.sum(axis=2), np.abs(terms).sum(axis=2)
                out = zo.gemm(fmt, w, x[:tokens], tokens, rows, cols)
                assert np.all(np.abs(out - ref) <= 2e-5 * np.maximum(1.0, mag))


def test_argmax_rule(zo):
    # src/adapters/dense_transformer_runtime.cpp:407-415: first maximum wins, non-finite never wins
    assert zo.argmax([1.0, 3.0, 3.0, 2.0]) == 1
    assert zo.argmax([float("nan"), float("inf"), -5.0, -5.0]) == 2
    assert zo.argmax([float("nan"), float("-inf")]) == -1
    assert zo.argmax([-0.0, 0.0]) == 0


def test_row_slices_tile_the_range(zo):
    # src/compute_pool.cpp:104-106
    for count, workers in ((128256, 8), (4096, 3), (67, 4), (5, 5)):
        cuts = [zo.row_slice(count, workers, i) for i in range(workers)]
        assert cuts[0][0] == 0 and cuts[-1][1] == count
        assert all(cuts[i][1] == cuts[i + 1][0] for i in range(workers - 1))
        assert cuts == [(count * i // workers, count * (i + 1) // workers) for i in range(workers)]


# ---- 2. committed outputs of the unmodified reference ------------------------

@pytest.fixture(scope="module")
def golden():
    with np.load(GOLDEN) as g:
        return {k: g[k] for k in g.files}


@pytest.mark.parametrize("name,fmt", [("q8_0", Q8_0), ("q4_0", Q4_0), ("q6_k", Q6_K)])
def test_golden_gemv_gemm_bit_exact(zo, golden, name, fmt):
    w, x = golden[f"{name}_w"], golden[f"{name}_x"]
    rows, cols, tokens = 37, 768, 5
    assert np.array_equal(zo.gemv(fmt, w, x[0], rows, cols), golden[f"{name}_gemv_y"])
    assert np.array_equal(zo.gemm(fmt, w, x, tokens, rows, cols), golden[f"{name}_gemm_y"])


def test_golden_kblk_route_bit_exact(zo, golden):
    from golden.make_golden import formula_acts
    x = formula_acts(64, 2048)
    assert np.array_equal(zo.gemm(Q8_0, golden["q8_0_kblk_w"], x, 64, 10, 2048), golden["q8_0_kblk_y"])


def test_golden_activation_codes_bit_exact(zo, golden):
    # An identity Q8_0 matrix with unit scales makes the reference return scale*code per
    # element, so its int8-activation GEMV exposes the quantiser's codes and scales.
    x = golden["i8_ident_x"]
    q, sc = zo.quantise_acts(x)
    deq = (q.astype(np.float32).reshape(x.shape[0], -1, 32) * sc[..., None]).reshape(x.shape)
    assert np.array_equal(deq, golden["i8_ident_y"])
    assert np.all(q[4, :32] == 0) and sc[4, 0] == 0  # the all-zero block (first of the edge rows)
    assert np.abs(q).max() <= 127


def test_golden_int8_gemv_bit_exact(zo, golden):
    w, x = golden["i8_gemv_w"], golden["i8_gemv_x"]
    y = np.stack([zo.gemv(Q8_0, w, xi, 67, 544, int8_acts=True) for xi in x])
    assert np.array_equal(y, golden["i8_gemv_y"])
    assert np.array_equal(y, golden["i8_gemv_y_w4"])  # worker count does not change the reference's result


# ---- 3. the compiled reference, bit for bit ----------------------------------

@pytest.mark.parametrize("fmt", [Q8_0, Q4_0, Q6_K])
def test_oracle_equals_compiled_reference(zo, zr, fmt):
    rng = np.random.default_rng(5 + fmt)
    for rows, cols, tokens in ((1, 256, 1), (3, 512, 2), (9, 1024, 4), (70, 768, 7), (33, 4096, 33)):
        w = blocks.quantize(fmt, rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02))
        x = rng.standard_normal((tokens, cols), dtype=np.float32)
        assert zo.row_bytes(fmt, cols) == zr.row_bytes(fmt, cols) == blocks.row_bytes(fmt, cols)
        assert np.array_equal(zo.dequantize(fmt, w, rows * cols), zr.dequantize(fmt, w, rows * cols))
        assert np.array_equal(zo.gemv(fmt, w, x[0], rows, cols), zr.gemv(fmt, w, x[0], rows, cols, workers=1))
        assert np.array_equal(zo.gemm(fmt, w, x, tokens, rows, cols), zr.gemm(fmt, w, x, tokens, rows, cols, workers=1))


def test_oracle_int8_sweep_equals_compiled_reference(zo, zr):
    rng = np.random.default_rng(9)
    for rows, cols in ((5, 96), (67, 544), (130, 4096)):
        w = blocks.quantize(Q8_0, rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02))
        xq, xsc = zo.quantise_acts(rng.standard_normal(cols, dtype=np.float32))
        assert np.array_equal(zo.gemv_q8_0_i8_prequant(w, xq, xsc, rows, cols), zr.gemv_q8_0_i8_prequant(w, xq, xsc, rows, cols))


def test_fp16_encode_equals_compiled_reference(zo, zr):
    rng = np.random.default_rng(3)
    v = np.concatenate([rng.standard_normal(4096).astype(np.float32) * np.float32(s) for s in (1e-8, 1e-4, 1.0, 1e4, 1e6)])
    ref = zr.encode_fp16(v)
    assert np.array_equal(ref, np.array([zo.float_to_half(float(f)) for f in v], np.uint16))
    with np.errstate(over="ignore"):
        as_half = v.astype(np.float16)
    finite = np.isfinite(as_half.astype(np.float32)) & (np.abs(v) >= 2.0 ** -126)
    assert np.array_equal(ref[finite], as_half.view(np.uint16)[finite])
    assert np.array_equal(zr.decode_fp16(np.arange(0x7C00, dtype=np.uint16)), np.arange(0x7C00, dtype=np.uint16).view(np.float16).astype(np.float32))


def test_quantiser_matches_reference_q8_requantiser(zo):
    # blocks.quantize_q8_0 restates src/quant.cpp:1265-1276; a Q8_0 matrix pushed through
    # dequantise -> quantise must come back byte-identical when codes reach +-127 in a block.
    rng = np.random.default_rng(12)
    w = rng.standard_normal((8, 512), dtype=np.float32) * np.float32(0.02)
    p1 = blocks.quantize_q8_0(w)
    deq = zo.dequantize(Q8_0, p1, 8 * 512).reshape(8, 512)
    codes = p1.reshape(8, 16, 34)[..., 2:].view(np.int8)
    assert np.abs(codes).max(axis=2).min() == 127  # amax element always lands on +-127
    err = np.abs(deq - w).reshape(8, 16, 32).max(axis=2)
    scale = p1.reshape(8, 16, 34)[..., :2].copy().view(np.float16).astype(np.float32)[..., 0]
    # half a step from rounding the code, plus up to 127 steps times the binary16 rounding of the scale
    assert np.all(err <= scale * (0.5 + 127 * 2.0 ** -11) * 1.001 + 1e-12)
