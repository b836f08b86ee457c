"""The two fused host-pointer submissions of the backend contract (include/zen/hip_backend.h:74-83 in the reference):
rms_norm and gemv_q8_0_ffn.  The reference's CPU path for the same work is rms_norm
(src/adapters/dense_transformer_runtime.cpp:117-125) and three gemv calls with silu(g) * u between them, which is what
the oracle composes here."""
import numpy as np
import pytest

from helpers import assert_parity, ref_fp32_f64, seeded_acts, seeded_weights
from oracle.llama import _rms_norm
from zeninfer_b200 import blocks
from zeninfer_b200.backend import ACT_FP32, ACT_INT8, BackendError

pytestmark = pytest.mark.gpu
Q8_0 = blocks.Q8_0


@pytest.fixture()
def be():
    from zeninfer_b200 import Backend
    b = Backend()
    yield b
    b.set_q8_act_mode(ACT_INT8)


@pytest.mark.parametrize("rows,cols", [(1, 4096), (1, 100), (7, 257), (3, 14336), (512, 4096), (16, 8)])
def test_rms_norm_matches_the_reference_arithmetic(be, rows, cols):
    rng = np.random.default_rng(rows * 131 + cols)
    x = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(3.0)
    w = rng.standard_normal(cols, dtype=np.float32)
    eps = 1e-5
    got = be.rms_norm(x, w, eps)
    ref = np.stack([_rms_norm(x[r], w, eps) for r in range(rows)])
    # same formula, float for float: the sum of squares is taken in double on both sides, so at most its last bit differs
    assert_parity(got, ref, 1e-6, f"rms_norm {rows}x{cols}")
    assert np.mean(got.view(np.uint32) == ref.view(np.uint32)) > 0.99
    x64 = x.astype(np.float64)
    assert_parity(got, x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + eps) * w, 1e-5, "rms_norm vs float64")


def test_rms_norm_edge_cases(be):
    before = be.stats()["fallbacks"]
    with pytest.raises(BackendError):
        be.rms_norm(np.empty((0, 64), np.float32), np.ones(64, np.float32), 1e-5)
    assert be.stats()["fallbacks"] == before + 1
    zeros = be.rms_norm(np.zeros((2, 64), np.float32), np.ones(64, np.float32), 1e-6)
    assert np.array_equal(zeros, np.zeros((2, 64), np.float32))


def _silu_mul(g, u):
    g = g.astype(np.float32)
    return (g / (np.float32(1.0) + np.exp(-g, dtype=np.float32)) * u).astype(np.float32)


@pytest.mark.parametrize("ffn_rows,cols,out_rows", [(96, 64, 5), (1024, 256, 256), (14336, 4096, 4096)])
def test_ffn_submission(be, zo, ffn_rows, cols, out_rows):
    gate = seeded_weights(Q8_0, ffn_rows, cols, 700)
    up = seeded_weights(Q8_0, ffn_rows, cols, 701)
    down = seeded_weights(Q8_0, out_rows, ffn_rows, 702)
    x = seeded_acts(1, cols, 703)[0]
    # fp32-equivalent activations against float64 end to end
    be.set_q8_act_mode(ACT_FP32)
    before = be.stats()
    y = be.gemv_ffn(gate, up, down, x, ffn_rows, cols, out_rows)
    after = be.stats()
    assert after["submits"] == before["submits"] + 1 and after["batches"] == before["batches"] + 1
    assert after["dispatches"] - before["dispatches"] <= 3 + 4      # fetch, gate|up, down, copy-out (+ the repacks of a first call)
    g64 = ref_fp32_f64(Q8_0, gate, x, ffn_rows, cols)[0]
    u64 = ref_fp32_f64(Q8_0, up, x, ffn_rows, cols)[0]
    a64 = g64 / (1.0 + np.exp(-g64)) * u64
    assert_parity(y, ref_fp32_f64(Q8_0, down, a64, out_rows, ffn_rows)[0], 1e-3, f"ffn fp32 activations {ffn_rows}x{cols}->{out_rows}")
    # the three separate host calls give the same numbers as the fused submission up to the float ops of silu(g) * u
    g, u = be.gemv_batch("Q8_0", [gate, up], x, [ffn_rows, ffn_rows], cols)
    assert_parity(y, be.gemv("Q8_0", down, _silu_mul(g, u), out_rows, ffn_rows), 1e-4, "fused vs three calls, fp32 activations")
    # int8 activations against the oracle's chain (one activation code that rounds the other way moves a result by a
    # block scale, hence the wider bar than for a single product)
    be.set_q8_act_mode(ACT_INT8)
    y8 = be.gemv_ffn(gate, up, down, x, ffn_rows, cols, out_rows)
    go = zo.gemv(Q8_0, gate, x, ffn_rows, cols, int8_acts=True)
    uo = zo.gemv(Q8_0, up, x, ffn_rows, cols, int8_acts=True)
    assert_parity(y8, zo.gemv(Q8_0, down, _silu_mul(go, uo), out_rows, ffn_rows, int8_acts=True), 5e-3, "ffn int8 activations vs the oracle chain")
    y8b = be.gemv_ffn(gate, up, down, x, ffn_rows, cols, out_rows)
    assert np.array_equal(y8, y8b)
    for w in (gate, up, down):
        be.release_weights(w)


def test_ffn_bad_arguments(be):
    w = seeded_weights(Q8_0, 32, 32, 1)
    x = np.ones(32, np.float32)
    with pytest.raises(BackendError):
        be.gemv_ffn(w, w, w, x, 0, 32, 32)
    with pytest.raises(BackendError):
        be.gemv_ffn(w, w, w, np.ones(48, np.float32), 32, 48, 32)      # columns not a multiple of 32
