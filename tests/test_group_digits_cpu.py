"""The arithmetic of the group-scale many-row product (zeninfer_b200/csrc/gemm_groups.cuh), restated in numpy and held to
its accuracy claim on the CPU: weights and activations as two int8 digits under one unit per 256 values, the low x low term
dropped, one fp32 multiply-add per group.  The GPU test compares the kernel with this restatement; here the restatement is
compared with float64 sums of the reference's arithmetic."""
import numpy as np
import pytest

from helpers import group_digits, group_product, ref_fp32_f64, ref_int8_f64, seeded_acts, seeded_weights
from zeninfer_b200 import blocks

Q8_0 = blocks.Q8_0


def test_digits_reconstruct_to_sixteen_bits():
    v = np.random.default_rng(1).standard_normal((7, 1024)).astype(np.float32)
    v[0, :256] = 0.0                       # an all-zero group: unit 0, digits 0
    v[1, 300] = 50.0                       # an outlier stretches its group's unit only
    hi, lo, unit = group_digits(v)
    assert hi.min() >= -127 and hi.max() <= 127 and lo.min() >= -128 and lo.max() <= 127
    assert unit[0, 0] == 0 and not hi[0, :256].any() and not lo[0, :256].any()
    back = (unit[..., None].astype(np.float64) * (256 * hi + lo).reshape(7, 4, 256)).reshape(7, 1024)
    amax = np.abs(v.reshape(7, 4, 256)).max(axis=2)
    bound = np.repeat(amax / 65278.0 * 1.001 + 1e-12, 256, axis=1)          # half a unit
    assert np.all(np.abs(back - v) <= bound)
    assert (256 * hi + lo)[1, 300] == 32639


@pytest.mark.parametrize("tokens,rows,cols", [(5, 64, 256), (16, 96, 4096), (9, 40, 14336)])
def test_group_product_meets_the_bar_in_both_activation_modes(zo, tokens, rows, cols):
    w = seeded_weights(Q8_0, rows, cols, 40 + rows)
    x = seeded_acts(tokens, cols, 50 + tokens)
    wv = blocks.dequantize(Q8_0, w, rows, cols)                              # d * q, exact in fp32
    # fp32-equivalent activations: x itself gets the digits
    got = group_product(wv, x).astype(np.float64)
    ref = ref_fp32_f64(Q8_0, w, x, rows, cols)
    assert np.abs(got - ref).max() / np.abs(ref).max() < 2e-4
    assert np.all(np.abs(got - ref) <= 1e-3 * np.maximum(1.0, np.abs(ref)))
    # int8 activations: the reference quantises per 32-block first (kernels/avx2.cpp:502-524); d_x * q_x gets the digits
    xq, xsc = zo.quantise_acts(x)
    xv = (xq.astype(np.float32).reshape(tokens, -1, 32) * xsc.astype(np.float32)[..., None]).reshape(tokens, cols)
    got8 = group_product(wv, xv).astype(np.float64)
    ref8 = ref_int8_f64(w, xq, xsc, rows, cols)
    assert np.abs(got8 - ref8).max() / np.abs(ref8).max() < 2e-4
    assert np.all(np.abs(got8 - ref8) <= 1e-3 * np.maximum(1.0, np.abs(ref8)))


@pytest.mark.parametrize("fmt", [blocks.Q4_0, blocks.Q6_K, blocks.Q4_K, blocks.Q5_K])
def test_group_product_on_the_other_formats(fmt):
    # the same arithmetic on the dequantised values of the other formats (w = d (n - 8), (d sc) q, (d sc) q - dmin m): the
    # error is relative to the largest result, which is how the GPU tests of these formats gate the group-scale kernel
    rows, cols, tokens = 48, 2048, 6
    if fmt in (blocks.Q4_K, blocks.Q5_K):
        w = blocks.random_k_blocks(fmt, rows, cols, 77)
    else:
        w = seeded_weights(fmt, rows, cols, 77)
    x = seeded_acts(tokens, cols, 78)
    got = group_product(blocks.dequantize(fmt, w, rows, cols), x).astype(np.float64)
    ref = ref_fp32_f64(fmt, w, x, rows, cols)
    assert np.abs(got - ref).max() / np.abs(ref).max() < 3e-4
