"""GPU parity for the Q4_0 and Q6_K decode paths, through the C-ABI.

The reference computes both formats with fp32 activations (Q4_0: dequantise the row, then a fp32 dot,
src/quant.cpp:1135-1162; Q6_K: gemv_q6k_avx2 / gemm_q6k_kblk_avx2), so the oracle here is always the
fp32-activation one.  Bar: 1e-3 under both gates of helpers.assert_parity; the integer kernels land near 1e-5.
"""
import os

import numpy as np
import pytest

from helpers import Q6KFixture as _Q6KFixture
from helpers import assert_parity, ref_fp32_f64, seeded_acts, seeded_weights
from conftest import lcg_bytes
from zeninfer_b200 import blocks

pytestmark = pytest.mark.gpu
Q4_0, Q6_K = blocks.Q4_0, blocks.Q6_K
NAMES = {Q4_0: "Q4_0", Q6_K: "Q6_K"}
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz")


@pytest.fixture(scope="module")
def be():
    from zeninfer_b200 import Backend
    return Backend()


@pytest.fixture(scope="module")
def golden():
    with np.load(GOLDEN) as g:
        return {k: g[k] for k in g.files}


@pytest.mark.parametrize("fmt,key", [(Q4_0, "q4_0"), (Q6_K, "q6_k")])
def test_against_reference_golden(be, golden, fmt, key):
    w = np.ascontiguousarray(golden[f"{key}_w"])
    x = golden[f"{key}_x"]
    assert_parity(be.gemv(NAMES[fmt], w, x[0], 37, 768), golden[f"{key}_gemv_y"], what=f"golden {key} gemv")
    assert_parity(be.gemm(NAMES[fmt], w, x, 5, 37, 768), golden[f"{key}_gemm_y"], what=f"golden {key} gemm")
    be.release_weights(w)


@pytest.mark.parametrize("rows,cols", [(1, 32), (3, 96), (5, 256), (67, 544), (130, 2048), (512, 4096), (1024, 4096), (64, 14336)])
def test_q4_0_gemv_vs_oracle(be, zo, rows, cols):
    w = seeded_weights(Q4_0, rows, cols, 110 + rows)
    x = seeded_acts(1, cols, 120 + cols)[0]
    rel = assert_parity(be.gemv("Q4_0", w, x, rows, cols), zo.gemv(Q4_0, w, x, rows, cols), what=f"Q4_0 gemv {rows}x{cols}")
    assert rel < 1e-4
    be.release_weights(w)


@pytest.mark.parametrize("rows,cols", [(1, 256), (3, 512), (5, 768), (67, 1280), (512, 4096), (1024, 4096), (64, 14336)])
def test_q6_k_gemv_vs_oracle(be, zo, rows, cols):
    w = seeded_weights(Q6_K, rows, cols, 130 + rows)
    x = seeded_acts(1, cols, 140 + cols)[0]
    rel = assert_parity(be.gemv("Q6_K", w, x, rows, cols), zo.gemv(Q6_K, w, x, rows, cols), what=f"Q6_K gemv {rows}x{cols}")
    assert rel < 1e-4
    be.release_weights(w)


@pytest.mark.parametrize("fmt", [Q4_0, Q6_K])
@pytest.mark.parametrize("tokens", [2, 3, 5, 8, 9, 17])
def test_small_batch_vs_oracle(be, zo, fmt, tokens):
    rows, cols = 100, 768
    w = seeded_weights(fmt, rows, cols, 150 + fmt)
    x = seeded_acts(tokens, cols, 160 + tokens)
    assert_parity(be.gemm(NAMES[fmt], w, x, tokens, rows, cols), zo.gemm(fmt, w, x, tokens, rows, cols), what=f"{NAMES[fmt]} T={tokens}")
    be.release_weights(w)


def test_q6_k_constructed_blocks(be):
    # tests/q6k_gemm_tests.cpp:16-45: blocks built from known codes and scales, expected weights computed
    # without any decoder; gate 2e-5 * max(1, sum|terms|)
    fx = _Q6KFixture()
    for cols in (256, 512, 1280):
        for rows in (1, 3, 5, 35):
            packed, expected = fx.weights(rows, cols)
            packed = np.ascontiguousarray(packed.reshape(rows, -1))
            for tokens in (1, 2, 5):
                x = np.array([(float((fx.u32() >> 24) - 128) / 128.0) for _ in range(tokens * cols)], np.float32).reshape(tokens, cols)
                terms = expected.astype(np.float64)[None, :, :] * x.astype(np.float64)[:, None, :]
                ref, mag = terms.sum(axis=2), np.abs(terms).sum(axis=2)
                got = be.gemm("Q6_K", packed, x, tokens, rows, cols)
                assert np.all(np.abs(got - ref) <= 2e-5 * np.maximum(1.0, mag)), (cols, rows, tokens)
            be.release_weights(packed)


@pytest.mark.parametrize("fmt", [Q4_0, Q6_K])
def test_all_format_sweep_fixture(be, zo, fmt):
    # tests/cpu_quant_sweep_tests.cpp:12-50 over tests/support/quant_fixture.h: random block bytes (LCG 1729),
    # every nibble / 6-bit code / int8 scale value occurs
    for cols in (256, 768):
        for rows in (1, 5, 67):
            rb = blocks.row_bytes(fmt, cols)
            w = lcg_bytes(1729, rows * rb).reshape(rows, cols // blocks.BLOCK_ELEMENTS[fmt], blocks.BLOCK_BYTES[fmt]).copy()
            at = 208 if fmt == Q6_K else 0
            w[..., at], w[..., at + 1] = 0, 0x30
            w = np.ascontiguousarray(w.reshape(rows, -1))
            decoded = zo.dequantize(fmt, w, rows * cols).reshape(rows, cols).astype(np.float64)
            x = (((np.arange(8 * cols) * 37 + 11) % 101 - 50) / 64.0).astype(np.float32).reshape(8, cols)
            for tokens in (1, 3, 8):
                terms = decoded[None] * x[:tokens].astype(np.float64)[:, None, :]
                ref, mag = terms.sum(axis=2), np.abs(terms).sum(axis=2)
                got = be.gemm(NAMES[fmt], w, x[:tokens], tokens, rows, cols)
                assert np.all(np.abs(got - ref) <= 2e-5 * np.maximum(1.0, mag)), (cols, rows, tokens)
            be.release_weights(w)


@pytest.mark.parametrize("fmt", [Q4_0, Q6_K])
def test_layer_shapes_full_size(be, fmt):
    # one Llama-3-8B layer (seed 4): q/o 4096x4096, k/v 1024x4096, gate/up 14336x4096, down 4096x14336
    for i, (rows, cols) in enumerate(((4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336))):
        w = seeded_weights(fmt, rows, cols, 4 + 10 * i)
        x = seeded_acts(1, cols, 4 + 10 * i + 1)
        y = be.gemv(NAMES[fmt], w, x[0], rows, cols)
        rel = assert_parity(y, ref_fp32_f64(fmt, w, x, rows, cols)[0], what=f"{NAMES[fmt]} {rows}x{cols}")
        assert rel < 1e-4  # max_abs/max_ref; two activation digits leave ~2e-5
        be.release_weights(w)


def test_int8_mode_is_q8_0_only(be):
    from zeninfer_b200 import BackendError
    from zeninfer_b200.backend import ACT_INT8
    w = seeded_weights(Q4_0, 16, 256, 170)
    h = be.dev_upload("Q4_0", w, 16, 256)
    with pytest.raises(BackendError):
        be.dev_gemv([h], [1], 1, 1, ACT_INT8)  # rejected on the host before any pointer is touched
    be.dev_free(h)


@pytest.mark.parametrize("fmt", [Q4_0, Q6_K])
def test_long_run_of_overlapped_launches_is_deterministic(be, zo, fmt):
    """Thousands of launches back to back on one stream over several weight copies: every launch must reproduce the first
    launch's bits and leave the error word clear (the ring protocol under overlap, as in the Q8_0 test of the same name)."""
    import torch
    rows = cols = 4096
    dev = torch.device("cuda", 0)
    copies, outs, rounds = 8, 64, 150
    w = seeded_weights(fmt, rows, cols, 60)
    handles = [be.dev_upload(NAMES[fmt], w, rows, cols) for _ in range(copies)]
    x = seeded_acts(1, cols, 61)
    d_x = torch.from_numpy(x).to(dev)
    d_y = torch.zeros((outs, rows), dtype=torch.float32, device=dev)
    ptrs = [d_y[i].data_ptr() for i in range(outs)]
    stream = torch.cuda.Stream(device=dev)
    bad = torch.zeros((), dtype=torch.int64, device=dev)
    with torch.cuda.stream(stream):
        be.dev_gemv([handles[0]], [ptrs[0]], d_x.data_ptr(), 1, 2, stream.cuda_stream)
        stream.synchronize()
        first = d_y[0].clone()
        for rnd in range(rounds):
            for i in range(outs):
                be.dev_gemv([handles[(rnd + i) % copies]], [ptrs[i]], d_x.data_ptr(), 1, 2, stream.cuda_stream)
            bad += (d_y != first[None, :]).sum()
            d_y.zero_()
            if rnd % 16 == 15:
                stream.synchronize()
        stream.synchronize()
    be.dev_check(stream.cuda_stream)
    assert int(bad.item()) == 0
    assert_parity(first.cpu().numpy(), zo.gemv(fmt, w, x[0], rows, cols), what=f"{NAMES[fmt]} first launch vs oracle")
    for h in handles:
        be.dev_free(h)


@pytest.mark.parametrize("rows,cols,tokens", [(1, 256, 1), (67, 1280, 1), (1027, 4096, 1), (64, 14336, 1), (130, 2048, 3), (300, 4096, 8), (9, 4352, 11)])
def test_q6_k_both_device_layouts_give_the_same_bits(be, zo, golden, rows, cols, tokens):
    # the default device layout keeps the 6-bit codes unpacked (one int8 per weight); the file's ql | qh planes remain
    # selectable.  Both kernels form the same integer sums, so the results are equal bit for bit, and both meet the oracle.
    import torch
    from zeninfer_b200.backend import ACT_FP32
    w = seeded_weights(Q6_K, rows, cols, 800 + rows)
    x = seeded_acts(tokens, cols, 810 + cols)
    outs, sizes = [], []
    before = be.set_q6k_codes(True)
    try:
        for codes in (True, False):
            be.set_q6k_codes(codes)
            h = be.dev_upload("Q6_K", w, rows, cols)
            sizes.append(be.dev_weight_bytes(h))
            d_x = torch.from_numpy(x).cuda()
            y = torch.zeros((tokens, rows), device="cuda")
            step = 8 if cols <= 4096 else 2      # the activation rows of a launch share shared memory with the weight ring
            for t0 in range(0, tokens, step):
                n = min(step, tokens - t0)
                be.dev_gemv([h], [y[t0:].data_ptr()], d_x[t0:].data_ptr(), n, ACT_FP32)
            be.dev_check()
            outs.append(y.cpu().numpy())
            be.dev_free(h)
        host = be.gemm("Q6_K", w, x, tokens, rows, cols)        # the host-pointer call, resident in the layout set last
        be.release_weights(w)
    finally:
        be.set_q6k_codes(before)
    assert np.array_equal(outs[0], outs[1])
    assert_parity(host, outs[1], 1e-5, "host-pointer call")    # its token chunks may differ: a one-token launch sums a row in another order
    assert sizes[0] >= sizes[1] and (rows * cols < 65536 or sizes[0] > 1.25 * sizes[1])     # 1.07 against 0.82 bytes per weight, plus 64 bytes of slack per plane
    ref = np.stack([zo.gemv(Q6_K, w, x[t], rows, cols) for t in range(tokens)])
    assert_parity(outs[0], ref, what=f"Q6_K unpacked codes {tokens}x{rows}x{cols}")


@pytest.mark.parametrize("fmt", [Q4_0, Q6_K])
@pytest.mark.parametrize("rows,cols,tokens", [(1027, 8192, 1), (77, 12288, 1), (301, 14336, 3), (4096, 14336, 1), (13, 4608, 1)])
def test_rows_of_several_segments(be, zo, fmt, rows, cols, tokens):
    # more than 4096 columns: a row group's segment arrives by one tiled copy per plane (partial groups by boxes of 4, 2
    # and 1 rows; 4608 columns have a pitch that is not a multiple of 256 in some planes and take the per-row copies)
    w = seeded_weights(fmt, rows, cols, 700 + rows)
    x = seeded_acts(tokens, cols, 710 + cols)
    for codes in ((True, False) if fmt == Q6_K else (True,)):
        before = be.set_q6k_codes(codes)
        try:
            got = be.gemm(NAMES[fmt], w, x, tokens, rows, cols)
            be.release_weights(w)
        finally:
            be.set_q6k_codes(before)
        ref = np.stack([zo.gemv(fmt, w, x[t], rows, cols) for t in range(tokens)])
        rel = assert_parity(got, ref, what=f"{NAMES[fmt]} {tokens}x{rows}x{cols} codes={codes}")
        assert rel < 1e-4


@pytest.mark.parametrize("rows,cols,tokens", [(1, 256, 2), (130, 2048, 3), (300, 4096, 8), (1027, 1280, 16), (64, 14336, 5), (9, 4352, 37), (19000, 512, 8), (130, 2048, 70), (300, 1024, 129)])
def test_q6_k_tensor_core_product_vs_oracle(be, zo, rows, cols, tokens):
    # two or more activation rows: the tcgen05 product with one column per token and group parity (the batched lm_head of
    # config 3, the reference's gemm_q6k_kblk_avx2); device pointers and a caller workspace, then the host-pointer call.
    # 19000 rows are 149 row tiles: one more than the SMs, so the K range of a tile is shared between two CTAs.  More than
    # sixteen rows take the 128-column tiles of the prefill GEMM (64 tokens a tile).
    import torch
    w = seeded_weights(Q6_K, rows, cols, 900 + rows)
    x = seeded_acts(tokens, cols, 910 + cols)
    ref = np.stack([zo.gemv(Q6_K, w, x[t], rows, cols) for t in range(tokens)])
    h = be.dev_upload("Q6_K", w, rows, cols)
    d_x = torch.from_numpy(x).cuda()
    y = torch.full((tokens, rows), float("nan"), device="cuda")
    ws_bytes = be.gemm_q6_k_workspace_bytes(tokens, cols)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
    # more than sixteen rows take the group-scale kernel (two digits per 256-weight group, ~5e-5); with it switched off, and
    # up to sixteen rows, the per-block kernel with one column per token and group parity (~1e-5)
    for groups in (True, False):
        before = be.set_gemm_groups(groups)
        try:
            y.fill_(float("nan"))
            be.dev_gemm_q6_k(h, y.data_ptr(), d_x.data_ptr(), tokens, ws.data_ptr(), ws_bytes)
            be.dev_check()
        finally:
            be.set_gemm_groups(before)
        rel = assert_parity(y.cpu().numpy(), ref, what=f"Q6_K tensor product {tokens}x{rows}x{cols} groups={groups}")
        assert rel < (3e-4 if groups and tokens > 16 else 1e-4)
    be.dev_free(h)
    host = be.gemm("Q6_K", w, x, tokens, rows, cols)
    assert_parity(host, ref, what="host-pointer call")
    be.release_weights(w)


def test_q6_k_tensor_core_product_needs_the_unpacked_codes(be):
    import torch
    rows, cols, tokens = 64, 512, 4
    w = seeded_weights(Q6_K, rows, cols, 950)
    before = be.set_q6k_codes(False)
    try:
        h = be.dev_upload("Q6_K", w, rows, cols)
    finally:
        be.set_q6k_codes(before)
    d_x = torch.zeros((tokens, cols), device="cuda")
    y = torch.zeros((tokens, rows), device="cuda")
    ws_bytes = be.gemm_q6_k_workspace_bytes(tokens, cols)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
    from zeninfer_b200.backend import BackendError
    with pytest.raises(BackendError, match="codes unpacked"):
        be.dev_gemm_q6_k(h, y.data_ptr(), d_x.data_ptr(), tokens, ws.data_ptr(), ws_bytes)
    be.dev_free(h)


@pytest.mark.parametrize("rows,cols,tokens", [(300, 4096, 40), (1027, 1280, 33), (64, 14336, 64), (130, 2048, 129), (7, 128, 12)])
def test_q4_0_tensor_core_product_vs_oracle(be, zo, rows, cols, tokens):
    # many activation rows: nibbles widened to int8 codes n - 8 in the workspace, then the Q8_0 GEMM with two activation
    # digits; the oracle is the reference's fp32-activation route for Q4_0.  Device entry point, then the host-pointer call
    # (which takes the same path from nine rows on).
    import torch
    w = seeded_weights(Q4_0, rows, cols, 960 + rows)
    x = seeded_acts(tokens, cols, 970 + cols)
    ref = np.stack([zo.gemv(Q4_0, w, x[t], rows, cols) for t in range(tokens)])
    h = be.dev_upload("Q4_0", w, rows, cols)
    d_x = torch.from_numpy(x).cuda()
    y = torch.full((tokens, rows), float("nan"), device="cuda")
    ws_bytes = be.gemm_q4_0_workspace_bytes(tokens, rows, cols)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
    # whole 256-weight groups: the group-scale kernel over the tensor's cached two-digit planes (~5e-5); otherwise, and with
    # it switched off, nibbles widened per call and the per-block Q8_0 kernel (~1e-5)
    outs = {}
    for groups in (False, True):
        before = be.set_gemm_groups(groups)
        try:
            y.fill_(float("nan"))
            be.dev_gemm_q4_0(h, y.data_ptr(), d_x.data_ptr(), tokens, ws.data_ptr(), ws_bytes)
            be.dev_check()
        finally:
            be.set_gemm_groups(before)
        outs[groups] = y.cpu().numpy()
        rel = assert_parity(outs[groups], ref, what=f"Q4_0 tensor product {tokens}x{rows}x{cols} groups={groups}")
        assert rel < (3e-4 if groups and cols % 256 == 0 else 1e-4)
    be.dev_free(h)
    host = be.gemm("Q4_0", w, x, tokens, rows, cols)
    assert np.array_equal(host, outs[True])       # the same kernels on the same bytes
    be.release_weights(w)
