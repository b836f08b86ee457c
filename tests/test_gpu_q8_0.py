"""GPU parity for the Q8_0 decode path, through the C-ABI (zeninfer_b200.Backend binds it with ctypes).

Bars: activation codes and scales bit-exact against the oracle; fp32 outputs within 1e-3 under the two
gates of helpers.assert_parity.  int8-activation kernels are compared with the int8-activation oracle,
fp32-activation kernels with the fp32-activation oracle -- never across.
"""
import os

import numpy as np
import pytest

from helpers import assert_parity, ref_fp32_f64, ref_int8_f64, seeded_acts, seeded_weights
from zeninfer_b200 import blocks
from zeninfer_b200.backend import ACT_FP32, ACT_INT8

pytestmark = pytest.mark.gpu
Q8_0 = blocks.Q8_0
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz")


@pytest.fixture(scope="module")
def be():
    from zeninfer_b200 import Backend
    b = Backend()
    assert b.enabled()
    assert b.info()["arch"] == "sm_100"
    yield b
    b.set_q8_act_mode(ACT_INT8)


@pytest.fixture(scope="module")
def golden():
    with np.load(GOLDEN) as g:
        return {k: g[k] for k in g.files}


def test_quantize_acts_bit_exact(be, zo):
    x = seeded_acts(8, 4096, 1)
    x[0, :32] = 0.0
    x[1, :32] = np.arange(32, dtype=np.float32) * 0.5 - 7.75    # lands on exact .5 ties
    x[2, :32] *= np.float32(1e30)
    x[3, :32] *= np.float32(1e-30)
    x[4, 100] = 1e4
    q, sc = be.quantize_acts(x)
    q_ref, sc_ref = zo.quantise_acts(x)
    assert np.array_equal(q, q_ref)
    assert np.array_equal(sc.view(np.uint32), sc_ref.view(np.uint32))


def test_quantize_acts_against_reference_golden(be, golden):
    x = golden["i8_ident_x"]
    q, sc = be.quantize_acts(x)
    deq = (q.astype(np.float32).reshape(x.shape[0], -1, 32) * sc[..., None]).reshape(x.shape)
    assert np.array_equal(deq, golden["i8_ident_y"])


def test_quantize_acts_prefill_shape(be, zo):
    x = seeded_acts(512, 4096, 2)  # the prefill activation matrix of the Llama-3-8B FFN-up case
    q, sc = be.quantize_acts(x)
    q_ref, sc_ref = zo.quantise_acts(x)
    assert np.array_equal(q, q_ref) and np.array_equal(sc.view(np.uint32), sc_ref.view(np.uint32))


def test_unit_row_is_exactly_32(be):
    # tests/core_tests.cpp:272-277, both activation modes
    blk = np.array([0x00, 0x3C] + [1] * 32, np.uint8)
    ones = np.ones(32, np.float32)
    for mode in (ACT_INT8, ACT_FP32):
        be.set_q8_act_mode(mode)
        assert be.gemv("Q8_0", blk, ones, 1, 32)[0] == np.float32(32.0)
    be.release_weights(blk)
    be.set_q8_act_mode(ACT_INT8)


@pytest.mark.parametrize("rows,cols", [(1, 32), (3, 96), (5, 256), (67, 544), (130, 2048), (512, 4096), (1024, 4096), (64, 14336)])
def test_gemv_int8_vs_oracle(be, zo, rows, cols):
    be.set_q8_act_mode(ACT_INT8)
    w = seeded_weights(Q8_0, rows, cols, 10 + rows)
    x = seeded_acts(1, cols, 20 + cols)[0]
    y = be.gemv("Q8_0", w, x, rows, cols)
    assert_parity(y, zo.gemv(Q8_0, w, x, rows, cols, int8_acts=True), what=f"int8 gemv {rows}x{cols}")
    be.release_weights(w)


@pytest.mark.parametrize("rows,cols", [(1, 32), (3, 96), (67, 544), (512, 4096), (64, 14336)])
def test_gemv_fp32_mode_vs_oracle(be, zo, rows, cols):
    be.set_q8_act_mode(ACT_FP32)
    w = seeded_weights(Q8_0, rows, cols, 30 + rows)
    x = seeded_acts(1, cols, 40 + cols)[0]
    y = be.gemv("Q8_0", w, x, rows, cols)
    rel = assert_parity(y, zo.gemv(Q8_0, w, x, rows, cols, int8_acts=False), what=f"fp32-act gemv {rows}x{cols}")
    assert rel < 1e-4  # two int8 digits: far inside the bar
    be.release_weights(w)
    be.set_q8_act_mode(ACT_INT8)


def test_gemv_against_reference_golden(be, golden):
    be.set_q8_act_mode(ACT_INT8)
    w = np.ascontiguousarray(golden["i8_gemv_w"])
    for xi, yi in zip(golden["i8_gemv_x"], golden["i8_gemv_y"]):
        assert_parity(be.gemv("Q8_0", w, xi, 67, 544), yi, what="golden int8 gemv")
    be.release_weights(w)
    be.set_q8_act_mode(ACT_FP32)
    w = np.ascontiguousarray(golden["q8_0_w"])
    assert_parity(be.gemv("Q8_0", w, golden["q8_0_x"][0], 37, 768), golden["q8_0_gemv_y"], what="golden fp32 gemv")
    assert_parity(be.gemm("Q8_0", w, golden["q8_0_x"], 5, 37, 768), golden["q8_0_gemm_y"], what="golden fp32 gemm")
    be.release_weights(w)
    be.set_q8_act_mode(ACT_INT8)


@pytest.mark.parametrize("tokens", [2, 3, 5, 8, 9, 17])
def test_small_batch_vs_oracle(be, zo, tokens):
    rows, cols = 100, 544  # the reference's token ladder shape (tests/core_tests.cpp:345-372)
    w = seeded_weights(Q8_0, rows, cols, 50)
    x = seeded_acts(tokens, cols, 60 + tokens)
    be.set_q8_act_mode(ACT_INT8)
    assert_parity(be.gemm("Q8_0", w, x, tokens, rows, cols), zo.gemm(Q8_0, w, x, tokens, rows, cols, int8_acts=True), what=f"int8 T={tokens}")
    be.set_q8_act_mode(ACT_FP32)
    assert_parity(be.gemm("Q8_0", w, x, tokens, rows, cols), zo.gemm(Q8_0, w, x, tokens, rows, cols, int8_acts=False), what=f"fp32 T={tokens}")
    be.release_weights(w)
    be.set_q8_act_mode(ACT_INT8)


def test_gemv_batch_shares_input(be, zo):
    # Q|K|V of one Llama-3-8B layer: rows {4096, 1024, 1024}, K = 4096 (src/quant.cpp:1441-1502)
    cols, rows = 4096, [4096, 1024, 1024]
    ws = [seeded_weights(Q8_0, r, cols, 70 + i) for i, r in enumerate(rows)]
    x = seeded_acts(1, cols, 80)[0]
    be.set_q8_act_mode(ACT_INT8)
    before = be.stats()
    ys = be.gemv_batch("Q8_0", ws, x, rows, cols)
    after = be.stats()
    assert after["batches"] == before["batches"] + 1
    for w, r, y in zip(ws, rows, ys):
        assert_parity(y, zo.gemv(Q8_0, w, x, r, cols, int8_acts=True), what=f"batched gemv rows={r}")
        assert np.array_equal(y, be.gemv("Q8_0", w, x, r, cols))  # same kernel, same order: bit-identical
        be.release_weights(w)


def test_config0_full_size_int8(be, zo):
    # BASELINE config 0: W 4096x4096 N(0,.02) seed 0 -> Q8_0, x N(0,1) seed 1, batch 1
    rows = cols = 4096
    w = seeded_weights(Q8_0, rows, cols, 0)
    x = seeded_acts(1, cols, 1)
    be.set_q8_act_mode(ACT_INT8)
    y = be.gemv("Q8_0", w, x[0], rows, cols)
    xq, xsc = zo.quantise_acts(x)
    assert_parity(y, ref_int8_f64(w, xq, xsc, rows, cols)[0], tol=1e-5, what="config 0 vs float64 int8 restatement")
    assert_parity(y, zo.gemv(Q8_0, w, x[0], rows, cols, int8_acts=True), what="config 0 vs oracle")
    be.set_q8_act_mode(ACT_FP32)
    y32 = be.gemv("Q8_0", w, x[0], rows, cols)
    assert_parity(y32, ref_fp32_f64(Q8_0, w, x, rows, cols)[0], tol=1e-4, what="config 0 fp32-act vs float64 dequant dot")
    be.release_weights(w)
    be.set_q8_act_mode(ACT_INT8)


def test_long_run_of_overlapped_launches_is_deterministic(be, zo):
    """Tens of thousands of launches back to back on one stream, each overlapping the tail of the one before
    (programmatic dependent launch), over several weight copies so the stream comes from HBM.  Every launch must give
    the first launch's bits, the error word must stay clear and the first result must match the oracle.  A ring protocol
    that lets a consumer team run ahead of a copy still in flight shows up here (about one launch in 10^4) and nowhere
    in a single-launch test."""
    import torch
    rows = cols = 4096
    dev = torch.device("cuda", 0)
    copies, outs, rounds = 8, 64, 400
    ws = [seeded_weights(Q8_0, rows, cols, 40)] * 1
    handles = [be.dev_upload("Q8_0", ws[0], rows, cols) for _ in range(copies)]
    x = seeded_acts(1, cols, 41)
    d_x = torch.from_numpy(x).to(dev)
    d_y = torch.zeros((outs, rows), dtype=torch.float32, device=dev)
    stream = torch.cuda.Stream(device=dev)
    ptrs = [d_y[i].data_ptr() for i in range(outs)]
    bad = torch.zeros((), dtype=torch.int64, device=dev)
    with torch.cuda.stream(stream):
        be.dev_gemv([handles[0]], [ptrs[0]], d_x.data_ptr(), 1, ACT_INT8, stream.cuda_stream)
        stream.synchronize()
        first = d_y[0].clone()
        for rnd in range(rounds):
            for i in range(outs):
                be.dev_gemv([handles[(rnd + i) % copies]], [ptrs[i]], d_x.data_ptr(), 1, ACT_INT8, stream.cuda_stream)
            bad += (d_y != first[None, :]).sum()
            d_y.zero_()
            if rnd % 16 == 15:
                stream.synchronize()
        stream.synchronize()
    be.dev_check(stream.cuda_stream)
    assert int(bad.item()) == 0, f"{int(bad.item())} output elements differed from the first launch over {rounds * outs} launches"
    assert_parity(first.cpu().numpy(), zo.gemv(Q8_0, ws[0], x[0], rows, cols, int8_acts=True), what="first launch vs oracle")
    for h in handles:
        be.dev_free(h)


def test_ffn_shapes_full_size(be, zo):
    # gate/up 14336x4096 and down 4096x14336 of config 2, checked through size-independent float64 references
    be.set_q8_act_mode(ACT_INT8)
    for rows, cols, seed in ((14336, 4096, 4), (4096, 14336, 5)):
        w = seeded_weights(Q8_0, rows, cols, seed)
        x = seeded_acts(2, cols, seed + 100)
        y = be.gemm("Q8_0", w, x, 2, rows, cols)
        xq, xsc = zo.quantise_acts(x)
        assert_parity(y, ref_int8_f64(w, xq, xsc, rows, cols), tol=1e-5, what=f"{rows}x{cols}")
        be.release_weights(w)


def test_residency_and_release(be):
    rows, cols = 64, 256
    w = seeded_weights(Q8_0, rows, cols, 90)
    x = seeded_acts(1, cols, 91)[0]
    s0 = be.stats()
    y1 = be.gemv("Q8_0", w, x, rows, cols)
    s1 = be.stats()
    y2 = be.gemv("Q8_0", w, x, rows, cols)
    s2 = be.stats()
    assert s1["upload_bytes"] - s0["upload_bytes"] == rows * (cols // 32) * 34  # raw GGUF bytes, uploaded once
    assert s2["upload_bytes"] == s1["upload_bytes"]
    assert np.array_equal(y1, y2)
    # same address, new contents: stale until released (include/zen/d3d12_backend.h:85-88), fresh after
    w[:] = seeded_weights(Q8_0, rows, cols, 92)
    assert np.array_equal(be.gemv("Q8_0", w, x, rows, cols), y1)
    be.release_weights(w)
    y3 = be.gemv("Q8_0", w, x, rows, cols)
    assert not np.array_equal(y3, y1)
    be.release_weights(w)


def test_bad_arguments_are_errors(be):
    from zeninfer_b200 import BackendError
    w = seeded_weights(Q8_0, 4, 64, 93)
    with pytest.raises(BackendError):
        be.gemm("Q8_0", w, np.zeros((1, 48), np.float32), 1, 4, 48)  # 48 is not a multiple of 32
    assert be.stats()["fallbacks"] >= 1


@pytest.mark.parametrize("rows,cols", [(4096, 14336), (1027, 4128), (300, 8192), (77, 12288), (5, 4128), (33, 14336)])
def test_rows_of_several_segments_int8(be, zo, rows, cols):
    # more than 4096 columns, one int8 token: a warp walks two rows segment by segment with the segment's activations in
    # registers (the down projection's shape class); plain, accumulating, and two tensors in one launch
    import torch
    be.set_q8_act_mode(ACT_INT8)
    w = seeded_weights(Q8_0, rows, cols, 60 + rows)
    w2 = seeded_weights(Q8_0, rows // 2 + 3, cols, 61 + rows)
    x = seeded_acts(1, cols, 70 + cols)[0]
    ref = zo.gemv(Q8_0, w, x, rows, cols, int8_acts=True)
    ref2 = zo.gemv(Q8_0, w2, x, w2.shape[0], cols, int8_acts=True)
    assert_parity(be.gemv("Q8_0", w, x, rows, cols), ref, what=f"host gemv {rows}x{cols}")
    h, h2 = be.dev_upload("Q8_0", w, rows, cols), be.dev_upload("Q8_0", w2, w2.shape[0], cols)
    d_x = torch.from_numpy(x).cuda()
    y, y2 = torch.zeros(rows, device="cuda"), torch.zeros(w2.shape[0], device="cuda")
    be.dev_gemv([h, h2], [y.data_ptr(), y2.data_ptr()], d_x.data_ptr(), 1, ACT_INT8)
    be.dev_check()
    assert_parity(y.cpu().numpy(), ref, what="two tensors in one launch, first")
    assert_parity(y2.cpu().numpy(), ref2, what="two tensors in one launch, second")
    base = torch.full((rows,), 0.5, device="cuda")
    be.dev_gemv_fused([h], [base.data_ptr()], d_x.data_ptr(), 1, ACT_INT8, accumulate=True)
    be.dev_check()
    assert torch.equal(base, y + 0.5)
    # eight tokens keep the activations in shared memory: a different summation order, the same oracle
    x8 = seeded_acts(2, cols, 71 + cols)
    got8 = be.gemm("Q8_0", w, x8, 2, rows, cols)
    assert_parity(got8, np.stack([zo.gemv(Q8_0, w, x8[t], rows, cols, int8_acts=True) for t in range(2)]), what="two tokens")
    be.dev_free(h); be.dev_free(h2)
    be.release_weights(w)
