"""GPU parity for the Q4_K and Q5_K decode products, through the C-ABI (zen_cuda_gemm_kquant, the device-pointer calls).

The reference computes both with fp32 activations (gemv_q4k_q5k_avx2, kernels/avx2.cpp:329-378); the checker is its C
restatement, pinned bit for bit to the compiled reference (tests/test_kquant_q4k_q5k_cpu.py), and the vectors the
unmodified reference produced.  Bar: 1e-3 under both gates of helpers.assert_parity.  The kernels keep the dot products in
integers with two int8 digits per activation (as for Q4_0 and Q6_K), so results land near 1e-5."""
import os

import numpy as np
import pytest

from helpers import assert_parity, seeded_acts
from zeninfer_b200 import blocks

pytestmark = pytest.mark.gpu
FORMATS = [(blocks.Q4_K, "Q4_K", "q4_k"), (blocks.Q5_K, "Q5_K", "q5_k")]
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "kquant_vectors.npz")


@pytest.fixture(scope="module")
def be():
    from zeninfer_b200 import Backend
    return Backend()


@pytest.mark.parametrize("fmt,name,tag", FORMATS)
def test_against_the_reference_vectors(be, fmt, name, tag):
    with np.load(GOLDEN) as g:
        w, x, y = np.ascontiguousarray(g[tag + "_w"]), g[tag + "_x"], g[tag + "_y"]
    rel = assert_parity(be.gemv(name, w, x, w.shape[0], x.size), y, what=f"{name} gemv vs the reference's vector")
    assert rel < 1e-4
    be.release_weights(w)


@pytest.mark.parametrize("fmt,name,tag", FORMATS)
@pytest.mark.parametrize("rows,cols,tokens", [(1, 256, 1), (5, 512, 1), (67, 1280, 3), (130, 2048, 8), (1024, 4096, 1), (64, 14336, 2), (300, 768, 11),
                                              (2050, 4096, 8), (33, 4096, 40), (9, 4352, 5), (8, 8192, 7), (1027, 8192, 1), (4096, 14336, 1), (77, 12288, 2)])
def test_host_pointer_product_vs_oracle(be, zo, fmt, name, tag, rows, cols, tokens):
    w = blocks.random_k_blocks(fmt, rows, cols, 500 + rows)
    x = seeded_acts(tokens, cols, 510 + cols)
    got = be.gemm(name, w, x, tokens, rows, cols)       # more than 8 tokens: several launches
    ref = np.stack([zo.gemv(fmt, w, x[t], rows, cols) for t in range(tokens)])
    rel = assert_parity(got, ref, what=f"{name} {tokens}x{rows}x{cols}")
    assert rel < (3e-4 if tokens >= 9 else 1e-4)        # nine rows and more: the group-scale tensor-core kernel (~5e-5)
    be.release_weights(w)


@pytest.mark.parametrize("fmt,name,tag", FORMATS)
def test_device_pointer_calls(be, zo, fmt, name, tag):
    import torch
    from zeninfer_b200 import BackendError
    from zeninfer_b200.backend import ACT_FP32, ACT_INT8
    rows, cols, tokens = [96, 40], 1024, 3
    ws = [blocks.random_k_blocks(fmt, r, cols, 520 + r) for r in rows]
    hs = [be.dev_upload(name, w, r, cols) for w, r in zip(ws, rows)]
    part = be.dev_upload(name, ws[0], rows[0], cols, 32, 48)            # rows 32..79 of the first tensor
    x = seeded_acts(tokens, cols, 530)
    d_x = torch.from_numpy(x).cuda()
    outs = [torch.zeros((tokens, r), dtype=torch.float32, device="cuda") for r in rows + [48]]
    stream = torch.cuda.Stream()
    be.dev_gemv(hs, [o.data_ptr() for o in outs[:2]], d_x.data_ptr(), tokens, ACT_FP32, stream.cuda_stream)
    be.dev_gemv([part], [outs[2].data_ptr()], d_x.data_ptr(), tokens, ACT_FP32, stream.cuda_stream)
    stream.synchronize()
    be.dev_check(stream.cuda_stream)
    for w, r, o in zip(ws, rows, outs):
        ref = np.stack([zo.gemv(fmt, w, x[t], r, cols) for t in range(tokens)])
        assert_parity(o.cpu().numpy(), ref, what=f"{name} device-pointer product rows={r}")
    assert torch.equal(outs[2], outs[0][:, 32:80])
    with pytest.raises(BackendError):
        be.dev_gemv(hs[:1], [outs[0].data_ptr()], d_x.data_ptr(), tokens, ACT_INT8, stream.cuda_stream)   # fp32-equivalent activations only
    for h in hs + [part]:
        be.dev_free(h)


@pytest.mark.parametrize("fmt,name,tag", FORMATS)
@pytest.mark.parametrize("rows,cols,tokens", [(300, 4096, 40), (1027, 1280, 12), (64, 14336, 64), (130, 2048, 129), (19000, 256, 16)])
def test_tensor_core_product_vs_oracle(be, zo, fmt, name, tag, rows, cols, tokens):
    # many activation rows: codes widened to int8 in the workspace with the fp32 factors d * sc and dmin * m of every
    # sub-block, then the tcgen05 GEMM with two activation digits whose epilogue subtracts the minimum term.  Device entry
    # point with a caller workspace, then the host-pointer call (the same path from nine rows on).  19000 rows are 149
    # row tiles: the K range of one tile is shared between two CTAs.
    import torch
    w = blocks.random_k_blocks(fmt, rows, cols, 600 + rows)
    x = seeded_acts(tokens, cols, 610 + cols)
    ref = np.stack([zo.gemv(fmt, w, x[t], rows, cols) for t in range(tokens)])
    h = be.dev_upload(name, w, rows, cols)
    d_x = torch.from_numpy(x).cuda()
    y = torch.full((tokens, rows), float("nan"), device="cuda")
    ws_bytes = be.gemm_kquant_workspace_bytes(tokens, rows, cols)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
    # the group-scale kernel over the tensor's cached two-digit planes (~5e-5); with it switched off, codes widened per call
    # and the per-block kernel with fp32 sub-block scales and the minimum term in its epilogue (~1e-5)
    outs = {}
    for groups in (False, True):
        before = be.set_gemm_groups(groups)
        try:
            y.fill_(float("nan"))
            be.dev_gemm_kquant(h, y.data_ptr(), d_x.data_ptr(), tokens, ws.data_ptr(), ws_bytes)
            be.dev_check()
        finally:
            be.set_gemm_groups(before)
        outs[groups] = y.cpu().numpy()
        if groups:
            # 16-bit fixed point per 256-weight group: the error scales with the LARGEST result (these random blocks give results
            # in the hundreds), so only the gate on max_abs / max_ref applies; the per-element gate is the other kernel's
            rel = float(np.abs(outs[groups].astype(np.float64) - ref).max() / np.abs(ref).max())
            assert np.all(np.isfinite(outs[groups])) and rel < 3e-4, rel
        else:
            rel = assert_parity(outs[groups], ref, what=f"{name} tensor product {tokens}x{rows}x{cols} groups={groups}")
            assert rel < 1e-4
    be.dev_free(h)
    host = be.gemm(name, w, x, tokens, rows, cols)
    assert np.array_equal(host, outs[True])       # the same kernels on the same bytes
    be.release_weights(w)
