"""GPU parity for the lm_head configuration at its own shape: Q6_K 128256 x 4096 (weights N(0, 0.02), seed 5), batch 1
and a speculative-verify block of 8 hidden states, through zen_cuda_gemm_q6_k, then the greedy pick.

Oracle: the reference's Q6_K kernels take fp32 activations (gemv_q6k_avx2, kernels/avx2.cpp:380-422; gemm_q6k_kblk_avx2
:1729-1770), so the checker is the fp32-activation restatement over ALL rows (a few seconds of CPU), plus the float64
dequantise-then-dot gate the reference's own sweeps use (tests/core_tests.cpp:360-367).  The picked ids follow the
reference's greedy rule (first maximum among finite logits, src/adapters/dense_transformer_runtime.cpp:407-415)."""
import numpy as np
import pytest

from helpers import assert_parity
from zeninfer_b200 import blocks
from zeninfer_b200.backend import ACT_FP32

pytestmark = pytest.mark.gpu
ROWS, COLS, CHUNK = 128256, 4096, 8016


@pytest.fixture(scope="module")
def be():
    from zeninfer_b200 import Backend
    return Backend()


@pytest.fixture(scope="module")
def lm_head():
    """(packed Q6_K rows, float64 logits of 8 hidden states): the matrix is drawn and packed in row chunks, and each
    chunk's float64 reference is taken while its decoded weights are at hand (the whole matrix in float64 would be 4 GB)."""
    rng = np.random.default_rng(5)
    hidden = np.random.default_rng([5, 1]).standard_normal((8, COLS), dtype=np.float32)
    packed, ref = [], []
    for r0 in range(0, ROWS, CHUNK):
        w = rng.standard_normal((min(CHUNK, ROWS - r0), COLS), dtype=np.float32) * np.float32(0.02)
        p = np.ascontiguousarray(blocks.quantize_q6_k(w))
        packed.append(p)
        ref.append(hidden.astype(np.float64) @ blocks.dequantize(blocks.Q6_K, p, p.shape[0], COLS).astype(np.float64).T)
    return np.ascontiguousarray(np.concatenate(packed, axis=0)), hidden, np.concatenate(ref, axis=1)


@pytest.mark.parametrize("tokens", [1, 8])
def test_lm_head_full_size_vs_oracle(be, zo, lm_head, tokens):
    import oracle
    packed, hidden, ref64 = lm_head
    x = hidden[:tokens]
    got = be.gemm("Q6_K", packed, x, tokens, ROWS, COLS)
    rel = assert_parity(got, ref64[:tokens], what=f"lm_head batch {tokens} vs float64 dequantise-dot")
    assert rel < 1e-4            # two activation digits leave about 2e-5
    want = zo.gemm(oracle.Q6_K, packed, x, tokens, ROWS, COLS)       # every row through the restatement of the reference kernel
    assert_parity(got, want, what=f"lm_head batch {tokens} vs the fp32-activation oracle")
    for t in range(tokens):
        pick = zo.argmax(got[t])
        assert pick == int(np.argmax(got[t]))
        top2 = np.sort(want[t])[-2:]
        if top2[1] - top2[0] > 1e-3 * max(1.0, abs(float(top2[1]))):   # no near-tie: both arithmetics must pick the same row
            assert pick == zo.argmax(want[t])


@pytest.mark.parametrize("tokens", [1, 8])
def test_lm_head_device_pick_matches_oracle_argmax(be, zo, lm_head, tokens):
    """The device path a decode step takes: resident tensor, logits in HBM, the pick on the device."""
    import torch
    packed, hidden, _ = lm_head
    dev = torch.device("cuda", 0)
    h = be.dev_upload("Q6_K", packed, ROWS, COLS)
    try:
        d_x = torch.from_numpy(hidden[:tokens].copy()).to(dev)
        d_y = torch.zeros((tokens, ROWS), dtype=torch.float32, device=dev)
        d_pick = torch.full((tokens,), -7, dtype=torch.int64, device=dev)
        stream = torch.cuda.Stream(device=dev)
        be.dev_gemv([h], [d_y.data_ptr()], d_x.data_ptr(), tokens, ACT_FP32, stream.cuda_stream)
        be.dev_greedy_pick([(d_y.data_ptr(), ROWS, 0, ROWS)], tokens, d_pick.data_ptr(), stream.cuda_stream)
        stream.synchronize()
        be.dev_check(stream.cuda_stream)
        logits = d_y.cpu().numpy()
        host = be.gemm("Q6_K", packed, hidden[:tokens], tokens, ROWS, COLS)
        if tokens == 1:
            assert np.array_equal(logits, host)   # host-pointer call = same kernel
        else:
            # from seven rows on the host-pointer call takes the tensor-core product: equal to the device entry point of
            # that product bit for bit, and to the decode kernel up to the order of the fp32 additions
            ws_bytes = be.gemm_q6_k_workspace_bytes(tokens, COLS)
            d_ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=dev)
            d_t = torch.zeros((tokens, ROWS), dtype=torch.float32, device=dev)
            be.dev_gemm_q6_k(h, d_t.data_ptr(), d_x.data_ptr(), tokens, d_ws.data_ptr(), ws_bytes, stream.cuda_stream)
            stream.synchronize()
            be.dev_check(stream.cuda_stream)
            assert np.array_equal(d_t.cpu().numpy(), host)
            assert assert_parity(host, logits, what="tensor-core product against the decode kernel") < 3e-4   # two digits per 256-weight group: ~5e-5
        assert d_pick.cpu().tolist() == [zo.argmax(logits[t]) for t in range(tokens)]
    finally:
        be.dev_free(h)
        be.release_weights(packed)
