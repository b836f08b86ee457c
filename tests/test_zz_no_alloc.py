"""The allocation-free prefill entry point (zen_cuda_dev_gemm_q8_0_noalloc) against the ordinary one.

Some callers of this library cannot allocate device memory when they call it -- a plug-in inside a host runtime that
has already handed out all of HBM, or a serving loop that must not trigger the device-wide synchronisation an
allocation implies -- so they have no workspace to pass.  For them the quantised activations live in a scratch array
built into the library.  This test drives that entry point through the C-ABI twice in a row, with different shapes, so
the second call meets the first call's bytes in the shared scratch, and compares each result with
zen_cuda_dev_gemm_q8_0 given an ordinary caller workspace.  Both run the same kernels on the same codes, so the bar is
the suite's parity bar (1e-3) and the results are in fact expected to be identical.  Each result is also held against
the CPU oracle's int8-activation product, so the test stands on its own, and the free device memory reported by the
driver must be the same before and after the calls.

The file name makes pytest collect it last: if it fails, a run that stops at the first failure has already run
everything else.  It builds its own inputs, so it also passes when run alone in a fresh process.
"""
import numpy as np
import pytest

from helpers import assert_parity, seeded_acts, seeded_weights
from zeninfer_b200 import blocks

pytestmark = pytest.mark.gpu


def test_noalloc_matches_workspace_entry_twice(zo):
    import torch
    from zeninfer_b200 import Backend, BackendError

    be = Backend()
    dev = torch.device("cuda", 0)
    rows, cols = 1000, 2048
    w = seeded_weights(blocks.Q8_0, rows, cols, 900)
    handle = be.dev_upload("Q8_0", w, rows, cols)  # residency (and backend start-up) happens here, outside the entry point under test
    stream = torch.cuda.Stream(device=dev)

    # first call: 150 tokens; second call: 37 tokens (shorter scale rows, stale bytes all around them)
    for call, tokens in enumerate((150, 37)):
        x = torch.from_numpy(seeded_acts(tokens, cols, 910 + call)).to(dev)
        out_ref = torch.full((tokens, rows), 123456.0, dtype=torch.float32, device=dev)
        out_new = torch.full((tokens, rows), 123456.0, dtype=torch.float32, device=dev)
        ws_bytes = be.gemm_workspace_bytes(tokens, cols)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        torch.cuda.synchronize()
        groups = be.set_gemm_groups(False)      # the allocation-free entry point takes the per-block kernel: compare with the same
        try:
            be.dev_gemm_q8_0([handle], [out_ref.data_ptr()], x.data_ptr(), tokens, ws.data_ptr(), ws_bytes, stream.cuda_stream)
        finally:
            be.set_gemm_groups(groups)
        stream.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]          # cudaMemGetInfo: what the driver still has to give
        be.dev_gemm_q8_0_noalloc(handle, out_new.data_ptr(), x.data_ptr(), tokens, stream.cuda_stream)
        stream.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before, "the allocation-free entry point changed the free device memory"
        be.dev_check(stream.cuda_stream)
        got, ref = out_new.cpu().numpy(), out_ref.cpu().numpy()
        assert not np.any(got == 123456.0)
        assert_parity(got, ref, what=f"no-alloc call {call + 1} ({tokens} tokens)")
        assert np.array_equal(got, ref)
        assert_parity(got, zo.gemm(blocks.Q8_0, w, x.cpu().numpy(), tokens, rows, cols, int8_acts=True), what=f"no-alloc call {call + 1} vs the int8 oracle")

    # a request larger than the built-in scratch is refused with a message, and nothing is launched
    too_many = 2097152 // cols + 1
    with pytest.raises(BackendError, match="exceeds the built-in scratch"):
        be.dev_gemm_q8_0_noalloc(handle, 1, 1, too_many, stream.cuda_stream)
    be.dev_free(handle)
    # the second limit: the activations fit the element count, but their scale rows (padded to four tokens) do not fit the array
    wide = 1 << 20
    w_wide = seeded_weights(blocks.Q8_0, 1, wide, 920)
    h_wide = be.dev_upload("Q8_0", w_wide, 1, wide)
    assert 2 * wide <= 2097152 and be.gemm_workspace_bytes(2, wide) > 2097152 + 262144
    with pytest.raises(BackendError, match="exceeds the built-in scratch"):
        be.dev_gemm_q8_0_noalloc(h_wide, 1, 1, 2, stream.cuda_stream)
    be.dev_free(h_wide)
