"""The device-side error channel: a bounded wait that runs out, reported through zen_cuda_dev_check, with the context
still usable afterwards; and calls arriving from a thread that is not the one that started the backend.

Nothing here faults or hangs the GPU: the wait budget is shortened to a few milliseconds, the kernel gives up after it,
sets the error word and returns."""
import threading

import numpy as np
import pytest

from helpers import assert_parity, seeded_acts, seeded_weights
from zeninfer_b200 import blocks
from zeninfer_b200.backend import ACT_INT8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from zeninfer_b200 import Backend
    return Backend()


def test_error_names_and_uninitialised_check(be):
    assert be.lib.zen_cuda_error_name(0) == b"none"
    assert b"peer" in be.lib.zen_cuda_error_name(5)
    assert be.lib.zen_cuda_dev_check(0) == 0


def test_peer_wait_runs_out_and_the_backend_stays_usable(be, zo):
    """A two-rank gather object whose second rank is a second region in this process that nobody ever publishes to: the
    all-gather stores its piece, then waits for rank 1's flag, which never rises.  With a 5 ms budget the kernel gives
    up, reports code 5, counts its launch, and everything after it works."""
    import torch
    from zeninfer_b200 import BackendError
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    slot = 1024
    nbytes = be.gather_region_bytes(2, slot)
    own, _ = be.ipc_alloc(nbytes)
    silent, _ = be.ipc_alloc(nbytes)          # stands in for a peer that never answers
    g = be.gather_create(2, 0, slot, [own, silent])
    piece = torch.arange(slot, dtype=torch.float32, device=dev)
    whole = torch.zeros(2 * slot, dtype=torch.float32, device=dev)
    be.set_wait_budget_ms(5)
    try:
        for attempt in range(2):              # the launch counter advances even when the wait gave up: a second launch times out the same way
            be.dev_allgather(g, piece.data_ptr(), slot, whole.data_ptr(), stream.cuda_stream)
            with pytest.raises(BackendError) as info:
                be.dev_check(stream.cuda_stream)
            assert info.value.code == 5
            be.dev_check(stream.cuda_stream)  # the word was cleared by the read
        # the fused-gather product waits the same way before it pushes (launch 2 needs rank 1's launch 1)
        rows = cols = 512
        w = seeded_weights(blocks.Q8_0, rows, cols, 700)
        x = torch.from_numpy(seeded_acts(1, cols, 701)).to(dev)
        h = be.dev_upload("Q8_0", w, rows, cols)
        own2, _ = be.ipc_alloc(be.gather_region_bytes(2, rows))
        silent2, _ = be.ipc_alloc(be.gather_region_bytes(2, rows))
        g2 = be.gather_create(2, 0, rows, [own2, silent2])
        y = torch.zeros(rows, dtype=torch.float32, device=dev)
        be.dev_gemv_gather(g2, [h], [y.data_ptr()], x.data_ptr(), 1, ACT_INT8, stream.cuda_stream)   # launch 1 needs nobody
        be.dev_check(stream.cuda_stream)
        be.dev_gemv_gather(g2, [h], [y.data_ptr()], x.data_ptr(), 1, ACT_INT8, stream.cuda_stream)   # launch 2 waits for rank 1's launch 1
        with pytest.raises(BackendError) as info:
            be.dev_check(stream.cuda_stream)
        assert info.value.code == 5
        assert_parity(y.cpu().numpy(), zo.gemv(blocks.Q8_0, w, x.cpu().numpy()[0], rows, cols, int8_acts=True), what="own outputs are still written")
    finally:
        be.set_wait_budget_ms(0)
    # an ordinary launch and a fresh, complete gather object work as before
    y2 = torch.zeros(rows, dtype=torch.float32, device=dev)
    be.dev_gemv([h], [y2.data_ptr()], x.data_ptr(), 1, ACT_INT8, stream.cuda_stream)
    be.dev_check(stream.cuda_stream)
    assert torch.equal(y, y2)
    from zeninfer_b200 import shard
    pg = shard.PeerGather(be, 1, 0, rows)
    got = torch.zeros(rows, dtype=torch.float32, device=dev)
    pg.gemv([h], x.data_ptr(), 1, ACT_INT8, stream.cuda_stream)
    pg.fetch(got.data_ptr(), stream.cuda_stream)
    be.dev_check(stream.cuda_stream)
    assert torch.equal(got, y2)
    pg.close()
    torch.cuda.synchronize()
    for obj in (g, g2):
        be.gather_destroy(obj)
    for region in (own, silent, own2, silent2):
        be.ipc_free(region)
    be.dev_free(h)


def test_calls_from_a_second_thread(be, zo):
    """The reference reaches its GPU hooks from runtime and server threads; every entry point makes the backend's device
    current for the calling thread."""
    rows, cols = 256, 1024
    w = seeded_weights(blocks.Q8_0, rows, cols, 710)
    x = seeded_acts(1, cols, 711)[0]
    out = {}

    def worker():
        try:
            out["y"] = be.gemv("Q8_0", w, x, rows, cols)          # uploads, allocates scratch and launches from this thread
        except Exception as e:                                    # noqa: BLE001 - reported in the main thread
            out["err"] = e

    t = threading.Thread(target=worker)
    t.start()
    t.join()
    assert "err" not in out, out.get("err")
    assert_parity(out["y"], zo.gemv(blocks.Q8_0, w, x, rows, cols, int8_acts=True), what="gemv from a second thread")
    assert np.array_equal(out["y"], be.gemv("Q8_0", w, x, rows, cols))
    be.release_weights(w)
