"""The residency budget of the pointer-keyed weights (the reference keeps them below 80 % of the device's memory,
src/backends/hip/hip_backend.hip:50 and :459-476): the whole keyed set is evicted when a new tensor would cross the
budget, a tensor larger than the budget is refused, and a batch whose lookups evict in the middle resolves its tensors
again before it launches, so that no launch reads a freed tensor.  Every product is checked against the oracle."""
import numpy as np
import pytest

from helpers import assert_parity, seeded_acts, seeded_weights
from zeninfer_b200 import blocks
from zeninfer_b200.backend import ACT_INT8, BackendError

pytestmark = pytest.mark.gpu
Q8_0 = blocks.Q8_0
ROWS, COLS = 256, 1024
TENSOR_BYTES = ROWS * COLS + 64 + ROWS * 32 * 2 + 64      # codes + f16 scales (padded to 8 per row), each with 64 bytes of slack


@pytest.fixture()
def be():
    from zeninfer_b200 import Backend
    b = Backend()
    b.set_q8_act_mode(ACT_INT8)
    yield b
    b.set_vram_budget(0)


def _check(be, zo, w, x, rows=ROWS, cols=COLS):
    assert_parity(be.gemv("Q8_0", w, x, rows, cols), zo.gemv(Q8_0, w, x, rows, cols, int8_acts=True), what="gemv under the budget")


def test_default_budget_is_80_percent_of_device_memory(be):
    be.set_vram_budget(0)
    assert be.residency()["budget_bytes"] == be.info()["dedicated_vram"] // 100 * 80


def test_keyed_set_is_evicted_whole_when_a_tensor_would_cross_the_budget(be, zo):
    ws = [seeded_weights(Q8_0, ROWS, COLS, 900 + i) for i in range(3)]
    x = seeded_acts(1, COLS, 77)[0]
    base = be.residency()
    be.set_vram_budget(base["held_bytes"] + 2 * TENSOR_BYTES + TENSOR_BYTES // 2)
    for w in ws[:2]:
        for _ in range(3):                      # the third call of each replays a captured graph
            _check(be, zo, w, x)
    r = be.residency()
    assert r["tensors"] == base["tensors"] + 2 and r["evictions"] == base["evictions"]
    assert r["held_bytes"] == base["held_bytes"] + 2 * TENSOR_BYTES
    uploaded = be.stats()["upload_bytes"]
    _check(be, zo, ws[2], x)                    # crosses the budget: everything keyed goes, then the new tensor comes in
    r = be.residency()
    assert r["evictions"] == base["evictions"] + 1 and r["tensors"] == 1
    assert r["held_bytes"] <= base["held_bytes"] + TENSOR_BYTES      # tensors other tests left keyed went too
    for _ in range(3):                          # the evicted tensor is uploaded again, and its stale graph is not replayed
        _check(be, zo, ws[0], x)
    assert be.stats()["upload_bytes"] == uploaded + 2 * ROWS * (COLS // 32) * 34
    assert be.residency()["tensors"] == 2
    for w in ws:
        be.release_weights(w)


def test_tensor_larger_than_the_budget_is_refused(be):
    w = seeded_weights(Q8_0, ROWS, COLS, 910)
    x = seeded_acts(1, COLS, 78)[0]
    be.set_vram_budget(be.residency()["held_bytes"] + TENSOR_BYTES - 1)
    before = be.stats()["fallbacks"]
    with pytest.raises(BackendError, match="residency budget"):
        be.gemv("Q8_0", w, x, ROWS, COLS)
    assert be.stats()["fallbacks"] == before + 1
    be.set_vram_budget(0)
    assert be.gemv("Q8_0", w, x, ROWS, COLS).shape == (ROWS,)     # the backend stays usable
    be.release_weights(w)


def test_eviction_in_the_middle_of_a_batch(be, zo):
    ws = [seeded_weights(Q8_0, ROWS, COLS, 920 + i) for i in range(4)]
    x = seeded_acts(1, COLS, 79)[0]
    be.set_vram_budget(be.residency()["held_bytes"] + 2 * TENSOR_BYTES + TENSOR_BYTES // 2)
    _check(be, zo, ws[0], x)                    # one tensor resident
    ev = be.residency()["evictions"]
    ys = be.gemv_batch("Q8_0", ws[1:3], x, [ROWS, ROWS], COLS)     # the second lookup evicts the first one's tensor
    for w, y in zip(ws[1:3], ys):
        assert_parity(y, zo.gemv(Q8_0, w, x, ROWS, COLS, int8_acts=True), what="batch across an eviction")
    r = be.residency()
    assert r["evictions"] == ev + 1 and r["tensors"] == 2
    with pytest.raises(BackendError, match="do not fit the residency budget together"):
        be.gemv_batch("Q8_0", ws[1:4], x, [ROWS] * 3, COLS)
    be.set_vram_budget(0)
    ys = be.gemv_batch("Q8_0", ws[1:4], x, [ROWS] * 3, COLS)
    for w, y in zip(ws[1:4], ys):
        assert_parity(y, zo.gemv(Q8_0, w, x, ROWS, COLS, int8_acts=True), what="batch after the budget was lifted")
    for w in ws:
        be.release_weights(w)


def test_caller_held_tensors_are_counted_and_never_evicted(be, zo):
    import torch
    w_dev = seeded_weights(Q8_0, ROWS, COLS, 930)
    keyed = [seeded_weights(Q8_0, ROWS, COLS, 931 + i) for i in range(2)]
    x = seeded_acts(1, COLS, 80)[0]
    base = be.residency()
    handle = be.dev_upload("Q8_0", w_dev, ROWS, COLS)
    assert be.residency()["held_bytes"] == base["held_bytes"] + TENSOR_BYTES
    be.set_vram_budget(base["held_bytes"] + 2 * TENSOR_BYTES + TENSOR_BYTES // 2)   # room for the handle and ONE keyed tensor
    _check(be, zo, keyed[0], x)
    _check(be, zo, keyed[1], x)                 # evicts keyed[0]; the handle stays
    assert be.residency()["tensors"] == 1
    d_x = torch.from_numpy(x).cuda()
    d_y = torch.empty(ROWS, device="cuda")
    be.dev_gemv([handle], [d_y.data_ptr()], d_x.data_ptr(), 1, ACT_INT8)
    be.dev_check()
    assert_parity(d_y.cpu().numpy(), zo.gemv(Q8_0, w_dev, x, ROWS, COLS, int8_acts=True), what="caller-held tensor after an eviction")
    be.dev_free(handle)
    for w in keyed:
        be.release_weights(w)
