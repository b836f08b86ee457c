"""The list launch (zen_cuda_dev_gemv_list): several batch-1 Q8_0 products in one persistent kernel.

Rows are independent and a lane meets its blocks in the same order as in the single-launch kernel, so every result must
equal, bit for bit, the same products launched one by one (zen_cuda_dev_gemv_fused); those are held to the oracle by
tests/test_gpu_q8_0.py, and the first case here is held to the oracle directly."""
import numpy as np
import pytest

from helpers import assert_parity, seeded_acts, seeded_weights
from zeninfer_b200 import blocks
from zeninfer_b200.backend import ACT_FP32, ACT_INT8

pytestmark = pytest.mark.gpu
Q8_0 = blocks.Q8_0


@pytest.fixture(scope="module")
def be():
    from zeninfer_b200 import Backend
    return Backend()


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("mode,int8", [(ACT_INT8, True), (ACT_FP32, False)])
def test_independent_items_equal_single_launches_and_the_oracle(be, zo, mode, int8):
    """Items that share nothing but their input: different shapes, one with three tensors (q|k|v), a ragged row count, a
    column count that is not a whole number of 128-block segments (K = 4608: two segments of 72 blocks) and the long-row
    class (K = 14336: four segments of 112)."""
    import torch
    shapes = [(4096, 4096), (520, 1024), (300, 4608), (64, 14336), (1027, 3584)]
    xs = {c: seeded_acts(1, c, 500 + c)[0] for c in {c for _, c in shapes}}
    d_xs = {c: dev(v) for c, v in xs.items()}
    ws = [seeded_weights(Q8_0, r, c, 510 + i) for i, (r, c) in enumerate(shapes)]
    hs = [be.dev_upload("Q8_0", w, r, c) for w, (r, c) in zip(ws, shapes)]
    qkv = [seeded_weights(Q8_0, r, 4096, 520 + i) for i, r in enumerate((512, 128, 136))]
    h_qkv = [be.dev_upload("Q8_0", w, r, 4096) for w, r in zip(qkv, (512, 128, 136))]
    ys = [torch.zeros(r, device="cuda") for r, _ in shapes]
    y_qkv = [torch.zeros(r, device="cuda") for r in (512, 128, 136)]
    items = [dict(handles=[h], d_y=[y.data_ptr()], d_x=d_xs[c].data_ptr()) for h, y, (_, c) in zip(hs, ys, shapes)]
    items.insert(2, dict(handles=h_qkv, d_y=[y.data_ptr() for y in y_qkv], d_x=d_xs[4096].data_ptr()))
    lst = be.gemv_list_create(items, mode)
    stream = torch.cuda.Stream()
    for _ in range(3):     # the counter word returns to zero after every launch
        be.dev_gemv_list(lst, stream.cuda_stream)
    be.dev_check(stream.cuda_stream)
    one = [torch.zeros(r, device="cuda") for r, _ in shapes]
    one_qkv = [torch.zeros(r, device="cuda") for r in (512, 128, 136)]
    for h, y, (_, c) in zip(hs, one, shapes):
        be.dev_gemv([h], [y.data_ptr()], d_xs[c].data_ptr(), 1, mode, stream.cuda_stream)
    be.dev_gemv(h_qkv, [y.data_ptr() for y in one_qkv], d_xs[4096].data_ptr(), 1, mode, stream.cuda_stream)
    be.dev_check(stream.cuda_stream)
    for got, want, w, (r, c) in zip(ys + y_qkv, one + one_qkv, ws + qkv, shapes + [(512, 4096), (128, 4096), (136, 4096)]):
        assert torch.equal(got, want), (r, c)
        assert_parity(got.cpu().numpy(), zo.gemv(Q8_0, w, xs[c], r, c, int8_acts=int8), what=f"list item {r}x{c}")
    assert be.gemv_list_bytes(lst) == sum(r * (c // 32) * 34 + 4 * r for r, c in shapes + [(512, 4096), (128, 4096), (136, 4096)]) + 4 * (sum(c for _, c in shapes) + 4096)
    be.gemv_list_destroy(lst)
    for h in hs + h_qkv:
        be.dev_free(h)


@pytest.mark.parametrize("mode", [ACT_INT8, ACT_FP32])
def test_dependent_chain_equals_single_launches(be, mode):
    """The matvec chain of a decoder layer as one list: x += o(att); gate, up = W(norm(x)); x += down(silu(gate) * up);
    q, k, v = W(norm(x)).  Every item but the first reads what the one before it wrote."""
    import torch
    E, F, KV = 1024, 3584, 256
    rng = np.random.default_rng(530)
    mats = {n: seeded_weights(Q8_0, r, c, 531 + i) for i, (n, r, c) in enumerate(
        (("o", E, E), ("gate", F, E), ("up", F, E), ("down", E, F), ("q", E, E), ("k", KV, E), ("v", KV, E)))}
    dims = {"o": (E, E), "gate": (F, E), "up": (F, E), "down": (E, F), "q": (E, E), "k": (KV, E), "v": (KV, E)}
    h = {n: be.dev_upload("Q8_0", w, *dims[n]) for n, w in mats.items()}
    att, x0 = dev(rng.standard_normal(E, dtype=np.float32)), dev(rng.standard_normal(E, dtype=np.float32))
    n1, n2 = dev(1 + 0.1 * rng.standard_normal(E, dtype=np.float32)), dev(1 + 0.1 * rng.standard_normal(E, dtype=np.float32))
    stream = torch.cuda.Stream()

    def buffers():
        return dict(x=x0.clone(), gate=torch.zeros(F, device="cuda"), up=torch.zeros(F, device="cuda"), q=torch.zeros(E, device="cuda"),
                    k=torch.zeros(KV, device="cuda"), v=torch.zeros(KV, device="cuda"))

    a, b = buffers(), buffers()
    P = lambda t: t.data_ptr()
    items = [dict(handles=[h["o"]], d_y=[P(a["x"])], d_x=P(att), accumulate=True),
             dict(handles=[h["gate"], h["up"]], d_y=[P(a["gate"]), P(a["up"])], d_x=P(a["x"]), norm_weight=P(n1), norm_eps=1e-5, depends=True),
             dict(handles=[h["down"]], d_y=[P(a["x"])], d_x=P(a["up"]), gate=P(a["gate"]), accumulate=True, depends=True),
             dict(handles=[h["q"], h["k"], h["v"]], d_y=[P(a["q"]), P(a["k"]), P(a["v"])], d_x=P(a["x"]), norm_weight=P(n2), norm_eps=1e-5, depends=True)]
    lst = be.gemv_list_create(items, mode)
    torch.cuda.synchronize()
    be.dev_gemv_list(lst, stream.cuda_stream)
    be.dev_check(stream.cuda_stream)
    st = stream.cuda_stream
    be.dev_gemv_fused([h["o"]], [P(b["x"])], P(att), 1, mode, st, accumulate=True)
    be.dev_gemv_fused([h["gate"], h["up"]], [P(b["gate"]), P(b["up"])], P(b["x"]), 1, mode, st, norm_weight=P(n1), norm_eps=1e-5)
    be.dev_gemv_fused([h["down"]], [P(b["x"])], P(b["up"]), 1, mode, st, gate=P(b["gate"]), accumulate=True)
    be.dev_gemv_fused([h["q"], h["k"], h["v"]], [P(b["q"]), P(b["k"]), P(b["v"])], P(b["x"]), 1, mode, st, norm_weight=P(n2), norm_eps=1e-5)
    be.dev_check(st)
    for name in a:
        assert torch.equal(a[name], b[name]), name
    assert bool(torch.isfinite(a["q"]).all()) and float(a["q"].abs().max()) > 0
    # replayed from a graph, many times over: the chain keeps accumulating into x, and must keep matching
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            be.dev_gemv_list(lst, stream.cuda_stream)
        for _ in range(50):
            graph.replay()
    be.dev_check(stream.cuda_stream)
    for _ in range(50):
        be.dev_gemv_fused([h["o"]], [P(b["x"])], P(att), 1, mode, st, accumulate=True)
        be.dev_gemv_fused([h["gate"], h["up"]], [P(b["gate"]), P(b["up"])], P(b["x"]), 1, mode, st, norm_weight=P(n1), norm_eps=1e-5)
        be.dev_gemv_fused([h["down"]], [P(b["x"])], P(b["up"]), 1, mode, st, gate=P(b["gate"]), accumulate=True)
        be.dev_gemv_fused([h["q"], h["k"], h["v"]], [P(b["q"]), P(b["k"]), P(b["v"])], P(b["x"]), 1, mode, st, norm_weight=P(n2), norm_eps=1e-5)
    be.dev_check(st)
    for name in a:
        assert torch.equal(a[name], b[name]), f"{name} after 51 chained launches"
    del graph
    be.gemv_list_destroy(lst)
    for v in h.values():
        be.dev_free(v)


def test_long_list_of_weight_copies_is_deterministic(be, zo):
    """The benchmark's shape of use: many copies of one 4096 x 4096 tensor, one input, 64 items per launch, launched over
    and over; every output must equal the first and the error word must stay clear."""
    import torch
    rows = cols = 4096
    w = seeded_weights(Q8_0, rows, cols, 540)
    x = seeded_acts(1, cols, 541)
    copies = [be.dev_upload("Q8_0", w, rows, cols) for _ in range(8)]
    d_x = dev(x[0])
    ys = torch.zeros((64, rows), device="cuda")
    lst = be.gemv_list_create([dict(handles=[copies[i % 8]], d_y=[ys[i].data_ptr()], d_x=d_x.data_ptr()) for i in range(64)], ACT_INT8)
    stream = torch.cuda.Stream()
    bad = torch.zeros((), dtype=torch.int64, device="cuda")
    with torch.cuda.stream(stream):
        be.dev_gemv_list(lst, stream.cuda_stream)
        stream.synchronize()
        first = ys[0].clone()
        for _ in range(40):
            bad += (ys != first[None, :]).sum()
            ys.zero_()
            be.dev_gemv_list(lst, stream.cuda_stream)
        bad += (ys != first[None, :]).sum()
    be.dev_check(stream.cuda_stream)
    assert int(bad.item()) == 0
    assert_parity(first.cpu().numpy(), zo.gemv(Q8_0, w, x[0], rows, cols, int8_acts=True), what="list of weight copies vs oracle")
    be.gemv_list_destroy(lst)
    for h in copies:
        be.dev_free(h)


def test_list_rejects_bad_items(be):
    from zeninfer_b200 import BackendError
    w8 = seeded_weights(Q8_0, 16, 256, 550)
    w4 = seeded_weights(blocks.Q4_0, 16, 256, 551)
    h8, h4 = be.dev_upload("Q8_0", w8, 16, 256), be.dev_upload("Q4_0", w4, 16, 256)
    with pytest.raises(BackendError):
        be.gemv_list_create([], ACT_INT8)
    with pytest.raises(BackendError):
        be.gemv_list_create([dict(handles=[h4], d_y=[256], d_x=256)], ACT_FP32)                       # Q8_0 only
    with pytest.raises(BackendError):
        be.gemv_list_create([dict(handles=[h8], d_y=[256], d_x=256, gate=512, norm_weight=768)], ACT_INT8)   # one fused input at most
    with pytest.raises(BackendError):
        be.gemv_list_create([dict(handles=[h8], d_y=[256], d_x=260)], ACT_INT8)                       # misaligned input
    be.dev_free(h8)
    be.dev_free(h4)
