"""The output all-gather fused into the decode kernels (zen_cuda_dev_gemv_gather / zen_cuda_dev_gather_fetch).

With one GPU the gather object has a single rank: the kernel stores into its own region, publishes to itself, and a
launch never has to wait (the launch it depends on has already ended), so the whole code path -- slot addressing, parity,
epoch, last-CTA publication, chained input -- runs without any kernel waiting on another.  With two or more GPUs the
same checks run with one process per GPU (spawned here), shards on different devices and real peer stores.
Rows are independent, so a sharded product must reproduce the unsharded one bit for bit.
"""
import os
import socket

import numpy as np
import pytest

from helpers import assert_parity, seeded_acts, seeded_weights
from zeninfer_b200 import blocks, shard
from zeninfer_b200.backend import ACT_FP32, ACT_INT8

pytestmark = pytest.mark.gpu
NAMES = {blocks.Q8_0: "Q8_0", blocks.Q4_0: "Q4_0", blocks.Q6_K: "Q6_K"}


@pytest.fixture(scope="module")
def be():
    from zeninfer_b200 import Backend
    return Backend()


@pytest.mark.parametrize("fmt,mode,tokens", [(blocks.Q8_0, ACT_INT8, 1), (blocks.Q8_0, ACT_FP32, 3), (blocks.Q6_K, ACT_FP32, 1),
                                             (blocks.Q4_0, ACT_FP32, 2)])
def test_single_rank_gather_equals_plain_product(be, fmt, mode, tokens):
    import torch
    dev = torch.device("cuda", 0)
    rows, cols = 520, 2048
    w = seeded_weights(fmt, rows, cols, 300)
    h = be.dev_upload(NAMES[fmt], w, rows, cols)
    pg = shard.PeerGather(be, 1, 0, tokens * rows + 24)  # a slot larger than the payload: the tail must stay zero
    stream = torch.cuda.Stream(device=dev)
    for launch in range(5):  # both parities, several epochs
        x = torch.from_numpy(seeded_acts(tokens, cols, 310 + launch)).to(dev)
        y_plain = torch.zeros((tokens, rows), dtype=torch.float32, device=dev)
        y_side = torch.zeros((tokens, rows), dtype=torch.float32, device=dev)
        got = torch.full((tokens * rows + 24,), 7.0, dtype=torch.float32, device=dev)
        be.dev_gemv([h], [y_plain.data_ptr()], x.data_ptr(), tokens, mode, stream.cuda_stream)
        pg.gemv([h], x.data_ptr(), tokens, mode, stream.cuda_stream, d_y=[y_side.data_ptr()] if launch % 2 else None)
        pg.fetch(got.data_ptr(), stream.cuda_stream)
        stream.synchronize()
        be.dev_check(stream.cuda_stream)  # raises if a bounded wait gave up
        assert torch.equal(got[: tokens * rows].view(tokens, rows), y_plain)
        assert bool((got[tokens * rows:] == 0).all())
        if launch % 2:
            assert torch.equal(y_side, y_plain)
    pg.close()
    be.dev_free(h)


def test_single_rank_chain_reads_previous_gather(be):
    """x of launch n+1 is what launch n gathered (d_x = None): a chain y <- W y against the same chain made of plain
    launches through an ordinary buffer."""
    import torch
    dev = torch.device("cuda", 0)
    n = 1024
    w = seeded_weights(blocks.Q8_0, n, n, 320)
    h = be.dev_upload("Q8_0", w, n, n)
    pg = shard.PeerGather(be, 1, 0, n)
    stream = torch.cuda.Stream(device=dev)
    x0 = torch.from_numpy(seeded_acts(1, n, 321)).to(dev)
    a, b = x0.clone(), torch.zeros_like(x0)
    steps = 9
    pg.gemv([h], x0.data_ptr(), 1, ACT_INT8, stream.cuda_stream)
    for _ in range(steps - 1):
        pg.gemv([h], None, 1, ACT_INT8, stream.cuda_stream)
    got = torch.zeros(n, dtype=torch.float32, device=dev)
    pg.fetch(got.data_ptr(), stream.cuda_stream)
    for _ in range(steps):
        be.dev_gemv([h], [b.data_ptr()], a.data_ptr(), 1, ACT_INT8, stream.cuda_stream)
        a, b = b, a
    stream.synchronize()
    be.dev_check(stream.cuda_stream)
    assert torch.equal(got, a[0])
    pg.close()
    be.dev_free(h)


def test_single_rank_allgather(be):
    """zen_cuda_dev_allgather with one rank: the piece goes through the rank's own slot (both parities, several launches,
    two sizes on one object) and lands in the whole vector; in place when the piece is the whole vector's slice."""
    import torch
    from zeninfer_b200 import BackendError
    dev = torch.device("cuda", 0)
    pg = shard.PeerGather(be, 1, 0, 4096)
    stream = torch.cuda.Stream(device=dev)
    for launch, n in enumerate((4096, 128, 4096, 2048, 4)):
        piece = torch.from_numpy(seeded_acts(1, n, 340 + launch)[0]).to(dev)
        whole = torch.zeros(n, dtype=torch.float32, device=dev)
        pg.allgather(piece.data_ptr(), n, whole.data_ptr(), stream.cuda_stream)
        keep = piece.clone()
        pg.allgather(piece.data_ptr(), n, piece.data_ptr(), stream.cuda_stream)      # in place
        stream.synchronize()
        be.dev_check(stream.cuda_stream)
        assert torch.equal(whole, keep) and torch.equal(piece, keep)
    # the all-reduce on the same object (the launch numbering is shared): with one rank, inout += partial
    part = torch.from_numpy(seeded_acts(1, 1024, 350)[0]).to(dev)
    acc = torch.from_numpy(seeded_acts(1, 1024, 351)[0]).to(dev)
    want = acc + part
    pg.allreduce_add(part.data_ptr(), 1024, acc.data_ptr(), stream.cuda_stream)
    stream.synchronize()
    be.dev_check(stream.cuda_stream)
    assert torch.equal(acc, want)
    with pytest.raises(BackendError, match="dev_allreduce_add"):
        pg.allreduce_add(acc.data_ptr(), 1024, acc.data_ptr())       # in place is not a sum
    buf = torch.zeros(8192, dtype=torch.float32, device=dev)
    with pytest.raises(BackendError, match="dev_allgather"):
        pg.allgather(buf.data_ptr(), 6, buf.data_ptr())               # not a multiple of 4 floats
    with pytest.raises(BackendError, match="dev_allgather"):
        pg.allgather(buf.data_ptr(), 8192, buf.data_ptr())            # larger than the slot
    with pytest.raises(BackendError, match="dev_allgather"):
        pg.allgather(buf.data_ptr() + 4, 8, buf.data_ptr())           # not 16-byte aligned
    pg.close()


def test_gather_rejects_bad_geometry(be):
    from zeninfer_b200 import BackendError
    rows, cols = 64, 256
    w = seeded_weights(blocks.Q8_0, rows, cols, 330)
    h = be.dev_upload("Q8_0", w, rows, cols)
    pg = shard.PeerGather(be, 1, 0, 32)
    with pytest.raises(BackendError, match="exceed the gather slot"):
        pg.gemv([h], 1, 1, ACT_INT8)
    pg64 = shard.PeerGather(be, 1, 0, 64)
    with pytest.raises(BackendError, match="chained input"):
        pg64.gemv([h], None, 1, ACT_INT8)  # columns 256 != world x slot 64
    assert be.gather_region_bytes(9, 16) == 0 and be.gather_region_bytes(0, 16) == 0
    pg.close()
    pg64.close()
    be.dev_free(h)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), LOCAL_RANK=str(rank), ZEN_CUDA_DEVICE=str(rank),
                      NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # handles are host bytes: no NCCL anywhere in this test
    from zeninfer_b200 import Backend
    be = Backend()
    result = {}
    try:
        stream = torch.cuda.Stream(device=dev)
        # (1) lm_head-like shard product, Q6_K, 3 tokens: every rank ends up with all logits
        rows, cols, tokens = 1000, 1024, 3
        w = seeded_weights(blocks.Q6_K, rows, cols, 400)
        first, last = shard.row_shard(rows, world, rank)
        widest = max(b - a for a, b in shard.shard_plan(rows, world))
        h = be.dev_upload("Q6_K", w, rows, cols, first, last - first)
        pg = shard.PeerGather(be, world, rank, tokens * widest)
        x = torch.from_numpy(seeded_acts(tokens, cols, 401)).to(dev)
        got = torch.zeros((world, tokens * widest), dtype=torch.float32, device=dev)
        for _ in range(4):
            pg.gemv([h], x.data_ptr(), tokens, ACT_FP32, stream.cuda_stream)
        pg.fetch(got.data_ptr(), stream.cuda_stream)
        stream.synchronize()
        be.dev_check(stream.cuda_stream)
        result["err1"] = 0
        full = torch.zeros((tokens, rows), dtype=torch.float32, device=dev)
        for r, (a, b) in enumerate(shard.shard_plan(rows, world)):
            full[:, a:b] = got[r, : tokens * (b - a)].view(tokens, b - a)
        result["logits"] = full.cpu()
        result["pick"] = shard.greedy_pick(full).cpu()
        dist.barrier()
        pg.close()
        be.dev_free(h)

        # (2) a chain y <- W y, K = n = world x shard rows, 40 launches deep, with programmatic overlap between launches
        n = 2048
        per = n // world
        w2 = seeded_weights(blocks.Q8_0, n, n, 410)
        h_shard = be.dev_upload("Q8_0", w2, n, n, rank * per, per)
        h_full = be.dev_upload("Q8_0", w2, n, n)
        pg = shard.PeerGather(be, world, rank, per)
        x0 = torch.from_numpy(seeded_acts(1, n, 411) * np.float32(0.05)).to(dev)
        steps = 40
        pg.gemv([h_shard], x0.data_ptr(), 1, ACT_INT8, stream.cuda_stream)
        for _ in range(steps - 1):
            pg.gemv([h_shard], None, 1, ACT_INT8, stream.cuda_stream)
        chain = torch.zeros(n, dtype=torch.float32, device=dev)
        pg.fetch(chain.data_ptr(), stream.cuda_stream)
        a, b = x0.clone(), torch.zeros_like(x0)
        for _ in range(steps):
            be.dev_gemv([h_full], [b.data_ptr()], a.data_ptr(), 1, ACT_INT8, stream.cuda_stream)
            a, b = b, a
        stream.synchronize()
        be.dev_check(stream.cuda_stream)
        result["err2"] = 0
        result["chain_equal"] = bool(torch.equal(chain, a[0]))
        result["chain_finite"] = bool(torch.isfinite(chain).all())
        dist.barrier()
        pg.close()
        torch.save(result, os.path.join(out_dir, f"rank{rank}.pt"))
    except BaseException:
        # no barrier on the error path (the other ranks may never reach it): leave a traceback for the parent and a
        # failing exit status, on which the spawner ends the remaining ranks
        import traceback
        with open(os.path.join(out_dir, f"rank{rank}.err"), "w") as f:
            traceback.print_exc(file=f)
        os._exit(1)
    dist.barrier()
    dist.destroy_process_group()


def test_two_or_more_gpus_gather_matches_oracle(zo, tmp_path):
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    try:
        mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    finally:
        errors = {f: open(os.path.join(tmp_path, f)).read() for f in sorted(os.listdir(tmp_path)) if f.endswith(".err")}
        assert not errors, "\n".join(f"{f}:\n{t}" for f, t in errors.items())
    rows, cols, tokens = 1000, 1024, 3
    w = seeded_weights(blocks.Q6_K, rows, cols, 400)
    x = seeded_acts(tokens, cols, 401)
    ref = zo.gemm(blocks.Q6_K, w, x, tokens, rows, cols)
    for r in range(world):
        got = torch.load(os.path.join(tmp_path, f"rank{r}.pt"))
        assert got["err1"] == 0 and got["err2"] == 0
        assert_parity(got["logits"].numpy(), ref, what=f"rank {r} gathered logits vs oracle")
        assert got["pick"].tolist() == [zo.argmax(row) for row in got["logits"].numpy()]
        assert got["chain_finite"] and got["chain_equal"], f"rank {r}: sharded chain differs from the unsharded chain"
