"""Host logic of the multi-GPU path on CPU: the shard plan, the all-gather of output shards (gloo, world size 2 and 3)
and the greedy pick.  The CPU oracle stands in for the kernels, so what is tested is the plumbing around them."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from zeninfer_b200 import blocks, shard


def test_shard_plan_tiles_any_row_count():
    for rows in (0, 1, 7, 8, 9, 264, 4096, 14336, 128256):
        for world in (1, 2, 3, 4, 8):
            plan = shard.shard_plan(rows, world)
            assert plan[0][0] == 0 and plan[-1][1] == rows
            assert all(plan[i][1] == plan[i + 1][0] for i in range(world - 1))
            assert all(a % shard.ROW_ALIGN == 0 for a, _ in plan)
    # the lm_head of the benchmark configuration splits evenly: 128256 / 8 = 16032 rows, a multiple of 8
    assert shard.shard_plan(128256, 8) == [(16032 * i, 16032 * (i + 1)) for i in range(8)]
    assert shard.raw_byte_range(16032, 32064, 3360) == (16032 * 3360, 32064 * 3360)


def test_row_shard_matches_pool_cut_when_aligned(zo):
    # src/compute_pool.cpp:104-106: slice i of n = [count*i/n, count*(i+1)/n)
    for rows, world in ((4096, 4), (128256, 8), (14336, 2)):
        for r in range(world):
            assert shard.row_shard(rows, world, r) == zo.row_slice(rows, world, r)


def test_greedy_pick_rule(zo):
    rows = torch.tensor([[1.0, 3.0, 3.0, 2.0], [float("nan"), float("inf"), -5.0, -5.0],
                         [float("nan"), float("-inf"), float("inf"), float("nan")], [-0.0, 0.0, -1.0, -2.0]])
    got = shard.greedy_pick(rows).tolist()
    assert got == [zo.argmax(r.numpy()) for r in rows] == [1, 2, -1, 0]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, rows: int, cols: int, tokens: int, fmt: int, out_dir: str):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        zo = oracle.Oracle()
        w = np.random.default_rng(5).standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
        packed = blocks.quantize(fmt, w)
        x = np.random.default_rng(6).standard_normal((tokens, cols), dtype=np.float32)
        first, last = shard.row_shard(rows, world, rank)
        lo, hi = shard.raw_byte_range(first, last, blocks.row_bytes(fmt, cols))
        mine = np.frombuffer(packed.tobytes()[lo:hi], np.uint8)  # a rank touches only its byte range
        local = torch.from_numpy(zo.gemm(fmt, mine, x, tokens, last - first, cols)) if last > first else torch.empty((tokens, 0))
        if first == 0 and last > 0:
            local[0, 0] = float("nan")  # a non-finite logit must never be picked, wherever it lives
        full = shard.all_gather_rows(local, rows, world, rank)
        pick_full = shard.greedy_pick(full)
        pick_sharded = shard.sharded_greedy_pick(local, rows, world, rank)
        torch.save({"full": full, "pick_full": pick_full, "pick_sharded": pick_sharded}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,rows", [(2, 264), (3, 100), (2, 8)])
def test_all_gather_and_pick_over_gloo(zo, tmp_path, world, rows):
    cols, tokens, fmt = 256, 3, blocks.Q6_K
    mp.spawn(_worker, args=(world, _free_port(), rows, cols, tokens, fmt, str(tmp_path)), nprocs=world, join=True)
    w = np.random.default_rng(5).standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
    packed = blocks.quantize(fmt, w)
    x = np.random.default_rng(6).standard_normal((tokens, cols), dtype=np.float32)
    ref = zo.gemm(fmt, packed, x, tokens, rows, cols)
    ref[0, 0] = np.nan
    expect = [zo.argmax(r) for r in ref]
    for r in range(world):
        got = torch.load(os.path.join(tmp_path, f"r{r}.pt"))
        assert np.array_equal(got["full"].numpy(), ref, equal_nan=True)  # shards come from the same code, bit for bit
        assert got["pick_full"].tolist() == expect
        assert got["pick_sharded"].tolist() == expect


class _FakeBackend:
    """Stands in for the CUDA library in the collective set-up of PeerGather: hands out fake addresses and records calls."""

    def __init__(self, rank):
        self.rank, self.calls = rank, []

    def gather_region_bytes(self, world, slot):
        return 2 * world * slot * 4 + 64

    def ipc_alloc(self, nbytes):
        self.calls.append(("alloc", nbytes))
        return 0x1000 * (self.rank + 1), bytes([self.rank]) * 64

    def ipc_open(self, handle):
        assert len(handle) == 64 and len(set(handle)) == 1
        self.calls.append(("open", handle[0]))
        return 0x100000 + handle[0]

    def gather_create(self, world, rank, slot, regions):
        self.calls.append(("create", world, rank, slot, tuple(regions)))
        return 77

    def gather_destroy(self, g):
        self.calls.append(("destroy", g))

    def ipc_close(self, p):
        self.calls.append(("close", p))

    def ipc_free(self, p):
        self.calls.append(("free", p))


def _gather_worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        be = _FakeBackend(rank)
        pg = shard.PeerGather(be, world, rank, 4096)
        pg.close()
        pg.close()  # idempotent
        torch.save(be.calls, os.path.join(out_dir, f"g{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_peer_gather_setup_exchanges_handles_over_gloo(tmp_path):
    world = 3
    mp.spawn(_gather_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        calls = torch.load(os.path.join(tmp_path, f"g{r}.pt"))
        own = 0x1000 * (r + 1)
        expect_regions = tuple(own if q == r else 0x100000 + q for q in range(world))
        assert calls[0] == ("alloc", 2 * world * 4096 * 4 + 64)
        assert [c for c in calls if c[0] == "open"] == [("open", q) for q in range(world) if q != r]  # each peer once, never itself
        assert ("create", world, r, 4096, expect_regions) in calls
        assert calls[-1] == ("free", own) and calls.count(("destroy", 77)) == 1
        assert sorted(c[1] for c in calls if c[0] == "close") == sorted(p for q, p in enumerate(expect_regions) if q != r)


def test_column_shard_partial_products_add_up():
    """The column cut of the sharded decoder's o and down projections: every rank's blocks times its slice of the input,
    summed over the ranks, is the whole product (same decoded weights, same codes and scales)."""
    rows, cols = 24, 1024
    for fmt in (blocks.Q8_0, blocks.Q4_0, blocks.Q6_K):
        w = np.random.default_rng(9).standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
        packed = blocks.quantize(fmt, w)
        x = np.random.default_rng(10).standard_normal(cols, dtype=np.float32)
        whole = blocks.dequantize(fmt, packed, rows, cols).astype(np.float64) @ x.astype(np.float64)
        for world in (1, 2, 4):
            total = np.zeros(rows)
            for rank in range(world):
                part, kept = shard.column_shard(packed, fmt, rows, cols, world, rank)
                assert kept == cols // world and part.shape == (rows, blocks.row_bytes(fmt, kept)) and part.flags["C_CONTIGUOUS"]
                dec = blocks.dequantize(fmt, part, rows, kept)
                assert np.array_equal(dec, blocks.dequantize(fmt, packed, rows, cols)[:, rank * kept:(rank + 1) * kept])
                total += dec.astype(np.float64) @ x[rank * kept:(rank + 1) * kept].astype(np.float64)
            assert np.allclose(total, whole, rtol=0, atol=1e-9 * np.abs(whole).max())
    with pytest.raises(ValueError):
        shard.column_shard(blocks.quantize(blocks.Q6_K, np.zeros((2, 768), np.float32)), blocks.Q6_K, 2, 768, 2, 0)   # three super-blocks over two ranks
