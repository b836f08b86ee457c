"""Row sharding of a projection across GPUs, and the one exchange step that follows it.

Output rows of a quantised product are independent (y[r] needs row r and x only), so a tensor is cut into
contiguous row ranges, one per rank; x is replicated; no collective runs inside the product.  The cut is the
reference's own worker cut, slice i of n = [rows*i/n, rows*(i+1)/n) (ComputePool::parallel_for,
src/compute_pool.cpp:104-106), rounded to the kernels' eight-row groups.  After the product every rank
all-gathers the fp32 output shards (NCCL over NVLink when the tensors are CUDA tensors, gloo on CPU), and the
lm_head then picks a token with the reference's greedy rule: the first maximum wins, non-finite logits never
win (sample_logits, src/adapters/dense_transformer_runtime.cpp:407-415).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from . import blocks

ROW_ALIGN = 8  # rows per group in the decode kernels


def row_shard(rows: int, world: int, rank: int, align: int = ROW_ALIGN) -> tuple[int, int]:
    """[first, last) of `rank`'s rows.  Boundaries are the pool's cut rounded down to `align`; the last shard
    takes the remainder, so shards tile [0, rows) exactly for any row count."""
    if not (0 <= rank < world) or rows < 0:
        raise ValueError("bad shard request")

    def cut(i: int) -> int:
        if i >= world:
            return rows
        return (rows * i // world) // align * align

    return cut(rank), cut(rank + 1)


def shard_plan(rows: int, world: int, align: int = ROW_ALIGN) -> list[tuple[int, int]]:
    return [row_shard(rows, world, r, align) for r in range(world)]


def raw_byte_range(first: int, last: int, row_bytes: int) -> tuple[int, int]:
    """Byte range of the file mapping a rank uploads: only its own rows are read."""
    return first * row_bytes, last * row_bytes


def all_gather_rows(local: torch.Tensor, rows: int, world: int, rank: int, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """local: [tokens, my_rows] fp32 -> [tokens, rows] on every rank.  Shards may differ in size; each is padded to
    the largest for the collective and trimmed afterwards."""
    plan = shard_plan(rows, world)
    widest = max(b - a for a, b in plan)
    tokens = local.shape[0]
    first, last = plan[rank]
    if local.shape[1] != last - first:
        raise ValueError(f"rank {rank} holds {local.shape[1]} rows, the plan says {last - first}")
    send = local if last - first == widest else torch.nn.functional.pad(local, (0, widest - (last - first)))
    send = send.contiguous()
    gathered = torch.empty((world, tokens, widest), dtype=local.dtype, device=local.device)
    if world == 1:
        gathered[0] = send
    else:
        dist.all_gather_into_tensor(gathered.view(world * tokens, widest), send, group=group)  # output = inputs stacked on dim 0
    full = out if out is not None else torch.empty((tokens, rows), dtype=local.dtype, device=local.device)
    for r, (a, b) in enumerate(plan):
        full[:, a:b] = gathered[r, :, : b - a]
    return full


def column_shard(packed: np.ndarray, fmt: int, rows: int, columns: int, world: int, rank: int) -> tuple[np.ndarray, int]:
    """The column cut that goes with an all-reduce: rank r keeps blocks [r * nb / world, (r + 1) * nb / world) of every
    row (whole quantisation blocks, so the codes and scales are untouched) as a contiguous [rows, bytes] copy, and
    multiplies them with the matching slice of the input.  Returns (rows of raw blocks, columns kept)."""
    be, bb = blocks.BLOCK_ELEMENTS[fmt], blocks.BLOCK_BYTES[fmt]
    nb = columns // be
    if columns % be or nb % world:
        raise ValueError(f"{columns} columns do not split into {world} runs of whole blocks")
    per = nb // world
    raw = np.asarray(packed).reshape(rows, nb, bb)[:, rank * per:(rank + 1) * per]
    return np.ascontiguousarray(raw).reshape(rows, per * bb), per * be


def greedy_pick(logits: torch.Tensor) -> torch.Tensor:
    """Per row: index of the first maximum among finite entries, -1 when a row has none.  [tokens, vocab] -> int64 [tokens]."""
    if logits.shape[1] == 0:  # an empty shard has no candidate
        return torch.full((logits.shape[0],), -1, dtype=torch.int64, device=logits.device)
    finite = torch.isfinite(logits)
    masked = torch.where(finite, logits, torch.full_like(logits, float("-inf")))
    best = masked.max(dim=1, keepdim=True).values
    idx = torch.arange(logits.shape[1], device=logits.device).expand_as(logits)
    first = torch.where((masked == best) & finite, idx, torch.full_like(idx, logits.shape[1])).min(dim=1).values
    return torch.where(first < logits.shape[1], first, torch.full_like(first, -1))


def sharded_greedy_pick(local: torch.Tensor, rows: int, world: int, rank: int, group=None) -> torch.Tensor:
    """The same pick without gathering the logits: each rank sends its best (value, global index) per token, 16 bytes,
    and every rank takes the first maximum over ranks.  Equal values resolve to the lowest index because shards are
    ordered by row."""
    first, _ = row_shard(rows, world, rank)
    local_idx = greedy_pick(local)
    has = local_idx >= 0
    safe = local_idx.clamp(min=0)
    neg_inf = torch.full((local.shape[0],), float("-inf"), dtype=torch.float64, device=local.device)
    val = torch.where(has, local.gather(1, safe[:, None])[:, 0].double(), neg_inf) if local.shape[1] else neg_inf
    pair = torch.stack([val, torch.where(has, (safe + first).double(), torch.full_like(val, -1.0))], dim=1)  # [tokens, 2]
    allp = torch.empty((world,) + pair.shape, dtype=pair.dtype, device=pair.device)
    if world == 1:
        allp[0] = pair
    else:
        dist.all_gather_into_tensor(allp.view(world * pair.shape[0], 2), pair.contiguous(), group=group)
    vals, idxs = allp[..., 0], allp[..., 1]                       # [world, tokens]
    best = vals.max(dim=0, keepdim=True).values
    cand = torch.where((vals == best) & (idxs >= 0), idxs, torch.full_like(idxs, float("inf")))
    pick = cand.min(dim=0).values
    return torch.where(torch.isfinite(pick), pick, torch.full_like(pick, -1.0)).long()


class PeerGather:
    """One rank's end of the all-gather that the decode kernels perform themselves (zen_cuda_dev_gemv_gather).

    Construction is collective: every rank allocates its gather region, the 64-byte IPC handles travel through
    torch.distributed (any backend: they are host bytes), every rank opens the others' regions and binds them.  After
    that no collective library is on the data path: a launch stores its outputs into every rank's region over NVLink
    and publishes an epoch; consumers wait on the device.  `slot_floats` is the capacity of one rank's slot,
    tokens x shard rows at most.  close() is collective too (no rank may free memory a peer can still write to).
    """

    def __init__(self, backend, world: int, rank: int, slot_floats: int, group=None):
        self.be, self.world, self.rank, self.slot_floats, self.group = backend, world, rank, slot_floats, group
        nbytes = backend.gather_region_bytes(world, slot_floats)
        if nbytes == 0:
            raise ValueError("bad gather geometry")
        self.own, handle = backend.ipc_alloc(nbytes)
        handles: list = [None] * world
        if world > 1:
            dist.all_gather_object(handles, handle, group=group)
        else:
            handles[0] = handle
        self.regions = [self.own if r == rank else backend.ipc_open(handles[r]) for r in range(world)]
        self.handle = backend.gather_create(world, rank, slot_floats, self.regions)
        if world > 1:
            dist.barrier(group=group)  # nobody launches before every rank has mapped every region

    def gemv(self, weights, d_x, tokens: int, act_mode: int, stream: int = 0, d_y=None) -> None:
        self.be.dev_gemv_gather(self.handle, weights, d_y, d_x, tokens, act_mode, stream)

    def fetch(self, d_out, stream: int = 0) -> None:
        """Device-side wait for every rank's latest launch, then a copy of the gathered [world][slot_floats] floats."""
        self.be.dev_gather_fetch(self.handle, d_out, stream)

    def allgather(self, d_piece: int, count: int, d_whole: int, stream: int = 0) -> None:
        """Plain all-gather of device vectors over this object's regions (zen_cuda_dev_allgather): rank r's `count` floats
        land at d_whole[r * count : (r + 1) * count] on every rank.  Not to be mixed with gemv() on one object."""
        self.be.dev_allgather(self.handle, d_piece, count, d_whole, stream)

    def allreduce_add(self, d_partial: int, count: int, d_inout: int, stream: int = 0) -> None:
        """d_inout += sum of every rank's d_partial, in rank order (zen_cuda_dev_allreduce_add)."""
        self.be.dev_allreduce_add(self.handle, d_partial, count, d_inout, stream)

    def close(self) -> None:
        if self.handle is None:
            return
        if self.world > 1:
            dist.barrier(group=self.group)  # callers synchronise their streams first; then nobody writes any more
        self.be.gather_destroy(self.handle)
        for r, p in enumerate(self.regions):
            if r != self.rank:
                self.be.ipc_close(p)
        if self.world > 1:
            dist.barrier(group=self.group)  # every mapping of the own region is gone before it is freed
        self.be.ipc_free(self.own)
        self.handle = None
