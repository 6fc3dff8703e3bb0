"""Chunk sharding for the chunked shortlist pipeline: one process per GPU, chunks split into
contiguous ranges, fixed-size promotion records and kept rows exchanged with all-gather
(NCCL over NVLink on GPUs; the same code runs over gloo on CPU tensors in the tests).

The reference has no distributed code; the single-device run with frozen prototypes is the
definition these functions must reproduce.  Received data always lands in this rank's own memory
before any kernel reads it: no kernel here touches peer memory."""
from __future__ import annotations

from typing import Any, Tuple

import torch
import torch.distributed as dist


def world_and_rank(group: Any = None) -> Tuple[int, int]:
    if not (dist.is_available() and dist.is_initialized()):
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def partition_chunks(n_chunks: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous chunk range [lo, hi) of ``rank``; the first ``n_chunks % world`` ranks get one extra."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    base, extra = divmod(n_chunks, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def max_chunks_per_rank(n_chunks: int, world: int) -> int:
    return -(-n_chunks // world)


def all_gather_records(group: Any, scores: torch.Tensor, idx: torch.Tensor, count: torch.Tensor, n_chunks: int,
                       world: int):
    """Local (n_local, budget) records -> (n_chunks, budget) records of every chunk, in chunk order.

    Ranks may own different chunk counts; each pads to the per-rank maximum with empty records
    (index -1, count 0) so one fixed-size all-gather suffices, then the padding is dropped."""
    if world == 1:
        return scores, idx, count
    rank = dist.get_rank(group)
    budget = scores.size(1)
    cap = max_chunks_per_rank(n_chunks, world)
    lo, hi = partition_chunks(n_chunks, world, rank)
    n_local = hi - lo

    def pad(t: torch.Tensor, fill) -> torch.Tensor:
        out = torch.full((cap,) + tuple(t.shape[1:]), fill, dtype=t.dtype, device=t.device)
        out[:n_local] = t[:n_local]
        return out

    sends = [pad(scores, 0.0), pad(idx, -1), pad(count, 0)]
    outs = []
    for s in sends:
        # concatenated (not stacked) layout: the form every backend accepts
        recv = torch.empty((world * s.shape[0],) + tuple(s.shape[1:]), dtype=s.dtype, device=s.device)
        dist.all_gather_into_tensor(recv, s.contiguous(), group=group)
        outs.append(recv)
    if cap * world == n_chunks:  # every rank owns `cap` chunks: the concatenation is already in chunk order
        return outs[0].view(n_chunks, budget), outs[1].view(n_chunks, budget), outs[2].view(n_chunks)
    sel = _padding_free_rows(n_chunks, world, cap, scores.device)
    return (outs[0].view(world * cap, budget)[sel].contiguous(), outs[1].view(world * cap, budget)[sel].contiguous(),
            outs[2].view(world * cap)[sel].contiguous())


_SEL_CACHE: dict = {}


def _padding_free_rows(n_chunks: int, world: int, cap: int, device: torch.device) -> torch.Tensor:
    """Rows of the (world * cap) gathered layout that hold real chunks; built once per shape (an upload from the
    host stalls the stream)."""
    key = (n_chunks, world, cap, str(device))
    sel = _SEL_CACHE.get(key)
    if sel is None:
        keep = []
        for r in range(world):
            rlo, rhi = partition_chunks(n_chunks, world, r)
            keep.extend(r * cap + j for j in range(rhi - rlo))
        sel = torch.tensor(keep, dtype=torch.long, device=device)
        _SEL_CACHE[key] = sel
    return sel


def sum_disjoint_rows(group: Any, rows: torch.Tensor, world: int) -> torch.Tensor:
    """All-reduce (sum) of per-rank (k, C) row blocks in which every row is non-zero on at most one rank: each rank
    fills the kept rows it owns and leaves the others zero, so the sum is the complete reduced sequence, exactly
    (x + 0 is exact in every float format).  Fixed shapes, no host synchronisation."""
    if world > 1:
        dist.all_reduce(rows, op=dist.ReduceOp.SUM, group=group)
    return rows


def all_gather_rows(group: Any, rows: torch.Tensor, total: int, world: int) -> torch.Tensor:
    """Concatenate per-rank row blocks (rank order) into the (total, C) reduced sequence.

    Kept indices ascend and every rank owns a contiguous index range, so rank order is index order."""
    if world == 1:
        return rows
    n = torch.tensor([rows.size(0)], dtype=torch.int64, device=rows.device)
    counts = torch.empty(world, dtype=torch.int64, device=rows.device)
    dist.all_gather_into_tensor(counts, n, group=group)
    counts_h = counts.tolist()
    cap = max(counts_h)
    send = rows.new_zeros((cap, rows.size(1)))
    send[: rows.size(0)] = rows
    recv = rows.new_empty((world * cap, rows.size(1)))
    dist.all_gather_into_tensor(recv, send, group=group)
    out = torch.cat([recv[r * cap: r * cap + counts_h[r]] for r in range(world)], dim=0)
    if out.size(0) != total:
        raise RuntimeError(f"ranks contributed {out.size(0)} kept rows, expected {total}")
    return out
