"""Chunk sharding for the chunked shortlist pipeline: one process per GPU, chunks split into
contiguous ranges, fixed-size promotion records and kept rows exchanged with all-gather
(NCCL over NVLink on GPUs; the same code runs over gloo on CPU tensors in the tests).

The reference has no distributed code; the single-device run with frozen prototypes is the
definition these functions must reproduce.  Received data always lands in this rank's own memory
before any kernel reads it: no kernel here touches peer memory."""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
import torch.distributed as dist


import os

POOL_EXCHANGE = os.environ.get("ASPA_POOL_EXCHANGE", "allgather")   # "allgather" (one NCCL all-gather) or "p2p" (grouped send/recv)


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


class PackedRecords:
    """The promotion records of up to ``n_slots`` chunks in ONE int64 buffer, so that a single all-gather moves them:
    ``[idx (n_slots, budget) int64 | scores (n_slots, budget) fp32 | count (n_slots) int32]``, each region contiguous
    and handed to the kernels as an ordinary tensor view."""

    def __init__(self, n_slots: int, budget: int, device: torch.device):
        self.n_slots, self.budget = n_slots, budget
        nb = n_slots * budget
        self._n_idx, self._n_sc, self._n_ct = nb, (nb + 1) // 2, (n_slots + 1) // 2
        self.buf = torch.zeros(self._n_idx + self._n_sc + self._n_ct, dtype=torch.int64, device=device)
        self.idx, self.scores, self.count = self.views(self.buf)

    def views(self, buf: torch.Tensor):
        """(idx, scores, count) views of a buffer with this layout (1-D, or 2-D with one buffer per row)."""
        lead = buf.shape[:-1]
        a, b = self._n_idx, self._n_idx + self._n_sc
        idx = buf[..., :a].reshape(*lead, self.n_slots, self.budget)
        sc = buf[..., a:b].view(torch.float32)[..., : self.n_slots * self.budget].reshape(*lead, self.n_slots, self.budget)
        ct = buf[..., b:].view(torch.int32)[..., : self.n_slots]
        return idx, sc, ct


def all_gather_packed_records(group: Any, rec: PackedRecords, n_chunks: int, world: int):
    """One all-gather of every rank's ``PackedRecords`` buffer (each rank holds ``rec.n_slots`` = the per-rank maximum
    of chunk slots; unused slots carry index -1 / count 0) -> (scores, idx, count) of all chunks in chunk order."""
    if world == 1:
        return rec.scores, rec.idx, rec.count
    cap, budget = rec.n_slots, rec.budget
    recv = torch.empty((world, rec.buf.numel()), dtype=rec.buf.dtype, device=rec.buf.device)
    dist.all_gather_into_tensor(recv.view(-1), rec.buf, group=group)
    idx, sc, ct = rec.views(recv)                                      # (world, cap, budget) x2, (world, cap)
    idx, sc, ct = idx.reshape(world * cap, budget), sc.reshape(world * cap, budget), ct.reshape(world * cap)
    if cap * world != n_chunks:
        sel = _padding_free_rows(n_chunks, world, cap, rec.buf.device)
        idx, sc, ct = idx[sel], sc[sel], ct[sel]
    return sc.contiguous(), idx.contiguous(), ct.contiguous()


def all_gather_pool(group: Any, pool: torch.Tensor, world: int, deferred: bool = False):
    """Per-rank pools of promoted rows ``(cap * budget, C)`` -> ``(world * cap * budget, C)``, rank-major.  Each rank
    sends only the rows it promoted (8 MiB per rank for 2 chunks x 2048 rows x 1024 bf16 channels), where summing
    zero-padded copies of the whole reduced sequence would move all of it through every rank.

    With ``deferred`` the collective is only started: the return value is ``(rows, wait)`` and the current stream sees
    the rows after ``wait()``, so that work which does not need them (the merge of the records) runs beside the transfer."""
    if world == 1:
        return (pool, lambda: None) if deferred else pool
    recv = torch.empty((world * pool.size(0), pool.size(1)), dtype=pool.dtype, device=pool.device)
    if POOL_EXCHANGE == "p2p" and pool.is_cuda:
        # one send and one receive per peer in a single group call: through NVSwitch every pair has its own full-rate
        # path, so the pools cross in one hop instead of travelling round a ring
        rank = dist.get_rank(group)
        n = pool.size(0)
        recv[rank * n:(rank + 1) * n].copy_(pool)
        ops_ = []
        for step in range(1, world):
            dst, src = (rank + step) % world, (rank - step) % world
            ops_.append(dist.P2POp(dist.isend, pool, dist.get_global_rank(group, dst) if group is not None else dst, group))
            ops_.append(dist.P2POp(dist.irecv, recv[src * n:(src + 1) * n],
                                   dist.get_global_rank(group, src) if group is not None else src, group))
        reqs = dist.batch_isend_irecv(ops_)

        def wait_all():
            for req in reqs:
                req.wait()
        if deferred:
            return recv, wait_all
        wait_all()
        return recv
    if deferred:
        work = dist.all_gather_into_tensor(recv, pool.contiguous(), group=group, async_op=True)
        return recv, work.wait
    dist.all_gather_into_tensor(recv, pool.contiguous(), group=group)
    return recv


def pool_row_of_position(n_chunks: int, world: int, budget: int, device: torch.device) -> Optional[torch.Tensor]:
    """Where chunk-major promotion position ``c * budget + i`` lies in the rank-major gathered pool: ``None`` when the
    two orders coincide (every rank owns the same number of chunks), else the int64 offset to ADD per chunk
    (n_chunks,), built once per shape."""
    cap = max_chunks_per_rank(n_chunks, world)
    if cap * world == n_chunks:
        return None
    key = ("pool", n_chunks, world, budget, str(device))
    off = _SEL_CACHE.get(key)
    if off is None:
        vals = []
        for r in range(world):
            lo, hi = partition_chunks(n_chunks, world, r)
            vals.extend((r * cap + (c - lo) - c) * budget for c in range(lo, hi))
        off = torch.tensor(vals, dtype=torch.int64, device=device)
        _SEL_CACHE[key] = off
    return off


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
