"""World-size-2 gloo test of the chunk sharding plumbing: partition, record all-gather and row
all-gather reproduce the single-process result.  The per-chunk scores come from the CPU oracle
(the checker); the product functions under test are the ones in distributed.py."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from proteus_flux_attention_b200 import distributed as D


def test_partition_covers_every_chunk_once():
    for n in (1, 5, 16, 17):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                lo, hi = D.partition_chunks(n, world, r)
                assert 0 <= lo <= hi <= n
                seen.extend(range(lo, hi))
            assert seen == list(range(n))
    with pytest.raises(ValueError):
        D.partition_chunks(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_chunks, chunk_len, budget, buffer_tokens, seed, out_q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import aspa_oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(seed)
        T = n_chunks * chunk_len
        seq = torch.randn(1, T, 16, generator=g)
        imp = torch.rand(T, generator=g)
        mask = torch.rand(T, generator=g) > 0.5
        lo, hi = D.partition_chunks(n_chunks, world, rank)
        n_local = hi - lo
        sc = torch.zeros(max(n_local, 1), budget)
        ix = torch.full((max(n_local, 1), budget), -1, dtype=torch.int64)
        ct = torch.zeros(max(n_local, 1), dtype=torch.int32)
        for j, c in enumerate(range(lo, hi)):
            s0 = c * chunk_len
            r = O.select_top_tokens(imp[s0:s0 + chunk_len], mask[s0:s0 + chunk_len], s0, budget=budget, top_p=0.9)
            if r is not None:
                n = r[0].numel()
                sc[j, :n], ix[j, :n], ct[j] = r[0], r[1], n
        a_sc, a_ix, a_ct = D.all_gather_records(None, sc, ix, ct, n_chunks, world)
        valid = a_ix.view(-1) >= 0
        keep_idx, keep_sc = O.finalise_indices(a_sc.view(-1)[valid], a_ix.view(-1)[valid], max_tokens=buffer_tokens)
        mine = (keep_idx >= lo * chunk_len) & (keep_idx < hi * chunk_len)
        shard = seq[0, lo * chunk_len: hi * chunk_len]
        rows = shard[keep_idx[mine] - lo * chunk_len]
        reduced = D.all_gather_rows(None, rows, keep_idx.numel(), world)
        # the exchange the runner uses: every rank fills its own rows, zeros elsewhere, then a sum over ranks
        filled = torch.zeros(keep_idx.numel(), seq.size(2))
        filled[mine] = rows
        summed = D.sum_disjoint_rows(None, filled, world)
        assert torch.equal(summed, reduced)
        # the exchange of the sharded runner: one packed record buffer and one pool of promoted rows per rank
        cap = D.max_chunks_per_rank(n_chunks, world)
        rec = D.PackedRecords(cap, budget, torch.device("cpu"))
        rec.idx.fill_(-1)
        rec.scores[:n_local], rec.idx[:n_local], rec.count[:n_local] = sc[:n_local], ix[:n_local], ct[:n_local]
        p_sc, p_ix, p_ct = D.all_gather_packed_records(None, rec, n_chunks, world)
        assert torch.equal(p_sc, a_sc) and torch.equal(p_ix, a_ix) and torch.equal(p_ct, a_ct)
        pool = torch.zeros(cap * budget, seq.size(2))
        for j in range(n_local):
            n = int(ct[j])
            pool[j * budget: j * budget + n] = seq[0, ix[j, :n]]
        all_pool = D.all_gather_pool(None, pool, world)
        # the deferred form (started, then waited for after other work) moves the same rows
        later, arrived = D.all_gather_pool(None, pool, world, deferred=True)
        arrived()
        assert torch.equal(later, all_pool)
        # position of every kept index in the chunk-major promotion list, then in the rank-major gathered pool
        flat_ix = a_ix.view(-1)
        pos = torch.tensor([int((flat_ix == t).nonzero()[0]) for t in keep_idx.tolist()], dtype=torch.int64)
        off = D.pool_row_of_position(n_chunks, world, budget, torch.device("cpu"))
        if off is not None:
            pos = pos + off[pos // budget]
        assert torch.equal(all_pool[pos], reduced)
        out_q.put((rank, a_ct.tolist(), keep_idx.tolist(), reduced.clone()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_chunks", [4, 5])
def test_two_rank_sharding_equals_single_process(n_chunks):
    from oracle import aspa_oracle as O
    chunk_len, budget, buffer_tokens, seed = 64, 12, 30, 3
    g = torch.Generator().manual_seed(seed)
    T = n_chunks * chunk_len
    seq = torch.randn(1, T, 16, generator=g)
    imp = torch.rand(T, generator=g)
    mask = torch.rand(T, generator=g) > 0.5
    ss, ii = [], []
    for c in range(n_chunks):
        r = O.select_top_tokens(imp[c * chunk_len:(c + 1) * chunk_len], mask[c * chunk_len:(c + 1) * chunk_len],
                                c * chunk_len, budget=budget, top_p=0.9)
        ss.append(r[0])
        ii.append(r[1])
    want_idx, _ = O.finalise_indices(torch.cat(ss), torch.cat(ii), max_tokens=buffer_tokens)
    want_rows = seq[0, want_idx]

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n_chunks, chunk_len, budget, buffer_tokens, seed, q))
             for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, counts, keep, reduced in results:
        assert counts == [int(s.numel()) for s in ss]
        assert keep == want_idx.tolist()
        assert torch.equal(reduced, want_rows)
