"""Two-GPU test of the sharded chunked pipeline: ranks own disjoint chunk ranges, exchange promotion
records and promoted rows with NCCL all-gathers (eagerly, and captured inside one graph for the whole run), and must
reproduce the single-GPU result bit for bit.
Skipped when fewer than two CUDA devices are visible.  NVLS is switched off for the child processes."""
import os
import socket
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _states():
    import proteus_flux_attention_b200 as P
    from proteus_flux_attention_b200.chunked_shortlist import _build_model_config
    torch.manual_seed(5)
    a = P.AdaptiveSparseAttention(_build_model_config(2048, 256, heads=4, sparse_ratio=0.05, shortlist_alpha=1.0, router_top_p=0.9))
    b = P.AdaptiveSparseAttention(_build_model_config(320, 256, heads=4, sparse_ratio=0.5, shortlist_alpha=1.0, router_top_p=0.9))
    return ({k: v.to(torch.bfloat16) if v.dtype == torch.float32 and "routing" not in k else v for k, v in a.state_dict().items()},
            {k: v.to(torch.bfloat16) if v.dtype == torch.float32 and "routing" not in k else v for k, v in b.state_dict().items()})


def _cfg(dev):
    import proteus_flux_attention_b200 as P
    return P.ChunkedShortlistConfig(seq_len=5 * 2048, d_model=256, chunk_len=2048, buffer_tokens=320, per_chunk_budget=64,
                                    device=dev, heads=4, freeze_prototypes=True, warmup=False)


def _worker(rank, world, port, q):
    import traceback
    import torch.distributed as dist
    import proteus_flux_attention_b200 as P
    from proteus_flux_attention_b200 import distributed as D
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    started = False
    try:
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        started = True
        cs, fs = _states()
        seq = torch.randn(1, 5 * 2048, 256, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
        lo, hi = D.partition_chunks(5, world, rank)
        shard = seq[:, lo * 2048: hi * 2048].contiguous()
        for where, src in (("hbm", shard.to(dev)), ("host", shard.pin_memory())):  # resident shard, streamed shard
            res = P.ChunkedShortlistRunner(_cfg(dev), process_group=dist.group.WORLD).run(
                src, chunk_state=cs, final_state=fs, sequence_is_local_shard=True)
            q.put((rank, where, res.keep_indices.clone(), res.final_output.float().cpu(),
                   res.reduced_sequence.float().cpu()))
        # the whole sharded run (both collectives included) replayed from one captured graph, twice
        import dataclasses
        gcfg = dataclasses.replace(_cfg(dev), use_cuda_graph=True, whole_run_graph=True, collect_summaries=False)
        runner = P.ChunkedShortlistRunner(gcfg, process_group=dist.group.WORLD, cache_layers=True)
        src = shard.to(dev)
        for _ in range(2):
            res = runner.run(src, chunk_state=cs, final_state=fs, sequence_is_local_shard=True)
            assert "whole_run_graph" in runner.last_phase_ms
        q.put((rank, "graph", res.keep_indices.clone(), res.final_output.float().cpu(), res.reduced_sequence.float().cpu()))
        del res
        runner.close()   # graphs that hold collectives go before the process group does
    except BaseException:   # the parent fails fast on this and tears the peer down
        q.put(("error", rank, traceback.format_exc()))
        raise
    finally:
        if started:
            dist.destroy_process_group()


def test_two_gpu_sharding_equals_single_gpu():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import queue
    import torch.multiprocessing as mp
    import proteus_flux_attention_b200 as P
    dev = torch.device("cuda:0")
    cs, fs = _states()
    seq = torch.randn(1, 5 * 2048, 256, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    want = P.ChunkedShortlistRunner(_cfg(dev)).run(seq.to(dev), chunk_state=cs, final_state=fs)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    results = []
    try:
        # a worker that dies leaves its peer blocked in a collective: collect with a deadline, fail on the first
        # reported error or dead child, and never leave a child behind
        deadline = time.monotonic() + 300
        while len(results) < 3 * len(procs):
            assert time.monotonic() < deadline, "workers did not report within 300 s"
            try:
                item = q.get(timeout=5)
            except queue.Empty:
                dead = [p for p in procs if p.exitcode not in (None, 0)]
                assert not dead, f"worker exited with code {dead[0].exitcode} before reporting"
                continue
            assert item[0] != "error", f"rank {item[1]} failed:\n{item[2]}"
            results.append(item)
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    assert sorted((r[0], r[1]) for r in results) == [(0, "graph"), (0, "hbm"), (0, "host"), (1, "graph"), (1, "hbm"), (1, "host")]
    for rank, where, keep, out, red in results:
        assert torch.equal(keep, want.keep_indices)
        assert torch.equal(red, want.reduced_sequence.float().cpu())
        assert torch.equal(out, want.final_output.float().cpu())
