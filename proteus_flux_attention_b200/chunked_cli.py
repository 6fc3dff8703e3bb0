"""Command line of the chunked shortlist pipeline: ``python -m proteus_flux_attention_b200.chunked_cli``.

Same flags, log lines and JSON report layout as the reference's ``scripts/chunked_shortlist.py`` (:70-101 flags,
:186-197 report), on the sm_100a runner.  Differences: the device must be a CUDA device (there is no CPU path),
``--storage device`` keeps the sequence in HBM (``disk`` stages it in a float32 memory-mapped file as the reference
does, ``--temp-dir`` and ``--ram-limit-mb`` included), and three additions of this runner are exposed: ``--cuda-graph``, ``--freeze-prototypes`` and ``--score-only``."""
from __future__ import annotations

import argparse
import json
import logging
from dataclasses import asdict
from pathlib import Path
from typing import Optional

import torch

from .chunked_shortlist import ChunkedShortlistConfig, ChunkedShortlistRunner


def _load_sequence(path: Path, *, seq_len: int, d_model: int) -> torch.Tensor:
    if path.suffix == ".npy":
        import numpy as np
        tensor = torch.from_numpy(np.load(path))
    else:
        tensor = torch.load(path, map_location="cpu")
    if tensor.dim() == 2:
        tensor = tensor.unsqueeze(0)
    if tensor.dim() != 3 or tensor.size(0) != 1 or tensor.size(2) != d_model:
        raise ValueError(f"input tensor must have shape (1, seq_len, {d_model}); got {tuple(tensor.shape)}")
    if tensor.size(1) < seq_len:
        raise ValueError(f"input tensor holds {tensor.size(1)} tokens, fewer than --seq-len {seq_len}")
    return tensor[:, :seq_len].contiguous()


def _save_tensor(path: Path, tensor: torch.Tensor) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    torch.save(tensor.detach().cpu(), path)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Chunked Shortlist pipeline utility.")
    p.add_argument("--seq-len", type=int, default=1_000_000, help="Total sequence length to process.")
    p.add_argument("--d-model", type=int, default=512, help="Model width for embeddings.")
    p.add_argument("--chunk-len", type=int, default=65_536,
                   help="Tokens per streaming chunk (the runner's limit is 65,536; the reference's script defaults to 131,072, "
                        "which its own runner refuses too).")
    p.add_argument("--buffer-tokens", type=int, default=32_768, help="Maximum tokens kept after chunking.")
    p.add_argument("--per-chunk-budget", type=int, default=4_096, help="Tokens promoted from each chunk.")
    p.add_argument("--heads", type=int, default=8, help="Number of attention heads for both passes.")
    p.add_argument("--chunk-sparse-ratio", type=float, default=0.05, help="Keep ratio used in the chunk streaming stage.")
    p.add_argument("--final-sparse-ratio", type=float, default=0.5, help="Keep ratio for the final pass.")
    p.add_argument("--seed", type=int, default=7, help="Seed used when generating synthetic inputs.")
    p.add_argument("--shortlist-alpha", type=float, default=1.0, help="Shortlist alpha slider (0=dense, 1=linear shortlist).")
    p.add_argument("--nucleus-top-p", type=float, default=0.9, help="Top-p (nucleus) filter applied during chunk promotion.")
    p.add_argument("--device", default=None, help="Target CUDA device (default cuda:0).")
    p.add_argument("--progress", action="store_true", help="Accepted for compatibility; chunks are not timed one by one.")
    p.add_argument("--report-latency", action="store_true", help="Accepted for compatibility; CUDA-event metrics are always on.")
    p.add_argument("--no-final-pass", action="store_true", help="Skip the final attention pass.")
    p.add_argument("--storage", choices=["auto", "cpu", "disk", "device"], default="auto",
                   help="Where the sequence lives while it is streamed (cpu: pinned host memory; disk: memory-mapped file; device: HBM).")
    p.add_argument("--temp-dir", type=Path, help="Directory for the memory-mapped file of disk staging.")
    p.add_argument("--ram-limit-mb", type=int, help="Host memory above which auto / cpu storage falls back to disk.")
    p.add_argument("--input", type=Path, help="Optional input tensor (.pt or .npy) with shape (1, seq_len, d_model).")
    p.add_argument("--save-indices", type=Path, help="Optional path to save the retained indices (.pt).")
    p.add_argument("--save-reduced", type=Path, help="Optional path to save the reduced sequence (.pt).")
    p.add_argument("--save-final", type=Path, help="Optional path to save the final pass output (.pt).")
    p.add_argument("--save-report", type=Path, help="Optional JSON report destination.")
    p.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16", help="Activation and weight dtype.")
    p.add_argument("--cuda-graph", action="store_true", help="Replay pass 1 and pass 2 from CUDA graphs (needs --freeze-prototypes).")
    p.add_argument("--freeze-prototypes", action="store_true", help="Prototype EMA decay 1.0 in pass 1 (chunks independent).")
    p.add_argument("--score-only", action="store_true", help="Pass 1 runs router + token keep only (its attention output is unused).")
    p.add_argument("--log-level", default="INFO", choices=["DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL"],
                   help="Logging verbosity.")
    return p


def main(argv: Optional[list] = None) -> dict:
    args = build_parser().parse_args(argv)
    logging.basicConfig(level=getattr(logging, args.log_level.upper(), logging.INFO),
                        format="%(asctime)s | %(levelname)s | %(name)s | %(message)s")
    device = torch.device(args.device if args.device else "cuda")
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    sequence: Optional[torch.Tensor] = None
    if args.input:
        sequence = _load_sequence(Path(args.input), seq_len=args.seq_len, d_model=args.d_model).to(dtype)
        logging.info("Loaded input tensor from %s", args.input)
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        config = ChunkedShortlistConfig(
            seq_len=args.seq_len, d_model=args.d_model, chunk_len=args.chunk_len, buffer_tokens=args.buffer_tokens,
            per_chunk_budget=args.per_chunk_budget, device=device, heads=args.heads,
            chunk_sparse_ratio=args.chunk_sparse_ratio, final_sparse_ratio=args.final_sparse_ratio, seed=args.seed,
            report_latency=args.report_latency, progress=args.progress, run_final_pass=not args.no_final_pass,
            shortlist_alpha=args.shortlist_alpha, nucleus_top_p=args.nucleus_top_p, storage=args.storage,
            temp_dir=args.temp_dir, ram_limit_bytes=int(args.ram_limit_mb * 1024 * 1024) if args.ram_limit_mb else None,
            freeze_prototypes=args.freeze_prototypes, use_cuda_graph=args.cuda_graph,
            pass1_full_forward=not args.score_only)
        result = ChunkedShortlistRunner(config).run(sequence=sequence)
    finally:
        torch.set_default_dtype(old)
    m = result.metrics
    logging.info("Chunked Shortlist complete: retained %s/%s tokens (%.2f%%) on %s", m.retained_tokens, m.original_tokens,
                 m.retention_ratio * 100.0, m.device)
    for label, value, fmt in (("Chunk streaming latency", m.chunk_time_ms, "%.1f ms"),
                              ("Chunk throughput", m.chunk_tokens_per_s, "%.2f tok/s"),
                              ("Final pass latency", m.final_time_ms, "%.1f ms"),
                              ("Final pass throughput", m.final_tokens_per_s, "%.2f tok/s"),
                              ("Final pass peak memory", m.peak_memory_mb, "%.1f MB"),
                              ("Overall throughput", m.total_tokens_per_s, "%.2f tok/s")):
        if value is not None:
            logging.info("%s: " + fmt, label, value)
    logging.info("Storage mode: %s", m.storage_mode)
    if m.host_required_mb is not None:
        logging.info("Host requirement: %.1f MB", m.host_required_mb)
    if m.host_allocated_mb is not None:
        logging.info("Host allocated: %.1f MB", m.host_allocated_mb)
    if args.save_indices:
        _save_tensor(Path(args.save_indices), result.keep_indices)
        logging.info("Saved keep indices to %s", args.save_indices)
    if args.save_reduced:
        _save_tensor(Path(args.save_reduced), result.reduced_sequence)
        logging.info("Saved reduced sequence to %s", args.save_reduced)
    if args.save_final and result.final_output is not None:
        _save_tensor(Path(args.save_final), result.final_output)
        logging.info("Saved final output tensor to %s", args.save_final)
    report = {"metrics": asdict(m), "keep_indices": result.keep_indices.detach().cpu().tolist(),
              "keep_scores": result.keep_scores.detach().cpu().tolist(), "chunks": [asdict(c) for c in result.chunks],
              "backend_info": result.backend_info, "final_stats": result.final_stats}
    if args.save_report:
        path = Path(args.save_report)
        path.parent.mkdir(parents=True, exist_ok=True)
        with path.open("w", encoding="utf-8") as handle:
            json.dump(report, handle, indent=2, sort_keys=True)
        logging.info("Saved JSON report to %s", args.save_report)
    return report


if __name__ == "__main__":
    main()
