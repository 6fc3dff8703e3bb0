"""Sequence-length sweep of the ASPA layer: ``python -m proteus_flux_attention_b200.tinytoy``.

The counterpart of the reference's benchmark harness (``kernels/tinytoy.py``): the same layer configuration per
sequence length (``build_aspa_config``, :274-347 - 32 heads, 64 gates, d_model 512, keep ratio and dense threshold
stepping with the length), the same batch rule (:487-495), BF16 and INT8 variants beside a dense
``nn.MultiheadAttention`` baseline, a table on stdout and a JSON summary with the reference's layout
(:1618-1634: ``device``, ``safe_*``, ``last_safe_*``, ``sequence_lengths``, ``base_batch_size``, ``d_model``,
``variant_labels``, ``runs``, ``auto_logs``, ``scaling_alpha``).  Not carried over: allocation probes, the Triton
autotuner, plotting, and the chunked-shortlist rows (see ``chunked_cli``).  Timing is by CUDA events."""
from __future__ import annotations

import argparse
import json
import math
import time
from pathlib import Path
from types import SimpleNamespace
from typing import Optional

import torch
import torch.nn as nn

from .aspa import AdaptiveSparseProtoAttention, ModelConfig

D_MODEL = 512
BASE_BATCH_SIZE = 4


def build_aspa_config(seq_len: int, seq_high: int, *, d_model: int, quantize: bool) -> SimpleNamespace:
    """The reference's per-length layer configuration (tinytoy.py:274-347), dense fast path off."""
    if seq_len <= 256:
        keep, keep_min, thr, dense_thr, act = 1.0, seq_len, 0.0, 0.20, 8
    elif seq_len <= 1024:
        keep, keep_min, thr, dense_thr, act = 0.8, 160, 0.04, 0.40, 6
    elif seq_len <= 4096:
        keep, keep_min, thr, dense_thr, act = 0.6, 192, 0.06, 0.60, 5
    else:
        keep, keep_min, thr, dense_thr, act = 0.45, 224, 0.08, 0.90, 4
    return SimpleNamespace(
        d_model=d_model, p_dropout=0.0, use_sdpa=False, attn_h_total=32, attn_h_active=act,
        attn_h_active_min=max(2, act // 2), attn_h_active_max=max(act, 8), attn_active_seq_low=256,
        attn_active_seq_high=seq_high, attn_small_seq_dense=0, n_ctx=seq_high, bias=False, attn_router_lambda=0.0,
        attn_router_beta=1.0, attn_router_reg_mode="entropy", attn_gates=64, attn_router_noise_std=0.0,
        attn_force_dense_threshold=dense_thr, attn_quantize_int8=quantize, attn_proto_enable=True,
        attn_proto_threshold=0.3, attn_proto_blend=0.6, attn_proto_temp=0.2, attn_proto_usage_boost=0.15,
        attn_proto_decay=0.97, attn_token_sparse=True, attn_token_keep_ratio=keep, attn_token_keep_min=keep_min,
        attn_token_keep_threshold=thr, attn_token_keep_guard=max(4, seq_len // 128), attn_linear_L_base=512,
        attn_linear_L_min=128, attn_linear_L_max=2048, attn_linear_L_schedule="sqrt", attn_linear_L_scale=1.0,
        attn_linear_L_scale_max=1.5, attn_linear_token_keep_schedule="sqrt", attn_linear_token_keep_min_ratio=0.2,
        attn_track_latency=False)


def effective_batch_size(seq_len: int, base: int = BASE_BATCH_SIZE) -> int:
    return 1 if seq_len >= 8192 else max(1, min(base, 4))


def runs_for(seq_len: int, num_runs: int = 50):
    """(warm-up runs, timed runs) of the reference's ``benchmark_forward_pass`` (:62-121)."""
    warm = 1 if seq_len >= 32768 else (2 if seq_len >= 16384 else (5 if seq_len >= 8192 else 10))
    if seq_len >= 524288:
        timed = 1
    elif seq_len >= 65536:
        timed = min(num_runs, 2)
    elif seq_len >= 32768:
        timed = min(num_runs, 3)
    elif seq_len >= 8192:
        timed = min(num_runs, 5)
    else:
        timed = num_runs
    return warm, timed


@torch.inference_mode()
def benchmark_forward_pass(model, x: torch.Tensor, num_runs: int = 50) -> float:
    warm, timed = runs_for(int(x.shape[1]), num_runs)
    for _ in range(warm):
        model(x)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(timed):
        model(x)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / timed


class _Dense(nn.Module):
    def __init__(self, d_model: int, heads: int):
        super().__init__()
        self.mha = nn.MultiheadAttention(d_model, heads, bias=False, batch_first=True)

    def forward(self, x):
        T = x.size(1)
        mask = torch.triu(torch.ones(T, T, dtype=torch.bool, device=x.device), diagonal=1)
        return self.mha(x, x, x, attn_mask=mask, need_weights=False)[0]


def _scaling_alpha(points) -> Optional[float]:
    """Slope of log(latency) over log(seq_len) (the reference's ``_estimate_alpha``)."""
    pts = [(math.log(s), math.log(l)) for s, l in points if s and l and l > 0]
    if len(pts) < 2:
        return None
    mx, my = sum(p[0] for p in pts) / len(pts), sum(p[1] for p in pts) / len(pts)
    den = sum((p[0] - mx) ** 2 for p in pts)
    return None if den == 0 else float(sum((p[0] - mx) * (p[1] - my) for p in pts) / den)


def main(argv: Optional[list] = None) -> dict:
    ap = argparse.ArgumentParser(description="Benchmark ASPA (Dynamic Mixture-of-Attention-Heads) kernels vs. standard attention.")
    ap.add_argument("--device", choices=["auto", "cuda"], default="auto", help="CUDA only: there is no CPU path.")
    ap.add_argument("--max-seq-len", type=int, default=262144, help="Limit the maximum sequence length.")
    ap.add_argument("--max-seq-count", type=int, default=None, help="Limit the number of sequence lengths to evaluate.")
    ap.add_argument("--disable-standard", action="store_true", help="Skip the dense attention baseline.")
    ap.add_argument("--disable-int8", action="store_true", help="Disable the INT8 variant.")
    ap.add_argument("--standard-max-seq-len", type=int, default=16384, help="Longest sequence the dense baseline is run on.")
    ap.add_argument("--report-dir", type=Path, default=None, help="Directory where the JSON summary is written.")
    ap.add_argument("--no-save", action="store_true", help="Disable writing the JSON summary to disk.")
    ap.add_argument("--cuda-fp32", action="store_true", help="float32 instead of the default bfloat16.")
    ap.add_argument("--num-runs", type=int, default=50)
    args = ap.parse_args(argv)
    device = torch.device("cuda")
    dtype = torch.float32 if args.cuda_fp32 else torch.bfloat16
    dtype_label = "FP32" if args.cuda_fp32 else "BF16"
    lengths = []
    s = 128
    while s <= args.max_seq_len:
        lengths.append(s)
        s *= 2
    if args.max_seq_count:
        lengths = lengths[: args.max_seq_count]
    seq_high = max(lengths)
    variants = [(f"ASPA ({dtype_label})", False, dtype_label.lower())]
    if not args.disable_int8 and not args.cuda_fp32:
        variants.append(("ASPA (INT8)", True, "int8"))
    runs, auto_logs = [], []
    header = f"{'Seq Len':<10} | {'Model':<24} | {'Latency (ms)':<15} | {'Tokens/s':<15} | {'Keep':<8} | {'k':<4} | {'Mode':<28}"
    print(header)
    print("-" * len(header))
    g = torch.Generator(device=device).manual_seed(0)
    for seq_len in lengths:
        batch = effective_batch_size(seq_len)
        x = torch.randn(batch, seq_len, D_MODEL, generator=g, device=device).to(dtype)
        if not args.disable_standard:
            rec = {"seq_len": seq_len, "model": "standard", "batch_size": batch}
            if seq_len <= args.standard_max_seq_len:
                try:
                    dense = _Dense(D_MODEL, 32).to(device=device, dtype=dtype).eval()
                    lat = benchmark_forward_pass(dense, x, args.num_runs)
                    rec.update(latency_ms=lat, tokens_per_s=batch * seq_len / (lat / 1e3), throughput_seq_s=batch / (lat / 1e3),
                               memory_mb=torch.cuda.max_memory_allocated() / 2 ** 20, backend="torch", status="ok")
                    print(f"{seq_len:<10} | {'Standard':<24} | {lat:<15.3f} | {rec['tokens_per_s']:<15.0f} | {'-':<8} | {'-':<4} | {'dense':<28}")
                    del dense
                except torch.OutOfMemoryError:
                    rec.update(latency_ms=None, tokens_per_s=None, status="oom", backend="torch")
                    torch.cuda.empty_cache()
            else:
                rec.update(latency_ms=None, tokens_per_s=None, status="limit", backend="std-limit")
            runs.append(rec)
        for label, quantize, key in variants:
            rec = {"seq_len": seq_len, "model": f"aspa_{key}", "variant": label, "quantized": quantize, "batch_size": batch}
            old = torch.get_default_dtype()
            torch.set_default_dtype(dtype)
            try:
                cfg = build_aspa_config(seq_len, seq_high, d_model=D_MODEL, quantize=quantize)
                layer = AdaptiveSparseProtoAttention(ModelConfig(**vars(cfg))).to(device).eval()
            finally:
                torch.set_default_dtype(old)
            torch.cuda.reset_peak_memory_stats()
            lat = benchmark_forward_pass(layer, x, args.num_runs)
            stats = dict(layer.last_head_stats or {})
            state = dict(layer._last_sparse_state or {})
            rec.update(latency_ms=lat, tokens_per_s=batch * seq_len / (lat / 1e3), throughput_seq_s=batch / (lat / 1e3),
                       memory_mb=torch.cuda.max_memory_allocated() / 2 ** 20, active_k=stats.get("target_k"),
                       token_fraction=stats.get("token_keep_fraction"), backend=state.get("backend"),
                       mode=stats.get("mode"), mode_selected=stats.get("mode_selected"), status="ok",
                       shortlist_alpha=stats.get("shortlist_alpha"))
            runs.append(rec)
            auto_logs.append({"label": label, "seq_len": seq_len, "batch_size": batch, "latency_ms": lat,
                              "tokens_per_s": rec["tokens_per_s"], "throughput_seq_s": rec["throughput_seq_s"],
                              "mode_setting": "auto", "mode_selected": rec["mode_selected"], "backend": rec["backend"],
                              "shortlist_backend": stats.get("linear_shortlist_backend"), "token_fraction": rec["token_fraction"],
                              "active_k": rec["active_k"], "quantized": quantize, "linear_L_effective": stats.get("linear_L"),
                              "shortlist_alpha": rec["shortlist_alpha"]})
            keep_s = "-" if rec["token_fraction"] is None else f"{rec['token_fraction']:.2f}"
            print(f"{seq_len:<10} | {label:<24} | {lat:<15.3f} | {rec['tokens_per_s']:<15.0f} | {keep_s:<8} | "
                  f"{str(rec['active_k']):<4} | {str(rec['mode_selected']):<28}")
            del layer
        del x
        torch.cuda.empty_cache()
        print("-" * len(header))
    ok = lambda model: [r for r in runs if r["model"] == model and r.get("status") == "ok"]  # noqa: E731
    record = {
        "device": str(device), "safe_standard": "none", "safe_aspa": "none", "safe_chunked_shortlist": "disabled",
        "last_safe_standard": max((r["seq_len"] for r in ok("standard")), default=None),
        "last_safe_variants": {key: max((r["seq_len"] for r in ok(f"aspa_{key}")), default=None) for _, _, key in variants},
        "last_safe_chunked_shortlist": None, "sequence_lengths": lengths, "base_batch_size": BASE_BATCH_SIZE,
        "d_model": D_MODEL, "variant_labels": {key: label for label, _, key in variants}, "runs": runs, "auto_logs": auto_logs,
        "scaling_alpha": {"standard": _scaling_alpha([(r["seq_len"], r["latency_ms"]) for r in ok("standard")]),
                          **{f"aspa_{key}": _scaling_alpha([(r["seq_len"], r["latency_ms"]) for r in ok(f"aspa_{key}")])
                             for _, _, key in variants}},
    }
    if not args.no_save:
        out_dir = args.report_dir or Path("reports") / "tinytoy"
        out_dir.mkdir(parents=True, exist_ok=True)
        path = out_dir / f"tinytoy_summary_{time.strftime('%Y%m%d-%H%M%S')}.json"
        with path.open("w", encoding="utf-8") as handle:
            json.dump(record, handle, indent=2)
            handle.write("\n")
        print(f"\n[Summary] Detailed JSON report saved to {path}")
    else:
        print("\n[Summary] JSON report saving disabled for this run.")
    return record


if __name__ == "__main__":
    main()
