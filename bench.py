"""Benchmark of the ASPA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl b200|reference]

Workloads (synthetic, seeded; shapes of the reference's headline configurations):
  chunked_1m     1,048,576 tokens, d_model 1024, 16 heads, chunk 65,536, 2,048 promoted per chunk, final pass over
                 the merged 32,768-token shortlist, bf16.  Chunks are sharded over the N ranks (strong scaling).
  shortlist_256k one INT8 shortlist layer, 262,144 tokens, L = 4096 (local + anchors + prototype picks), bf16.
  sparse_16k     one sparse layer, batch 4 x 16,384 tokens, top-4 of 16 heads, keep 0.2, RoPE, bf16.
  sparse_4k_fp32 the reference's CPU-runnable case on the GPU: one sparse layer, 1 x 4096 x 512, fp32.
  lm_12l         a 12-layer decoder (d_model 768, 12 heads) around the drop-in module, 2 x 32,768 tokens, with a sweep
                 over sequence lengths naming the mode each resolves to.
  attn_dense_8k  the tile attention kernel alone (--attn-kernel auto|tcgen05|warp_mma), tensor roofline.
  chunk_64k, router_64k   one chunk step of pass 1 / the router alone, for profiler captures (--profile-mode).
A step is one pass of the hot path over one batch.  `value` is measured with inputs resident in HBM; `e2e` goes
through the public API with host buffers (host->device copies of the inputs and device->host reads of the results
inside the timed region).  One JSON line is printed by rank 0.  Besides the contract's keys it carries: `roofline`
(dominant kernel; `kernels_ms_per_step` and `kernels_frac_of_peak` from a strictly serial pass of the same steps),
`cpu_baseline`, `config.phases_ms_last_step` (CUDA-event phases of the last timed step; for sharded runs also
`phases_ms_chunk_by_chunk`), `config.self_check` (N = 1: the timed path against an eager run) or
`config.parity_vs_1rank` (N > 1: against a 1-rank run on rank 0), `config.cold_first_run_ms`.

`--run-graph auto|on|off` (chunked_1m): the whole sharded run from one CUDA graph (auto: on for N > 1).  The
environment variables ASPA_ATTN_TC_MODE and ASPA_ATTN_PICKS_MODE select attention kernels for A/B runs.

`--impl reference` times the reference's own CPU implementation on the host cores, all threads, on a bounded sample
of the same workload: the unmodified reference package out of `oracle/_ref` (installed there by `oracle/build_ref.py`;
`cpu_baseline.kind` "reference") - its `ChunkedShortlistRunner` with router-importance scoring, or its layer module -
and, only where that directory is missing, the CPU port under `oracle/` (`kind` "port").
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

try:
    METRIC = json.loads((ROOT / "BASELINE.json").read_text())["metric"]
except Exception:
    METRIC = "ASPA fwd tokens/sec (256K shortlist, 1M chunked @1/2/4/8 GPU); % HBM/TC roof"
SEQ_1M, CHUNK, BUDGET, BUFFER, D_MODEL, HEADS = 1 << 20, 65536, 2048, 32768, 1024, 16


# ----------------------------------------------------------------------------------------------- helpers
_NVML_CHILD = r"""
import sys, time, datetime
import pynvml as nv
nv.nvmlInit()
target, period = sys.argv[1], float(sys.argv[2])
try:
    h = nv.nvmlDeviceGetHandleByUUID(target.encode() if target.startswith("GPU-") else target)
except Exception:
    h = nv.nvmlDeviceGetHandleByIndex(int(target) if target.isdigit() else 0)
mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
while True:
    sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
    r = int(get(h))
    f = lambda bit: "Active" if r & bit else "Not Active"
    # NVML reason bits: 0x8 hw slowdown, 0x40 hw thermal slowdown, 0x20 sw thermal slowdown, 0x4 sw power cap
    print(datetime.datetime.now().strftime("%Y/%m/%d %H:%M:%S.%f"), sm, mx, hex(r), f(0x8), f(0x40), f(0x20), f(0x4),
          sep=", ", flush=True)
    time.sleep(period)
"""


class ClockSampler:
    """SM clock and throttle reasons, sampled by a separate process while the benchmark runs (a sampling thread in
    this process competes for the interpreter lock with the timed loop).  `nvml`: a small python child polling NVML;
    `smi`: one `nvidia-smi -lms` process.  Start it early - either needs a moment before its first line - and mark
    the timed region with begin()/end(); only samples whose timestamps fall inside that window are summarised."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, kind: str = "nvml", period_ms: int = 20):
        import datetime
        self.dt = datetime
        self.t0 = self.t1 = None
        self.kind = kind
        self.proc = None
        try:
            gpu = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
        except Exception:
            gpu = str(index)
        try:
            if kind == "nvml":
                self.proc = subprocess.Popen([sys.executable, "-c", _NVML_CHILD, gpu, str(period_ms / 1e3)],
                                             stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            elif kind == "smi":
                self.proc = subprocess.Popen(["nvidia-smi", "-i", gpu, f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                              "-lms", str(period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                             text=True)
        except Exception:
            self.proc = None
        # the child's lines are collected as they come, so that summary() can tell whether a sample exists yet
        self.lines = []
        if self.proc is not None:
            import threading

            def pump(stream, sink):
                for line in stream:
                    sink.append(line)
            threading.Thread(target=pump, args=(self.proc.stdout, self.lines), daemon=True).start()

    def begin(self):
        self.t0 = self.dt.datetime.now()

    def end(self):
        self.t1 = self.dt.datetime.now()

    def summary(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        # a timed region of a few tens of milliseconds can end before the child's first line: wait for one (the sample
        # nearest to the region is then reported, and says so)
        deadline = time.time() + 5.0
        time.sleep(0.05)
        while not self.lines and time.time() < deadline and self.proc.poll() is None:
            time.sleep(0.02)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=10)
        except Exception:
            self.proc.kill()
        rows, near = [], []
        for line in list(self.lines):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = self.dt.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
            except ValueError:
                continue
            near.append((ts, parts[1:]))
            if self.t0 is not None and self.t1 is not None and self.t0 <= ts <= self.t1:
                rows.append(parts[1:])
        window = "timed region"
        if not rows and near and self.t0 is not None:  # region shorter than the sampling period: the closest samples
            near.sort(key=lambda r: abs((r[0] - self.t0).total_seconds()))
            rows = [r[1] for r in near[:3]]
            window = "nearest to the timed region"
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": float(rows[0][1]),
                "reasons": reasons, "samples": len(rows), "window": window, "sampler": self.kind}


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the main kernels of one 65536-token chunk
# of the chunked_1m workload, from one-kernel ncu captures on B200 of the chunk_64k workload (the same chunk step alone;
# summaries: profiles/ncu_attn_rows64_chunk_64k.md, ncu_rope_inplace_chunk_64k.md, ncu_router_tc_chunk_64k.md,
# ncu_chunk_select_cluster_chunk_64k.md).
NCU_DRAM_BYTES_PER_LAUNCH = {
    "chunked_1m": {"attention": 224.7e6, "rope_inplace": 237.2e6, "router_tc": 138.8e6, "chunk_select": 0.4e6},
}


def bind_to_gpu_node(index: int):
    """Pin this process to the CPUs NVML reports as local to GPU `index` (read-only query), so that the pinned host
    buffers of a rank are first touched on the NUMA node its GPU hangs off.  Returns the CPU count, or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def peak_hbm():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def xavier_state(layer, dtype, seed):
    """Seeded Xavier-uniform weights for the layer's four matrices; identical on every rank."""
    g = torch.Generator().manual_seed(seed)
    sd = {k: v.clone() for k, v in layer.state_dict().items()}
    for k in ("qkv.weight", "proj.weight", "head_router.linear.weight", "routing_prototypes"):
        w = sd[k].float()
        bound = (6.0 / (w.size(0) + w.size(1))) ** 0.5
        w = (torch.rand(w.shape, generator=g) * 2 - 1) * bound
        sd[k] = w.to(dtype if k != "routing_prototypes" else torch.float32)
    return sd


def chunk_data(c: int, device, dtype):
    """Chunk c of the synthetic 1M sequence: N(0,1), seeded by the chunk index (independent of the rank count)."""
    g = torch.Generator(device=device).manual_seed(1000 + c)
    return torch.randn(CHUNK, D_MODEL, generator=g, device=device, dtype=torch.float32).to(dtype)


# ----------------------------------------------------------------------------------------------- workloads
class ChunkedWorkload:
    name = "chunked_1m"

    def __init__(self, device, world, rank, group, run_graph=True, full_forward=True, shard=None):
        import proteus_flux_attention_b200 as P
        from proteus_flux_attention_b200 import distributed as D
        from proteus_flux_attention_b200.chunked_shortlist import _build_model_config
        self.P, self.device, self.world, self.rank = P, device, world, rank
        self.tokens = SEQ_1M
        cfg = P.ChunkedShortlistConfig(seq_len=SEQ_1M, d_model=D_MODEL, chunk_len=CHUNK, buffer_tokens=BUFFER,
                                       per_chunk_budget=BUDGET, device=device, heads=HEADS, freeze_prototypes=True,
                                       warmup=False, collect_summaries=False, pass1_full_forward=bool(full_forward),
                                       use_cuda_graph=True, whole_run_graph=bool(run_graph))
        self.runner = P.ChunkedShortlistRunner(cfg, process_group=group, cache_layers=True)
        mk = lambda n, r: P.AdaptiveSparseAttention(_build_model_config(n, D_MODEL, heads=HEADS, sparse_ratio=r,  # noqa: E731
                                                                       shortlist_alpha=1.0, router_top_p=0.9))
        self.chunk_state = xavier_state(mk(CHUNK, 0.05), torch.bfloat16, 0)
        self.final_state = xavier_state(mk(BUFFER, 0.5), torch.bfloat16, 1)
        lo, hi = D.partition_chunks(SEQ_1M // CHUNK, world, rank)
        self.shard = shard if shard is not None else \
            torch.stack([chunk_data(c, device, torch.bfloat16) for c in range(lo, hi)]).view(1, -1, D_MODEL)
        self.host_shard = None
        self.config = {"workload": self.name, "seq_len": SEQ_1M, "d_model": D_MODEL, "heads": HEADS, "chunk_len": CHUNK,
                       "per_chunk_budget": BUDGET, "buffer_tokens": BUFFER,
                       "pass1": "full layer forward per chunk" if full_forward else "router + token keep per chunk",
                       "prototypes": "frozen during pass 1",
                       "pass1_launch": "one CUDA graph per run (both passes and the exchange)" if run_graph else "CUDA graph replay per chunk", "sharding": f"chunks over {world} rank(s)",
                       "l2": "inputs (2 GiB) larger than L2"}

    def step(self):
        res = self.runner.run(self.shard, chunk_state=self.chunk_state, final_state=self.final_state,
                              sequence_is_local_shard=True)
        self.phases_ms = dict(getattr(self.runner, "last_phase_ms", {}))
        if res.metrics.chunk_time_ms is not None:
            self.phases_ms["pass1_exchange_merge"] = round(res.metrics.chunk_time_ms, 3)
        return res

    def step_e2e(self):
        if self.host_shard is None:
            self.host_shard = self.shard.cpu().pin_memory()
            self.host_out = torch.empty((1, BUFFER, D_MODEL), dtype=torch.bfloat16, pin_memory=True)
        res = self.runner.run(self.host_shard, chunk_state=self.chunk_state, final_state=self.final_state,
                              sequence_is_local_shard=True)
        out = self.host_out[:, : res.final_output.size(1)]
        out.copy_(res.final_output, non_blocking=True)
        torch.cuda.synchronize()
        return self.host_shard.numel() * 2, out.numel() * 2 + res.keep_indices.numel() * 12


class LayerWorkload:
    # The layer call is issued on a stream of elevated priority: the layer puts its large projection GEMM on a second
    # stream one priority level lower, so the routing chain of the same call runs beside the GEMM instead of behind it.
    high_priority = True
    # ... and replayed from a captured CUDA graph when the call never waits for the host (both workloads here): at
    # 4 x 16384 tokens the host cost of the few dozen launches exceeds their device time.
    use_graph = True

    def __init__(self, name, device, seq_len=None):
        import proteus_flux_attention_b200 as P
        self.name, self.device = name, device
        self.B, self.T = {"sparse_16k": (4, 16384), "shortlist_256k": (1, 262144), "sparse_4k_fp32": (1, 4096)}[name]
        if seq_len:   # a shorter sequence through the same kernels, for profiler captures
            self.T = int(seq_len)
        cfg = dict(LAYER_CFGS[name])
        self.dtype = torch.float32 if name == "sparse_4k_fp32" else torch.bfloat16
        self.tokens = self.B * self.T
        layer = P.AdaptiveSparseProtoAttention(P.ModelConfig(**cfg))
        C = cfg["d_model"]
        self.state = xavier_state(layer, self.dtype, 0)
        self.layer = layer.to(self.dtype)
        self.layer.load_state_dict(self.state)
        self.layer = self.layer.to(device).eval()
        g = torch.Generator(device=device).manual_seed(0)
        x = torch.randn(self.B, self.T, C, generator=g, device=device)
        if name == "shortlist_256k":
            pos = torch.randperm(self.T, generator=torch.Generator().manual_seed(1))[:64].to(device)
            x[:, pos] *= 4.0
        self.x = x.to(self.dtype)
        self.host_x = None
        self.hp = torch.cuda.Stream(device=device, priority=-2) if self.high_priority else None
        self.step_events = []
        self.captured = None
        if self.use_graph:
            try:
                self.captured = P.CapturedLayerCall(self.layer, self.x)
                self.x = self.captured.static_in   # the resident input is the graph's own input: no copy per step
            except RuntimeError as e:
                print(f"[bench] {name}: layer call not capturable ({e}); eager calls", file=sys.stderr)
        self.config = {"workload": name, "batch": self.B, "seq_len": self.T, "d_model": C, "heads": cfg["attn_h_total"],
                       "l2": ("activations (>= 128 MiB per tensor) larger than L2" if self.B * self.T * C * 2 >= (128 << 20)
                              else "L2 flushed between steps (a 256 MiB buffer is rewritten)"),
                       "stream": "layer call on a priority -2 stream" if self.high_priority else "default priority",
                       "launch": "CUDA graph replay" if self.captured is not None else "eager"}

    def _call(self, x):
        if self.captured is not None:
            return self.captured(x)
        if self.hp is None:
            return self.layer(x)
        cur = torch.cuda.current_stream()
        self.hp.wait_stream(cur)
        with torch.cuda.stream(self.hp):
            y = self.layer(x)
        cur.wait_stream(self.hp)
        y.record_stream(cur)
        return y

    def _reset(self):
        # every forward moves the prototype EMA; restore it so each step does identical work
        for k in ("routing_prototypes", "routing_usage_ema", "routing_confidence"):
            getattr(self.layer, k).copy_(self.state[k])

    def step(self):
        self._reset()
        if self.B * self.T * self.x.size(2) * 2 < (128 << 20):   # inputs fit in L2: flush it between steps
            if not hasattr(self, "_flush"):
                self._flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.device)
            self._flush.zero_()
            # the flush is not part of the step: bracket the call itself; the caller sums these instead of one bracket
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            y = self._call(self.x)
            b.record()
            self.step_events.append((a, b))
            return y
        return self._call(self.x)

    def step_e2e(self):
        if self.host_x is None:
            self.host_x = self.x.cpu().pin_memory()
            self.host_y = torch.empty_like(self.host_x)  # pinned, like the input
        self._reset()
        y = self._call(self.host_x.to(self.device, non_blocking=True))
        self.host_y.copy_(y, non_blocking=True)
        torch.cuda.synchronize()
        return self.host_x.numel() * self.host_x.element_size(), y.numel() * y.element_size()


class LMWorkload:
    """BASELINE configuration 5: a 12-layer decoder (d_model 768, 12 heads x 64, RMSNorm, SwiGLU 3072, vocabulary
    32000) with the drop-in attention module in every layer and its automatic mode choice (dense fast path up to
    1024 tokens, dense / sparse below 16K, linear shortlist above), bf16, forward only, random N(0, 0.02) weights.
    Everything around the attention module is plain PyTorch, as it would be in a model that adopts the module."""
    name = "lm_12l"

    def __init__(self, device, B=2, T=32768):
        import torch.nn as nn
        import proteus_flux_attention_b200 as P
        self.device, self.B, self.T = device, B, T
        self.tokens = B * T
        d, H, L, V, F_ = 768, 12, 12, 32000, 3072

        class Block(nn.Module):
            def __init__(self):
                super().__init__()
                self.n1, self.n2 = nn.RMSNorm(d), nn.RMSNorm(d)
                self.attn = P.CausalASPAMultiheadAttention(d, H, bias=False, max_seq_len=32768, attn_small_seq_dense=1024,
                                                           attn_active_seq_low=1024, attn_linear_switch_ctx=16384,
                                                           attn_use_rope=True, attn_track_latency=False)
                self.w1, self.w3, self.w2 = nn.Linear(d, F_, bias=False), nn.Linear(d, F_, bias=False), nn.Linear(F_, d, bias=False)

            def forward(self, x):
                x = x + self.attn(self.n1(x), need_weights=False)[0]
                h = self.n2(x)
                return x + self.w2(torch.nn.functional.silu(self.w1(h)) * self.w3(h))

        class LM(nn.Module):
            def __init__(self):
                super().__init__()
                self.emb = nn.Embedding(V, d)
                self.blocks = nn.ModuleList(Block() for _ in range(L))
                self.norm, self.head = nn.RMSNorm(d), nn.Linear(d, V, bias=False)

            def forward(self, ids):
                x = self.emb(ids)
                for blk in self.blocks:
                    x = blk(x)
                return self.head(self.norm(x))

        torch.manual_seed(0)
        model = LM()
        with torch.no_grad():
            for prm in model.parameters():
                if prm.dim() >= 2:
                    prm.normal_(0.0, 0.02)
        self.model = model.to(torch.bfloat16).to(device).eval()
        self.ids = torch.randint(0, V, (B, T), generator=torch.Generator().manual_seed(0)).to(device)
        self.host_ids = None
        self.config = {"workload": self.name, "layers": L, "d_model": d, "heads": H, "mlp": "SwiGLU 3072", "vocab": V,
                       "batch": B, "seq_len": T, "l2": "activations (96 MiB per layer tensor, 4 GiB of logits) larger than L2"}
        # The whole forward from one CUDA graph where every attention call is one that never waits for the host
        # (shortlist mode at this length); eager otherwise.  `captured` is switched off by the kernel-timing passes.
        self.captured = None
        try:
            self.captured = P.CapturedModelCall(self.model, self.ids)
            self.config["launch"] = "one CUDA graph for the whole forward"
        except RuntimeError as err:
            self.config["launch"] = f"eager ({str(err)[:80]})"

    @torch.no_grad()
    def step(self):
        if self.captured is not None:
            return self.captured(self.ids)
        return self.model(self.ids)

    @torch.no_grad()
    def step_e2e(self):
        if self.host_ids is None:
            self.host_ids = self.ids.cpu().pin_memory()
            self.host_last = torch.empty((self.B, 32000), dtype=torch.bfloat16, pin_memory=True)
        ids = self.host_ids.to(self.device, non_blocking=True)
        logits = self.captured(ids) if self.captured is not None else self.model(ids)
        self.host_last.copy_(logits[:, -1], non_blocking=True)     # what a caller reads back: next-token logits
        torch.cuda.synchronize()
        return self.host_ids.numel() * 8, self.host_last.numel() * 2

    @torch.no_grad()
    def mode_sweep(self):
        """Attention mode the first layer picks at 512 / 2048 / 8192 / 32768 tokens, with the forward time of the model."""
        out = {}
        for T in (512, 2048, 8192, 32768):
            ids = self.ids[:, :T].contiguous()
            for _ in range(2):
                self.model(ids)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(3):
                self.model(ids)
            b.record()
            torch.cuda.synchronize()
            st = self.model.blocks[0].attn.attention._last_sparse_state or {}
            out[str(T)] = {"mode": st.get("mode"), "ms_per_forward": round(a.elapsed_time(b) / 3, 3),
                           "tokens_per_s": round(self.B * T / (a.elapsed_time(b) / 3e3))}
        return out


class AttentionWorkload:
    """The window-attention kernel alone, for profiling (--profile-mode): dense causal attention over 16 heads x 8192
    tokens x 64 channels, bf16 - 50 MB of q, k, v, resident in L2, which is the regime in which the tile products
    rather than HBM bound the kernel.  `--attn-kernel` forces the tcgen05 or the warp-MMA kernel."""
    name = "attn_dense_8k"

    def __init__(self, device, kernel="auto"):
        from proteus_flux_attention_b200 import _native as N
        from proteus_flux_attention_b200.sparse_attn import attention_packed
        self.device, self.call = device, attention_packed
        heads, T = 16, 8192
        self.heads, self.T, self.tokens = heads, T, T
        g = torch.Generator(device=device).manual_seed(0)
        self.q, self.k, self.v = (torch.randn(heads, T, 64, generator=g, device=device).to(torch.bfloat16) for _ in range(3))
        self.offs = torch.arange(0, (heads + 1) * T, T, dtype=torch.int32, device=device)
        self.tok = torch.arange(T, dtype=torch.int32, device=device).repeat(heads)
        self.out = torch.zeros(heads, T, 64, dtype=torch.bfloat16, device=device)
        N.lib().aspa_attn_tc_mode({"auto": 1, "tcgen05": 2, "warp_mma": 0}[kernel])
        self.flops = 4 * 64 * heads * T * (T + 1) / 2
        self.config = {"workload": self.name, "heads": heads, "seq_len": T, "head_dim": 64, "kernel": kernel,
                       "useful_flops_per_step": self.flops, "l2": "q, k, v (50 MB) resident in L2 on purpose"}

    def step(self):
        return self.call(self.q, self.k, self.v, row_offsets=self.offs, token_idx=self.tok, max_rows=self.T,
                         total_rows=self.heads * self.T, H=self.heads, plan=None, out=self.out)

    def step_e2e(self):
        self.step()
        torch.cuda.synchronize()
        return 0, 0


class ChunkStepWorkload:
    """One pass-1 chunk of the chunked pipeline alone, eagerly on one stream: the chunk layer over 65536 tokens plus
    the promotion of 2048 of them.  Holds about 1 GB on the device: the case profiler captures of the chunk kernels
    (`--profile-mode`) are taken on."""
    name = "chunk_64k"

    def __init__(self, device):
        import proteus_flux_attention_b200 as P
        from proteus_flux_attention_b200 import ops
        from proteus_flux_attention_b200.chunked_shortlist import _build_model_config
        self.ops, self.device, self.tokens = ops, device, CHUNK
        mc = _build_model_config(CHUNK, D_MODEL, heads=HEADS, sparse_ratio=0.05, shortlist_alpha=1.0, router_top_p=0.9)
        mc.attn_proto_decay = 1.0
        layer = P.AdaptiveSparseAttention(mc)
        layer.load_state_dict(xavier_state(layer, torch.bfloat16, 0))
        self.layer = layer.to(device=device, dtype=torch.bfloat16).eval()
        self.layer.set_shortlist_alpha(1.0)
        self.x = chunk_data(0, device, torch.bfloat16).view(1, CHUNK, D_MODEL)
        self.rec = (torch.zeros(1, BUDGET, device=device), torch.full((1, BUDGET), -1, dtype=torch.int64, device=device),
                    torch.zeros(1, dtype=torch.int32, device=device), torch.zeros(1, dtype=torch.int32, device=device),
                    torch.zeros(1, dtype=torch.int64, device=device))
        self.config = {"workload": self.name, "tokens": CHUNK, "d_model": D_MODEL, "heads": HEADS,
                       "l2": "activations (128 MiB per tensor) larger than L2"}

    def step(self):
        self.ops.SERIAL_STREAMS = True
        try:
            y = self.layer(self.x)
            sc, ix, ct, slot, offs = self.rec
            self.ops.chunk_select_slot(self.layer._last_token_importance.view(-1),
                                       self.layer._last_token_mask.view(torch.uint8).view(-1), BUDGET, 0.9, slot, offs, sc, ix, ct)
        finally:
            self.ops.SERIAL_STREAMS = False
        return y

    def step_e2e(self):
        self.step()
        torch.cuda.synchronize()
        return 0, 0


class RouterWorkload:
    """The router alone on 65536 tokens x 1024 channels (bf16, 16 gates with prototypes): the shape of one chunk of the
    chunked pipeline.  For profiling the tcgen05 kernel in isolation (--profile-mode)."""
    name = "router_64k"

    def __init__(self, device):
        from proteus_flux_attention_b200 import ops
        self.ops, self.device = ops, device
        self.tokens = 65536
        g = torch.Generator(device=device).manual_seed(0)
        self.x = torch.randn(self.tokens, D_MODEL, generator=g, device=device).to(torch.bfloat16)
        self.w = (torch.randn(16, D_MODEL, generator=g, device=device) * 0.03).to(torch.bfloat16)
        self.p = torch.nn.functional.normalize(torch.randn(16, D_MODEL, generator=g, device=device), dim=-1)
        self.conf = torch.full((16,), 1e-6, device=device)
        self.ub = torch.full((16,), 1.0 / 16, device=device)
        self.host_x = None
        self.config = {"workload": self.name, "tokens": self.tokens, "d_model": D_MODEL, "gates": 16,
                       "l2": "activations (134 MB) larger than L2"}

    def step(self):
        return self.ops.router_fwd(self.x, self.w, self.p, self.conf, self.ub, temp=0.3, threshold=0.2, span=0.8, blend=0.5,
                                   usage_boost=0.1, raw_stats=True)

    def step_e2e(self):
        if self.host_x is None:
            self.host_x = self.x.cpu().pin_memory()
            self.host_imp = torch.empty(self.tokens, dtype=torch.float32, pin_memory=True)
        x = self.host_x.to(self.device, non_blocking=True)
        out = self.ops.router_fwd(x, self.w, self.p, self.conf, self.ub, temp=0.3, threshold=0.2, span=0.8, blend=0.5,
                                  usage_boost=0.1, raw_stats=True)
        self.host_imp.copy_(out[1], non_blocking=True)
        torch.cuda.synchronize()
        return self.host_x.numel() * 2, self.host_imp.numel() * 4


# ----------------------------------------------------------------------------------------------- CPU baselines
LAYER_CFGS = {
    "sparse_16k": dict(d_model=1024, n_head=16, attn_h_total=16, attn_gates=16, attn_h_active=4, attn_h_active_min=4,
                       attn_h_active_max=4, attn_linear_head_k=4, attn_token_sparse=True, attn_token_keep_ratio=0.2,
                       attn_mode="auto", attn_small_seq_dense=0, attn_router_top_p=0.0, attn_use_rope=True,
                       attn_rope_base=10000.0, n_ctx=16384, attn_track_latency=False, attn_proto_enable=True),
    "shortlist_256k": dict(d_model=1024, n_head=16, attn_h_total=16, attn_mode="linear", attn_quantize_int8=True,
                           attn_linear_L=4096, attn_linear_L_base=4096, attn_linear_L_max=4096, attn_linear_window=4096,
                           attn_linear_anchor_stride=128, attn_linear_policy="local+anchors+proto", attn_h_active=2,
                           attn_h_active_min=2, attn_h_active_max=2, attn_token_sparse=True, attn_token_keep_ratio=0.2,
                           n_ctx=262144, attn_track_latency=False, attn_proto_enable=True),
    "sparse_4k_fp32": dict(d_model=512, n_head=8, attn_h_total=8, attn_h_active=2, attn_h_active_min=2, attn_h_active_max=2,
                           attn_gates=8, attn_token_sparse=True, attn_token_keep_ratio=0.25, attn_mode="auto",
                           attn_small_seq_dense=0, attn_router_top_p=0.0, n_ctx=4096, attn_track_latency=False,
                           attn_proto_enable=True),
}
REF_DIR = ROOT / "oracle" / "_ref"


def reference_package():
    """The unmodified reference, importable from oracle/_ref, forced onto its PyTorch CPU path; None if not installed."""
    if not (REF_DIR / "proteus_attention" / "__init__.py").exists():
        return None
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    import proteus_attention.kernels.sparse_attn as sa
    import proteus_attention.tools.chunked_shortlist as cs
    sa.TRITON_AVAILABLE = False
    if not getattr(cs, "_bench_importance_scoring", False):
        # On CPU the stock tool scores chunks by L2 norm (tools/chunked_shortlist.py:149-154).  The GPU semantics -
        # router importance - are what is benchmarked, so the selection is swapped for the importance-based CPU twin the
        # reference ships in scripts/chunked_shortlist_tests.py:58-84 (restated here: that script is not part of the package).
        def select_cpu(model, global_offset, *, per_chunk_budget, nucleus_top_p):
            imp = model._last_token_importance
            if imp is None:
                return None
            scores = imp.squeeze(0).to(torch.float32)
            m = model._last_token_mask
            if m is not None:
                scores = torch.where(m.squeeze(0).bool(), scores, torch.full_like(scores, float("-inf")))
            sel = cs._nucleus_select(scores, per_chunk_budget, nucleus_top_p)
            if sel is None:
                return None
            vals, idx = sel
            fin = torch.isfinite(vals)
            if not bool(fin.any()):
                return None
            return vals[fin], idx[fin] + int(global_offset)
        cs._select_top_tokens = select_cpu
        cs._bench_importance_scoring = True
    return cs


def _xav(shape, g):
    bound = (6.0 / (shape[0] + shape[1])) ** 0.5
    return (torch.rand(shape, generator=g) * 2 - 1) * bound


def _cpu_weights(C, G, g, dtype):
    return {"qkv.weight": _xav((3 * C, C), g).to(dtype), "proj.weight": _xav((C, C), g).to(dtype),
            "head_router.linear.weight": _xav((G, C), g).to(dtype), "routing_prototypes": _xav((G, C), g)}


def cpu_chunked_sample(n_chunks: int):
    """The chunked pipeline on the host cores over `n_chunks` chunks of the real size (65536 tokens, d_model 1024,
    16 heads, 2048 promoted per chunk, final pass over all promoted tokens), bf16.  Returns (tokens/s over the
    pipeline's two timed phases, seconds they took, kind, description)."""
    T = n_chunks * CHUNK
    seq = torch.randn(1, T, D_MODEL, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
    cs = reference_package()
    if cs is not None:
        cfg = cs.ChunkedShortlistConfig(seq_len=T, d_model=D_MODEL, chunk_len=CHUNK, buffer_tokens=n_chunks * BUDGET,
                                        per_chunk_budget=BUDGET, device=torch.device("cpu"), heads=HEADS, storage="cpu")
        torch.manual_seed(0)
        res = cs.ChunkedShortlistRunner(cfg).run(seq)
        secs = (float(res.metrics.chunk_time_ms) + float(res.metrics.final_time_ms or 0.0)) / 1e3
        return T / secs, secs, "reference", (
            f"the reference's ChunkedShortlistRunner (oracle/_ref, PyTorch CPU path, router-importance scoring) on "
            f"{n_chunks} of the 16 chunks: {n_chunks} x {CHUNK} tokens, d_model {D_MODEL}, {HEADS} heads, {BUDGET} promoted "
            f"per chunk, final pass over {n_chunks * BUDGET} tokens, bf16; time = its chunk stage + its final pass")
    from oracle import aspa_oracle as O
    g = torch.Generator().manual_seed(0)
    cw, fw = _cpu_weights(D_MODEL, 2 * HEADS, g, torch.bfloat16), _cpu_weights(D_MODEL, 2 * HEADS, g, torch.bfloat16)
    t0 = time.perf_counter()
    O.chunked_run(seq, chunk_len=CHUNK, buffer_tokens=n_chunks * BUDGET, per_chunk_budget=BUDGET, heads=HEADS,
                  chunk_weights=cw, final_weights=fw, freeze_prototypes=True)
    secs = time.perf_counter() - t0
    return T / secs, secs, "port", (f"CPU port of the reference (oracle/) on {n_chunks} of the 16 chunks: {n_chunks} x {CHUNK} "
                                    f"tokens, {BUDGET} promoted per chunk, final pass over {n_chunks * BUDGET} tokens, bf16")


def cpu_layer_sample(workload: str):
    """One layer call on the host cores on a bounded slice of the workload's input."""
    cfg = LAYER_CFGS[workload]
    dtype = torch.float32 if workload == "sparse_4k_fp32" else torch.bfloat16
    C = cfg["d_model"]
    T = {"sparse_16k": 16384, "shortlist_256k": 8192, "sparse_4k_fp32": 4096}[workload]
    what = {"sparse_16k": "one of the four batch rows (1 x 16384 tokens)", "shortlist_256k": f"the first {T} tokens",
            "sparse_4k_fp32": "the whole input (1 x 4096 tokens)"}[workload]
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, T, C, generator=g).to(dtype)
    gates = cfg.get("attn_gates", 2 * cfg["attn_h_total"])
    w = _cpu_weights(C, gates, g, dtype)
    if reference_package() is not None:
        from proteus_attention.models.aspa import AdaptiveSparseProtoAttention, ModelConfig
        old = torch.get_default_dtype()
        torch.set_default_dtype(dtype)
        try:
            mod = AdaptiveSparseProtoAttention(ModelConfig(**cfg)).eval()
        finally:
            torch.set_default_dtype(old)
        sd = mod.state_dict()
        sd.update(w)
        mod.load_state_dict(sd)
        with torch.no_grad():
            t0 = time.perf_counter()
            mod(x)
            secs = time.perf_counter() - t0
        return T / secs, secs, "reference", f"the reference's layer module (oracle/_ref, PyTorch CPU path) on {what}"
    from oracle import aspa_oracle as O
    lay = O.OracleLayer(w, **cfg)
    t0 = time.perf_counter()
    lay.forward(x)
    secs = time.perf_counter() - t0
    return T / secs, secs, "port", f"CPU port of the reference (oracle/) on {what}"


def cpu_sample(workload: str, n_chunks: int = 2):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    v, secs, kind, desc = cpu_chunked_sample(n_chunks) if workload == "chunked_1m" else cpu_layer_sample(workload)
    return v, secs, cores, kind, desc


def reference_arm(args):
    """`--impl reference`: K timed steps (after W // 3 untimed ones) of the CPU baseline, each on a sample sized so that
    the whole run stays within a few minutes; for the chunked pipeline the sample is as many whole chunks as fit."""
    budget_s = 200.0
    runs = args.steps + max(1, args.warmup // 3)
    n_chunks = 1
    v, secs, cores, kind, desc = cpu_sample(args.workload, 1)     # calibration run, also the first warm-up
    if args.workload == "chunked_1m":
        n_chunks = int(max(1, min(SEQ_1M // CHUNK, (budget_s / runs) // max(secs, 1e-3))))
    for _ in range(max(0, args.warmup // 3 - 1)):
        cpu_sample(args.workload, n_chunks)
    vals = []
    for _ in range(args.steps):
        v, secs, cores, kind, desc = cpu_sample(args.workload, n_chunks)
        vals.append(v)
    v = statistics.mean(vals)
    cfg = {"workload": args.workload}
    if args.workload == "chunked_1m":
        cfg.update({"seq_len": n_chunks * CHUNK, "d_model": D_MODEL, "heads": HEADS, "chunk_len": CHUNK,
                    "per_chunk_budget": BUDGET, "buffer_tokens": n_chunks * BUDGET,
                    "sample_of": f"{n_chunks} of the {SEQ_1M // CHUNK} chunks of the 1,048,576-token job per step"})
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
                      "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
                      "scaling": "strong" if args.workload == "chunked_1m" else "replicas",
                      "vs_baseline": None, "dtype": "f32" if args.workload == "sparse_4k_fp32" else "bf16", "data": "synthetic",
                      "config": cfg,
                      "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": desc},
                      "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


# ----------------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--run-graph", default="auto", choices=["auto", "on", "off"],
                    help="chunked_1m: replay the whole run from one CUDA graph (on) or launch it chunk by chunk, one graph "
                         "per chunk (off); auto = on for sharded runs, where a rank's few chunks leave the host behind "
                         "the device, off on one GPU, where sixteen chunks keep it ahead (measured: 7.6 against 7.9 ms)")
    ap.add_argument("--workload", default="chunked_1m", choices=["chunked_1m", "shortlist_256k", "sparse_16k", "sparse_4k_fp32", "lm_12l", "attn_dense_8k", "chunk_64k", "router_64k"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--layer-seq-len", type=int, default=None,
                    help="single-layer workloads: run the same layer on a shorter sequence (for profiler captures)")
    ap.add_argument("--attn-kernel", default="auto", choices=["auto", "tcgen05", "warp_mma"],
                    help="attn_dense_8k only: which tile kernel runs the window pass")
    ap.add_argument("--no-parity-check", action="store_true",
                    help="multi-GPU runs: skip the untimed comparison of the N-rank result with a 1-rank run on rank 0")
    ap.add_argument("--no-other-workloads", action="store_true",
                    help="skip the shortlist_256k / sparse_16k side measurements of the default run")
    ap.add_argument("--clock-sampler", default="nvml", choices=["nvml", "smi", "none"],
                    help="how SM clocks / throttle reasons are sampled during the timed region")
    ap.add_argument("--clock-period-ms", type=int, default=20)
    ap.add_argument("--bind-numa", action="store_true",
                    help="multi-GPU runs: pin each rank to the CPUs NVML reports as local to its GPU before the pinned "
                         "host buffers of the end-to-end measurement are allocated (off by default)")
    ap.add_argument("--profile-mode", action="store_true",
                    help="for runs under a profiler: exactly --warmup + --steps passes, no timing pass, e2e or CPU baseline")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            reference_arm(args)
        return

    import torch.distributed as dist
    from proteus_flux_attention_b200 import _native, ops
    _native.lib()  # no fallback: fail here if the CUDA library is missing
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    # started this early because its child needs about a second before its first sample, and the timed region of a
    # sharded run lasts a few tens of milliseconds
    clocks = ClockSampler(local_rank, args.clock_sampler, args.clock_period_ms)
    cpu_affinity = bind_to_gpu_node(local_rank) if (world > 1 and args.bind_numa) else None
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
    if args.workload == "chunked_1m":
        wl = ChunkedWorkload(device, world, rank, group, run_graph=args.run_graph == "on" or (args.run_graph == "auto" and world > 1))
    else:
        if world > 1:
            raise SystemExit("layer workloads do not shard: run them with --gpus 1 (replicas only)")
        if args.workload == "router_64k":
            wl = RouterWorkload(device)
        elif args.workload == "lm_12l":
            wl = LMWorkload(device)
        elif args.workload == "attn_dense_8k":
            wl = AttentionWorkload(device, args.attn_kernel)
        elif args.workload == "chunk_64k":
            wl = ChunkStepWorkload(device)
        else:
            wl = LayerWorkload(args.workload, device, args.layer_seq_len)
    # Sharded runs: outside the timed region, rank 0 repeats the whole job alone (a one-member process group, the full
    # sequence regenerated from the same per-chunk seeds) and the kept indices and the final output of the N-rank run
    # must be bit-equal to it.
    if world > 1 and args.workload == "chunked_1m" and not args.no_parity_check:
        solo = dist.new_group([0])
        res_n = wl.step()
        torch.cuda.synchronize()
        ok = True
        if rank == 0:
            wl1 = ChunkedWorkload(device, 1, 0, solo, run_graph=False)
            res_1 = wl1.step()
            torch.cuda.synchronize()
            ok = (torch.equal(res_n.keep_indices, res_1.keep_indices) and torch.equal(res_n.final_output, res_1.final_output)
                  and torch.equal(res_n.reduced_sequence, res_1.reduced_sequence))
            del wl1, res_1
            torch.cuda.empty_cache()
        wl.config["parity_vs_1rank"] = bool(ok)
        dist.barrier()
    # One GPU: outside the timed region, the run as it is timed (graph replay, lanes, speculative pass 2) must give
    # exactly what the same job gives eagerly on one stream, and a well-formed result.
    if world == 1 and args.workload == "chunked_1m" and not args.profile_mode:
        res_g = wl.step()
        wl.runner.config.use_cuda_graph = False
        res_e = wl.step()
        wl.runner.config.use_cuda_graph = True
        ki = res_g.keep_indices
        wl.config["self_check"] = bool(
            torch.equal(ki, res_e.keep_indices) and torch.equal(res_g.final_output, res_e.final_output)
            and ki.numel() == BUFFER and bool((ki[1:] > ki[:-1]).all()) and int(ki.min()) >= 0 and int(ki.max()) < SEQ_1M
            and bool(torch.isfinite(res_g.final_output.float()).all()) and bool(torch.isfinite(res_g.keep_scores).all())
            and torch.equal(res_g.reduced_sequence[0], wl.shard[0][ki.to(device)]))
        del res_g, res_e
    if cpu_affinity is not None:
        wl.config["host_binding"] = f"each rank pinned to the {cpu_affinity} CPUs local to its GPU (NVML affinity)"

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.profile_mode:
        if clocks.proc is not None:   # no sampling under a profiler
            clocks.proc.terminate()
        for _ in range(args.warmup + args.steps):
            wl.step()
        sync()
        if rank == 0:
            print(json.dumps({"profile_mode": True, "workload": args.workload, "passes": args.warmup + args.steps}))
        return
    for _ in range(max(3, args.warmup)):
        wl.step()
    sync()
    launches0 = ops.LAUNCHES
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    clocks.begin()
    e0.record()
    for _ in range(args.steps):
        wl.step()
    e1.record()
    sync()
    clocks.end()
    ms = e0.elapsed_time(e1)
    if getattr(wl, "step_events", None):   # steps that flush L2 in between time each call on its own
        ms = sum(a.elapsed_time(b) for a, b in wl.step_events[-args.steps:])
    launches = ops.LAUNCHES - launches0
    clock_summary = clocks.summary()
    if hasattr(wl, "phases_ms"):  # device time of the phases of the last timed step, on this rank
        wl.config["phases_ms_last_step"] = wl.phases_ms
        if getattr(wl.runner.config, "whole_run_graph", False):   # ... and of one step launched chunk by chunk
            wl.runner.config.whole_run_graph = False
            for _ in range(4):
                wl.step()
            wl.config["phases_ms_chunk_by_chunk"] = wl.phases_ms
            wl.runner.config.whole_run_graph = True
    t = torch.tensor([ms], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ms_per_step = ms / args.steps
    value = wl.tokens / (ms_per_step / 1e3)

    # per-kernel timing over the same steps (separate pass: events between kernels perturb overlap slightly).
    # Kernels replayed from a CUDA graph cannot be bracketed by events, so this pass launches them eagerly; it also
    # gives the launch count of one step (a graph replay launches exactly the kernels that were captured).
    if hasattr(wl, "runner"):
        wl.runner.config.use_cuda_graph = False
    captured = getattr(wl, "captured", None)
    if captured is not None:
        wl.captured = None
    launches0 = ops.LAUNCHES
    for _ in range(args.steps):     # launch count of a step as it really runs (forked streams, lanes), eagerly
        wl.step()
    launches = ops.LAUNCHES - launches0
    # ... and the kernel times from a strictly serial pass (nothing forked onto other streams): an event bracket around
    # a kernel that shares the GPU with another stream's GEMM would time the queueing, not the kernel
    ops.SERIAL_STREAMS = True
    ops.start_timing()
    for _ in range(args.steps):
        wl.step()
    kt = ops.stop_timing()
    ops.SERIAL_STREAMS = False
    if hasattr(wl, "runner"):
        wl.runner.config.use_cuda_graph = True
    if captured is not None:
        wl.captured = captured
    top = max(kt.items(), key=lambda kv: kv[1][1]) if kt else None
    peak, peak_kind = peak_hbm()
    roofline = None
    if top is not None:
        name, (n, tot_ms, nbytes) = top
        achieved = (nbytes / n) / (tot_ms / n * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                    "frac_of_nominal_8tbs": achieved / 8000.0,
                    "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload, {}).get(name) if world == 1 else None,
                    "launch_ms": tot_ms / n, "algorithmic_bytes_per_launch": nbytes / n,
                    "kernels_ms_per_step": {k: round(v[1] / args.steps, 4) for k, v in sorted(kt.items(), key=lambda kv: -kv[1][1])},
                    # the same serial pass per kernel: algorithmic bytes of its launches over their CUDA-event time, as a
                    # fraction of the peak (kernels that move next to nothing - selections, scans - read near zero here)
                    "kernels_frac_of_peak": {k: round((v[2] / max(v[1], 1e-9) / 1e6) / peak, 3)
                                             for k, v in sorted(kt.items(), key=lambda kv: -kv[1][1]) if v[2] > 0}}

    if args.workload == "attn_dense_8k":   # the tile products bound this one: useful flops against the measured GEMM peak
        pk = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"] if (ROOT / "MEASURED_PEAKS.json").exists() else 1590.0
        ach = wl.flops / (ms_per_step * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": "attention", "achieved": ach, "peak": pk, "unit": "TFLOP/s", "frac": ach / pk,
                    "peak_kind": "of measured" if (ROOT / "MEASURED_PEAKS.json").exists() else "of fallback", "traffic": None,
                    "note": "useful flops 4 * D * sum of row lengths; the kernel also multiplies the masked half of diagonal tiles"}
    if args.workload == "lm_12l":
        wl.config["mode_sweep"] = wl.mode_sweep()
    e2e = None
    if not args.no_e2e:
        for _ in range(2):
            wl.step_e2e()
        sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            h2d, d2h = wl.step_e2e()
        sync()
        dt = torch.tensor([time.perf_counter() - t0], device=device)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {"value": wl.tokens / (float(dt.item()) / args.steps), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h)}

    # one cold number: the first run() on a sequence at a NEW address (per-chunk graphs are keyed by address, so all
    # of pass 1 is captured afresh); layers stay cached.  Outside every timed region above.
    if args.workload == "chunked_1m" and not args.no_e2e:
        fresh = wl.shard.clone()
        sync()
        t0 = time.perf_counter()
        wl.runner.run(fresh, chunk_state=wl.chunk_state, final_state=wl.final_state, sequence_is_local_shard=True)
        torch.cuda.synchronize()
        wl.config["cold_first_run_ms"] = round((time.perf_counter() - t0) * 1e3, 2)
        wl.runner.run(wl.shard, chunk_state=wl.chunk_state, final_state=wl.final_state, sequence_is_local_shard=True)
        del fresh
        sync()

    # Beside the headline (never in its place): the same job with pass 1 reduced to what its result depends on.  The
    # reference runs a full layer forward per chunk and throws the output away (tools/chunked_shortlist.py:624-625);
    # router + token keep alone give the same promotions, hence the same kept tokens and the same final output, which
    # is checked here before the variant is timed.
    if args.workload == "chunked_1m" and not args.no_e2e:
        wl_so = ChunkedWorkload(device, world, rank, group, run_graph=wl.runner.config.whole_run_graph, full_forward=False,
                                shard=wl.shard)
        res_full, res_so = wl.step(), wl_so.step()
        same = bool(torch.equal(res_full.keep_indices, res_so.keep_indices) and torch.equal(res_full.final_output, res_so.final_output))
        del res_full, res_so
        for _ in range(3):
            wl_so.step()
        sync()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            wl_so.step()
        s1.record()
        sync()
        st = torch.tensor([s0.elapsed_time(s1) / args.steps], device=device)
        if world > 1:
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
        wl.config["pass1_score_only_variant"] = {"ms_per_step": round(float(st.item()), 4),
                                                 "tokens_per_s": round(wl.tokens / (float(st.item()) * 1e-3), 1),
                                                 "same_kept_tokens_and_output": same,
                                                 "note": "not the headline: pass 1 without the attention whose output the reference discards"}
        wl_so.runner.close()
        del wl_so
        sync()

    # the single-layer workloads of the same metric, measured in the same run (one GPU; they do not shard)
    others = None
    if rank == 0 and world == 1 and args.workload == "chunked_1m" and not args.no_other_workloads:
        others = {}
        for name, k in (("shortlist_256k", 5), ("sparse_16k", 20), ("sparse_4k_fp32", 20)):
            lw = LayerWorkload(name, device)
            for _ in range(3):
                lw.step()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(k):
                lw.step()
            b.record()
            torch.cuda.synchronize()
            ms_l = a.elapsed_time(b) / k
            if lw.step_events:
                ms_l = sum(x.elapsed_time(y) for x, y in lw.step_events[-k:]) / k
            others[name] = {"tokens_per_s": lw.tokens / (ms_l / 1e3), "ms_per_step": ms_l, "steps": k, "warmup": 3,
                            "config": lw.config}
            del lw
            torch.cuda.empty_cache()
        lm = LMWorkload(device)
        for _ in range(2):
            lm.step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            lm.step()
        b.record()
        torch.cuda.synchronize()
        ms_l = a.elapsed_time(b) / 3
        others["lm_12l"] = {"tokens_per_s": lm.tokens / (ms_l / 1e3), "ms_per_step": ms_l, "steps": 3, "warmup": 2,
                            "config": lm.config, "mode_sweep": lm.mode_sweep()}
        del lm
        torch.cuda.empty_cache()
        wl.config["other_workloads"] = others

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.workload in ("chunked_1m", *LAYER_CFGS):
        v, _, cores, kind, desc = cpu_sample(args.workload, 2)
        cpu = {"value": v, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": desc}
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                          "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
                          "scaling": "strong" if args.workload == "chunked_1m" else "replicas", "vs_baseline": None,
                          "dtype": "f32" if args.workload == "sparse_4k_fp32" else "bf16", "data": "synthetic",
                          "config": wl.config, "clocks": clock_summary,
                          "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu}))
    if world > 1:
        if hasattr(wl, "runner"):
            wl.runner.close()   # captured graphs that hold collectives go before the process group does
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
