"""Two-pass chunked shortlist pipeline on the sm_100a kernels.

Same public surface as the reference tool
(src/proteus_attention/tools/chunked_shortlist.py): ``ChunkedShortlistConfig``
(:314-366), ``ChunkedShortlistRunner.run`` (:382-827), ``ChunkedShortlistResult``
(:300-311), ``ChunkedShortlistMetrics`` (:276-297), ``ChunkSummary`` (:265-273).

Pass 1 runs the chunk layer over every chunk, promotes up to ``per_chunk_budget``
tokens per chunk by router importance (nucleus count + top-k, on the device) and
writes fixed-size ``(score, index)`` records.  The records of all chunks are merged
(``aspa_merge_finalise``), the kept rows are gathered into the reduced sequence and
pass 2 runs a fresh layer over it.

What is different from the reference, on purpose:
  * scoring always uses router importance (the reference silently switches to L2-norm
    scoring when its importance tensor is not on a CUDA device, :149-154, :632-647);
  * the sequence stays resident in HBM when it is given as a CUDA tensor; a CPU tensor is
    streamed chunk by chunk through pinned double buffers on a copy stream;
  * no host synchronisation per chunk: per-chunk summaries are built after the loop from
    one device-to-host copy;
  * chunks can be sharded over the ranks of a ``torch.distributed`` process group: rank r
    owns a contiguous range of chunks, the promotion records (one packed buffer) and the
    promoted rows (one pool per rank) are exchanged with two all-gathers, the merge and pass 2
    run replicated (see ``distributed.py``).
"""
from __future__ import annotations

import logging
import math
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Literal, Optional, Sequence, Tuple

import torch

from . import distributed as dist_utils
from . import ops
from .aspa import AdaptiveSparseAttention, ModelConfig
from .sparse_attn import get_last_backend_info

LOGGER = logging.getLogger(__name__)
MAX_SHORTLIST_CHUNK_TOKENS = 65_536
BYTES_PER_MB = 1024.0 * 1024.0


def _build_model_config(seq_len: int, d_model: int, *, heads: int, sparse_ratio: float, shortlist_alpha: float,
                        router_top_p: float) -> ModelConfig:
    """Layer configuration used for both passes (reference :88-137)."""
    return ModelConfig(
        vocab_size=0, n_ctx=seq_len, n_layer=1, n_head=heads, d_model=d_model, p_dropout=0.0, bias=False,
        attn_variant="aspa", attn_h_total=heads, attn_h_active=heads, attn_h_active_min=heads,
        attn_h_active_max=heads, attn_active_seq_low=max(128, seq_len // 4), attn_active_seq_high=seq_len,
        attn_mode="linear", attn_token_sparse=True, attn_token_keep_ratio=max(0.0, min(1.0, sparse_ratio)),
        attn_token_keep_min=max(4, int(seq_len * sparse_ratio * 0.5)), attn_token_keep_guard=4,
        attn_token_keep_threshold=0.0, attn_linear_L=256, attn_linear_L_base=256, attn_linear_L_min=64,
        attn_linear_L_max=256, attn_linear_switch_ctx=max(512, min(seq_len, 4096)),
        attn_linear_policy="local+anchors", attn_proto_enable=True, attn_proto_threshold=0.2, attn_proto_blend=0.5,
        attn_proto_temp=0.3, attn_linear_token_keep_schedule="sqrt", attn_linear_token_keep_min_ratio=0.05,
        attn_track_latency=False, attn_small_seq_dense=0, use_sdpa=False, attn_shortlist_alpha=shortlist_alpha,
        attn_router_top_p=router_top_p)


def _system_available_ram() -> Optional[int]:
    """Best-effort estimate of the available host memory in bytes (psutil, else sysconf)."""
    try:
        import psutil
        return int(psutil.virtual_memory().available)
    except Exception:
        pass
    try:
        import os
        return int(os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_AVPHYS_PAGES"))
    except (AttributeError, ValueError, TypeError, OSError):
        return None


def _sanitize_mapping(mapping: Dict[str, Any]) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    for key, value in mapping.items():
        if isinstance(value, torch.Tensor):
            out[key] = value.detach().cpu().item() if value.numel() == 1 else value.detach().cpu().tolist()
        elif isinstance(value, dict):
            out[key] = _sanitize_mapping(value)
        else:
            out[key] = value
    return out


@dataclass
class ChunkSummary:
    index: int
    start: int
    end: int
    promoted: Sequence[int] = field(default_factory=list)
    scores: Sequence[float] = field(default_factory=list)


@dataclass
class ChunkedShortlistMetrics:
    original_tokens: int
    retained_tokens: int
    retention_ratio: float
    chunk_count: int
    device: str
    chunk_time_ms: Optional[float] = None
    final_time_ms: Optional[float] = None
    total_time_ms: Optional[float] = None
    peak_memory_mb: Optional[float] = None
    used_fallback: bool = False
    chunk_tokens_per_s: Optional[float] = None
    final_tokens_per_s: Optional[float] = None
    total_tokens_per_s: Optional[float] = None
    storage_mode: str = "cpu"
    host_required_mb: Optional[float] = None
    host_allocated_mb: Optional[float] = None
    host_limit_mb: Optional[float] = None
    storage_reason: Optional[str] = None
    world_size: int = 1


@dataclass
class ChunkedShortlistResult:
    keep_indices: torch.Tensor
    keep_scores: torch.Tensor
    reduced_sequence: torch.Tensor
    metrics: ChunkedShortlistMetrics
    chunks: Sequence[ChunkSummary]
    final_output: Optional[torch.Tensor] = None
    final_stats: Optional[Dict[str, Any]] = None
    backend_info: Optional[Dict[str, Any]] = None


@dataclass
class ChunkedShortlistConfig:
    seq_len: int
    d_model: int
    chunk_len: int
    buffer_tokens: int
    per_chunk_budget: int
    device: torch.device
    heads: int = 8
    nucleus_top_p: float = 0.9
    chunk_sparse_ratio: float = 0.05
    final_sparse_ratio: float = 0.5
    seed: Optional[int] = 7
    report_latency: bool = False
    progress: bool = False
    run_final_pass: bool = True
    shortlist_alpha: float = 1.0
    storage: Literal["cpu", "disk", "auto", "device"] = "auto"
    temp_dir: Optional[Path] = None
    ram_limit_bytes: Optional[int] = None
    # --- additions of this implementation ---
    freeze_prototypes: bool = False      # EMA decay 1.0 in pass 1: chunks become independent (needed for sharding)
    pass1_full_forward: bool = True      # False: pass 1 runs only router + token keep (its attention output is unused)
    warmup: bool = True                  # the reference's untimed warm-up forward on noise (:583-589)
    collect_summaries: bool = True       # build the python-side summaries after the run: per-chunk lists and final_stats
                                         # (False: the final layer's telemetry stays readable on the layer object)
    use_cuda_graph: bool = False         # replay pass 1's per-chunk layer call from a captured CUDA graph
    whole_run_graph: bool = False        # with use_cuda_graph, a device-resident sequence and a caching runner: the whole
                                         # run (both passes, the exchange between ranks, the read-backs) is ONE graph

    def validate(self) -> None:
        if self.seq_len <= 0:
            raise ValueError("seq_len must be positive.")
        if self.d_model <= 0:
            raise ValueError("d_model must be positive.")
        if self.chunk_len <= 0:
            raise ValueError("chunk_len must be positive.")
        if self.chunk_len > MAX_SHORTLIST_CHUNK_TOKENS:
            raise ValueError(f"chunk_len={self.chunk_len} exceeds MAX_SHORTLIST_CHUNK_TOKENS={MAX_SHORTLIST_CHUNK_TOKENS}.")
        if self.buffer_tokens <= 0:
            raise ValueError("buffer_tokens must be positive.")
        if self.per_chunk_budget <= 0:
            raise ValueError("per_chunk_budget must be positive.")
        if not (0.0 < float(self.nucleus_top_p) <= 1.0):
            raise ValueError("nucleus_top_p must be within (0, 1].")
        if self.chunk_sparse_ratio <= 0.0:
            raise ValueError("chunk_sparse_ratio must be positive.")
        if self.final_sparse_ratio <= 0.0:
            raise ValueError("final_sparse_ratio must be positive.")
        if not (0.0 <= self.shortlist_alpha <= 1.0):
            raise ValueError("shortlist_alpha must be within [0, 1].")
        if self.use_cuda_graph and not self.freeze_prototypes:
            raise ValueError("use_cuda_graph needs freeze_prototypes=True (capture runs the layer extra times, which "
                             "would move the prototype state)")
        if self.storage not in {"cpu", "disk", "auto", "device"}:
            raise ValueError("storage must be 'cpu', 'disk', 'auto' or 'device'.")
        if self.ram_limit_bytes is not None and self.ram_limit_bytes <= 0:
            raise ValueError("ram_limit_bytes must be positive when provided.")


PASS1_LANES = 2   # chunks of pass 1 in flight at once (streams, record slots, memory pools)


class _ChunkFeeder:
    """Hands out (1, len, C) device views of the chunks this rank owns.

    A sequence that is resident in HBM is handed out as views of itself.  A host sequence is uploaded chunk by chunk
    on a copy stream, one chunk ahead of the compute stream, into two device buffers.  With ``targets`` (the static
    inputs of captured graphs, chunk i going to ``targets[i % len(targets)]``) every chunk, resident or not, is copied
    there on that copy stream, half the ring ahead: with four targets and two chunks in flight the copy of chunk i+2
    runs while chunks i and i+1 are being worked on."""

    def __init__(self, source: torch.Tensor, local_start: int, device: torch.device, chunk_len: int,
                 targets: Optional[List[torch.Tensor]] = None, dtype: Optional[torch.dtype] = None):
        dtype = dtype or source.dtype   # a disk-staged sequence is float32 and is converted while it is staged
        self.src = source
        self.off = local_start  # global index of source[:, 0]
        self.device = device
        self.on_device = source.is_cuda
        self.copying = targets is not None or not self.on_device
        if self.copying:
            self.copy_stream = torch.cuda.Stream(device=device)
            shape = (1, chunk_len, source.size(2))
            self.dev = targets if targets is not None else [torch.empty(shape, dtype=dtype, device=device) for _ in range(2)]
            self.nbuf = len(self.dev)
            self.ahead = max(1, self.nbuf // 2)
            self.pinned_source = self.on_device or (source.is_pinned() and source.dtype == dtype)  # uploads straight from the caller's buffer
            self.stage = [] if self.pinned_source else [torch.empty(shape, dtype=dtype, pin_memory=True)
                                                        for _ in range(self.nbuf)]
            self.ready = [torch.cuda.Event() for _ in range(self.nbuf)]
            self.consumed = [torch.cuda.Event() for _ in range(self.nbuf)]
            self.issued = 0   # chunks 0 .. issued-1 have their copy on the copy stream
            if self.on_device:  # the source must be complete before the copy stream reads it
                self.copy_stream.wait_stream(torch.cuda.current_stream())

    def _issue(self, slot: int, start: int, end: int) -> None:
        n = end - start
        if self.pinned_source:
            host = self.src[:, start - self.off:end - self.off]
        else:
            self.ready[slot].synchronize()  # the previous upload out of this pinned buffer has finished
            self.stage[slot][:, :n].copy_(self.src[:, start - self.off:end - self.off])
            host = self.stage[slot][:, :n]
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.consumed[slot])
            self.dev[slot][:, :n].copy_(host, non_blocking=True)
            self.ready[slot].record(self.copy_stream)

    def get(self, i: int, bounds: Sequence[Tuple[int, int]]) -> torch.Tensor:
        """Chunk i (``bounds[i]`` = its global start and end) on the device, ordered after its copy on the current
        stream; starts the copies of the chunks up to ``ahead`` behind it."""
        start, end = bounds[i]
        if not self.copying:
            return self.src[:, start - self.off:end - self.off]
        while self.issued < min(len(bounds), i + self.ahead + 1):
            j = self.issued
            self._issue(j % self.nbuf, bounds[j][0], bounds[j][1])
            self.issued += 1
        slot = i % self.nbuf
        torch.cuda.current_stream().wait_event(self.ready[slot])
        return self.dev[slot][:, :end - start]

    def done(self, i: int) -> None:
        if self.copying:
            self.consumed[i % self.nbuf].record(torch.cuda.current_stream())


class _Pass1Records:
    """Fixed-size promotion records of the chunks this rank owns, filled by ``aspa_chunk_select_slot``: the chunk's
    slot number lives in device memory, so the same launch - eager or a node of a captured graph - serves every chunk.
    The promotion only needs token importance and the token mask, which are final early in the layer call; it runs on
    its own stream beside the rest of that call (it occupies 8 SMs)."""

    def __init__(self, n_slots: int, budget: int, device: torch.device, top_p: float):
        self.n_slots, self.budget, self.top_p = n_slots, budget, top_p
        self.packed = dist_utils.PackedRecords(n_slots, budget, device)   # one buffer: one all-gather moves all three
        self.scores, self.idx, self.count = self.packed.scores, self.packed.idx, self.packed.count
        self.idx.fill_(-1)
        # two slot numbers: two chunks can be in flight at once, each on its own lane (stream + captured graph)
        self.slots = [torch.zeros((1,), dtype=torch.int32, device=device) for _ in range(PASS1_LANES)]
        self.slot = self.slots[0]
        self.offsets = torch.zeros((n_slots,), dtype=torch.int64, device=device)
        self._template = None
        self._offsets_template = torch.zeros((n_slots,), dtype=torch.int64, device=device)
        self._offsets_for = None
        self.stream = torch.cuda.Stream(device=device, priority=-2)

    def reset(self, first_chunk: int, chunk_len: int) -> None:
        """Empty records (scores 0, indices -1, counts 0) and the global offset of every slot: two copies from
        templates built once (this runs at the head of every call, with the GPU idle until the first chunk starts)."""
        if self._template is None:
            self._template = self.packed.buf.clone()
            idx_t, _, _ = self.packed.views(self._template)
            self._template.zero_()
            idx_t.fill_(-1)
        key = (first_chunk, chunk_len)
        if self._offsets_for != key:
            torch.arange(first_chunk, first_chunk + self.n_slots, out=self._offsets_template)
            self._offsets_template.mul_(chunk_len)
            self._offsets_for = key
        self.packed.buf.copy_(self._template)
        self.offsets.copy_(self._offsets_template)

    def use_lane(self, lane: int) -> None:
        self.slot = self.slots[lane]

    def hook(self, layer: AdaptiveSparseAttention) -> None:
        """Called by the layer right after its token keep: fork the promotion of this chunk."""
        main = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        self.stream.wait_event(ready)
        mask = layer._last_token_mask
        with torch.cuda.stream(main if ops.SERIAL_STREAMS else self.stream):
            ops.chunk_select_slot(layer._last_token_importance.view(-1),
                                  mask.view(torch.uint8).view(-1) if mask is not None else None, self.budget, self.top_p,
                                  self.slot, self.offsets, self.scores, self.idx, self.count)

    def join(self) -> None:
        torch.cuda.current_stream().wait_stream(self.stream)


class ChunkedShortlistRunner:
    def __init__(self, config: ChunkedShortlistConfig, *, logger: Optional[logging.Logger] = None,
                 process_group: Any = None, cache_layers: bool = False) -> None:
        """``cache_layers`` keeps the two layers between calls of ``run`` (the reference builds fresh ones
        every call): their ``state_dict`` arguments are then read on first use only, and prototype state
        carries over from call to call unless ``freeze_prototypes`` is set."""
        self.config = config
        self.config.validate()
        self.logger = logger or LOGGER
        self.group = process_group
        self._layer_cache: Optional[Dict[Tuple, AdaptiveSparseAttention]] = {} if cache_layers else None

    def close(self) -> None:
        """Drop the cached layers and captured graphs.  A sharded runner with ``whole_run_graph`` must be closed before
        its process group is destroyed: a captured graph that holds collectives keeps the communicator busy, and the
        communicator's teardown waits for it."""
        if self._layer_cache is not None:
            self._layer_cache.clear()
        self.__dict__.pop("_graph_tmp", None)
        torch.cuda.synchronize(torch.device(self.config.device))

    def _make_layer(self, seq_len: int, ratio: float, dtype: torch.dtype, state: Optional[Dict[str, torch.Tensor]],
                    frozen: bool) -> AdaptiveSparseAttention:
        cfg = self.config
        key = (seq_len, ratio, dtype, frozen)
        if self._layer_cache is not None and key in self._layer_cache:
            return self._layer_cache[key]
        mc = _build_model_config(seq_len, cfg.d_model, heads=cfg.heads, sparse_ratio=ratio,
                                 shortlist_alpha=cfg.shortlist_alpha, router_top_p=cfg.nucleus_top_p)
        if frozen:
            mc.attn_proto_decay = 1.0
        layer = AdaptiveSparseAttention(mc)
        if state is not None:
            layer.load_state_dict(state)
        layer = layer.to(device=cfg.device, dtype=dtype).eval()
        layer.use_sdpa = False
        layer.set_shortlist_alpha(float(cfg.shortlist_alpha))
        if self._layer_cache is not None:
            self._layer_cache[key] = layer
        return layer

    def _records(self, n_slots: int) -> _Pass1Records:
        cfg = self.config
        key = ("records", n_slots, cfg.per_chunk_budget, float(cfg.nucleus_top_p))
        cache = self._layer_cache if self._layer_cache is not None else self.__dict__.setdefault("_graph_tmp", {})
        if key not in cache:
            cache[key] = _Pass1Records(n_slots, cfg.per_chunk_budget, torch.device(cfg.device), float(cfg.nucleus_top_p))
        return cache[key]

    def _chunk_step(self, layer: AdaptiveSparseAttention, x: torch.Tensor, records: _Pass1Records) -> None:
        """Layer call (or scoring only) of one chunk with the promotion forked off inside it, joined at the end."""
        layer.after_token_keep = records.hook
        try:
            layer(x) if self.config.pass1_full_forward else self._score_only(layer, x)
        finally:
            layer.after_token_keep = None
        records.join()

    def _chunk_graph(self, layer: AdaptiveSparseAttention, dtype: torch.dtype, records: _Pass1Records,
                     resident: Optional[List[torch.Tensor]] = None):
        """(graphs, static inputs, lanes) for the full chunks of pass 1.  The layer call is launch-bound (about 45
        small launches around two GEMMs), so replaying a captured graph removes the host from the loop.  Capture needs
        a call that never waits for the host, which holds for the chunk layer (alpha = 1, no keep threshold).  The
        promotion of the chunk is part of the graph; it finds its record slot in device memory.

        A host sequence goes through a ring of four static inputs (chunk i: input and graph i % 4).  For a sequence
        that is resident in HBM, ``resident`` lists its chunks and every chunk gets a graph of its own that reads the
        chunk where it lies (static inputs: None): copying 128 MiB per chunk into a static input costs a sixth of the
        chunk's memory traffic, and at the lowest priority, beside two chunks in flight, the copy became the slowest
        stage.  Those graphs are valid for that address only; a sequence at another address is captured afresh."""
        cfg = self.config
        cache = self._layer_cache if self._layer_cache is not None else self.__dict__.setdefault("_graph_tmp", {})
        if resident is not None:
            key = ("graph_resident", cfg.chunk_len, dtype, cfg.pass1_full_forward, id(records))
            signature = tuple(int(t.data_ptr()) for t in resident)
            if key in cache and cache[key][3] == signature:
                return cache[key]
            cache.pop(key, None)
            statics = list(resident)
        else:
            key = ("graph", cfg.chunk_len, dtype, cfg.pass1_full_forward, id(records))
            signature = None
            if key in cache:
                return cache[key]
            statics = [torch.zeros(1, cfg.chunk_len, cfg.d_model, device=cfg.device, dtype=dtype) for _ in range(2 * PASS1_LANES)]
        # Two lanes, each a stream of priority -2 with its own record slot and memory for the intermediates: chunk i+1
        # starts on the other lane while chunk i is still running, so its GEMM (compute bound) runs beside the
        # attention and the row scatter of chunk i (memory and latency bound).  Graph k runs on lane k % PASS1_LANES; the graphs
        # of a lane never overlap and share the lane's memory.  With the ring the copy of a chunk runs two chunks ahead.
        # Priorities: the layer forks its key/value GEMM onto a stream one level below the caller's, and the copy of
        # the next chunk runs at priority 0; captured kernel nodes keep the priority of the stream they came from.
        # So the short selection kernels of the main line take SMs as GEMM blocks retire instead of queueing behind
        # all of them, and the GEMM in turn is not held up by the copy.
        lanes = [torch.cuda.Stream(device=cfg.device, priority=-2) for _ in range(PASS1_LANES)]
        graphs: List[Any] = [None] * len(statics)
        for k in range(len(statics)):
            lane = k % PASS1_LANES
            records.use_lane(lane)
            if k < PASS1_LANES:
                lanes[lane].wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(lanes[lane]):  # eager warm-up on a side stream, as graph capture requires
                    for _ in range(2):
                        self._chunk_step(layer, statics[k], records)
                torch.cuda.current_stream().wait_stream(lanes[lane])
                torch.cuda.synchronize(cfg.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=graphs[lane].pool() if k >= PASS1_LANES else None, stream=lanes[lane]):
                self._chunk_step(layer, statics[k], records)
            graphs[k] = g
        records.use_lane(0)
        cache[key] = (graphs, statics if resident is None else None, lanes, signature)
        return cache[key]

    def _final_replay(self, layer: AdaptiveSparseAttention, reduced: torch.Tensor) -> torch.Tensor:
        """Pass 2 from a captured graph (one per reduced length): about sixty launches whose host cost would otherwise
        exceed their device time.  The telemetry record of the call is re-armed after every replay."""
        key = ("final_graph", reduced.size(1), reduced.dtype)
        cache = self._layer_cache if self._layer_cache is not None else self.__dict__.setdefault("_graph_tmp", {})
        if key not in cache:
            static_in = torch.empty_like(reduced)
            static_in.copy_(reduced)
            side = torch.cuda.Stream(device=reduced.device, priority=-2)   # see _chunk_graph
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    layer(static_in)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize(reduced.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                static_out = layer(static_in)
            cache[key] = (g, static_in, static_out, layer.__dict__.get("_pending"))
        g, static_in, static_out, ctx = cache[key]
        static_in.copy_(reduced, non_blocking=True)
        g.replay()
        if ctx is not None:  # the replay refreshed the pinned record: decode it again on the next telemetry access
            layer.__dict__["_pending"] = dict(ctx)
            layer.__dict__["_head_stats_value"] = None
            layer.__dict__["_sparse_state_value"] = None
        return static_out.detach().clone()

    @staticmethod
    def _score_only(layer: AdaptiveSparseAttention, x: torch.Tensor) -> None:
        """Router + token keep + prototype EMA of one chunk, without the attention whose output pass 1 discards."""
        B, T, C = x.shape
        alpha = layer._compute_cvt_alpha(T)
        layer._current_alpha = alpha
        ratio = (1.0 - alpha) * float(layer.token_keep_ratio_base) + alpha * float(layer._linear_token_keep_ratio(T))
        ratio = float(max(0.0, min(1.0, ratio)))
        x2d = x.contiguous().view(B * T, C)
        proto_hat = ops.normalize_rows(layer.routing_prototypes)
        conf_eps = (layer.routing_confidence + 1e-6).to(torch.float32)
        gate, imp, sim, bs, _ = ops.router_fwd(
            x2d, layer.head_router.linear.weight.contiguous(), proto_hat, conf_eps, None, temp=layer.proto_temp,
            threshold=layer.proto_threshold, span=max(1e-6, 1.0 - layer.proto_threshold), blend=layer.proto_blend,
            usage_boost=0.0, want_stats=False)
        layer._last_token_importance = imp.view(B, T)
        guard = min(max(0, layer.token_keep_guard), T)
        min_keep = max(min(max(0, layer.token_keep_min), T), guard)
        from .aspa import _py_round_f32
        need = max(1, min(max(_py_round_f32(ratio * T), min_keep), T))
        if ratio >= 0.999 and layer.token_keep_threshold <= 0.0:
            mask = torch.ones((B, T), dtype=torch.uint8, device=x.device)
        else:
            mask, _ = ops.token_select(layer._last_token_importance, need, layer.token_keep_threshold, guard)
        layer._last_token_mask = mask.view(torch.bool)
        if layer.after_token_keep is not None:
            layer.after_token_keep(layer)
        if layer.proto_decay != 1.0:
            ops.proto_ema_update(x2d, gate, layer.proto_decay, layer.routing_prototypes, layer.routing_usage_ema,
                                 layer.routing_confidence)

    def run(self, sequence: Optional[torch.Tensor] = None, *, chunk_state: Optional[Dict[str, torch.Tensor]] = None,
            final_state: Optional[Dict[str, torch.Tensor]] = None, warmup_input: Optional[torch.Tensor] = None,
            sequence_is_local_shard: bool = False) -> ChunkedShortlistResult:
        """Run both passes (see ``_run``).  Without ``cache_layers`` the layers are built afresh on every call, so
        whatever was captured against them - graphs, record buffers - lives for this call only: a graph replayed
        after its layer is gone would read freed weights."""
        if self._layer_cache is not None:
            try:
                return self._run(sequence, chunk_state=chunk_state, final_state=final_state, warmup_input=warmup_input,
                                 sequence_is_local_shard=sequence_is_local_shard)
            finally:
                self._drop_disk_stage()
        self.__dict__["_graph_tmp"] = {}
        try:
            return self._run(sequence, chunk_state=chunk_state, final_state=final_state, warmup_input=warmup_input,
                             sequence_is_local_shard=sequence_is_local_shard)
        finally:
            if torch.device(self.config.device).type == "cuda":   # nothing of this call is still replaying
                torch.cuda.synchronize(torch.device(self.config.device))
            self.__dict__.pop("_graph_tmp", None)
            self._drop_disk_stage()

    # ------------------------------------------------------------------------------------------ host staging
    def _resolve_storage(self, required_bytes: int, on_device: bool):
        """Where the sequence lives while it is streamed: the reference's rules (cs.py:420-451) for host sequences -
        ``auto`` goes to disk when the sequence exceeds ``ram_limit_bytes`` (or the available RAM), ``cpu`` when it
        exceeds an explicit limit, ``disk`` always - plus ``device`` for a sequence that is (or is asked to be) resident
        in HBM.  Returns (mode, reason, limit in bytes)."""
        cfg = self.config
        available = _system_available_ram()
        limit = cfg.ram_limit_bytes
        host_limit = limit if limit is not None else available
        if cfg.storage == "device" or (on_device and cfg.storage != "disk"):
            return "device", None, host_limit
        mode, reason = cfg.storage, None
        if mode == "auto":
            if host_limit is not None and required_bytes > host_limit:
                mode, reason = "disk", f"required={required_bytes:,}B exceeds limit={host_limit:,}B; staging on disk"
            else:
                mode = "cpu"
                if limit is not None:
                    reason = f"limit={limit:,}B, required={required_bytes:,}B"
                elif available is not None:
                    reason = f"available≈{available:,}B, required={required_bytes:,}B"
        elif mode == "cpu" and limit is not None and required_bytes > limit:
            mode, reason = "disk", f"required={required_bytes:,}B exceeds ram_limit={limit:,}B; staging on disk"
        return mode, reason, host_limit

    def _stage_on_disk(self, source: Optional[torch.Tensor], n_tokens: int):
        """The sequence as a float32 memory-mapped file (cs.py:497-541): written in blocks of at most 64 MiB, seeded
        noise block by block when no sequence was given.  Returns (a CPU tensor over the mapping, bytes of one
        block); the file is removed when the call ends."""
        import tempfile
        import numpy as np
        cfg = self.config
        tmp_dir = Path(cfg.temp_dir) if cfg.temp_dir is not None else Path(tempfile.gettempdir())
        tmp_dir.mkdir(parents=True, exist_ok=True)
        handle = tempfile.NamedTemporaryFile(dir=tmp_dir, prefix="chunked_shortlist_", suffix=".mmap", delete=False)
        handle.close()
        path = Path(handle.name)
        array = np.memmap(path, dtype=np.float32, mode="w+", shape=(n_tokens, cfg.d_model))
        self.__dict__.setdefault("_disk_stage", []).append((path, array))
        rows_per_block = max(1, min(cfg.chunk_len, int((64 * 1024 * 1024) / max(cfg.d_model * 4, 1))))
        gen = None
        if source is None:
            gen = torch.Generator(device="cpu")
            if cfg.seed is not None:
                gen.manual_seed(int(cfg.seed))
        for start in range(0, n_tokens, rows_per_block):
            end = min(n_tokens, start + rows_per_block)
            if source is not None:
                block = source[0, start:end].to("cpu", dtype=torch.float32)
            else:
                block = torch.randn(end - start, cfg.d_model, generator=gen, device="cpu").to(torch.float32)
            array[start:end] = block.numpy()
        array.flush()
        return torch.from_numpy(array).unsqueeze(0), rows_per_block * cfg.d_model * 4

    def _drop_disk_stage(self) -> None:
        import contextlib
        import os
        for path, array in self.__dict__.pop("_disk_stage", []):
            with contextlib.suppress(Exception):
                array.flush()
            del array
            with contextlib.suppress(OSError):
                os.remove(path)

    def _run(self, sequence: Optional[torch.Tensor] = None, *, chunk_state: Optional[Dict[str, torch.Tensor]] = None,
             final_state: Optional[Dict[str, torch.Tensor]] = None, warmup_input: Optional[torch.Tensor] = None,
             sequence_is_local_shard: bool = False) -> ChunkedShortlistResult:
        """Run both passes.  ``sequence``: (1, T, C) on the host or the device; ``None`` generates seeded noise as
        the reference does.  ``chunk_state`` / ``final_state`` optionally supply the layers' ``state_dict`` (the
        reference draws fresh random weights inside ``run``; ranks of a sharded run must agree on them).  With
        ``sequence_is_local_shard`` the tensor holds only the chunks this rank owns."""
        cfg = self.config
        device = torch.device(cfg.device)
        if device.type != "cuda":
            raise RuntimeError("proteus_flux_attention_b200 has no CPU path: ChunkedShortlistConfig.device must be a CUDA device")
        world, rank = dist_utils.world_and_rank(self.group)
        if world > 1 and not cfg.freeze_prototypes:
            raise ValueError("sharding chunks over ranks needs freeze_prototypes=True (chunks must be independent)")
        n_chunks = math.ceil(cfg.seq_len / cfg.chunk_len)
        c_lo, c_hi = dist_utils.partition_chunks(n_chunks, world, rank)
        local_start = c_lo * cfg.chunk_len

        if sequence is not None:
            if sequence.dim() != 3:
                raise ValueError("sequence tensor must have shape (B, T, D)")
            if sequence.size(2) != cfg.d_model:
                raise ValueError(f"sequence hidden size {sequence.size(2)} does not match d_model={cfg.d_model}")
            if sequence.size(0) != 1:
                raise ValueError("Chunked Shortlist runner currently expects batch size of 1.")
            if not sequence_is_local_shard:
                if sequence.size(1) < cfg.seq_len:
                    raise ValueError(f"sequence length {sequence.size(1)} smaller than configured seq_len {cfg.seq_len}")
                sequence = sequence[:, :cfg.seq_len].detach()
                source, source_off = sequence, 0
            else:
                source, source_off = sequence.detach(), local_start
            base_dtype = sequence.dtype
        else:
            base_dtype = torch.get_default_dtype()
            source, source_off = None, 0
        self.__dict__["_base_dtype"] = base_dtype
        elem = torch.tensor([], dtype=base_dtype).element_size()
        host_bytes = int(cfg.seq_len * cfg.d_model * elem)
        storage_mode, storage_reason, host_limit = self._resolve_storage(host_bytes, source is not None and source.is_cuda)
        host_allocated = None
        if storage_mode == "disk":
            # float32 on disk, converted to the activation dtype chunk by chunk on the way to the device (cs.py:543-552)
            n_stage = source.size(1) if source is not None else cfg.seq_len
            source, host_allocated = self._stage_on_disk(source, n_stage)
            host_bytes = int(cfg.seq_len * cfg.d_model * 4)
        elif source is None:
            gen = torch.Generator(device="cpu")
            if cfg.seed is not None:
                gen.manual_seed(int(cfg.seed))
            source = torch.randn(1, cfg.seq_len, cfg.d_model, generator=gen, device="cpu").to(base_dtype)
        if storage_mode == "device" and not source.is_cuda:
            source = source.to(device)
        if storage_mode == "cpu":
            host_allocated = int(source.numel() * source.element_size())
        if storage_reason is not None:
            self.logger.info("Host staging: %s (%s)", storage_mode, storage_reason)

        chunk_model = self._make_layer(cfg.chunk_len, cfg.chunk_sparse_ratio, base_dtype, chunk_state, cfg.freeze_prototypes)
        if cfg.warmup:
            dummy = warmup_input.to(device=device, dtype=base_dtype) if warmup_input is not None else \
                torch.randn(1, cfg.chunk_len, cfg.d_model, device=device, dtype=base_dtype)
            chunk_model(dummy)
            torch.cuda.synchronize(device)

        n_local = c_hi - c_lo
        budget = cfg.per_chunk_budget
        cap = dist_utils.max_chunks_per_rank(n_chunks, world)   # slots per rank: the same on every rank (fixed-size exchange)
        records = self._records(max(cap, 1))
        rec_scores, rec_idx, rec_count = records.scores, records.idx, records.count
        bounds = [(c * cfg.chunk_len, min(cfg.seq_len, (c + 1) * cfg.chunk_len)) for c in range(c_lo, c_hi)]
        if (cfg.whole_run_graph and cfg.use_cuda_graph and cfg.freeze_prototypes and self._layer_cache is not None
                and source.is_cuda and source.is_contiguous() and not cfg.collect_summaries and not cfg.report_latency
                and n_local >= 1 and all(e - s == cfg.chunk_len for s, e in bounds)
                and n_chunks * budget <= ops.MERGE_POS_MAX and not ops.SERIAL_STREAMS):
            t0 = time.perf_counter()
            wr = self._whole_run(source=source, source_off=source_off, bounds=bounds, c_lo=c_lo, c_hi=c_hi,
                                 chunk_model=chunk_model, final_state=final_state, base_dtype=base_dtype, records=records,
                                 n_chunks=n_chunks, world=world, rank=rank, device=device)
            if wr is not None:
                total_s = time.perf_counter() - t0
                self.last_phase_ms = {"whole_run_graph": round(wr["device_ms"], 3), "host_wall": round(total_s * 1e3, 3)}
                metrics = ChunkedShortlistMetrics(
                    original_tokens=cfg.seq_len, retained_tokens=wr["k"], retention_ratio=float(wr["k"] / max(cfg.seq_len, 1)),
                    chunk_count=n_chunks, device=str(device), chunk_time_ms=None, final_time_ms=None,
                    total_time_ms=float(total_s * 1e3), peak_memory_mb=None, used_fallback=False, chunk_tokens_per_s=None,
                    final_tokens_per_s=None, total_tokens_per_s=float(cfg.seq_len / total_s) if total_s > 0 else None,
                    storage_mode=storage_mode, host_required_mb=host_bytes / BYTES_PER_MB, host_allocated_mb=None,
                    host_limit_mb=None, storage_reason=None, world_size=world)
                return ChunkedShortlistResult(keep_indices=wr["keep_idx_host"], keep_scores=wr["keep_sc_host"],
                                              reduced_sequence=wr["reduced"], metrics=metrics, chunks=[],
                                              final_output=wr["final_output"], final_stats=None,
                                              backend_info=wr["backend_info"])
        # Host-resident input: the rows of every promoted token are set aside while their chunk is on the device,
        # so that the reduced sequence is assembled from device memory instead of a second trip to the host.
        # Sharded runs do the same whatever the source: each rank then contributes exactly the rows it promoted.
        pool = None
        if (not source.is_cuda or world > 1) and n_chunks * budget <= ops.MERGE_POS_MAX:
            pool = torch.empty((max(cap, 1) * budget, cfg.d_model), dtype=base_dtype, device=device)

        ev_a = torch.cuda.Event(enable_timing=True)
        ev_b = torch.cuda.Event(enable_timing=True)
        ev_c = torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        ev_a.record()
        graph = None
        if cfg.use_cuda_graph:
            resident = None
            if source.is_cuda and source.is_contiguous():
                resident = [source[:, s - source_off:e - source_off] for s, e in bounds if e - s == cfg.chunk_len]
            graph = self._chunk_graph(chunk_model, base_dtype, records, resident)
        feeder = _ChunkFeeder(source, source_off, device, cfg.chunk_len, targets=graph[1] if graph is not None else None,
                              dtype=base_dtype)
        records.reset(c_lo, cfg.chunk_len)  # after a possible capture, whose warm-up calls wrote into slot 0
        main = torch.cuda.current_stream()
        lanes = graph[2] if graph is not None else [main]
        for lane in lanes:
            if lane is not main:
                lane.wait_stream(main)
        for i, (start, end) in enumerate(bounds):
            k = i % len(lanes)
            records.use_lane(k)
            with torch.cuda.stream(lanes[k]):
                xc = feeder.get(i, bounds)
                records.slot.fill_(i)
                if graph is not None and end - start == cfg.chunk_len:
                    graph[0][i % len(graph[0])].replay()   # xc is the static input of that graph
                else:
                    self._chunk_step(chunk_model, xc, records)
                if pool is not None:
                    ops.gather_rows(xc[0], (rec_idx[i] - start).clamp_(min=0), rec_count[i:i + 1], budget,
                                    out=pool[i * budget:(i + 1) * budget])
                feeder.done(i)
        records.use_lane(0)
        for lane in lanes:
            if lane is not main:
                main.wait_stream(lane)

        # exchange: every rank ends up with the records of all chunks, in chunk order
        ev_p1 = torch.cuda.Event(enable_timing=True)
        ev_x1 = torch.cuda.Event(enable_timing=True)
        ev_x2 = torch.cuda.Event(enable_timing=True)
        ev_p1.record()
        all_scores, all_idx, all_count = dist_utils.all_gather_packed_records(self.group, records.packed, n_chunks, world)
        ev_x1.record()
        all_pool = dist_utils.all_gather_pool(self.group, pool, world) if (pool is not None and world > 1) else pool
        ev_x2.record()
        keep_pos = None
        if pool is not None:
            keep_idx, keep_sc, keep_count, keep_pos = ops.merge_finalise(all_scores.view(-1), all_idx.view(-1), cfg.seq_len,
                                                                         cfg.buffer_tokens, want_pos=True)
        else:
            keep_idx, keep_sc, keep_count = ops.merge_finalise(all_scores.view(-1), all_idx.view(-1), cfg.seq_len,
                                                               cfg.buffer_tokens)
        ev_b.record()

        # the allocator's statistics cost the host 0.1-0.2 ms per call: kept for eager runs and on request
        track_peak = cfg.report_latency or not cfg.use_cuda_graph

        def second_half(k_host: int):
            """Gather the kept rows and run pass 2 for a kept count of ``k_host``."""
            kidx, ksc = keep_idx[:k_host], keep_sc[:k_host]
            if pool is not None:
                red = self._gather_pooled(all_pool, keep_pos[:k_host], k_host, budget, world, n_chunks)
            else:
                red = self._gather_reduced(source, source_off, kidx, k_host, device, world, rank, c_lo, c_hi)
            out = info = stats = None
            if cfg.run_final_pass:
                final_model = self._make_layer(k_host, cfg.final_sparse_ratio, base_dtype, final_state, cfg.freeze_prototypes)
                if track_peak:
                    torch.cuda.reset_peak_memory_stats(device)
                if cfg.use_cuda_graph:
                    out = self._final_replay(final_model, red)
                else:
                    out = final_model(red).detach()
                info = get_last_backend_info()
                stats = (final_model,)
            return kidx, ksc, red, out, info, stats

        # The kept count is a device value.  Waiting for it here leaves the GPU idle for a host round trip (about
        # 0.1 ms before pass 2 can even be enqueued).  With graphs on, pass 2 is enqueued for the count that holds
        # whenever the chunks promote at least `buffer_tokens` tokens in all, min(buffer, chunks * budget), while the
        # real count travels to a pinned word; it is checked once the stream has drained, and only a run that guessed
        # wrong (indices beyond the real count are -1 and gather zero rows) repeats the second half.  Every rank sees
        # the same records, so every rank takes the same branch.
        speculate = cfg.use_cuda_graph and (pool is not None or source.is_cuda)
        if speculate:
            k_guess = min(cfg.buffer_tokens, n_chunks * budget)
            count_pin = self.__dict__.get("_count_pin")
            if count_pin is None:
                count_pin = self.__dict__["_count_pin"] = torch.zeros(1, dtype=torch.int32, pin_memory=True)
            count_pin.copy_(keep_count, non_blocking=True)
            counted = torch.cuda.Event()
            counted.record()
            result = second_half(k_guess)
            counted.synchronize()
            k_host = int(count_pin.item())
        else:
            k_host = int(keep_count.item())
            k_guess = k_host
            result = None
        if k_host == 0:
            raise RuntimeError("Chunked pipeline selected zero tokens; adjust per_chunk_budget or sparse ratios.")
        if result is None or k_host != k_guess:
            result = second_half(k_host)
        keep_idx, keep_sc, reduced, final_output, backend_info, fm = result
        chunk_time_ms = None
        final_stats = None
        final_time_ms = peak_mb = None
        ev_c.record()
        # Everything the host reads back travels to pinned memory behind the last kernel, so that ONE wait for the
        # device ends the call: router status, kept indices and scores (the telemetry record of pass 2 is pinned already).
        status_pin = self.__dict__.get("_status_pin")
        if status_pin is None:
            status_pin = self.__dict__["_status_pin"] = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        status_pin.copy_(ops.router_status(device), non_blocking=True)
        keep_pin = self.__dict__.get("_keep_pin")
        if keep_pin is None or keep_pin[0].numel() < keep_idx.numel():
            keep_pin = self.__dict__["_keep_pin"] = (torch.empty(max(keep_idx.numel(), cfg.buffer_tokens), dtype=torch.int64, pin_memory=True),
                                                     torch.empty(max(keep_idx.numel(), cfg.buffer_tokens), dtype=torch.float32, pin_memory=True))
        keep_pin[0][: keep_idx.numel()].copy_(keep_idx, non_blocking=True)
        keep_pin[1][: keep_sc.numel()].copy_(keep_sc, non_blocking=True)
        torch.cuda.synchronize(device)
        if int(status_pin.item()) != 0:   # a bounded wait ran out in some chunk's router: nothing of this run is valid
            ops.check_router_status(device)
        t1 = time.perf_counter()
        keep_idx_host, keep_sc_host = keep_pin[0][: keep_idx.numel()].clone(), keep_pin[1][: keep_sc.numel()].clone()
        if fm is not None and cfg.collect_summaries:
            final_model = fm[0]
            final_stats = _sanitize_mapping(dict(final_model.last_head_stats or {}))
            st = {k: v for k, v in (final_model._last_sparse_state or {}).items() if not isinstance(v, torch.Tensor)}
            if st:
                final_stats["sparse_state"] = _sanitize_mapping(st)
        chunk_time_ms = float(ev_a.elapsed_time(ev_b))
        self.last_phase_ms = {"pass1": round(ev_a.elapsed_time(ev_p1), 3), "exchange_records": round(ev_p1.elapsed_time(ev_x1), 3),
                              "exchange_rows": round(ev_x1.elapsed_time(ev_x2), 3), "merge": round(ev_x2.elapsed_time(ev_b), 3),
                              "gather_pass2": round(ev_b.elapsed_time(ev_c), 3), "host_wall": round((t1 - t0) * 1e3, 3)}
        if cfg.run_final_pass:
            final_time_ms = float(ev_b.elapsed_time(ev_c))
            peak_mb = torch.cuda.max_memory_allocated(device) / BYTES_PER_MB if track_peak else None
        total_s = t1 - t0

        summaries: List[ChunkSummary] = []
        if cfg.collect_summaries:
            sc_h, ix_h, ct_h = all_scores.cpu(), all_idx.cpu(), all_count.cpu().tolist()
            for c in range(n_chunks):
                n = int(ct_h[c])
                if n == 0:
                    continue
                summaries.append(ChunkSummary(index=c, start=c * cfg.chunk_len, end=min(cfg.seq_len, (c + 1) * cfg.chunk_len),
                                              promoted=ix_h[c, :n].tolist(), scores=sc_h[c, :n].tolist()))
        metrics = ChunkedShortlistMetrics(
            original_tokens=cfg.seq_len, retained_tokens=k_host, retention_ratio=float(k_host / max(cfg.seq_len, 1)),
            chunk_count=len(summaries) if cfg.collect_summaries else n_chunks, device=str(device),
            chunk_time_ms=chunk_time_ms, final_time_ms=final_time_ms, total_time_ms=float(total_s * 1e3),
            peak_memory_mb=peak_mb, used_fallback=False,
            chunk_tokens_per_s=float(cfg.seq_len * 1e3 / chunk_time_ms) if chunk_time_ms and chunk_time_ms > 0 else None,
            final_tokens_per_s=float(k_host * 1e3 / final_time_ms) if final_time_ms and final_time_ms > 0 else None,
            total_tokens_per_s=float(cfg.seq_len / total_s) if total_s > 0 else None, storage_mode=storage_mode,
            host_required_mb=host_bytes / BYTES_PER_MB,
            host_allocated_mb=host_allocated / BYTES_PER_MB if host_allocated is not None else None,
            host_limit_mb=host_limit / BYTES_PER_MB if host_limit is not None else None, storage_reason=storage_reason,
            world_size=world)
        self.logger.info("Chunked Shortlist retained %s/%s tokens (%.3f) across %s chunks", metrics.retained_tokens,
                         metrics.original_tokens, metrics.retention_ratio, n_chunks)
        return ChunkedShortlistResult(keep_indices=keep_idx_host, keep_scores=keep_sc_host,
                                      reduced_sequence=reduced, metrics=metrics, chunks=summaries,
                                      final_output=final_output, final_stats=final_stats, backend_info=backend_info)

    def _whole_run(self, *, source: torch.Tensor, source_off: int, bounds, c_lo: int, c_hi: int,
                   chunk_model: AdaptiveSparseAttention, final_state, base_dtype: torch.dtype, records: _Pass1Records,
                   n_chunks: int, world: int, rank: int, device: torch.device):
        """The whole run as ONE captured CUDA graph, replayed: record reset, pass 1 of this rank's chunks on two lanes,
        both exchanges (NCCL collectives are captured like kernels), merge, row gather, pass 2 and the copies of
        everything the host reads into pinned memory.  Per run the host then launches one graph and waits once, where
        the chunk-by-chunk path enqueues a few dozen operations - about 0.4 ms of host time, which at eight ranks (two
        chunks each) is a fifth of the step.  Valid for one sequence address, one rank layout and frozen prototypes; the
        kept count is assumed to be ``min(buffer_tokens, chunks * budget)`` (true whenever the chunks promote that
        many tokens) and checked after the replay: on a mismatch ``None`` is returned and the caller runs the
        chunk-by-chunk path.  Output tensors live in the graph's memory and are cloned for the caller."""
        cfg = self.config
        budget = cfg.per_chunk_budget
        k_guess = min(cfg.buffer_tokens, n_chunks * budget)
        cache = self._layer_cache
        key = ("run_graph", int(source.data_ptr()), tuple(source.shape), base_dtype, world, rank, c_lo, c_hi, id(records))
        entry = cache.get(key)
        if entry is None:
            use_pool = world > 1
            pool = torch.empty((max(records.n_slots, 1) * budget, cfg.d_model), dtype=base_dtype, device=device) if use_pool else None
            final_model = self._make_layer(k_guess, cfg.final_sparse_ratio, base_dtype, final_state, cfg.freeze_prototypes) \
                if cfg.run_final_pass else None
            lanes = [torch.cuda.Stream(device=device, priority=-2) for _ in range(PASS1_LANES)]
            pins = {"count": torch.zeros(1, dtype=torch.int32, pin_memory=True),
                    "status": torch.zeros(1, dtype=torch.int32, pin_memory=True),
                    "idx": torch.empty(k_guess, dtype=torch.int64, pin_memory=True),
                    "sc": torch.empty(k_guess, dtype=torch.float32, pin_memory=True)}

            def enqueue():
                main = torch.cuda.current_stream()
                records.reset(c_lo, cfg.chunk_len)
                for lane in lanes:
                    lane.wait_stream(main)
                for i, (start, end) in enumerate(bounds):
                    k = i % len(lanes)
                    records.use_lane(k)
                    with torch.cuda.stream(lanes[k]):
                        xc = source[:, start - source_off:end - source_off]
                        records.slot.fill_(i)
                        self._chunk_step(chunk_model, xc, records)
                        if pool is not None:
                            ops.gather_rows(xc[0], (records.idx[i] - start).clamp_(min=0), records.count[i:i + 1], budget,
                                            out=pool[i * budget:(i + 1) * budget])
                records.use_lane(0)
                for lane in lanes:
                    main.wait_stream(lane)
                all_scores, all_idx, _ = dist_utils.all_gather_packed_records(self.group, records.packed, n_chunks, world)
                if pool is not None:
                    all_pool, rows_arrived = dist_utils.all_gather_pool(self.group, pool, world, deferred=True)
                    keep_idx, keep_sc, keep_count, keep_pos = ops.merge_finalise(all_scores.view(-1), all_idx.view(-1), cfg.seq_len,
                                                                                 cfg.buffer_tokens, want_pos=True)
                    rows_arrived()   # the merge ran beside the row exchange
                    red = self._gather_pooled(all_pool, keep_pos[:k_guess], k_guess, budget, world, n_chunks)
                else:
                    keep_idx, keep_sc, keep_count = ops.merge_finalise(all_scores.view(-1), all_idx.view(-1), cfg.seq_len,
                                                                       cfg.buffer_tokens)
                    red = self._gather_reduced(source, source_off, keep_idx[:k_guess], k_guess, device, world, rank, c_lo, c_hi)
                out = final_model(red).detach() if final_model is not None else None
                pins["count"].copy_(keep_count, non_blocking=True)
                pins["status"].copy_(ops.router_status(device), non_blocking=True)
                pins["idx"].copy_(keep_idx[:k_guess], non_blocking=True)
                pins["sc"].copy_(keep_sc[:k_guess], non_blocking=True)
                return keep_idx[:k_guess], keep_sc[:k_guess], red, out

            side = torch.cuda.Stream(device=device, priority=-2)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):   # eager warm-up on the capture stream: communicators, workspaces, caches
                for _ in range(2):
                    enqueue()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize(device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
                outs = enqueue()
            ctx = [(m, m.__dict__.get("_pending")) for m in (chunk_model, final_model) if m is not None]
            info = get_last_backend_info() if final_model is not None else None
            if world > 1 and not self.__dict__.get("_close_at_exit"):
                import atexit
                import weakref
                ref = weakref.ref(self)
                atexit.register(lambda: ref() is not None and ref().close())   # best effort for callers that never close
                self.__dict__["_close_at_exit"] = True
            # one graph per sequence address: keep the two most recent (each holds its intermediates in a memory pool)
            stale = [k for k in cache if isinstance(k, tuple) and k and k[0] == "run_graph"]
            for k in stale[:-1]:
                del cache[k]
            # everything the captured kernels address by raw pointer stays alive with the graph: the pool of promoted
            # rows, the pinned read-back buffers, both layers, the lanes (the sequence itself belongs to the caller)
            entry = cache[key] = {"graph": g, "outs": outs, "pins": pins, "final_model": final_model, "ctx": ctx, "info": info,
                                  "pool": pool, "lanes": lanes, "side": side, "chunk_model": chunk_model,
                                  "ev": (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))}
        ev0, ev1 = entry["ev"]
        ev0.record()
        entry["graph"].replay()
        ev1.record()
        # the caller's copies of the two large outputs are enqueued behind the graph, before the one wait of the run
        keep_idx, keep_sc, red, out = entry["outs"]
        red_copy = red.clone()
        out_copy = out.clone() if out is not None else None
        torch.cuda.synchronize(device)
        for m, pending in entry["ctx"]:   # the replay refreshed the pinned telemetry records: decode on next access
            if pending is not None:
                m.__dict__["_pending"] = dict(pending)
                m.__dict__["_head_stats_value"] = None
                m.__dict__["_sparse_state_value"] = None
        pins = entry["pins"]
        if int(pins["status"].item()) != 0:
            ops.check_router_status(device)
        if int(pins["count"].item()) != k_guess:
            return None
        return {"k": k_guess, "keep_idx_host": pins["idx"].clone(), "keep_sc_host": pins["sc"].clone(), "reduced": red_copy,
                "final_output": out_copy, "backend_info": entry["info"],
                "final_model": entry["final_model"], "device_ms": float(ev0.elapsed_time(ev1))}

    def _gather_pooled(self, pool: torch.Tensor, keep_pos: torch.Tensor, k: int, budget: int, world: int,
                       n_chunks: int) -> torch.Tensor:
        """(1, k, C) rows of the kept tokens from the pool of promoted rows (all ranks' pools after the all-gather).
        ``keep_pos`` holds, for every kept index, its position in the chunk-major list of all promotions
        (chunk * budget + rank within the chunk); the gathered pool is rank-major, which is the same order whenever
        every rank owns the same number of chunks."""
        if world > 1:
            off = dist_utils.pool_row_of_position(n_chunks, world, budget, pool.device)
            if off is not None:
                chunk = torch.div(keep_pos.clamp(min=0), budget, rounding_mode="floor")
                keep_pos = torch.where(keep_pos >= 0, keep_pos + off[chunk], keep_pos)
        return ops.gather_rows(pool, keep_pos, None, k).unsqueeze(0)

    def _activation_dtype(self, source: torch.Tensor) -> torch.dtype:
        """dtype of the rows handed to the layers: the source's own, except for a disk-staged (float32) sequence."""
        return self.__dict__.get("_base_dtype", source.dtype)

    def _gather_reduced(self, source: torch.Tensor, source_off: int, keep_idx: torch.Tensor, k: int,
                        device: torch.device, world: int, rank: int, c_lo: int, c_hi: int) -> torch.Tensor:
        """(1, k, C) rows of the kept tokens, in ascending index order (reference :688-689)."""
        cfg = self.config
        full_local = source_off == 0 and source.size(1) >= cfg.seq_len
        if full_local:
            if source.is_cuda:
                return ops.gather_rows(source[0], keep_idx, None, k).unsqueeze(0)
            return source[:, keep_idx.cpu()].to(self._activation_dtype(source)).to(device, non_blocking=True)
        # sharded input: every rank fills the kept rows that fall inside its own chunks and leaves zeros elsewhere;
        # the sum over ranks is the full reduced sequence
        lo, hi = c_lo * cfg.chunk_len, min(cfg.seq_len, c_hi * cfg.chunk_len)
        local_idx = torch.where((keep_idx >= lo) & (keep_idx < hi), keep_idx - source_off, torch.full_like(keep_idx, -1))
        if source.is_cuda:
            rows = ops.gather_rows(source[0], local_idx, None, k)
        else:
            li = local_idx.cpu()
            rows = torch.zeros((k, cfg.d_model), dtype=self._activation_dtype(source))
            rows[li >= 0] = source[0, li[li >= 0]].to(rows.dtype)
            rows = rows.to(device)
        return dist_utils.sum_disjoint_rows(self.group, rows, world).unsqueeze(0)


__all__ = ["ChunkedShortlistConfig", "ChunkedShortlistMetrics", "ChunkedShortlistResult", "ChunkedShortlistRunner",
           "ChunkSummary", "MAX_SHORTLIST_CHUNK_TOKENS"]
