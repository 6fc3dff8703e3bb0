"""Thin tensor-level wrappers over the C ABI: allocate outputs with torch, pass raw
pointers, raise on a non-zero status.  Everything here runs on the current CUDA
stream and never synchronises."""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple

import torch

from . import _native as N

# ---- optional instrumentation (used by bench.py): launch counter and per-op CUDA-event timing ----------
LAUNCHES = 0                      # kernels of libaspa_b200.so launched through this module
_TIMING: Optional[dict] = None    # name -> list of (start_event, end_event, algorithmic_bytes)
# ASPA_NVTX=1: every op of this module is wrapped in an NVTX range named after it (off by default: two host calls per op)
NVTX = os.environ.get("ASPA_NVTX", "0") not in ("", "0")


def start_timing() -> None:
    global _TIMING
    _TIMING = {}


def stop_timing() -> dict:
    """Returns name -> (launches, total_ms, algorithmic_bytes); synchronises the device."""
    global _TIMING
    rec, _TIMING = _TIMING or {}, None
    torch.cuda.synchronize()
    return {k: (len(v), sum(a.elapsed_time(b) for a, b, _ in v), sum(n for _, _, n in v)) for k, v in rec.items()}


class _timed:
    """Counts launches; when timing is on, brackets the op with CUDA events on the current stream."""

    def __init__(self, name: str, launches: int, nbytes: int = 0):
        self.name, self.launches, self.nbytes = name, launches, nbytes

    def __enter__(self):
        global LAUNCHES
        LAUNCHES += self.launches
        if NVTX:
            torch.cuda.nvtx.range_push("aspa:" + self.name)
        if _TIMING is not None:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if NVTX:
            torch.cuda.nvtx.range_pop()
        if _TIMING is not None and exc[0] is None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            _TIMING.setdefault(self.name, []).append((self.e0, e1, self.nbytes))
        return False


def _nb(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def _empty(shape, dtype, device):
    return torch.empty(shape, dtype=dtype, device=device)


def normalize_rows(p: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    p = p.to(torch.float32).contiguous()
    out = torch.empty_like(p)
    with _timed('normalize_rows', 1, 0):
        N.check(N.lib().aspa_normalize_rows(N.ptr(p), p.size(0), p.size(1), eps, N.ptr(out), N.stream()), "normalize_rows")
    return out


def reduce_partials(partials: torch.Tensor, n_series: int) -> torch.Tensor:
    n_blocks = partials.numel() // n_series
    out = _empty((n_series,), torch.float32, partials.device)
    with _timed('reduce_partials', 1, 0):
        N.check(N.lib().aspa_reduce_partials(N.ptr(partials), n_series, n_blocks, N.ptr(out), N.stream()), "reduce_partials")
    return out


SERIAL_STREAMS = False           # True: nothing is forked onto side streams (per-kernel timing passes need one serial stream)
USE_ANCHOR_TILES = True          # strided anchor keys of a plan go through the tile kernel when groups are large enough
USE_TC_ROUTER = True             # bf16 activations take the tcgen05 router when the shape allows
_ROUTER_STATUS: dict = {}        # device -> int32[1], raised by the tensor-core router if a bounded wait ran out


def router_status(device) -> torch.Tensor:
    key = str(device)
    if key not in _ROUTER_STATUS:
        _ROUTER_STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _ROUTER_STATUS[key]


def check_router_status(device) -> None:
    """Raise ``DeviceWaitTimeout`` if a bounded wait of the tensor-core router ran out since the last check, and
    clear the word so that later, healthy calls are not blamed for it.  Waits for the current stream: call it where
    the host synchronises anyway."""
    key = str(device)
    if key in _ROUTER_STATUS:
        N.check(N.lib().aspa_read_status(N.ptr(_ROUTER_STATUS[key]), 1, N.stream()), "tensor-core router")


def router_fwd(x2d: torch.Tensor, w_router: torch.Tensor, proto_hat: Optional[torch.Tensor],
               conf_eps: Optional[torch.Tensor], usage_bias: Optional[torch.Tensor], *, temp: float,
               threshold: float, span: float, blend: float, usage_boost: float, want_stats: bool = True,
               raw_stats: bool = False):
    """x2d (n, C) fp32/bf16 -> gate (n, G) fp32, importance (n), sim (n)|None, blend (n)|None, stats (3,)|None.
    With ``raw_stats`` the last item is the (3 * blocks) tensor of per-block partial sums instead of their sums."""
    n, Cdim = x2d.shape
    G = w_router.size(0)
    dev = x2d.device
    gate = _empty((n, G), torch.float32, dev)
    imp = _empty((n,), torch.float32, dev)
    has_proto = proto_hat is not None
    sim = _empty((n,), torch.float32, dev) if has_proto else None
    bs = _empty((n,), torch.float32, dev) if has_proto else None
    tc_bytes = 0
    if USE_TC_ROUTER and x2d.dtype == torch.bfloat16 and n >= 128 and x2d.data_ptr() % 16 == 0:
        tc_bytes = int(N.lib().aspa_router_tc_scratch_bytes(Cdim, G, int(has_proto)))
    ntile = (n + 31) // 32 if tc_bytes > 0 else (n + 63) // 64  # statistics partials: per 32 / per 64 tokens
    partials = _empty((3 * ntile,), torch.float32, dev) if (want_stats and has_proto) else None
    if tc_bytes > 0:
        scratch = _empty((tc_bytes,), torch.uint8, dev)
        with _timed('router_tc', 2, _nb(x2d, w_router, proto_hat, gate, imp, sim, bs)):
            N.check(N.lib().aspa_router_fwd_tc(
                N.ptr(x2d), n, Cdim, N.ptr(w_router), G, N.ptr(proto_hat), N.ptr(conf_eps), N.ptr(usage_bias), temp,
                threshold, span, blend, usage_boost, N.ptr(gate), N.ptr(imp), N.ptr(sim), N.ptr(bs), N.ptr(partials),
                N.ptr(scratch), N.ptr(router_status(dev)), N.stream()), "router_fwd_tc")
        stats = (partials if raw_stats else reduce_partials(partials, 3)) if partials is not None else None
        return gate, imp, sim, bs, stats
    with _timed('router', 1, _nb(x2d, w_router, proto_hat, gate, imp, sim, bs)):
        N.check(N.lib().aspa_router_fwd(
            N.ptr(x2d), N.dtype_code(x2d.dtype), n, Cdim, N.ptr(w_router), G, N.ptr(proto_hat), N.ptr(conf_eps),
            N.ptr(usage_bias), temp, threshold, span, blend, usage_boost, N.ptr(gate), N.ptr(imp), N.ptr(sim), N.ptr(bs),
            N.ptr(partials), N.stream()), "router_fwd")
    stats = (partials if raw_stats else reduce_partials(partials, 3)) if partials is not None else None
    return gate, imp, sim, bs, stats


def token_select(importance: torch.Tensor, need: int, threshold: float, guard: int):
    B, T = importance.shape
    mask = _empty((B, T), torch.uint8, importance.device)
    kept = _empty((B,), torch.int32, importance.device)
    with _timed('token_select', 1, _nb(importance, mask)):
        N.check(N.lib().aspa_token_select(N.ptr(importance), B, T, int(need), float(threshold), int(guard), N.ptr(mask),
                                          N.ptr(kept), N.stream()), "token_select")
    return mask, kept


def head_budget(gate: torch.Tensor, g2h: torch.Tensor, H: int, *, top_p: float, dense_k: int, h_min: int,
                linear_head_k: int, alpha: float) -> torch.Tensor:
    n, G = gate.shape
    scratch = _empty((H * ((n + 1023) // 1024),), torch.float32, gate.device)
    k_out = _empty((2,), torch.int32, gate.device)
    with _timed('head_budget', 2, _nb(gate)):
        N.check(N.lib().aspa_head_budget(N.ptr(gate), n, G, N.ptr(g2h), H, float(top_p), int(dense_k), int(h_min),
                                         int(linear_head_k), float(alpha), N.ptr(scratch), N.ptr(k_out), N.stream()),
                "head_budget")
    return k_out


def head_select(gate: torch.Tensor, g2h: torch.Tensor, H: int, *, k_host: int, k_dev: Optional[torch.Tensor],
                kmax: int, token_mask: Optional[torch.Tensor], want_stats: bool = True):
    n, G = gate.shape
    dev = gate.device
    bits = _empty((n,), torch.int64, dev)  # uint64 bit masks stored in an int64 tensor
    top_idx = _empty((n, kmax), torch.int32, dev)
    top_score = _empty((n, kmax), torch.float32, dev)
    nblk = (n + 255) // 256
    partials = _empty((2 * nblk,), torch.float32, dev) if want_stats else None
    with _timed('head_select', 1, _nb(gate, bits, top_idx, top_score)):
        N.check(N.lib().aspa_head_select(N.ptr(gate), n, G, N.ptr(g2h), H, int(k_host), N.ptr(k_dev), int(kmax),
                                         N.ptr(token_mask), N.ptr(bits), N.ptr(top_idx), N.ptr(top_score),
                                         N.ptr(partials), N.stream()), "head_select")
    stats = reduce_partials(partials, 2) if partials is not None else None
    return bits, top_idx, top_score, stats


def pack_rows(head_bits: torch.Tensor, B: int, T: int, H: int, capacity: int):
    dev = head_bits.device
    scratch = _empty((int(N.lib().aspa_pack_rows_scratch(B, H, T)),), torch.int32, dev)
    offs = _empty((B * H + 1,), torch.int32, dev)
    tok = _empty((max(1, capacity),), torch.int32, dev)
    with _timed('pack_rows', 3, 2 * _nb(head_bits)):
        N.check(N.lib().aspa_pack_rows(N.ptr(head_bits), B, T, H, N.ptr(scratch), N.ptr(offs), N.ptr(tok), capacity,
                                       N.stream()), "pack_rows")
    return offs, tok


def pack_mask(mask_u8: torch.Tensor):
    heads, T = mask_u8.shape
    dev = mask_u8.device
    scratch = _empty((heads * ((T + 255) // 256) + 1,), torch.int32, dev)
    offs = _empty((heads + 1,), torch.int32, dev)
    tok = _empty((heads * T,), torch.int32, dev)
    with _timed('pack_mask', 3, 2 * _nb(mask_u8)):
        N.check(N.lib().aspa_pack_mask(N.ptr(mask_u8), heads, T, N.ptr(scratch), N.ptr(offs), N.ptr(tok), heads * T,
                                       N.stream()), "pack_mask")
    return offs, tok


def rope_table(inv_freq: torch.Tensor, T: int, D: int, dtype: torch.dtype):
    dev = inv_freq.device
    cos = _empty((T, D // 2), torch.float32, dev)
    sin = _empty((T, D // 2), torch.float32, dev)
    with _timed('rope_table', 1, _nb(cos, sin)):
        N.check(N.lib().aspa_rope_table(N.ptr(inv_freq), T, D, N.dtype_code(dtype), N.ptr(cos), N.ptr(sin), N.stream()),
                "rope_table")
    return cos, sin


def rope_relayout(qkv: torch.Tensor, H: int, D: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                  want_amax: bool = False, q_keep: Optional[torch.Tensor] = None, q_fraction: float = 1.0):
    B, T, _ = qkv.shape
    dev = qkv.device
    q = _empty((B * H, T, D), qkv.dtype, dev)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    amax = torch.zeros((3, B * H), dtype=torch.float32, device=dev) if want_amax else None
    frac = (2.0 + (q_fraction if q_keep is not None else 1.0)) / 3.0  # share of the buffers that is actually moved
    with _timed('rope_relayout', 1, int(frac * _nb(qkv, q, k, v))):
        N.check(N.lib().aspa_rope_relayout(N.ptr(qkv), N.dtype_code(qkv.dtype), B, T, H, D, N.ptr(cos), N.ptr(sin),
                                           N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(amax), N.ptr(q_keep), N.stream()), "rope_relayout")
    return q, k, v, amax


def head_amax(x: torch.Tensor) -> torch.Tensor:
    heads = x.size(0)
    amax = _empty((heads,), torch.float32, x.device)
    with _timed('head_amax', 1, _nb(x)):
        N.check(N.lib().aspa_head_amax(N.ptr(x), N.dtype_code(x.dtype), heads, x.numel() // heads, N.ptr(amax),
                                       N.stream()), "head_amax")
    return amax


def quantize_int8(x: torch.Tensor, amax: torch.Tensor):
    heads = x.size(0)
    out = _empty(x.shape, torch.int8, x.device)
    scales = _empty((heads,), torch.float32, x.device)
    with _timed('quantize_int8', 1, _nb(x, out)):
        N.check(N.lib().aspa_quantize_int8(N.ptr(x), N.dtype_code(x.dtype), heads, x.numel() // heads, N.ptr(amax),
                                           N.ptr(out), N.ptr(scales), N.stream()), "quantize_int8")
    return out, scales


def head_abs_quantile(x: torch.Tensor, q: float, amax: torch.Tensor) -> torch.Tensor:
    """(heads,) fp32: torch.quantile(|x_h|, q) per head (linear interpolation), the head's maximum where that is zero."""
    heads = x.size(0)
    base = _empty((heads,), torch.float32, x.device)
    scratch = _empty((int(N.lib().aspa_head_abs_quantile_scratch(heads)),), torch.uint8, x.device)
    with _timed('head_abs_quantile', 10, 4 * _nb(x)):
        N.check(N.lib().aspa_head_abs_quantile(N.ptr(x), N.dtype_code(x.dtype), heads, x.numel() // heads, float(q),
                                               N.ptr(amax), N.ptr(scratch), N.ptr(base), N.stream()), "head_abs_quantile")
    return base


PROTO_BLOCK = 128


def proto_plan(scores: torch.Tensor, cap: int):
    """scores (B, T) fp32 -> lists (B, nblk, cap+128) int32, limits (B, T) int32."""
    B, T = scores.shape
    dev = scores.device
    nblk = (T + PROTO_BLOCK - 1) // PROTO_BLOCK
    lists = _empty((B, nblk, cap + PROTO_BLOCK), torch.int32, dev)
    limits = _empty((B, T), torch.int32, dev)
    scratch = _empty((max(16, int(N.lib().aspa_proto_plan_scratch(B, T, cap))),), torch.uint8, dev)
    with _timed('proto_plan', 1, _nb(scores, lists, limits)):
        N.check(N.lib().aspa_proto_plan(N.ptr(scores), B, T, int(cap), N.ptr(scratch), N.ptr(lists), N.ptr(limits),
                                        N.stream()), "proto_plan")
    return lists, limits


def make_plan(window: int, anchor_slots: int, anchor_stride: int, proto_cap: int = 0,
              lists: Optional[torch.Tensor] = None, limits: Optional[torch.Tensor] = None) -> N.ShortlistPlan:
    p = N.ShortlistPlan()
    p.window, p.anchor_slots, p.anchor_stride = int(window), int(anchor_slots), int(anchor_stride)
    p.proto_cap = int(proto_cap) if lists is not None else 0
    p.proto_block = PROTO_BLOCK
    p.proto_list_stride = int(proto_cap) + PROTO_BLOCK
    p.proto_lists = lists.data_ptr() if lists is not None else None
    p.proto_limit = limits.data_ptr() if limits is not None else None
    return p


def build_candidates(rows: torch.Tensor, row_batch: Optional[torch.Tensor], seq_len: int, L: int, *,
                     linear_window: int, anchor_stride: int, use_local: bool, use_anchors: bool,
                     proto_scores: Optional[torch.Tensor], local_cap: Optional[int], anchor_cap: Optional[int],
                     proto_cap: Optional[int]):
    n = rows.numel()
    dev = rows.device
    cand = _empty((n, L), torch.int64, dev)
    lens = _empty((n,), torch.int64, dev)

    def cap(v):
        return -1 if v is None else max(0, int(v))

    with _timed('build_candidates', 1, _nb(cand, lens)):
        N.check(N.lib().aspa_build_candidates(
            N.ptr(rows), N.ptr(row_batch), n, int(seq_len), int(L), int(linear_window), int(anchor_stride),
            int(bool(use_local)), int(bool(use_anchors)), N.ptr(proto_scores), cap(local_cap), cap(anchor_cap),
            cap(proto_cap), N.ptr(cand), N.ptr(lens), N.stream()), "build_candidates")
    return cand, lens


def regroup_rows(plan: N.ShortlistPlan, dtype: torch.dtype, heads: int, T: int, D: int, row_offsets: torch.Tensor,
                 token_idx: torch.Tensor, total_rows: int):
    """The regrouping of the anchor tile pass of a planned attention call, ahead of the call (it needs the packed rows
    and the plan, not q, k, v).  Returns (scratch, prepared) for ``gather_attn(regroup=...)``, or None when the plan
    has no anchors."""
    if not (plan.anchor_slots > 0 and plan.anchor_stride > 0 and USE_ANCHOR_TILES):
        return None
    rb = int(N.lib().aspa_attn_regroup_bytes(int(total_rows), heads, int(plan.anchor_stride)))
    if rb <= 0:
        return None
    ws = _empty((rb,), torch.uint8, row_offsets.device)
    prepared = C.c_int32(0)
    with _timed('regroup_rows', 3, 0):
        N.check(N.lib().aspa_attn_regroup_rows(N.dtype_code(dtype), heads, int(T), int(D), N.ptr(row_offsets),
                                               N.ptr(token_idx), int(total_rows), C.byref(plan), N.ptr(ws),
                                               C.byref(prepared), N.stream()), "attn_regroup_rows")
    return ws, int(prepared.value)


def gather_attn(q, k, v, *, scales: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]], H: int,
                row_offsets: torch.Tensor, token_idx: torch.Tensor, max_rows: int, total_rows: int,
                cand: Optional[torch.Tensor] = None, cand_len: Optional[torch.Tensor] = None,
                plan: Optional[N.ShortlistPlan] = None, add_mask: Optional[torch.Tensor] = None,
                out: torch.Tensor, out_layout: int, out_row_map: Optional[torch.Tensor] = None,
                kv_layout: Optional[N.KVLayout] = None, regroup=None):
    """Launch the attention kernels; `out` must be zero-filled by the caller.  ``out_row_map`` (B*T int32)
    redirects token-major output rows to compact slots.  With ``kv_layout`` k and v are any tensors holding the
    rows at those element strides (q stays (heads, T, D))."""
    heads, T, D = q.shape
    ws = None
    nbytes = int(N.lib().aspa_attn_workspace_bytes(int(total_rows), D))
    if plan is not None and cand is None and nbytes > 0:
        ws = _empty((nbytes,), torch.uint8, q.device)
    prepared = 0
    if regroup is not None:
        regroup, prepared = regroup
    elif ws is not None and plan.anchor_slots > 0 and plan.anchor_stride > 0 and USE_ANCHOR_TILES:
        rb = int(N.lib().aspa_attn_regroup_bytes(int(total_rows), heads, int(plan.anchor_stride)))
        if rb > 0:
            regroup = _empty((rb,), torch.uint8, q.device)
    qs, ks, vs = scales if scales is not None else (None, None, None)
    L = cand.size(1) if cand is not None else 0
    e = q.element_size()
    two_pass = plan is not None and cand is None and (plan.anchor_slots > 0 or plan.proto_cap > 0) and D == 64 \
        and q.dtype in (torch.bfloat16, torch.int8)
    # algorithmic bytes: each active row's q once, every key and value row once, each active output row once
    nbytes = int(total_rows) * D * (e + out.element_size()) + 2 * heads * T * D * e
    with _timed("attention", 2 if two_pass else 1, nbytes):
        N.check(N.lib().aspa_gather_attn_fwd_prepared(
            N.ptr(q), N.ptr(k), N.ptr(v), N.dtype_code(q.dtype), N.ptr(qs), N.ptr(ks), N.ptr(vs), heads, T, D, int(H),
            N.ptr(row_offsets), N.ptr(token_idx), int(max_rows), int(total_rows), N.ptr(cand), N.ptr(cand_len), int(L),
            C.byref(plan) if plan is not None else None, N.ptr(add_mask), N.ptr(out), N.dtype_code(out.dtype),
            int(out_layout), N.ptr(out_row_map), C.byref(kv_layout) if kv_layout is not None else None, N.ptr(ws),
            N.ptr(regroup), int(prepared), N.stream()), "gather_attn_fwd")
    return out


def proto_ema_update(x2d: torch.Tensor, gate: torch.Tensor, decay: float, protos: torch.Tensor,
                     usage: torch.Tensor, conf: torch.Tensor) -> torch.Tensor:
    n, Cdim = x2d.shape
    G = gate.size(1)
    nbytes = int(N.lib().aspa_proto_ema_scratch(n, Cdim, G))
    scratch = _empty((nbytes,), torch.uint8, x2d.device)
    updated = _empty((1,), torch.int32, x2d.device)
    with _timed('proto_ema', 2, _nb(x2d, gate, protos)):
        N.check(N.lib().aspa_proto_ema_update(N.ptr(x2d), N.dtype_code(x2d.dtype), n, Cdim, N.ptr(gate), G, float(decay),
                                              N.ptr(protos), N.ptr(usage), N.ptr(conf), N.ptr(scratch), N.ptr(updated),
                                              N.stream()), "proto_ema_update")
    return updated


def chunk_select(importance: torch.Tensor, token_mask: Optional[torch.Tensor], budget: int, top_p: float, offset: int,
                 out_scores: torch.Tensor, out_idx: torch.Tensor, out_count: torch.Tensor) -> None:
    T = importance.numel()
    with _timed('chunk_select', 1, _nb(importance)):
        N.check(N.lib().aspa_chunk_select(N.ptr(importance), N.ptr(token_mask), T, int(budget), float(top_p), int(offset),
                                          N.ptr(out_scores), N.ptr(out_idx), N.ptr(out_count), N.stream()), "chunk_select")


MERGE_POS_MAX = 65536  # ASPA_MERGE_POS_MAX of the C header


def merge_finalise(scores: torch.Tensor, indices: torch.Tensor, seq_len: int, max_tokens: int, want_pos: bool = False):
    """Returns (keep_idx, keep_scores, count) and, with ``want_pos``, the candidate position of every kept index."""
    dev = scores.device
    table = _empty((int(N.lib().aspa_merge_finalise_scratch(int(seq_len))),), torch.uint8, dev)
    # entries beyond the kept count stay -1 (a gather by them reads nothing)
    keep_idx = torch.full((max_tokens,), -1, dtype=torch.int64, device=dev)
    keep_sc = _empty((max_tokens,), torch.float32, dev)
    keep_pos = torch.full((max_tokens,), -1, dtype=torch.int64, device=dev) if want_pos else None
    count = _empty((1,), torch.int32, dev)
    with _timed('merge_finalise', 2, _nb(scores, indices)):
        N.check(N.lib().aspa_merge_finalise(N.ptr(scores), N.ptr(indices), scores.numel(), int(seq_len), int(max_tokens),
                                            N.ptr(table), N.ptr(keep_idx), N.ptr(keep_sc), N.ptr(keep_pos), N.ptr(count),
                                            N.stream()), "merge_finalise")
    if want_pos:
        return keep_idx, keep_sc, count, keep_pos
    return keep_idx, keep_sc, count


def gather_rows(src2d: torch.Tensor, idx: torch.Tensor, count_dev: Optional[torch.Tensor], max_rows: int,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dst[i] = src2d[idx[i]] for i < count (all max_rows when count_dev is None); other rows are left as they are."""
    row_bytes = src2d.size(1) * src2d.element_size()
    dst = out if out is not None else _empty((max_rows, src2d.size(1)), src2d.dtype, src2d.device)
    with _timed('gather_rows', 1, 2 * _nb(dst)):
        N.check(N.lib().aspa_gather_rows(N.ptr(src2d), N.ptr(idx), N.ptr(count_dev), int(max_rows), int(row_bytes),
                                         N.ptr(dst), N.stream()), "gather_rows")
    return dst


def rope_relayout_kv(kv: torch.Tensor, H: int, D: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                     out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """kv (B, T, 2*H*D) -> rotated k and v, both (B*H, T, D)."""
    B, T, _ = kv.shape
    if out is not None:
        k, v = out
    else:
        k = _empty((B * H, T, D), kv.dtype, kv.device)
        v = torch.empty_like(k)
    with _timed('rope_relayout', 1, _nb(kv, k, v)):
        N.check(N.lib().aspa_rope_relayout_kv(N.ptr(kv), N.dtype_code(kv.dtype), B, T, H, D, N.ptr(cos), N.ptr(sin),
                                              N.ptr(k), N.ptr(v), N.stream()), "rope_relayout_kv")
    return k, v


def rope_rows_q(q_rows: torch.Tensor, kept_idx: torch.Tensor, count_dev: Optional[torch.Tensor], B: int, T: int, H: int,
                D: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor]) -> torch.Tensor:
    """Compact query rows -> (B*H, T, D) with only the kept tokens' rows written."""
    q = _empty((B * H, T, D), q_rows.dtype, q_rows.device)
    with _timed('rope_rows_q', 1, 2 * _nb(q_rows)):
        N.check(N.lib().aspa_rope_rows_q(N.ptr(q_rows), N.dtype_code(q_rows.dtype), N.ptr(kept_idx), N.ptr(count_dev),
                                         q_rows.size(0), B, T, H, D, N.ptr(cos), N.ptr(sin), N.ptr(q), N.stream()),
                "rope_rows_q")
    return q


def compact_mask(mask_u8: torch.Tensor, capacity: int):
    """Ordered indices of the non-zero mask bytes: (kept_idx int64 (capacity) padded with n, slot_of int32 (n), count)."""
    n = mask_u8.numel()
    dev = mask_u8.device
    kept_idx = _empty((capacity,), torch.int64, dev)
    slot_of = _empty((n,), torch.int32, dev)
    count = _empty((1,), torch.int32, dev)
    scratch = _empty((int(N.lib().aspa_compact_mask_scratch(n)),), torch.uint8, dev)
    with _timed('compact_mask', 2, 2 * n + 4 * n + 8 * capacity):
        N.check(N.lib().aspa_compact_mask(N.ptr(mask_u8), n, int(capacity), N.ptr(kept_idx), N.ptr(slot_of), N.ptr(count),
                                          N.ptr(scratch), N.stream()), "compact_mask")
    return kept_idx, slot_of, count


def scatter_rows_fill(src2d: torch.Tensor, slot_of: torch.Tensor, mask_u8: torch.Tensor, fill: Optional[torch.Tensor],
                      n: int) -> torch.Tensor:
    """(n, C): row i = src2d[slot_of[i]] where mask_u8[i] != 0, else ``fill`` (a (C,) row; None = zeros)."""
    Cdim = src2d.size(1)
    dst = _empty((n, Cdim), src2d.dtype, src2d.device)
    with _timed('scatter_rows_fill', 1, _nb(dst)):
        N.check(N.lib().aspa_scatter_rows_fill(N.ptr(src2d), N.ptr(slot_of), N.ptr(mask_u8), N.ptr(fill), n,
                                               Cdim * src2d.element_size(), N.ptr(dst), N.stream()), "scatter_rows_fill")
    return dst


def rope_inplace(x_rows: torch.Tensor, n_rows: int, T: int, row_stride: int, H: int, D: int, cos: torch.Tensor,
                 sin: torch.Tensor, heads_out: Optional[torch.Tensor] = None) -> None:
    """Rotate ``n_rows`` rows of H*D elements that start at ``x_rows`` and lie ``row_stride`` elements apart: in
    place, or into ``heads_out`` (n_rows / T * H, T, D) when given."""
    e = x_rows.element_size()
    with _timed('rope_inplace', 1, 2 * n_rows * H * D * e):
        N.check(N.lib().aspa_rope_rows_to_heads(N.ptr(x_rows), N.dtype_code(x_rows.dtype), int(n_rows), int(T),
                                                int(row_stride), H, D, N.ptr(cos), N.ptr(sin), N.ptr(heads_out),
                                                N.stream()), "rope_rows_to_heads")


def memory_update(k: torch.Tensor, v: torch.Tensor, kv_layout: Optional[N.KVLayout], B: int, H: int, T: int, D: int,
                  row_offsets: torch.Tensor, token_idx: torch.Tensor, decay: float, mem_keys: torch.Tensor,
                  mem_values: torch.Tensor, mem_counts: torch.Tensor, mem_ptr: torch.Tensor) -> None:
    """Push the mean key / value of every (batch, head) pair that has packed rows into the head's ring (in place)."""
    with _timed('memory_update', 1, 0):
        N.check(N.lib().aspa_memory_update(
            N.ptr(k), N.ptr(v), N.dtype_code(k.dtype), C.byref(kv_layout) if kv_layout is not None else None, B, H, T, D,
            N.ptr(row_offsets), N.ptr(token_idx), float(decay), N.ptr(mem_keys), N.ptr(mem_values), N.ptr(mem_counts),
            N.ptr(mem_ptr), int(mem_keys.size(1)), N.stream()), "memory_update")


def memory_fold_amax(mem_keys: torch.Tensor, mem_values: torch.Tensor, mem_counts: torch.Tensor, mem_ptr: torch.Tensor,
                     B: int, dtype: torch.dtype, row_offsets: torch.Tensor, amax_k: torch.Tensor,
                     amax_v: torch.Tensor) -> None:
    """amax_k, amax_v (B*H) fp32, in place: max with the amax of the ring rows the reference appends to k and v."""
    H, S, D = mem_keys.shape
    with _timed('memory_fold_amax', 1, 0):
        N.check(N.lib().aspa_memory_fold_amax(
            N.ptr(mem_keys), N.ptr(mem_values), N.ptr(mem_counts), N.ptr(mem_ptr), B, H, S, D, N.dtype_code(dtype),
            N.ptr(row_offsets), N.ptr(amax_k), N.ptr(amax_v), N.stream()), "memory_fold_amax")


TOKEN_COMPACT_MAX_T = 65536  # ASPA_TOKEN_COMPACT_MAX_T of the C header


def token_select_compact(importance: torch.Tensor, need: int, threshold: float, guard: int, slots_per_row: int):
    """Token keep plus the ordered kept-token list in one launch: (mask, kept, kept_idx padded with -1, slot_of)."""
    B, T = importance.shape
    dev = importance.device
    mask = _empty((B, T), torch.uint8, dev)
    kept = _empty((B,), torch.int32, dev)
    kept_idx = _empty((B * slots_per_row,), torch.int64, dev)
    slot_of = _empty((B * T,), torch.int32, dev)
    with _timed('token_select', 1, _nb(importance, mask, kept_idx, slot_of)):
        N.check(N.lib().aspa_token_select_compact(N.ptr(importance), B, T, int(need), float(threshold), int(guard),
                                                  N.ptr(mask), N.ptr(kept), N.ptr(kept_idx), N.ptr(slot_of),
                                                  int(slots_per_row), N.stream()), "token_select_compact")
    return mask, kept, kept_idx, slot_of


def head_select_pack(gate: torch.Tensor, g2h: torch.Tensor, B: int, T: int, H: int, *, k_host: int,
                     k_dev: Optional[torch.Tensor], kmax: int, token_mask: Optional[torch.Tensor], capacity: int):
    """Per-token head choice and row packing.  Returns (bits, top_idx, top_score, stat partials (2 * blocks),
    row_offsets, token_idx)."""
    n, G = gate.shape
    dev = gate.device
    bits = _empty((n,), torch.int64, dev)
    top_idx = _empty((n, kmax), torch.int32, dev)
    top_score = _empty((n, kmax), torch.float32, dev)
    partials = _empty((2 * ((n + 255) // 256),), torch.float32, dev)
    scratch = _empty((int(N.lib().aspa_pack_rows_scratch(B, H, T)),), torch.int32, dev)
    offs = _empty((B * H + 1,), torch.int32, dev)
    tok = _empty((max(1, capacity),), torch.int32, dev)
    with _timed('head_select_pack', 3 if T % 256 == 0 else 4, _nb(gate, bits, top_idx, top_score) + 2 * _nb(bits)):
        N.check(N.lib().aspa_head_select_pack(N.ptr(gate), B, T, G, N.ptr(g2h), H, int(k_host), N.ptr(k_dev), int(kmax),
                                              N.ptr(token_mask), N.ptr(bits), N.ptr(top_idx), N.ptr(top_score),
                                              N.ptr(partials), N.ptr(scratch), N.ptr(offs), N.ptr(tok), int(capacity),
                                              N.stream()), "head_select_pack")
    return bits, top_idx, top_score, partials, offs, tok


def stats_record(row_offsets: torch.Tensor, kept: Optional[torch.Tensor], n_kept: int, kept_fill: float,
                 k_dev: Optional[torch.Tensor], k_fill: float, head_partials: torch.Tensor,
                 proto_partials: Optional[torch.Tensor], status: Optional[torch.Tensor]) -> torch.Tensor:
    """fp64 record [row offsets | kept | k, adaptive k | score, entropy sums | 3 prototype sums | status]."""
    rec = _empty((row_offsets.numel() + n_kept + 8,), torch.float64, row_offsets.device)
    with _timed('stats_record', 1, 0):
        N.check(N.lib().aspa_stats_record(
            N.ptr(row_offsets), row_offsets.numel(), N.ptr(kept), int(n_kept), float(kept_fill), N.ptr(k_dev), float(k_fill),
            N.ptr(head_partials), head_partials.numel() // 2, N.ptr(proto_partials),
            proto_partials.numel() // 3 if proto_partials is not None else 0, N.ptr(status), N.ptr(rec), N.stream()),
            "stats_record")
    return rec


def chunk_select_slot(importance: torch.Tensor, token_mask: Optional[torch.Tensor], budget: int, top_p: float,
                      slot_dev: torch.Tensor, slot_offsets: torch.Tensor, rec_scores: torch.Tensor, rec_idx: torch.Tensor,
                      rec_count: torch.Tensor) -> None:
    """Chunk promotion into record slot ``slot_dev[0]`` (int32 on the device); ``slot_offsets`` (n_slots) int64."""
    T = importance.numel()
    with _timed('chunk_select', 1, _nb(importance)):
        N.check(N.lib().aspa_chunk_select_slot(N.ptr(importance), N.ptr(token_mask), T, int(budget), float(top_p),
                                               N.ptr(slot_dev), N.ptr(slot_offsets), N.ptr(rec_scores), N.ptr(rec_idx),
                                               N.ptr(rec_count), N.stream()), "chunk_select_slot")


def rope_quantize_outputs(B: int, T: int, H: int, D: int, dev: torch.device):
    """(q8, k8, v8, scales) for ``rope_quantize(out=...)``, allocated on the current stream."""
    q8 = _empty((B * H, T, D), torch.int8, dev)
    return q8, torch.empty_like(q8), torch.empty_like(q8), _empty((3, B * H), torch.float32, dev)


def rope_quantize(qkv: torch.Tensor, H: int, D: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], out=None):
    """Fused bf16 projection (B, T, 3*H*D) -> rotated, head-major INT8 q, k, v (B*H, T, D) and their per-head scales."""
    B, T, _ = qkv.shape
    dev = qkv.device
    q8, k8, v8, scales = out if out is not None else rope_quantize_outputs(B, T, H, D, dev)
    amax = _empty((3, B * H), torch.float32, dev)
    with _timed('rope_quantize', 3, 2 * _nb(qkv) + _nb(q8, k8, v8)):
        N.check(N.lib().aspa_rope_quantize(N.ptr(qkv), B, T, H, D, N.ptr(cos), N.ptr(sin), N.ptr(q8), N.ptr(k8), N.ptr(v8),
                                           N.ptr(amax), N.ptr(scales), N.stream()), "rope_quantize")
    return q8, k8, v8, scales
