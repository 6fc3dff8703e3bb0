"""CPU oracle for the ASPA hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch-on-CPU code, the algorithm of the reference
project's ASPA attention layer and chunked shortlist tool.  It exists so that
the CUDA path can be checked against something independent.  Only the test
suite, the smoke entry and the CPU-baseline leg of the benchmark may import
it; the product package never does.

Parity status: PINNED.  ``tests/golden/make_golden.py`` runs the reference
implementation itself (imported from its source tree) on seeded inputs and
stores inputs and outputs under ``tests/golden/``; ``tests/test_oracle_golden.py``
checks every function below against those vectors.

Where the reference leaves an order unspecified (``torch.topk`` /
``torch.argsort`` on tied keys) this oracle fixes it: among equal keys the
lowest index wins.  The CUDA kernels use the same rule.

Citations are ``file:line`` inside the reference project:
  aspa.py = src/proteus_attention/models/aspa.py
  sa.py   = src/proteus_attention/kernels/sparse_attn.py
  cs.py   = src/proteus_attention/tools/chunked_shortlist.py
"""
from __future__ import annotations

import math
from types import SimpleNamespace
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

NEG_INF = float("-inf")


# ----------------------------------------------------------------------------
# configuration (aspa.py:180-567)
# ----------------------------------------------------------------------------

def _get(cfg: Dict[str, Any], key: str, default: Any) -> Any:
    return cfg[key] if key in cfg else default


def _f(cfg, key, default):
    """``float(getattr(cfg, key, default) or default)`` idiom of the reference."""
    return float(_get(cfg, key, default) or default)


def _i(cfg, key, default):
    return int(_get(cfg, key, default) or default)


_MODEL_DEFAULTS = {  # aspa.py:42-64
    "n_ctx": 0, "n_head": 1, "d_model": 0, "p_dropout": 0.0, "bias": False,
    "attn_mode": "auto", "attn_linear_L": 512, "attn_linear_window": 512,
    "attn_linear_anchor_stride": 256, "attn_linear_head_k": 2,
    "attn_linear_switch_ctx": 20000, "attn_linear_latency_budget_ms": None,
    "attn_linear_policy": "local+anchors", "attn_use_rope": True,
    "attn_rope_base": 10000.0, "attn_router_top_p": 0.9,
}


def derive_config(**kwargs: Any) -> SimpleNamespace:
    """Resolve every knob the layer reads.  Follows aspa.py:180-567."""
    cfg = dict(_MODEL_DEFAULTS)
    cfg.update(kwargs)
    s = SimpleNamespace()
    s.d_model = int(cfg["d_model"])
    s.bias = bool(_get(cfg, "bias", False))
    h = int(_get(cfg, "attn_h_total", 0) or _get(cfg, "n_head", 1) or 1)
    if h <= 0:
        h = max(1, int(_get(cfg, "n_head", 1)))
    s.h_total = h
    if s.d_model % h:
        raise ValueError("d_model must be divisible by the total number of attention heads (attn_h_total)")
    act = int(_get(cfg, "attn_h_active", 0))
    if act <= 0 or act > h:
        act = max(1, min(4, h))
    lo = int(_get(cfg, "attn_h_active_min", 0) or 0)
    hi = int(_get(cfg, "attn_h_active_max", 0) or 0)
    if hi <= 0:
        hi = min(16, h)
    hi = max(1, min(hi, h))
    if lo <= 0:
        lo = max(1, min(2, hi))
    lo = max(1, min(lo, hi))
    s.h_active_min, s.h_active_max = lo, hi
    s.h_active = max(lo, min(act, hi))
    curve = _get(cfg, "attn_active_curve", None)
    try:
        curve = float(curve) if curve is not None else 0.25
    except (TypeError, ValueError):
        curve = 0.25
    s.h_active_curve = curve if curve > 0.0 else 1.0
    s.force_dense_when_full = bool(_get(cfg, "attn_force_dense_when_full", False))
    s.d_head = s.d_model // h
    s.use_rope = bool(_get(cfg, "attn_use_rope", True)) and s.d_head % 2 == 0
    base = _f(cfg, "attn_rope_base", 10000.0)
    s.rope_base = base if base > 0.0 else 10000.0
    s.p_dropout = float(_get(cfg, "p_dropout", 0.0))
    top_p = _get(cfg, "attn_router_top_p", 0.0)
    try:
        top_p = float(top_p)
    except (TypeError, ValueError):
        top_p = 0.0
    if not math.isfinite(top_p):
        top_p = 0.0
    s.router_top_p = max(0.0, min(top_p, 1.0))
    mode = str(_get(cfg, "attn_mode", "auto") or "auto").lower()
    s.mode_setting = mode if mode in ("auto", "subquad", "linear") else "auto"
    s.linear_L = max(1, _i(cfg, "attn_linear_L", 512))
    sched = str(_get(cfg, "attn_linear_L_schedule", "fixed") or "fixed").lower()
    s.linear_L_schedule = sched if sched in ("fixed", "sqrt", "log", "mem_cap") else "fixed"
    s.linear_L_base = max(1, _i(cfg, "attn_linear_L_base", s.linear_L))
    dflt_min = min(64, s.linear_L_base)
    s.linear_L_min = max(1, _i(cfg, "attn_linear_L_min", dflt_min))
    lmax = _get(cfg, "attn_linear_L_max", s.linear_L)
    s.linear_L_max = max(s.linear_L_min, int(lmax if lmax is not None else s.linear_L))
    s.linear_L_scale_init = max(0.1, _f(cfg, "attn_linear_L_scale", 1.0))
    dflt_smax = max(1.0, s.linear_L_scale_init)
    s.linear_L_scale_max = _f(cfg, "attn_linear_L_scale_max", dflt_smax)
    s.linear_scale_min = max(0.05, s.linear_L_min / max(1.0, s.linear_L_base))
    s.linear_latency_shrink = min(max(_f(cfg, "attn_linear_latency_shrink", 0.8), 0.1), 0.99)
    s.linear_latency_growth = max(1.0, _f(cfg, "attn_linear_latency_growth", 1.05))
    mb = _get(cfg, "attn_linear_mem_budget_mb", None)
    s.linear_mem_budget_mb = float(mb) if mb is not None else None
    pl = max(0.0, min(1.0, _f(cfg, "attn_linear_piece_local_frac", 0.6)))
    pa = max(0.0, min(1.0, _f(cfg, "attn_linear_piece_anchor_frac", 0.3)))
    pp = float(_get(cfg, "attn_linear_piece_proto_frac", max(0.0, 1.0 - pl - pa)))
    pp = max(0.0, min(1.0, pp))
    tot = pl + pa + pp
    if tot <= 0.0:
        pl, pa, pp, tot = 1.0, 0.0, 0.0, 1.0
    pl /= tot
    pa /= tot
    pp = max(0.0, 1.0 - pl - pa)
    win = _i(cfg, "attn_linear_window", s.linear_L_base)
    if win <= 0:
        win = s.linear_L_base
    s.linear_window_base = max(1, win)
    stride = int(_get(cfg, "attn_linear_anchor_stride", _get(cfg, "attn_linear_anchors_every", 256)) or 0)
    s.linear_anchor_stride = max(0, stride)
    s.linear_head_k = max(1, min(_i(cfg, "attn_linear_head_k", 2), h))
    s.linear_switch_ctx = max(0, _i(cfg, "attn_linear_switch_ctx", 20000))
    lb = _get(cfg, "attn_linear_latency_budget_ms", None)
    s.linear_latency_budget_ms = float(lb) if lb is not None else None
    pol = str(_get(cfg, "attn_linear_policy", "local+anchors") or "local+anchors").lower()
    toks = {p.strip() for p in pol.replace("|", ",").replace("+", ",").split(",") if p.strip()}
    if not toks:
        toks = {"local", "anchors"}
    s.linear_use_anchors = bool(toks & {"anchors", "anchor", "global"})
    s.linear_use_proto = bool(toks & {"proto", "prototype", "semantic", "dna"})
    s.linear_use_local = bool(toks & {"local", "window"}) or not (s.linear_use_anchors or s.linear_use_proto)
    if not s.linear_use_local:
        pl = 0.0
    if not s.linear_use_anchors:
        pa = 0.0
    if not s.linear_use_proto:
        pp = 0.0
    tot = pl + pa + pp
    if tot <= 0.0:
        pl, pa, pp = 1.0, 0.0, 0.0
    else:
        pl /= tot
        pa /= tot
        pp = max(0.0, 1.0 - pl - pa)
    s.piece_local, s.piece_anchor, s.piece_proto = pl, pa, pp
    cut = _get(cfg, "attn_dense_alpha_cutoff", 0.0)
    try:
        cut = float(cut)
    except (TypeError, ValueError):
        cut = 0.25
    s.dense_alpha_cutoff = max(0.0, min(0.95, cut))
    s.quantize_int8 = bool(_get(cfg, "attn_quantize_int8", False))
    qm = str(_get(cfg, "attn_quantize_int8_mode", "max") or "max").lower()
    s.quantize_mode = qm if qm in ("max", "percentile", "ema_percentile") else "max"
    s.quantize_percentile = min(max(_f(cfg, "attn_quantize_int8_percentile", 1.0), 0.0), 1.0)
    s.quantize_ema_decay = min(max(_f(cfg, "attn_quantize_int8_ema_decay", 0.9), 0.0), 0.9999)
    seq_low = _i(cfg, "attn_active_seq_low", 0)
    seq_high = _i(cfg, "attn_active_seq_high", 0)
    if seq_low <= 0:
        seq_low = max(64, s.d_head)
    if seq_high <= 0:
        seq_high = int(_get(cfg, "n_ctx", 0) or seq_low * 4)
    s.seq_low, s.seq_high = seq_low, max(seq_high, seq_low)
    dc = _get(cfg, "attn_small_seq_dense", None)
    try:
        dc = int(dc) if dc is not None else max(0, s.seq_low // 2)
    except (TypeError, ValueError):
        dc = max(0, s.seq_low // 2)
    s.small_seq_dense = max(0, dc)
    dt = _get(cfg, "attn_force_dense_threshold", None)
    dt = float(dt) if dt is not None else None
    s.dense_threshold = dt if (dt is not None and dt > 0.0) else None
    g = int(_get(cfg, "attn_gates", 0))
    if g <= 0:
        g = max(h, s.h_active_max, s.h_active) * 2
    s.attn_gates = max(g, h, s.h_active_max)
    s.proto_enabled = bool(_get(cfg, "attn_proto_enable", False))
    s.proto_decay = float(_get(cfg, "attn_proto_decay", 0.97))
    s.proto_threshold = float(_get(cfg, "attn_proto_threshold", 0.25))
    s.proto_blend = float(_get(cfg, "attn_proto_blend", 0.6))
    s.proto_temp = float(max(_get(cfg, "attn_proto_temp", 0.2), 1e-3))
    s.proto_usage_boost = float(max(_get(cfg, "attn_proto_usage_boost", 0.0), 0.0))
    s.proto_init_scale = float(_get(cfg, "attn_proto_init_scale", 0.02))
    s.token_sparse = bool(_get(cfg, "attn_token_sparse", False))
    s.token_keep_ratio_base = min(max(_f(cfg, "attn_token_keep_ratio", 1.0), 0.0), 1.0)
    ks = str(_get(cfg, "attn_linear_token_keep_schedule", "sqrt") or "sqrt").lower()
    s.token_keep_schedule = ks if ks in ("fixed", "sqrt", "log") else "sqrt"
    s.token_keep_ratio_min = min(max(_f(cfg, "attn_linear_token_keep_min_ratio", 0.2), 0.0), s.token_keep_ratio_base)
    s.token_keep_ref = _i(cfg, "attn_linear_token_keep_ref", 2048)
    kmin = max(0, _i(cfg, "attn_token_keep_min", 0))
    guard = max(0, _i(cfg, "attn_token_keep_guard", 1))
    s.token_keep_guard = guard
    s.token_keep_min = max(kmin, guard if s.token_sparse else kmin)
    s.token_keep_threshold = max(0.0, _f(cfg, "attn_token_keep_threshold", 0.0))
    # key/value memory bank (aspa.py:389-416)
    s.memory_enabled = bool(_get(cfg, "attn_memory_enable", False))
    slots = int(_get(cfg, "attn_memory_slots", 0) or 0)
    if slots <= 0:
        s.memory_enabled, slots = False, 1
    s.memory_slots = slots
    s.memory_decay = float(max(0.0, min(1.0, float(_get(cfg, "attn_memory_decay", 0.9) or 0.9))))
    return s


def gate_to_head(gates: int, heads: int) -> torch.Tensor:
    """aspa.py:621-626."""
    idx = torch.arange(gates, dtype=torch.long)
    return torch.clamp((idx * max(heads, 1)) // max(gates, 1), 0, max(heads, 1) - 1)


# ----------------------------------------------------------------------------
# host-side schedules (aspa.py:731-747, 862-923, 1037-1145)
# ----------------------------------------------------------------------------

def choose_active_k(s, seq_len: int) -> int:
    if seq_len <= s.seq_low:
        k = s.h_active_max
    elif seq_len >= s.seq_high:
        k = s.h_active_min
    else:
        r = float(seq_len - s.seq_low) / float(max(1, s.seq_high - s.seq_low))
        if s.h_active_curve != 1.0:
            r = max(0.0, min(1.0, r)) ** s.h_active_curve
        k = int(math.floor(s.h_active_max - r * (s.h_active_max - s.h_active_min) + 1e-6))
    return max(s.h_active_min, min(k, s.h_active_max))


def shortlist_alpha(s, seq_len: int, override: Optional[float]) -> float:
    if override is not None:
        return float(max(0.0, min(1.0, override)))
    seq_len = int(max(1, seq_len))
    low = max(1, int(s.seq_low))
    high = max(low + 1, int(s.linear_switch_ctx)) if s.linear_switch_ctx > 0 else max(low + 1, seq_len)
    if seq_len <= low:
        return 0.0
    if seq_len >= high:
        return 1.0
    return float((seq_len - low) / (high - low))


def cvt_alpha(s, seq_len: int, state) -> float:
    """aspa.py:892-923.  ``state`` carries latency_ema/current_alpha/L scale/override."""
    seq_len = int(max(1, seq_len))
    if s.mode_setting == "linear":
        alpha = 1.0
    elif s.mode_setting == "subquad":
        alpha = 0.0
    else:
        alpha = shortlist_alpha(s, seq_len, state.alpha_override)
    if s.linear_latency_budget_ms is not None and state.latency_ema is not None:
        b, lat = s.linear_latency_budget_ms, state.latency_ema
        if lat > b * 1.05:
            if state.L_scale > s.linear_scale_min + 1e-3:
                state.L_scale = _clamp_scale(s, state.L_scale * s.linear_latency_shrink)
            alpha = 1.0
        elif lat < b * 0.80 and seq_len < max(1, s.linear_switch_ctx):
            if state.L_scale < s.linear_L_scale_max:
                state.L_scale = _clamp_scale(s, state.L_scale * s.linear_latency_growth)
            alpha = min(alpha, 0.0)
    if s.linear_switch_ctx > 0:
        if state.current_alpha >= 0.95 and seq_len >= max(1, int(s.linear_switch_ctx * 0.75)):
            alpha = max(alpha, 0.95)
        if seq_len >= s.linear_switch_ctx:
            alpha = 1.0
    return float(max(0.0, min(1.0, alpha)))


def _clamp_scale(s, v: float) -> float:
    return float(min(max(v, s.linear_scale_min), max(s.linear_scale_min, s.linear_L_scale_max)))


def linear_token_keep_ratio(s, seq_len: int) -> float:
    if not s.token_sparse:
        return s.token_keep_ratio_base
    ref = max(1, s.token_keep_ref)
    base = s.token_keep_ratio_base
    seq = max(1, int(seq_len))
    if s.token_keep_schedule == "sqrt":
        r = base * math.sqrt(ref / float(seq))
    elif s.token_keep_schedule == "log":
        r = base * (math.log2(ref + 1.0) / math.log2(seq + 1.0))
    else:
        r = base
    return float(max(min(base, s.token_keep_ratio_min), min(base, r)))


def effective_linear_params(s, seq_len: int, batch: Optional[int], alpha: float,
                            L_scale: float, last_target_k: Optional[int]) -> Dict[str, Any]:
    """aspa.py:1037-1145."""
    seq_len = max(1, int(seq_len))
    coeff = float(max(1.0, s.linear_L_base))
    if s.linear_L_schedule == "sqrt":
        base_val = coeff * math.sqrt(float(seq_len))
    elif s.linear_L_schedule == "log":
        base_val = coeff * math.log2(float(seq_len) + 1.0)
    elif s.linear_L_schedule == "mem_cap" and s.linear_mem_budget_mb:
        heads_est = max(1, int(last_target_k if last_target_k is not None else s.linear_head_k))
        batch_est = max(1, int(batch) if batch is not None else 1)
        denom = heads_est * batch_est * seq_len * max(1, s.d_head) * 8
        cap = int(s.linear_mem_budget_mb * 1024 * 1024 // denom) if denom > 0 else s.linear_L_max
        base_val = max(1, min(cap, s.linear_L_max))
    else:
        base_val = coeff
    eff = max(s.linear_L_min, min(s.linear_L_max, int(math.ceil(L_scale * max(1.0, base_val)))))
    window = min(s.linear_window_base, eff)
    dense_cap = int(min(seq_len, max(s.linear_L_min, s.linear_window_base + seq_len // 32)))
    dense_cap = max(s.linear_L_min, min(s.linear_L_max, dense_cap))
    eff = int(alpha * eff + (1.0 - alpha) * dense_cap)
    eff = max(s.linear_L_min, min(s.linear_L_max, eff))
    window_dense = max(1, min(seq_len, max(s.linear_window_base, seq_len // 8)))
    window = int(alpha * window + (1.0 - alpha) * window_dense)
    window = max(1, min(eff, window))
    use = (s.linear_use_local, s.linear_use_anchors, s.linear_use_proto)
    dense_w = (0.85, 0.10, 0.05)
    target_w = (s.piece_local, s.piece_anchor, s.piece_proto)
    w = [(1.0 - alpha) * (dense_w[i] if use[i] else 0.0) + alpha * (target_w[i] if use[i] else 0.0) for i in range(3)]
    tw = w[0] + w[1] + w[2]
    if tw <= 0.0:
        w, tw = [1.0, 0.0, 0.0], 1.0
    wl, wa = w[0] / tw, w[1] / tw
    wp = max(0.0, 1.0 - wl - wa)
    caps = [int(round(eff * wl)) if use[0] else 0,
            int(round(eff * wa)) if use[1] else 0,
            int(round(eff * wp)) if use[2] else 0]
    total = sum(caps)
    if total > eff and total > 0:
        sd = eff / total
        caps = [int(max(0, math.floor(c * sd))) for c in caps]
        total = sum(caps)
    remaining = eff - total
    for i in range(3):
        if remaining <= 0:
            break
        if not use[i]:
            continue
        caps[i] += 1
        remaining -= 1
    if remaining > 0:
        caps[0 if use[0] else 1 if use[1] else 2] += remaining
    if use[0]:
        caps[0] = min(caps[0], window)
        if caps[0] <= 0 and eff > 0:
            caps[0] = min(window, max(1, eff // 4))
    return {"effective_L": eff, "local_cap": max(0, caps[0]), "anchor_cap": max(0, caps[1]),
            "proto_cap": max(0, caps[2]), "window": max(1, int(window)), "shortlist_alpha": float(alpha)}


# ----------------------------------------------------------------------------
# deterministic selection helpers
# ----------------------------------------------------------------------------

def topk_lowest_index(values: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the ``k`` largest entries of a 1-D tensor, ordered by value
    descending; equal values are ordered by ascending index."""
    order = torch.sort(values, descending=True, stable=True).indices
    return order[:k]


# ----------------------------------------------------------------------------
# router (aspa.py:149-157, 628-690) and importance (aspa.py:1521-1530)
# ----------------------------------------------------------------------------

def route_tokens(s, x: torch.Tensor, w_router: torch.Tensor, protos: Optional[torch.Tensor],
                 confidence: Optional[torch.Tensor], usage: Optional[torch.Tensor]):
    """Return (gate_probs fp32 (B,T,G), proto_sim (B,T) or None, blend_scalar (B,T) or None)."""
    logits = F.linear(x, w_router)
    gate = F.softmax(logits, dim=-1).to(torch.float32)
    if not (s.proto_enabled and protos is not None):
        return gate, None, None
    xn = F.normalize(x.to(torch.float32), dim=-1, eps=1e-6)
    pn = F.normalize(protos.to(torch.float32), dim=-1, eps=1e-6)
    sims = xn @ pn.t()
    sim = sims.max(dim=-1).values
    pprob = F.softmax(sims / s.proto_temp, dim=-1)
    blend_scalar = torch.clamp((sim - s.proto_threshold) / max(1e-6, 1.0 - s.proto_threshold), 0.0, 1.0)
    if confidence is not None:
        pprob = pprob * (confidence.view(1, 1, -1) + 1e-6).to(torch.float32)
        pprob = pprob / pprob.sum(dim=-1, keepdim=True).clamp_min(1e-6)
    blend = s.proto_blend * blend_scalar.unsqueeze(-1)
    gate = gate * (1.0 - blend) + pprob * blend
    if s.proto_usage_boost > 0.0 and usage is not None:
        ub = torch.softmax(-(usage + 1e-6), dim=0).to(torch.float32)
        gate = gate + ub.view(1, 1, -1) * ((1.0 - blend_scalar).unsqueeze(-1) * s.proto_usage_boost)
    gate = gate.clamp_min(0.0)
    gate = gate / gate.sum(dim=-1, keepdim=True).clamp_min(1e-6)
    return gate, sim, blend_scalar


def token_importance(gate: torch.Tensor, sim: Optional[torch.Tensor], blend: Optional[torch.Tensor]) -> torch.Tensor:
    gmax = gate.amax(dim=-1)
    if sim is None:
        return gmax
    if blend is None:
        return torch.maximum(gmax, sim)
    return gmax * (1.0 - blend) + sim * blend


def select_active_tokens(s, importance: torch.Tensor, ratio: float) -> Optional[torch.Tensor]:
    """aspa.py:790-842.  Ties at the cut go to the lowest token index."""
    if not s.token_sparse:
        return None
    B, T = importance.shape
    if ratio >= 0.999 and s.token_keep_threshold <= 0.0:
        return torch.ones(B, T, dtype=torch.bool)
    guard = min(max(0, s.token_keep_guard), T)
    min_keep = max(min(max(0, s.token_keep_min), T), guard)
    need0 = int(torch.full((1,), ratio * T, dtype=torch.float32).round().item())
    if min_keep > 0:
        need0 = max(need0, min_keep)
    need0 = max(1, min(need0, T))
    mask = torch.zeros(B, T, dtype=torch.bool)
    imp = importance.to(torch.float32)
    for b in range(B):
        base = torch.zeros(T, dtype=torch.bool)
        if s.token_keep_threshold > 0.0:
            base = imp[b] >= s.token_keep_threshold
        need = min(max(1, max(need0, int(base.sum()), guard)), T)
        if need >= T:
            base = torch.ones(T, dtype=torch.bool)
        else:
            base[topk_lowest_index(imp[b], need)] = True
        if guard > 0:
            base[:guard] = True
        mask[b] = base
    return mask


def nucleus_head_count(head_probs: torch.Tensor, target_p: float, max_cap: int) -> int:
    """aspa.py:749-780."""
    if max_cap <= 1:
        return max(1, max_cap)
    mean = head_probs.to(torch.float32).mean(dim=(0, 1))
    mean = torch.where(torch.isfinite(mean), mean, torch.zeros_like(mean))
    total = float(mean.sum())
    if total <= 0.0:
        return 1
    sv = torch.sort(mean, descending=True).values
    keep = int((torch.cumsum(sv, 0) < total * float(target_p)).sum())
    if keep < sv.numel():
        keep += 1
    return min(max_cap, max(1, keep))


def head_topk(head_probs: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token top-k heads, ties to the lowest head index.  aspa.py:1590."""
    order = torch.sort(head_probs, dim=-1, descending=True, stable=True)
    return order.values[..., :k], order.indices[..., :k]


# ----------------------------------------------------------------------------
# RoPE (aspa.py:570-618)
# ----------------------------------------------------------------------------

def rope_tables(s, seq_len: int, dtype: torch.dtype):
    inv = 1.0 / (s.rope_base ** (torch.arange(0, s.d_head, 2, dtype=torch.float32) / max(s.d_head, 1)))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32), inv)
    cos = torch.repeat_interleave(ang.cos(), 2, dim=-1).to(dtype)
    sin = torch.repeat_interleave(ang.sin(), 2, dim=-1).to(dtype)
    return cos, sin


def apply_rope(s, q: torch.Tensor, k: torch.Tensor):
    """q, k: (B,T,H,D)."""
    if not s.use_rope:
        return q, k
    T = q.size(1)
    cos, sin = rope_tables(s, T, q.dtype)
    cos = cos.view(1, T, 1, s.d_head)
    sin = sin.view(1, T, 1, s.d_head)

    def rot(t):
        return torch.stack((-t[..., 1::2], t[..., ::2]), dim=-1).reshape_as(t)

    return q * cos + rot(q) * sin, k * cos + rot(k) * sin


# ----------------------------------------------------------------------------
# packing and candidates (sa.py:924-947, 260-596)
# ----------------------------------------------------------------------------

def pack_active_rows(mask: torch.Tensor):
    """mask: (heads, T) bool → (head_idx, token_idx, row_offsets int32, max_rows) or None."""
    pos = mask.nonzero(as_tuple=False)
    if pos.numel() == 0:
        return None
    counts = torch.bincount(pos[:, 0], minlength=mask.size(0)).to(torch.int32)
    offs = torch.zeros(mask.size(0) + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(counts, 0)
    return pos[:, 0].to(torch.int64), pos[:, 1].to(torch.int64), offs, int(counts.max())


def _proto_candidates(rows: torch.Tensor, seq_len: int, max_candidates: int,
                      proto: Optional[torch.Tensor], proto_cap: int) -> Optional[torch.Tensor]:
    """Per row ``t``: the ``min(t+1, cap)`` best-scoring positions ``<= t``; unused
    slots hold ``t``.  sa.py:260-299.  Ties by lowest index."""
    if proto is None or proto.numel() == 0 or proto_cap <= 0 or max_candidates <= 0:
        return None
    p = proto.to(torch.float32).reshape(-1)[:seq_len]
    if p.numel() == 0:
        return None
    cap = min(max_candidates, proto_cap, p.numel())
    if cap <= 0:
        return None
    out = rows.unsqueeze(1).expand(-1, cap).clone()
    order = torch.sort(p, descending=True, stable=True).indices  # global order, ties by index
    for i, t in enumerate(rows.tolist()):
        sel = order[order <= t][:cap]
        out[i, : sel.numel()] = sel
    return out


def build_candidates(rows: torch.Tensor, row_batch_ids: Optional[torch.Tensor], seq_len: int, *,
                     max_candidates: int, linear_window: int, anchor_stride: int,
                     use_local: bool, use_anchors: bool, proto_scores: Optional[torch.Tensor] = None,
                     local_cap: Optional[int] = None, anchor_cap: Optional[int] = None,
                     proto_cap: Optional[int] = None,
                     extra_candidates: Optional[torch.Tensor] = None,
                     extra_lengths: Optional[torch.Tensor] = None):
    """sa.py:376-596: (N, L) candidate table + lengths.  Row ``t`` gets its
    local window, strided anchors, prototype picks and itself, clamped to
    ``[0, min(t, seq_len-1)]``, sorted, de-duplicated and cut to the ``L``
    smallest; unused slots hold ``t``."""
    L = max_candidates
    if rows.numel() == 0 or L <= 0:
        return rows.new_empty(rows.shape + (0,)), rows.new_zeros(rows.shape, dtype=torch.long)
    lc = max(0, int(local_cap)) if local_cap is not None else (L if use_local else 0)
    ac = max(0, int(anchor_cap)) if anchor_cap is not None else (L if use_anchors else 0)
    pc = max(0, int(proto_cap)) if proto_cap is not None else (L if proto_scores is not None else 0)
    pieces: List[torch.Tensor] = []
    if use_local and lc > 0:
        w = min(linear_window, L, lc)
        if w > 0:
            steps = torch.arange(w, dtype=rows.dtype)
            ln = torch.clamp(rows + 1, max=w)
            start = torch.clamp(rows - ln + 1, min=0)
            loc = start[:, None] + steps[None, :]
            pieces.append(torch.where(steps[None, :] < ln[:, None], loc, rows[:, None]))
    if use_anchors and anchor_stride > 0 and ac > 0:
        slots = min(ac, L, max(1, seq_len))
        steps = torch.arange(1, slots + 1, dtype=rows.dtype)
        pieces.append(torch.clamp(rows[:, None] - steps[None, :] * anchor_stride, min=0))
    if proto_scores is not None and pc > 0:
        ps = proto_scores if proto_scores.dim() > 1 else proto_scores.unsqueeze(0)
        bids = row_batch_ids if row_batch_ids is not None else torch.zeros_like(rows)
        cap = min(L, pc, seq_len)
        if cap > 0 and ps.numel() > 0:
            blockp = rows.unsqueeze(1).expand(-1, cap).clone()
            for b in torch.unique(bids).tolist():
                m = bids == b
                c = _proto_candidates(rows[m], seq_len, L, ps[b], pc)
                if c is not None:
                    wdt = min(c.size(1), cap)
                    tmp = blockp[m]
                    tmp[:, :wdt] = c[:, :wdt]
                    blockp[m] = tmp
            pieces.append(blockp)
    if extra_candidates is not None and extra_candidates.numel() > 0:
        ex = extra_candidates.to(rows.dtype)
        if extra_lengths is not None:
            st = torch.arange(ex.size(1))
            ex = torch.where(st[None, :] < extra_lengths[:, None], ex, rows[:, None].expand_as(ex))
        pieces.append(ex)
    cand = torch.cat(pieces, dim=1) if pieces else rows[:, None]
    cand = torch.clamp(cand, min=0, max=max(seq_len - 1, 0))
    cand = torch.minimum(cand, rows[:, None])
    cand = torch.cat([cand, rows[:, None]], dim=1)
    out = rows[:, None].expand(-1, L).clone()
    lengths = torch.ones(rows.numel(), dtype=torch.long)
    for i in range(rows.numel()):
        u = torch.unique(cand[i])[:L]  # sorted ascending
        out[i, : u.numel()] = u
        lengths[i] = max(1, u.numel())
    return out.contiguous(), lengths


# ----------------------------------------------------------------------------
# key/value memory bank (aspa.py:932-1035)
# ----------------------------------------------------------------------------
def new_memory_bank(s) -> SimpleNamespace:
    return SimpleNamespace(keys=torch.zeros(s.h_total, s.memory_slots, s.d_head),
                           values=torch.zeros(s.h_total, s.memory_slots, s.d_head),
                           counts=torch.zeros(s.h_total, s.memory_slots),
                           ptr=torch.zeros(s.h_total, dtype=torch.long))


def memory_update(s, mem, active_heads: torch.Tensor, k_comp: torch.Tensor, v_comp: torch.Tensor,
                  mask_comp: torch.Tensor) -> None:
    """aspa.py:932-969.  For every active (batch, head) pair in ascending order: the head's whole bank decays, the
    mean key / value over the pair's active tokens goes into the slot under the ring pointer, the pointer advances.
    The sums are taken in the dtype of k.  With a decay of 1.0 nothing is written at all (the writes sit inside the
    ``decay < 1`` branch of the reference)."""
    if not s.memory_enabled or active_heads.numel() == 0 or mask_comp.numel() == 0:
        return
    counts = mask_comp.sum(dim=1)
    if not bool((counts > 0).any()):
        return
    mf = mask_comp.to(k_comp.dtype)
    sums_k = torch.einsum("ht,htd->hd", mf, k_comp)
    sums_v = torch.einsum("ht,htd->hd", mf, v_comp)
    for i, head in enumerate((active_heads % s.h_total).tolist()):
        c = counts[i].item()
        if c <= 0 or not s.memory_decay < 1.0:
            continue
        mem.keys[head] *= s.memory_decay
        mem.values[head] *= s.memory_decay
        mem.counts[head] *= s.memory_decay
        slot = int(mem.ptr[head])
        mem.keys[head, slot] = (sums_k[i] / c).to(torch.float32)
        mem.values[head, slot] = (sums_v[i] / c).to(torch.float32)
        mem.counts[head, slot] = float(c)
        mem.ptr[head] = (mem.ptr[head] + 1) % s.memory_slots


def memory_candidates(s, mem, active_heads: torch.Tensor, token_idx: torch.Tensor, row_offsets: torch.Tensor,
                      k_comp: torch.Tensor, v_comp: torch.Tensor, seq_len: int):
    """aspa.py:971-1035: k, v with ``max_mem`` memory rows appended per active head (the ring read from the pointer
    on, the first ``count`` rows of it, ``count`` = slots whose count is positive), and per packed row the extra
    candidate ids ``seq_len + j``.  Returns (k_aug, v_aug, extra, extra_len, max_mem)."""
    if not s.memory_enabled or active_heads.numel() == 0:
        return k_comp, v_comp, None, None, 0
    hid = (active_heads % s.h_total).long()
    per_head = (mem.counts.index_select(0, hid) > 0).sum(dim=1)
    max_mem = int(per_head.max()) if per_head.numel() else 0
    if max_mem <= 0:
        return k_comp, v_comp, None, None, 0
    A, D = k_comp.size(0), k_comp.size(2)
    mk, mv = k_comp.new_zeros(A, max_mem, D), v_comp.new_zeros(A, max_mem, D)
    valid = torch.zeros(A, max_mem, dtype=torch.bool)
    for i, head in enumerate(hid.tolist()):
        c = int(per_head[i])
        if c <= 0:
            continue
        p_ = int(mem.ptr[head])
        keys = torch.cat([mem.keys[head, p_:], mem.keys[head, :p_]], dim=0).to(k_comp.dtype)
        vals = torch.cat([mem.values[head, p_:], mem.values[head, :p_]], dim=0).to(v_comp.dtype)
        mk[i, :c], mv[i, :c], valid[i, :c] = keys[:c], vals[:c], True
    k_aug, v_aug = torch.cat([k_comp, mk], dim=1), torch.cat([v_comp, mv], dim=1)
    ids = (torch.arange(max_mem) + seq_len).unsqueeze(0).expand(A, -1)
    row_head = torch.repeat_interleave(torch.arange(A), (row_offsets[1:] - row_offsets[:-1]).long())
    extra = torch.where(valid[row_head], ids[row_head].to(token_idx.dtype), token_idx.unsqueeze(1).expand(-1, max_mem))
    return k_aug, v_aug, extra, valid[row_head].long().sum(dim=1).to(token_idx.dtype), max_mem


# ----------------------------------------------------------------------------
# INT8 per-head quantiser (aspa.py:1312-1363)
# ----------------------------------------------------------------------------

def quantize_per_head_int8(t: torch.Tensor, mode: str = "max", percentile: float = 1.0, ema: Optional[dict] = None,
                           ema_key: str = "", ema_decay: float = 0.9):
    """``ema`` (mode "ema_percentile") is the layer's dictionary of running bases; an entry that is missing or has
    another head count starts from this call's maximum (aspa.py:1339-1356)."""
    flat = t.to(torch.float32).reshape(t.size(0), -1)
    a = flat.abs()
    amax = a.amax(dim=1, keepdim=True)
    if mode == "max" or percentile <= 0.0:
        base = amax
    else:
        q = torch.quantile(a, percentile, dim=1, keepdim=True)
        base = torch.where(q > 0.0, q, amax)
    if mode == "ema_percentile" and ema is not None:
        prev = ema.get(ema_key)
        if prev is None or prev.numel() != flat.size(0):
            prev = amax.squeeze(1)
        updated = ema_decay * prev + (1.0 - ema_decay) * base.squeeze(1)
        ema[ema_key] = updated
        base = updated.unsqueeze(1)
    scales = torch.clamp(base / 127.0, min=1e-6)
    quant = torch.clamp((flat / scales).round(), -127.0, 127.0).to(torch.int8).view_as(t)
    return quant.contiguous(), scales.squeeze(1).contiguous()


# ----------------------------------------------------------------------------
# attention over packed rows (sa.py:950-1046, 1373-1646)
# ----------------------------------------------------------------------------

def sparse_attention(q, k, v, *, packed, causal_mask=None, candidates=None, lengths=None,
                     q_scale=None, k_scale=None, v_scale=None, out_dtype=None):
    """q,k,v: (heads, T, D).  ``packed`` = (head_idx, token_idx, row_offsets, max_rows).
    Shortlist branch: softmax over each row's own candidate keys.  Otherwise
    softmax over keys ``0..max_token`` under ``causal_mask`` rows (or ``j<=t``)."""
    heads, T, D = q.shape
    quant = q.dtype == torch.int8
    if out_dtype is None:
        out_dtype = q.dtype if q.dtype.is_floating_point else torch.float32
    if quant:
        q = q.to(torch.float32) * q_scale.view(-1, 1, 1)
        k = k.to(torch.float32) * k_scale.view(-1, 1, 1)
        v = v.to(torch.float32) * v_scale.view(-1, 1, 1)
    if causal_mask is not None:
        causal_mask = causal_mask.to(out_dtype)
    head_idx, token_idx, offs, _ = packed
    qa = q[head_idx, token_idx]
    scale = 1.0 / (D ** 0.5)
    res = torch.zeros_like(q)
    use_sl = candidates is not None and lengths is not None and candidates.numel() > 0
    for h in range(heads):
        a, b = int(offs[h]), int(offs[h + 1])
        if a == b:
            continue
        rt = token_idx[a:b]
        qs = qa[a:b]
        if use_sl:
            cr = candidates[a:b].long().clamp(0, T - 1)
            ln = lengths[a:b].long()
            inval = torch.arange(cr.size(1))[None, :] >= ln[:, None]
            ks = k[h][cr].masked_fill(inval[..., None], 0.0)
            vs = v[h][cr].masked_fill(inval[..., None], 0.0)
            sc = torch.einsum("rd,rld->rl", qs, ks) * scale
            if causal_mask is not None:
                sc = sc + torch.gather(causal_mask.index_select(0, rt), 1, cr).to(sc.dtype)
            pr = torch.softmax(sc.masked_fill(inval, NEG_INF), dim=-1)
            res[h].index_copy_(0, rt, torch.bmm(pr.unsqueeze(1), vs).squeeze(1))
        else:
            mt = int(rt.max())
            if causal_mask is not None:
                am = causal_mask.index_select(0, rt)[:, : mt + 1].unsqueeze(0)
            else:
                fut = torch.arange(mt + 1)[None, :] > rt[:, None]
                am = None
                if fut.any():
                    am = torch.zeros(1, rt.numel(), mt + 1, dtype=qs.dtype).masked_fill(fut[None], NEG_INF)
            o = F.scaled_dot_product_attention(qs[None], k[h][None, : mt + 1], v[h][None, : mt + 1],
                                               attn_mask=am, dropout_p=0.0, is_causal=False)[0]
            res[h].index_copy_(0, rt, o)
    return res.to(out_dtype)


# ----------------------------------------------------------------------------
# prototype EMA (aspa.py:692-718)
# ----------------------------------------------------------------------------

def update_prototypes(s, x, gate, protos, usage, confidence):
    """In-place EMA update of the three state tensors; returns #updated gates."""
    feats = x.to(torch.float32).reshape(-1, s.d_model)
    probs = gate.to(torch.float32).reshape(-1, s.attn_gates)
    counts = probs.sum(dim=0)
    m = counts > 1e-6
    if not m.any():
        return 0
    weighted = probs.t() @ feats
    mean = torch.zeros_like(protos, dtype=torch.float32)
    mean[m] = weighted[m] / counts[m].unsqueeze(-1)
    d = s.proto_decay
    protos[m] = protos[m] * d + mean[m].to(protos.dtype) * (1.0 - d)
    usage.mul_(d)
    usage[m] += counts[m] * (1.0 - d)
    confidence.mul_(d)
    confidence[m] += (1.0 - d)
    return int(m.sum())


# ----------------------------------------------------------------------------
# the layer (aspa.py:1365-1932)
# ----------------------------------------------------------------------------

class OracleLayer:
    """Stateful restatement of ``AdaptiveSparseAttention`` in eval mode."""

    def __init__(self, weights: Dict[str, torch.Tensor], **config: Any) -> None:
        self.s = derive_config(**config)
        s = self.s
        self.w_qkv = weights["qkv.weight"]
        self.b_qkv = weights.get("qkv.bias")
        self.w_proj = weights["proj.weight"]
        self.b_proj = weights.get("proj.bias")
        self.w_router = weights["head_router.linear.weight"]
        if s.proto_enabled:
            self.protos = weights["routing_prototypes"].clone()
            self.usage = weights.get("routing_usage_ema", torch.zeros(s.attn_gates)).clone()
            self.conf = weights.get("routing_confidence", torch.zeros(s.attn_gates)).clone()
        else:
            self.protos = self.usage = self.conf = None
        self.g2h = gate_to_head(s.attn_gates, s.h_total)
        self.onehot = F.one_hot(self.g2h, num_classes=s.h_total).to(torch.float32)
        self.state = SimpleNamespace(latency_ema=None, current_alpha=0.0, L_scale=s.linear_L_scale_init,
                                     alpha_override=None, last_target_k=None)
        self.memory = new_memory_bank(s) if s.memory_enabled else None
        self.quant_ema: Dict[str, torch.Tensor] = {}
        self.trace: Dict[str, Any] = {}

    def set_shortlist_alpha(self, v: float) -> None:
        self.state.alpha_override = float(max(0.0, min(1.0, v)))

    def _dense_fastpath(self, x):
        s = self.s
        B, T, C = x.shape
        qkv = F.linear(x, self.w_qkv, self.b_qkv)
        q, k, v = (t.view(B, T, s.h_total, s.d_head) for t in qkv.chunk(3, dim=2))
        q, k = apply_rope(s, q, k)
        o = F.scaled_dot_product_attention(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3),
                                           v.permute(0, 2, 1, 3), is_causal=True)
        self.trace = {"mode": "dense_fastpath"}
        return F.linear(o.permute(0, 2, 1, 3).reshape(B, T, C), self.w_proj, self.b_proj)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        s, st = self.s, self.state
        B, T, C = x.shape
        if s.small_seq_dense and T <= s.small_seq_dense:
            return self._dense_fastpath(x)
        alpha = cvt_alpha(s, T, st)
        st.current_alpha = alpha
        ratio = None
        if s.token_sparse:
            ratio = (1.0 - alpha) * float(s.token_keep_ratio_base) + alpha * float(linear_token_keep_ratio(s, T))
            ratio = float(max(0.0, min(1.0, ratio)))
        gate, sim, blend = route_tokens(s, x, self.w_router, self.protos, self.conf, self.usage)
        imp = token_importance(gate, sim, blend).to(torch.float32)
        tmask = select_active_tokens(s, imp, ratio) if s.token_sparse else None
        keep_frac = float(tmask.float().mean()) if tmask is not None else 1.0
        head_probs = gate @ self.onehot
        dense_k = choose_active_k(s, T)
        adaptive = dense_k
        if s.router_top_p > 0.0:
            adaptive = max(s.h_active_min, min(dense_k, nucleus_head_count(head_probs, s.router_top_p, dense_k)))
        lin_k = max(1, min(adaptive, s.linear_head_k))
        topk = min(adaptive, max(1, int(round((1.0 - alpha) * float(adaptive) + alpha * float(lin_k)))))
        st.last_target_k = topk
        hscores, hidx = head_topk(head_probs, topk)
        hmask = torch.zeros(B, T, s.h_total, dtype=torch.bool)
        hmask.scatter_(2, hidx, True)
        if tmask is not None:
            hmask &= tmask.unsqueeze(-1)
        flat = hmask.permute(0, 2, 1).reshape(B * s.h_total, T)
        counts = flat.sum(dim=1)
        max_rows = int(counts.max()) if counts.numel() else 0
        density = float(max_rows) / float(max(1, T))
        force_dense, reason = False, None
        if alpha <= s.dense_alpha_cutoff and not s.quantize_int8:
            force_dense, reason = True, "alpha"
        if s.dense_threshold is not None and density >= s.dense_threshold:
            force_dense, reason = True, reason or "density"
        elif bool(flat.all()) and s.force_dense_when_full:
            force_dense, reason = True, reason or "full"
        if alpha >= 0.95:
            force_dense, reason = False, (None if reason == "alpha" else reason)
        qkv = F.linear(x, self.w_qkv, self.b_qkv)
        q, k, v = (t.view(B, T, s.h_total, s.d_head) for t in qkv.chunk(3, dim=2))
        q, k = apply_rope(s, q, k)
        qf, kf, vf = (t.permute(0, 2, 1, 3).reshape(B * s.h_total, T, s.d_head) for t in (q, k, v))
        tr: Dict[str, Any] = {"alpha": alpha, "keep_ratio": ratio, "gate_probs": gate, "importance": imp,
                              "proto_sim": sim, "blend": blend, "token_mask": tmask, "topk": topk,
                              "head_idx": hidx, "head_scores": hscores, "max_rows": max_rows,
                              "density": density, "keep_fraction": keep_frac, "nucleus_k": adaptive}
        if force_dense:
            HT = B * s.h_total
            packed = (torch.arange(HT).repeat_interleave(T), torch.arange(T).repeat(HT),
                      torch.arange(0, (HT + 1) * T, T, dtype=torch.int32), T)
            cm = torch.triu(torch.full((T, T), NEG_INF, dtype=qf.dtype), diagonal=1)
            att = sparse_attention(qf, kf, vf, packed=packed, causal_mask=cm)
            tr["mode"] = "dense_alpha" if reason == "alpha" else ("dense" if int((counts > 0).sum()) == HT else "dense_auto")
        else:
            packed = pack_active_rows(flat)
            att = torch.zeros_like(qf)
            tr["mode"] = "sparse"
            if packed is not None:
                rt = effective_linear_params(s, T, B, alpha, st.L_scale, st.last_target_k)
                tr["runtime"] = rt
                bids = (packed[0] // s.h_total) if (s.linear_use_proto and sim is not None) else None
                extra = extra_len = None
                T_eff = T
                if self.memory is not None:   # aspa.py:1220-1260, on the heads that have active rows
                    act = torch.nonzero(counts > 0).flatten()
                    offs_comp = torch.cat([counts.new_zeros(1), counts[act].cumsum(0)])
                    memory_update(s, self.memory, act, kf[act], vf[act], flat[act])
                    k_aug, v_aug, extra, extra_len, mm = memory_candidates(
                        s, self.memory, act, packed[1], offs_comp, kf[act], vf[act], T)
                    if mm > 0:
                        T_eff = T + mm
                        pad = qf.new_zeros(qf.size(0), mm, qf.size(2))
                        qf = torch.cat([qf, pad], dim=1)
                        kf, vf = torch.cat([kf, pad], dim=1), torch.cat([vf, pad.to(vf.dtype)], dim=1)
                        kf[act], vf[act] = k_aug, v_aug
                cands, lens = build_candidates(
                    packed[1], bids, T_eff, max_candidates=rt["effective_L"], linear_window=rt["window"],
                    anchor_stride=s.linear_anchor_stride, use_local=s.linear_use_local,
                    use_anchors=s.linear_use_anchors,
                    proto_scores=sim if (s.linear_use_proto and sim is not None) else None,
                    local_cap=rt["local_cap"], anchor_cap=rt["anchor_cap"], proto_cap=rt["proto_cap"],
                    extra_candidates=extra, extra_lengths=extra_len)
                tr["candidates"], tr["lengths"], tr["packed"] = cands, lens, packed
                if s.quantize_int8:
                    kw = dict(ema=self.quant_ema, ema_decay=s.quantize_ema_decay)
                    qq, qs_ = quantize_per_head_int8(qf, s.quantize_mode, s.quantize_percentile, ema_key="q", **kw)
                    kq, ks_ = quantize_per_head_int8(kf, s.quantize_mode, s.quantize_percentile, ema_key="k", **kw)
                    vq, vs_ = quantize_per_head_int8(vf, s.quantize_mode, s.quantize_percentile, ema_key="v", **kw)
                    tr["quant_scales"] = (qs_, ks_, vs_)
                    att = sparse_attention(qq, kq, vq, packed=packed, candidates=cands, lengths=lens,
                                           q_scale=qs_, k_scale=ks_, v_scale=vs_, out_dtype=qf.dtype)
                else:
                    att = sparse_attention(qf, kf, vf, packed=packed, candidates=cands, lengths=lens)
                att = att[:, :T].contiguous()
                tr["mode"] = "shortlist"
        out = att.view(B, s.h_total, T, s.d_head).permute(0, 2, 1, 3)
        if tmask is not None:
            out = out * tmask.unsqueeze(-1).unsqueeze(-1)
        cons = out.reshape(B, T, C)
        tr["consensus"] = cons
        y = F.linear(cons, self.w_proj, self.b_proj)
        if s.proto_enabled and self.protos is not None:
            update_prototypes(s, x, gate, self.protos, self.usage, self.conf)
        self.trace = tr
        return y


# ----------------------------------------------------------------------------
# chunked shortlist tool (cs.py:88-254, 382-827)
# ----------------------------------------------------------------------------

def chunk_model_config(seq_len: int, d_model: int, *, heads: int, sparse_ratio: float,
                       router_top_p: float) -> Dict[str, Any]:
    """cs.py:88-137."""
    return dict(
        n_ctx=seq_len, n_head=heads, d_model=d_model, p_dropout=0.0, bias=False,
        attn_h_total=heads, attn_h_active=heads, attn_h_active_min=heads, attn_h_active_max=heads,
        attn_active_seq_low=max(128, seq_len // 4), attn_active_seq_high=seq_len, attn_mode="linear",
        attn_token_sparse=True, attn_token_keep_ratio=max(0.0, min(1.0, sparse_ratio)),
        attn_token_keep_min=max(4, int(seq_len * sparse_ratio * 0.5)), attn_token_keep_guard=4,
        attn_token_keep_threshold=0.0, attn_linear_L=256, attn_linear_L_base=256, attn_linear_L_min=64,
        attn_linear_L_max=256, attn_linear_switch_ctx=max(512, min(seq_len, 4096)),
        attn_linear_policy="local+anchors", attn_proto_enable=True, attn_proto_threshold=0.2,
        attn_proto_blend=0.5, attn_proto_temp=0.3, attn_linear_token_keep_schedule="sqrt",
        attn_linear_token_keep_min_ratio=0.05, attn_track_latency=False, attn_small_seq_dense=0,
        attn_router_top_p=router_top_p)


def nucleus_select(scores: torch.Tensor, max_tokens: int, top_p: float):
    """cs.py:175-208 with ties ordered by index."""
    limit = min(max_tokens, int(scores.numel()))
    if limit <= 0:
        return None
    fin = torch.isfinite(scores)
    if not fin.any():
        return None
    safe = scores.clone()
    safe[~fin] = -1e9
    order = torch.sort(safe, descending=True, stable=True).indices
    if top_p >= 1.0:
        keep = limit
    else:
        mass = torch.cumsum(torch.softmax(safe, dim=-1)[order], dim=-1)
        keep = int((mass < torch.tensor(float(top_p), dtype=scores.dtype)).sum())
        if keep < order.numel():
            keep += 1
        keep = max(1, keep)
    sel = order[: min(limit, keep)]
    return scores[sel], sel


def select_top_tokens(importance: torch.Tensor, mask: Optional[torch.Tensor], offset: int, *,
                      budget: int, top_p: float):
    """cs.py:140-172 (device check dropped: scores always come from the router)."""
    sc = importance.reshape(-1).to(torch.float32)
    if mask is not None:
        sc = torch.where(mask.reshape(-1).bool(), sc, torch.full_like(sc, NEG_INF))
    r = nucleus_select(sc, budget, top_p)
    if r is None:
        return None
    vals, idx = r
    f = torch.isfinite(vals)
    if not f.any():
        return None
    return vals[f], idx[f] + int(offset)


def finalise_indices(scores: torch.Tensor, indices: torch.Tensor, *, max_tokens: int):
    """cs.py:211-254.  The reference sorts by the key ``index*(n+1) - rank`` where
    ``rank`` is the position in score-descending order, then keeps the first
    entry of every run of equal indices.  Within a run the LARGEST rank sorts
    first, so a duplicated index is represented by its LOWEST score (its
    docstring says otherwise; the code is what is followed here).  The
    ``max_tokens`` best representatives (ties to the lower index) are returned
    in ascending index order."""
    if scores.numel() == 0:
        raise RuntimeError("No candidate tokens captured during chunking.")
    best: Dict[int, float] = {}
    for sc, ix in zip(scores.tolist(), indices.tolist()):
        if ix not in best or sc < best[ix]:
            best[ix] = sc
    ids = torch.tensor(sorted(best), dtype=torch.long)
    vals = torch.tensor([best[i] for i in ids.tolist()], dtype=scores.dtype)
    pick = torch.sort(vals, descending=True, stable=True).indices[:max_tokens]
    pick = torch.sort(pick).values
    return ids[pick], vals[pick]


def chunked_run(sequence: torch.Tensor, *, chunk_len: int, buffer_tokens: int, per_chunk_budget: int,
                heads: int, chunk_weights: Dict[str, torch.Tensor], final_weights: Dict[str, torch.Tensor],
                nucleus_top_p: float = 0.9, chunk_sparse_ratio: float = 0.05, final_sparse_ratio: float = 0.5,
                shortlist_alpha: float = 1.0, freeze_prototypes: bool = False, run_final_pass: bool = True,
                scoring_only: bool = False, warmup_input: Optional[torch.Tensor] = None):
    """cs.py:382-827 with router-importance scoring (the reference's GPU
    semantics; its CPU run silently scores by L2 norm instead).  The warm-up
    forward on unseeded noise (cs.py:583-587) runs only when ``warmup_input`` is
    given, so both sides of a comparison can be fed the same noise.
    ``freeze_prototypes`` sets the EMA decay to 1.0 so chunks are independent."""
    _, T, C = sequence.shape
    extra = {"attn_proto_decay": 1.0} if freeze_prototypes else {}
    cm = OracleLayer(chunk_weights, **chunk_model_config(chunk_len, C, heads=heads, sparse_ratio=chunk_sparse_ratio,
                                                         router_top_p=nucleus_top_p), **extra)
    cm.set_shortlist_alpha(shortlist_alpha)
    if warmup_input is not None:
        cm.forward(warmup_input)
    all_s, all_i = [], []
    for start in range(0, T, chunk_len):
        end = min(T, start + chunk_len)
        xc = sequence[:, start:end]
        if scoring_only:
            s = cm.s
            alpha = cvt_alpha(s, end - start, cm.state)
            ratio = (1.0 - alpha) * s.token_keep_ratio_base + alpha * linear_token_keep_ratio(s, end - start)
            gate, sim, blend = route_tokens(s, xc, cm.w_router, cm.protos, cm.conf, cm.usage)
            imp = token_importance(gate, sim, blend).to(torch.float32)
            tm = select_active_tokens(s, imp, float(max(0.0, min(1.0, ratio))))
            update_prototypes(s, xc, gate, cm.protos, cm.usage, cm.conf)
        else:
            cm.forward(xc)
            imp, tm = cm.trace["importance"], cm.trace["token_mask"]
        r = select_top_tokens(imp, tm, start, budget=per_chunk_budget, top_p=nucleus_top_p)
        if r is not None:
            all_s.append(r[0])
            all_i.append(r[1])
    keep_idx, keep_sc = finalise_indices(torch.cat(all_s), torch.cat(all_i), max_tokens=buffer_tokens)
    reduced = sequence[:, keep_idx]
    final_out = None
    if run_final_pass:
        fm = OracleLayer(final_weights, **chunk_model_config(reduced.size(1), C, heads=heads,
                                                             sparse_ratio=final_sparse_ratio,
                                                             router_top_p=nucleus_top_p), **extra)
        fm.set_shortlist_alpha(shortlist_alpha)
        final_out = fm.forward(reduced)
    return {"keep_indices": keep_idx, "keep_scores": keep_sc, "reduced_sequence": reduced,
            "final_output": final_out, "chunk_scores": all_s, "chunk_indices": all_i}
