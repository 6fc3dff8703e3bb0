"""ASPA attention layer on the sm_100a kernels.

Drop-in for the reference classes in ``src/proteus_attention/models/aspa.py``:
``ModelConfig`` (:33-72), ``AdaptiveSparseAttention`` (:170-1932),
``AdaptiveSparseProtoAttention`` (:1935-1944) and ``AdaptiveSparseAttentionBlock``
(:1947-1990).  Constructor knobs, attribute names read by callers and
controllers, ``state_dict`` keys, mode selection and the telemetry dictionaries
follow the reference; the arithmetic runs in libaspa_b200.so.

Differences that are deliberate:
  * forward only (the reference's kernel path has no autograd either); attention
    dropout raises ``NotImplementedError``;
  * the key/value memory bank (:932-1035) is kept as state (four buffers, updated by every shortlist call) and
    enters the INT8 scales of k and v; its rows never reach the attention in the reference either, because the
    candidate builder clamps the memory ids onto the row's own token (kernels/sparse_attn.py:570-571);
  * one device-to-host read per call (a small statistics record) instead of the
    reference's ~20 ``.item()`` calls; it is issued before the QKV projection and
    waited on after it, so the GPU does not idle;
  * float buffers (RoPE frequencies, prototypes, EMAs) stay fp32 under ``.to(bfloat16)``;
  * ties in top-k selections go to the lowest index.
"""
from __future__ import annotations

import math
import time
import warnings
from typing import Any, Dict, Optional, Tuple

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _native as N
from . import ops
from .sparse_attn import BACKEND_NAME, _record_backend, attention_packed, get_last_backend_info


class ModelConfig:
    """Attribute bag with the reference's defaults (aspa.py:42-64)."""

    _DEFAULTS: Dict[str, Any] = {
        "vocab_size": 0, "n_ctx": 0, "n_layer": 0, "n_head": 1, "d_model": 0, "p_dropout": 0.0, "bias": False,
        "attn_variant": "standard", "moe_n_experts": 0, "attn_mode": "auto", "attn_linear_L": 512,
        "attn_linear_window": 512, "attn_linear_anchor_stride": 256, "attn_linear_head_k": 2,
        "attn_linear_switch_ctx": 20000, "attn_linear_latency_budget_ms": None,
        "attn_linear_policy": "local+anchors", "attn_use_rope": True, "attn_rope_base": 10000.0,
        "attn_router_top_p": 0.9,
    }

    def __init__(self, **kwargs: Any) -> None:
        data = dict(self._DEFAULTS)
        data.update(kwargs)
        self.__dict__.update(data)

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.__dict__)


class LayerNorm(nn.Module):
    def __init__(self, ndim: int, bias: bool, eps: float = 1e-5) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(ndim))
        self.bias = nn.Parameter(torch.zeros(ndim)) if bias else None
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.layer_norm(x, x.shape[-1:], self.weight, self.bias, eps=self.eps)


class RMSNorm(nn.Module):
    def __init__(self, ndim: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(ndim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.weight * (x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + self.eps))


def _build_norm(config: ModelConfig) -> nn.Module:
    kind = str(getattr(config, "norm_type", "layernorm") or "layernorm").lower()
    eps = float(getattr(config, "norm_eps", 1e-5))
    if kind == "rmsnorm":
        return RMSNorm(config.d_model, eps=eps)
    return LayerNorm(config.d_model, bias=bool(getattr(config, "bias", False)), eps=eps)


class MLP(nn.Module):
    def __init__(self, config: ModelConfig) -> None:
        super().__init__()
        hidden = int(getattr(config, "mlp_hidden_mult", 4)) * config.d_model
        self.fc1 = nn.Linear(config.d_model, hidden, bias=bool(config.bias))
        self.act = nn.GELU()
        self.fc2 = nn.Linear(hidden, config.d_model, bias=bool(config.bias))
        self.dropout = nn.Dropout(config.p_dropout)
        self.last_aux_loss: Optional[torch.Tensor] = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.dropout(self.fc2(self.act(self.fc1(x))))


class SwitchRouter(nn.Module):
    """Holds the router weight (``head_router.linear.weight``); the product and softmax run inside
    the fused router kernel, so ``forward`` here exists only for API compatibility."""

    def __init__(self, d_model: int, n_gates: int, noise_std: float = 0.0) -> None:
        super().__init__()
        self.linear = nn.Linear(d_model, n_gates, bias=False)
        self.noise_std = float(noise_std)

    def forward(self, x: torch.Tensor):
        probs = F.softmax(self.linear(x), dim=-1)
        scores, indices = torch.max(probs, dim=-1)
        return indices, scores, probs


# ---- config parsing helpers ------------------------------------------------------------------
K_HEAD_MAJOR = True   # rotated keys are written head-major (a window of keys becomes one contiguous run)
_SIDE_STREAMS: Dict[Tuple[str, int], "torch.cuda.Stream"] = {}  # second streams per (device, priority), shared by all layers


def _num(config, name, default, kind=float):
    """``kind(getattr(config, name, default) or default)`` — zero and None select the default."""
    return kind(getattr(config, name, default) or default)


def _policy_tokens(raw: str):
    parts = {p.strip() for p in raw.replace("|", ",").replace("+", ",").split(",") if p.strip()}
    return parts or {"local", "anchors"}


def _py_round_f32(value: float) -> int:
    """round() of a value first rounded to fp32, half to even — what ``torch.full(.., fp32).round()`` gives."""
    return int(np.rint(np.float32(value)))


class AdaptiveSparseAttention(nn.Module):
    """Adaptive Sparse Proto Attention layer; ``forward(x: (B, T, C)) -> (B, T, C)``."""

    def __init__(self, config: ModelConfig):
        super().__init__()
        g = lambda name, default=None: getattr(config, name, default)  # noqa: E731
        self.d_model = int(config.d_model)
        self.bias = bool(g("bias", False))
        heads = int(g("attn_h_total", 0) or g("n_head", 1) or 1)
        if heads <= 0:
            heads = max(1, int(g("n_head", 1)))
        self.h_total = heads
        if self.d_model % heads != 0:
            raise ValueError("d_model must be divisible by the total number of attention heads (attn_h_total)")
        if heads > 64:
            raise ValueError("the sm_100a kernels support at most 64 heads per layer")
        act = int(g("attn_h_active", 0))
        if act <= 0 or act > heads:
            act = max(1, min(4, heads))
        lo, hi = int(g("attn_h_active_min", 0) or 0), int(g("attn_h_active_max", 0) or 0)
        hi = max(1, min(hi if hi > 0 else min(16, heads), heads))
        lo = max(1, min(lo if lo > 0 else max(1, min(2, hi)), hi))
        self.h_active_min, self.h_active_max = lo, hi
        self.h_active = max(lo, min(act, hi))
        try:
            curve = float(g("attn_active_curve")) if g("attn_active_curve") is not None else 0.25
        except (TypeError, ValueError):
            curve = 0.25
        self.h_active_curve = curve if curve > 0.0 else 1.0
        self.force_dense_when_full = bool(g("attn_force_dense_when_full", False))
        self.d_head = self.d_model // heads
        self.use_rope = bool(g("attn_use_rope", True))
        base = _num(config, "attn_rope_base", 10000.0)
        self.rope_base = base if base > 0.0 else 10000.0
        if self.use_rope and self.d_head % 2 != 0:
            warnings.warn("Disabling RoPE because attention head dimension is not even.", RuntimeWarning)
            self.use_rope = False
        inv_freq = 1.0 / (self.rope_base ** (torch.arange(0, self.d_head, 2, dtype=torch.float32) / max(self.d_head, 1)))
        self.register_buffer("_rope_inv_freq", inv_freq, persistent=False)
        self._rope_cache: Dict[Tuple[str, int, str], Tuple[int, torch.Tensor, torch.Tensor]] = {}
        self._rope_retired: list = []   # outgrown tables, kept alive for graphs captured with them
        self._n_ctx_hint = int(g("n_ctx", 0) or 0)

        self.dropout = nn.Dropout(config.p_dropout)
        self.use_sdpa = bool(g("use_sdpa", True))
        self.router_reg_lambda = _num(config, "attn_router_lambda", 0.0) if g("attn_router_lambda", 0.0) else 0.0
        self.router_reg_beta = _num(config, "attn_router_beta", 1.0)
        self.router_reg_mode = str(g("attn_router_reg_mode", "entropy"))
        try:
            top_p = float(g("attn_router_top_p", 0.0))
        except (TypeError, ValueError):
            top_p = 0.0
        self.router_top_p = max(0.0, min(top_p if math.isfinite(top_p) else 0.0, 1.0))
        mode = str(g("attn_mode", "auto") or "auto").lower()
        self.mode_setting = mode if mode in {"auto", "subquad", "linear"} else "auto"

        # shortlist sizing
        self.linear_L = max(1, _num(config, "attn_linear_L", 512, int))
        sched = str(g("attn_linear_L_schedule", "fixed") or "fixed").lower()
        self.linear_L_schedule = sched if sched in {"fixed", "sqrt", "log", "mem_cap"} else "fixed"
        self.linear_L_base = max(1, _num(config, "attn_linear_L_base", self.linear_L, int))
        self.linear_L_min = max(1, _num(config, "attn_linear_L_min", min(64, self.linear_L_base), int))
        lmax = g("attn_linear_L_max", self.linear_L)
        self.linear_L_max = max(self.linear_L_min, int(lmax if lmax is not None else self.linear_L))
        self.linear_L_scale_init = max(0.1, _num(config, "attn_linear_L_scale", 1.0))
        self.linear_L_scale_max = _num(config, "attn_linear_L_scale_max", max(1.0, self.linear_L_scale_init))
        self._linear_scale_min = max(0.05, self.linear_L_min / max(1.0, self.linear_L_base))
        self._linear_L_scale_runtime = self.linear_L_scale_init
        self.linear_latency_shrink = min(max(_num(config, "attn_linear_latency_shrink", 0.8), 0.1), 0.99)
        self.linear_latency_growth = max(1.0, _num(config, "attn_linear_latency_growth", 1.05))
        mb = g("attn_linear_mem_budget_mb")
        self.linear_mem_budget_mb = float(mb) if mb is not None else None
        fl = max(0.0, min(1.0, _num(config, "attn_linear_piece_local_frac", 0.6)))
        fa = max(0.0, min(1.0, _num(config, "attn_linear_piece_anchor_frac", 0.3)))
        fp = max(0.0, min(1.0, float(g("attn_linear_piece_proto_frac", max(0.0, 1.0 - fl - fa)))))
        fl, fa, fp = self._normalise_fracs(fl, fa, fp)
        window = _num(config, "attn_linear_window", self.linear_L_base, int)
        self.linear_window_base = max(1, window if window > 0 else self.linear_L_base)
        self.linear_window = self.linear_window_base
        self.linear_anchor_stride = max(0, int(g("attn_linear_anchor_stride", g("attn_linear_anchors_every", 256)) or 0))
        self.linear_head_k = max(1, min(_num(config, "attn_linear_head_k", 2, int), heads))
        self.linear_switch_ctx = max(0, _num(config, "attn_linear_switch_ctx", 20000, int))
        lb = g("attn_linear_latency_budget_ms")
        self.linear_latency_budget_ms = float(lb) if lb is not None else None
        tokens = _policy_tokens(str(g("attn_linear_policy", "local+anchors") or "local+anchors").lower())
        self.linear_policy_tokens = tokens
        self.linear_use_anchors = bool(tokens & {"anchors", "anchor", "global"})
        self.linear_use_proto = bool(tokens & {"proto", "prototype", "semantic", "dna"})
        self.linear_use_local = bool(tokens & {"local", "window"}) or not (self.linear_use_anchors or self.linear_use_proto)
        fl = fl if self.linear_use_local else 0.0
        fa = fa if self.linear_use_anchors else 0.0
        fp = fp if self.linear_use_proto else 0.0
        if fl + fa + fp <= 0.0:
            fl, fa, fp = 1.0, 0.0, 0.0
        else:
            tot = fl + fa + fp
            fl, fa = fl / tot, fa / tot
            fp = max(0.0, 1.0 - fl - fa)
        self.linear_piece_local_frac, self.linear_piece_anchor_frac, self.linear_piece_proto_frac = fl, fa, fp
        self._linear_runtime: Optional[dict] = None
        self._linear_runtime_seq_len: Optional[int] = None
        self._linear_runtime_alpha: Optional[float] = None
        self._current_alpha: float = 0.0
        try:
            cutoff = float(g("attn_dense_alpha_cutoff", 0.0))
        except (TypeError, ValueError):
            cutoff = 0.25
        self.dense_alpha_cutoff = float(max(0.0, min(0.95, cutoff)))

        # key/value memory bank (aspa.py:389-416): non-persistent fp32 buffers, ring pointer per head
        self.memory_enabled = bool(g("attn_memory_enable", False)) and int(g("attn_memory_slots", 0) or 0) > 0
        self.memory_slots = int(g("attn_memory_slots", 0) or 0) if self.memory_enabled else 1
        self.memory_decay = float(max(0.0, min(1.0, float(g("attn_memory_decay", 0.9) or 0.9))))
        self.register_buffer("memory_keys", torch.zeros(heads, self.memory_slots, self.d_head, dtype=torch.float32),
                             persistent=False)
        self.register_buffer("memory_values", torch.zeros(heads, self.memory_slots, self.d_head, dtype=torch.float32),
                             persistent=False)
        self.register_buffer("memory_counts", torch.zeros(heads, self.memory_slots, dtype=torch.float32), persistent=False)
        self.register_buffer("memory_ptr", torch.zeros(heads, dtype=torch.long), persistent=False)
        self.quantize_sparse_int8 = bool(g("attn_quantize_int8", False))
        qmode = str(g("attn_quantize_int8_mode", "max") or "max").lower()
        self.quantize_sparse_int8_mode = qmode if qmode in {"max", "percentile", "ema_percentile"} else "max"
        self.quantize_sparse_int8_percentile = min(max(_num(config, "attn_quantize_int8_percentile", 1.0), 0.0), 1.0)
        self.quantize_sparse_int8_ema_decay = min(max(_num(config, "attn_quantize_int8_ema_decay", 0.9), 0.0), 0.9999)
        for name in ("_quant_ema_q", "_quant_ema_k", "_quant_ema_v"):
            self.register_buffer(name, torch.zeros(heads, dtype=torch.float32), persistent=False)
        self._quant_ema_flags = {"_quant_ema_q": False, "_quant_ema_k": False, "_quant_ema_v": False}

        seq_low, seq_high = _num(config, "attn_active_seq_low", 0, int), _num(config, "attn_active_seq_high", 0, int)
        if seq_low <= 0:
            seq_low = max(64, self.d_head)
        if seq_high <= 0:
            seq_high = int(g("n_ctx", 0) or (seq_low * 4))
        self.seq_low, self.seq_high = seq_low, max(seq_high, seq_low)
        hint = g("attn_small_seq_dense")
        try:
            dense_cut = int(hint) if hint is not None else max(0, self.seq_low // 2)
        except (TypeError, ValueError):
            dense_cut = max(0, self.seq_low // 2)
        self.small_seq_dense = max(0, dense_cut)
        self._density_ema: Optional[float] = None
        self._last_density: Optional[float] = None
        self._last_target_k: Optional[int] = None
        dt = g("attn_force_dense_threshold")
        dt = float(dt) if dt is not None else None
        self._dense_threshold: Optional[float] = dt if (dt is not None and dt > 0.0) else None

        gates = int(g("attn_gates", 0))
        if gates <= 0:
            gates = max(heads, self.h_active_max, self.h_active) * 2
        self.attn_gates = max(gates, heads, self.h_active_max)
        if self.attn_gates > 64:
            raise ValueError("the sm_100a router supports at most 64 gates")
        self.head_router = SwitchRouter(self.d_model, self.attn_gates, noise_std=float(g("attn_router_noise_std", 0.01)))
        idx = torch.arange(self.attn_gates, dtype=torch.long)
        gate_to_head = torch.clamp((idx * heads) // max(self.attn_gates, 1), 0, heads - 1)
        self.register_buffer("gate_to_head", gate_to_head, persistent=False)
        self.register_buffer("gate_to_head_onehot", F.one_hot(gate_to_head, num_classes=heads).to(torch.float32),
                             persistent=False)
        self.register_buffer("_gate_to_head_i32", gate_to_head.to(torch.int32), persistent=False)
        self._shortlist_alpha_override: Optional[float] = None

        self.qkv = nn.Linear(self.d_model, 3 * self.d_model, bias=self.bias)
        self.proj = nn.Linear(self.d_model, self.d_model, bias=self.bias)

        self.__dict__["_pending"] = None
        self.last_head_stats = None
        self._last_sparse_state = None
        self.last_aux_loss: Optional[torch.Tensor] = None
        self.last_router_reg: Optional[torch.Tensor] = None
        self._latency_ema: Optional[float] = None
        self.track_latency = bool(g("attn_track_latency", True))
        self.proto_enabled = bool(g("attn_proto_enable", False))
        self.proto_decay = float(g("attn_proto_decay", 0.97))
        self.proto_threshold = float(g("attn_proto_threshold", 0.25))
        self.proto_blend = float(g("attn_proto_blend", 0.6))
        self.proto_temp = float(max(g("attn_proto_temp", 0.2), 1e-3))
        self.proto_usage_boost = float(max(g("attn_proto_usage_boost", 0.0), 0.0))
        self.proto_init_scale = float(g("attn_proto_init_scale", 0.02))
        if self.proto_enabled:
            self.register_buffer("routing_prototypes",
                                 torch.randn(self.attn_gates, self.d_model, dtype=torch.float32) * self.proto_init_scale)
            self.register_buffer("routing_usage_ema", torch.zeros(self.attn_gates, dtype=torch.float32))
            self.register_buffer("routing_confidence", torch.zeros(self.attn_gates, dtype=torch.float32))
        else:
            self.routing_prototypes = None  # type: ignore[assignment]
            self.routing_usage_ema = None  # type: ignore[assignment]
            self.routing_confidence = None  # type: ignore[assignment]
        self._last_proto_stats: Optional[dict] = None
        self.token_sparse = bool(g("attn_token_sparse", False))
        self.token_keep_ratio_base = min(max(_num(config, "attn_token_keep_ratio", 1.0), 0.0), 1.0)
        self._token_keep_ratio_runtime: Optional[float] = None
        ks = str(g("attn_linear_token_keep_schedule", "sqrt") or "sqrt").lower()
        self.linear_token_keep_schedule = ks if ks in {"fixed", "sqrt", "log"} else "sqrt"
        self.linear_token_keep_ratio_min = min(max(_num(config, "attn_linear_token_keep_min_ratio", 0.2), 0.0),
                                               self.token_keep_ratio_base)
        self.linear_token_keep_ratio_ref = _num(config, "attn_linear_token_keep_ref", 2048, int)
        keep_min = max(0, _num(config, "attn_token_keep_min", 0, int))
        guard = max(0, _num(config, "attn_token_keep_guard", 1, int))
        self.token_keep_guard = guard
        self.token_keep_min = max(keep_min, guard if self.token_sparse else keep_min)
        self.token_keep_threshold = float(max(0.0, _num(config, "attn_token_keep_threshold", 0.0)))
        self._last_token_importance: Optional[torch.Tensor] = None
        self._last_token_mask: Optional[torch.Tensor] = None
        self._last_token_blend: Optional[torch.Tensor] = None
        self._last_token_similarity: Optional[torch.Tensor] = None
        self._last_shortlist_backend_info: Optional[Dict[str, object]] = None
        self._last_batch_size: Optional[int] = None
        self.last_head_consensus: Optional[torch.Tensor] = None
        # project queries / outputs for kept tokens only when at most 3/4 of the tokens can survive the token keep
        self.compact_projection = True
        # optional callable(layer), invoked as soon as token importance and the token mask of a call are launched
        self.after_token_keep = None
        self._identity_pack: Dict[Tuple[int, int, str], Tuple[torch.Tensor, torch.Tensor]] = {}
        self._pin: Optional[torch.Tensor] = None

    # float buffers keep fp32 whatever dtype the module is cast to (see module docstring)
    def _apply(self, fn, *args, **kwargs):
        keep = {n: b for n, b in self.named_buffers(recurse=False) if b is not None and b.dtype == torch.float32}
        super()._apply(fn, *args, **kwargs)
        for name, old in keep.items():
            new = getattr(self, name)
            if new.dtype != torch.float32:
                setattr(self, name, old.to(device=new.device))
        self._rope_cache.clear()
        self._identity_pack.clear()
        self._pin = None
        return self

    @staticmethod
    def _normalise_fracs(fl: float, fa: float, fp: float):
        tot = fl + fa + fp
        if tot <= 0.0:
            return 1.0, 0.0, 0.0
        fl, fa = fl / tot, fa / tot
        return fl, fa, max(0.0, 1.0 - fl - fa)

    # ---- host-side schedules (reference aspa.py:731-747, 844-930, 1037-1173) --------------------
    def _choose_active_k(self, seq_len: int) -> int:
        if seq_len <= self.seq_low:
            k = self.h_active_max
        elif seq_len >= self.seq_high:
            k = self.h_active_min
        else:
            r = float(seq_len - self.seq_low) / float(max(1, self.seq_high - self.seq_low))
            if self.h_active_curve != 1.0:
                r = max(0.0, min(1.0, r)) ** self.h_active_curve
            k = int(math.floor(self.h_active_max - r * (self.h_active_max - self.h_active_min) + 1e-6))
        k = max(self.h_active_min, min(k, self.h_active_max))
        self._last_target_k = k
        return k

    def _update_density(self, value: float) -> None:
        value = float(max(0.0, value))
        self._last_density = value
        self._density_ema = value if self._density_ema is None else 0.8 * self._density_ema + 0.2 * value

    def _density_threshold(self) -> Optional[float]:
        return self._dense_threshold

    def _set_linear_scale(self, value: float) -> None:
        lo = self._linear_scale_min
        self._linear_L_scale_runtime = float(min(max(value, lo), max(lo, self.linear_L_scale_max)))
        self._linear_runtime_seq_len = None
        self._linear_runtime_alpha = None

    def adjust_linear_L_scale(self, factor: float) -> None:
        """Multiply the shortlist-length scale (used by controllers)."""
        if factor == 0.0:
            return
        self._set_linear_scale(self._linear_L_scale_runtime * factor)

    def _linear_token_keep_ratio(self, seq_len: int) -> float:
        if not self.token_sparse:
            return self.token_keep_ratio_base
        ref, base, seq = max(1, self.linear_token_keep_ratio_ref), self.token_keep_ratio_base, max(1, int(seq_len))
        if self.linear_token_keep_schedule == "sqrt":
            r = base * math.sqrt(ref / float(seq))
        elif self.linear_token_keep_schedule == "log":
            r = base * (math.log2(ref + 1.0) / math.log2(seq + 1.0))
        else:
            r = base
        return float(max(min(base, self.linear_token_keep_ratio_min), min(base, r)))

    def _get_shortlist_alpha(self, seq_len: int) -> float:
        if self._shortlist_alpha_override is not None:
            return float(max(0.0, min(1.0, self._shortlist_alpha_override)))
        seq_len = int(max(1, seq_len))
        low = max(1, int(self.seq_low))
        high = max(low + 1, int(self.linear_switch_ctx)) if self.linear_switch_ctx > 0 else max(low + 1, seq_len)
        if seq_len <= low:
            return 0.0
        if seq_len >= high:
            return 1.0
        return float((seq_len - low) / (high - low))

    def _compute_cvt_alpha(self, seq_len: int) -> float:
        seq_len = int(max(1, seq_len))
        alpha = {"linear": 1.0, "subquad": 0.0}.get(self.mode_setting)
        if alpha is None:
            alpha = self._get_shortlist_alpha(seq_len)
        if self.linear_latency_budget_ms is not None and self._latency_ema is not None:
            budget, lat = self.linear_latency_budget_ms, self._latency_ema
            if lat > budget * 1.05:
                if self._linear_L_scale_runtime > self._linear_scale_min + 1e-3:
                    self.adjust_linear_L_scale(self.linear_latency_shrink)
                alpha = 1.0
            elif lat < budget * 0.80 and seq_len < max(1, self.linear_switch_ctx):
                if self._linear_L_scale_runtime < self.linear_L_scale_max:
                    self.adjust_linear_L_scale(self.linear_latency_growth)
                alpha = min(alpha, 0.0)
        if self.linear_switch_ctx > 0:
            if self._current_alpha >= 0.95 and seq_len >= max(1, int(self.linear_switch_ctx * 0.75)):
                alpha = max(alpha, 0.95)
            if seq_len >= self.linear_switch_ctx:
                alpha = 1.0
        return float(max(0.0, min(1.0, alpha)))

    def set_shortlist_alpha(self, value: float) -> None:
        """Externally pin the dense<->shortlist slider (0 = dense, 1 = linear)."""
        self._shortlist_alpha_override = float(max(0.0, min(1.0, value)))
        self._linear_runtime = None
        self._linear_runtime_seq_len = None
        self._linear_runtime_alpha = None

    def _compute_effective_linear_params(self, seq_len: int, batch_size: Optional[int], alpha: float) -> dict:
        seq_len = max(1, int(seq_len))
        coeff = float(max(1.0, self.linear_L_base))
        sched = self.linear_L_schedule
        if sched == "sqrt":
            base_val = coeff * math.sqrt(float(seq_len))
        elif sched == "log":
            base_val = coeff * math.log2(float(seq_len) + 1.0)
        elif sched == "mem_cap" and self.linear_mem_budget_mb:
            heads_est = max(1, int(getattr(self, "_last_target_k", self.linear_head_k)))
            batch_est = max(1, int(batch_size) if batch_size is not None else 1)
            denom = heads_est * batch_est * seq_len * max(1, self.d_head) * 8
            cap_mem = int(self.linear_mem_budget_mb * 1024 * 1024 // denom) if denom > 0 else self.linear_L_max
            base_val = max(1, min(cap_mem, self.linear_L_max))
        else:
            base_val = coeff
        clampL = lambda v: max(self.linear_L_min, min(self.linear_L_max, v))  # noqa: E731
        eff = clampL(int(math.ceil(self._linear_L_scale_runtime * max(1.0, base_val))))
        window = min(self.linear_window_base, eff)
        dense_cap = clampL(int(min(seq_len, max(self.linear_L_min, self.linear_window_base + seq_len // 32))))
        eff = clampL(int(alpha * eff + (1.0 - alpha) * dense_cap))
        window_dense = max(1, min(seq_len, max(self.linear_window_base, seq_len // 8)))
        window = max(1, min(eff, int(alpha * window + (1.0 - alpha) * window_dense)))
        use = (self.linear_use_local, self.linear_use_anchors, self.linear_use_proto)
        dense_w = (0.85, 0.10, 0.05)
        target_w = (self.linear_piece_local_frac, self.linear_piece_anchor_frac, self.linear_piece_proto_frac)
        w = [(1.0 - alpha) * (dense_w[i] if use[i] else 0.0) + alpha * (target_w[i] if use[i] else 0.0) for i in range(3)]
        tw = w[0] + w[1] + w[2]
        if tw <= 0.0:
            w, tw = [1.0, 0.0, 0.0], 1.0
        wl, wa = w[0] / tw, w[1] / tw
        weights = (wl, wa, max(0.0, 1.0 - wl - wa))
        caps = [int(round(eff * weights[i])) if use[i] else 0 for i in range(3)]
        total = sum(caps)
        if total > eff and total > 0:
            caps = [int(max(0, math.floor(c * (eff / total)))) for c in caps]
            total = sum(caps)
        remaining = eff - total
        for i in range(3):
            if remaining <= 0:
                break
            if use[i]:
                caps[i] += 1
                remaining -= 1
        if remaining > 0:
            caps[0 if use[0] else 1 if use[1] else 2] += remaining
        if use[0]:
            caps[0] = min(caps[0], window)
            if caps[0] <= 0 and eff > 0:
                caps[0] = min(window, max(1, eff // 4))
        return {"effective_L": eff, "local_cap": max(0, int(caps[0])), "anchor_cap": max(0, int(caps[1])),
                "proto_cap": max(0, int(caps[2])), "window": max(1, int(window)), "shortlist_alpha": float(alpha)}

    def _prepare_linear_runtime(self, seq_len: int, batch_size: Optional[int], alpha: float) -> dict:
        if (self._linear_runtime is not None and self._linear_runtime_seq_len == seq_len
                and self._linear_runtime_alpha is not None and abs(self._linear_runtime_alpha - float(alpha)) < 1e-4):
            return self._linear_runtime
        alpha = float(max(0.0, min(1.0, alpha)))
        p = self._compute_effective_linear_params(seq_len, batch_size, alpha)
        self.linear_L, self.linear_window = p["effective_L"], p["window"]
        rt = dict(p, anchor_stride=self.linear_anchor_stride)
        self._linear_runtime, self._linear_runtime_seq_len, self._linear_runtime_alpha = rt, seq_len, alpha
        return rt

    # ---- device helpers ---------------------------------------------------------------------------
    def _rope_factors(self, seq_len: int, device: torch.device, dtype: torch.dtype):
        """fp32 (T, D/2) cos/sin tables whose values are rounded to ``dtype`` (reference aspa.py:576-604)."""
        if seq_len <= 0:
            raise ValueError("RoPE requires a positive sequence length.")
        key = (device.type, int(device.index) if device.index is not None else -1, str(dtype))
        cached = self._rope_cache.get(key)
        if cached is None or cached[0] < seq_len:
            # A captured CUDA graph holds the raw address of the table it was captured with, so a table that is
            # outgrown is retired, never freed: it stays alive for as long as the layer does.  The first table
            # already spans the configured context, which makes growth the exception.
            if cached is not None:
                self._rope_retired.append(cached)
            span = max(seq_len, self._n_ctx_hint) if cached is None else seq_len
            span = min(span, max(seq_len, 1 << 20))
            cos, sin = ops.rope_table(self._rope_inv_freq.to(device), span, self.d_head, dtype)
            cached = (span, cos, sin)
            self._rope_cache[key] = cached
        return cached[1][:seq_len], cached[2][:seq_len]

    def _identity_rows(self, B: int, T: int, device: torch.device):
        key = (B, T, str(device))
        hit = self._identity_pack.get(key)
        if hit is None:
            HT = B * self.h_total
            hit = (torch.arange(0, (HT + 1) * T, T, device=device, dtype=torch.int32),
                   torch.arange(T, device=device, dtype=torch.int32).repeat(HT))
            self._identity_pack = {key: hit}
        return hit

    def _project_qkv(self, x: torch.Tensor, want_amax: bool = False, q_keep: Optional[torch.Tensor] = None):
        B, T, _ = x.shape
        qkv = self.qkv(x)
        cos = sin = None
        if self.use_rope:
            cos, sin = self._rope_factors(T, x.device, x.dtype)
        return ops.rope_relayout(qkv.contiguous(), self.h_total, self.d_head, cos, sin, want_amax,
                                 None if want_amax else q_keep,
                                 q_fraction=float(self._token_keep_ratio_runtime or 1.0))

    def _fork_kv_projection(self, x: torch.Tensor) -> dict:
        """K/V projection + RoPE/relayout of every token on a second stream.  Nothing in it depends on the routing
        chain (router, token keep, head choice, packing), whose kernels are small or latency-bound and leave most of
        the GPU idle; the two run side by side and meet before the attention.  The outputs are allocated on the
        calling stream, so the allocator's stream bookkeeping stays with the caller.  No head-major copies are made:
        the attention kernels read keys and values out of the (B*T, 2, H, D) projection through element strides."""
        B, T, C = x.shape
        H, D = self.h_total, self.d_head
        dev = x.device
        w, b = self.qkv.weight, self.qkv.bias
        kv = torch.empty((B * T, 2 * C), dtype=x.dtype, device=dev)
        cos = sin = None
        k_heads = None
        if self.use_rope:
            cos, sin = self._rope_factors(T, dev, x.dtype)
            if K_HEAD_MAJOR:
                k_heads = torch.empty((B * H, T, D), dtype=x.dtype, device=dev)
        main = torch.cuda.current_stream()
        # One priority level below the caller's stream when that one is elevated: the GEMM fills the GPU, and the
        # short kernels of the calling stream then take SMs as its blocks retire instead of waiting for all of them.
        # Still above priority 0, where bulk copies run.
        prio = min(0, int(main.priority) + 1)
        side = _SIDE_STREAMS.get((str(dev), prio))
        if side is None:
            side = _SIDE_STREAMS[(str(dev), prio)] = torch.cuda.Stream(device=dev, priority=prio)
        if ops.SERIAL_STREAMS:
            side = main
        ready, done = torch.cuda.Event(), torch.cuda.Event()
        ready.record(main)
        side.wait_event(ready)
        with torch.cuda.stream(side):
            if b is None:
                torch.mm(x.view(B * T, C), w[C:].t(), out=kv)
            else:
                torch.addmm(b[C:], x.view(B * T, C), w[C:].t(), out=kv)
            if cos is not None:  # keys are rotated where the projection left them; values are used as they are
                ops.rope_inplace(kv.view(-1), B * T, T, 2 * C, H, D, cos, sin, heads_out=k_heads)
            done.record(side)
        flat = kv.view(-1)
        if k_heads is not None:
            layout = N.KVLayout(k_batch=H * T * D, k_head=T * D, k_token=D, v_batch=T * 2 * C, v_head=D, v_token=2 * C)
            return {"k": k_heads.view(-1), "v": flat[C:], "kv": kv, "layout": layout, "done": done}
        layout = N.KVLayout(k_batch=T * 2 * C, k_head=D, k_token=2 * C, v_batch=T * 2 * C, v_head=D, v_token=2 * C)
        return {"k": flat, "v": flat[C:], "kv": kv, "layout": layout, "done": done}

    def _fork_qkv_quantize(self, x: torch.Tensor) -> dict:
        """Fused QKV projection, RoPE, head-major split and per-head INT8 quantisation of one call on the second
        stream (see ``_fork_kv_projection``).  The results are allocated on the calling stream, where they are used."""
        B, T, C = x.shape
        H, D = self.h_total, self.d_head
        dev = x.device
        cos = sin = None
        if self.use_rope:
            cos, sin = self._rope_factors(T, dev, x.dtype)
        main = torch.cuda.current_stream()
        prio = min(0, int(main.priority) + 1)
        side = _SIDE_STREAMS.get((str(dev), prio))
        if side is None:
            side = _SIDE_STREAMS[(str(dev), prio)] = torch.cuda.Stream(device=dev, priority=prio)
        if ops.SERIAL_STREAMS:
            side = main
        ready, done = torch.cuda.Event(), torch.cuda.Event()
        ready.record(main)
        side.wait_event(ready)
        pack = ops.rope_quantize_outputs(B, T, H, D, dev)   # on the calling stream, where they are used
        with torch.cuda.stream(side):
            ops.rope_quantize(self.qkv(x).contiguous(), H, D, cos, sin, out=pack)
            done.record(side)
        return {"pack": pack, "done": done}

    def _percentile_bases(self, tensors, amax: torch.Tensor) -> torch.Tensor:
        """Per-head quantisation bases of q, k, v in the "percentile" and "ema_percentile" modes (reference
        aspa.py:1329-1356): the percentile of |x| (the maximum when the percentile is 0 or the quantile is 0), and in
        the EMA mode its running average, which starts from the maximum of the first call (or of any call whose head
        count differs from the stored one)."""
        pct = float(self.quantize_sparse_int8_percentile)
        out = []
        for i, (t_, name) in enumerate(zip(tensors, ("_quant_ema_q", "_quant_ema_k", "_quant_ema_v"))):
            base = amax[i].contiguous() if pct <= 0.0 else ops.head_abs_quantile(t_, pct, amax[i].contiguous())
            if self.quantize_sparse_int8_mode == "ema_percentile":
                ema = getattr(self, name)
                if ema is None or ema.numel() != base.numel() or not self._quant_ema_flags.get(name, False):
                    ema = amax[i]
                base = self.quantize_sparse_int8_ema_decay * ema.to(torch.float32) + \
                    (1.0 - self.quantize_sparse_int8_ema_decay) * base
                setattr(self, name, base.detach())
                self._quant_ema_flags[name] = True
            out.append(base)
        return torch.stack(out)

    def _project_compact_q(self, x: torch.Tensor, compact: dict) -> torch.Tensor:
        """q for the kept tokens only; the q rows of dropped tokens stay unwritten."""
        B, T, C = x.shape
        H, D = self.h_total, self.d_head
        w, b = self.qkv.weight, self.qkv.bias
        if compact["count"] is None:   # -1 padded list: the gather writes zeros into the unused slots itself
            x_rows = ops.gather_rows(x.view(B * T, C), compact["idx"], None, compact["slots"])
        else:
            x_rows = ops.gather_rows(x.view(B * T, C), compact["idx"], compact["count"], compact["slots"],
                                     out=torch.zeros((compact["slots"], C), dtype=x.dtype, device=x.device))
        q_rows = F.linear(x_rows, w[:C], None if b is None else b[:C])
        cos = sin = None
        if self.use_rope:
            cos, sin = self._rope_factors(T, x.device, x.dtype)
        return ops.rope_rows_q(q_rows, compact["idx"], compact["count"], B, T, H, D, cos, sin)

    @property
    def last_head_consensus(self) -> Optional[torch.Tensor]:
        """(B, T, C) attention output before the projection (eval mode only, aspa.py:1849); rebuilt on first use
        when the call kept it as rows of kept tokens."""
        pending = self.__dict__.get("_consensus_pending")
        if pending is not None:
            rows, slot_of, mask, (B, T, C) = pending
            self.__dict__["_consensus_value"] = ops.scatter_rows_fill(rows, slot_of, mask, None, B * T).view(B, T, C)
            self.__dict__["_consensus_pending"] = None
        return self.__dict__.get("_consensus_value")

    @last_head_consensus.setter
    def last_head_consensus(self, value: Optional[torch.Tensor]) -> None:
        self.__dict__["_consensus_pending"] = None
        self.__dict__["_consensus_value"] = value

    def _check_input(self, x: torch.Tensor) -> None:
        if not x.is_cuda:
            raise RuntimeError("proteus_flux_attention_b200 has no CPU path: move the module and input to a CUDA device")
        if x.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("ASPA kernels take float32 or bfloat16 activations")
        if self.qkv.weight.dtype != x.dtype:
            raise TypeError(f"activation dtype {x.dtype} does not match the layer weights ({self.qkv.weight.dtype})")
        if self.training and self.dropout.p > 0.0:
            raise NotImplementedError("attention dropout is not implemented in the sm_100a kernels (forward-only build)")

    def _forward_dense_fastpath(self, x: torch.Tensor) -> torch.Tensor:
        """Causal attention over every head for short sequences (reference aspa.py:1365-1440)."""
        B, T, C = x.shape
        q, k, v, _ = self._project_qkv(x)
        offs, tok = self._identity_rows(B, T, x.device)
        out = torch.zeros((B, T, C), dtype=x.dtype, device=x.device)
        attention_packed(q, k, v, row_offsets=offs, token_idx=tok, max_rows=T, total_rows=B * self.h_total * T,
                         H=self.h_total, out=out, out_layout=N.OUT_TOKEN_MAJOR)
        y = self.dropout(self.proj(out))
        thr = None if self._dense_threshold is None else float(self._dense_threshold)
        self._last_target_k = self.h_total
        self._last_sparse_state = {"mode": "dense_fastpath", "backend": BACKEND_NAME, "max_rows": T, "density": 1.0,
                                   "target_k": self.h_total, "force_dense_threshold": thr,
                                   "cutoff": int(self.small_seq_dense), "quantized": False, "token_keep_fraction": 1.0}
        self._update_density(1.0)
        self.last_head_stats = {
            "top_k": int(self.h_total), "mean_gate_prob": 1.0, "router_entropy": 0.0,
            "mean_active_per_token": float(self.h_total), "unique_heads": int(self.h_total), "active_fraction": 1.0,
            "max_active_rows": int(T), "max_active_density": 1.0, "target_k": int(self.h_total), "seq_len": int(T),
            "active_min": int(self.h_active_min), "active_max": int(self.h_active_max), "force_dense_threshold": thr,
            "active_curve": float(self.h_active_curve), "token_keep_fraction": 1.0,
            "router_top_p": float(self.router_top_p), "nucleus_k": int(self.h_total), "top_a_consensus": True}
        self.last_router_reg = None
        return y

    # ---- telemetry: filled from one small host record, lazily when the call did not need it ------------------
    @property
    def last_head_stats(self) -> Optional[dict]:
        self._materialize()
        return self.__dict__.get("_head_stats_value")

    @last_head_stats.setter
    def last_head_stats(self, value: Optional[dict]) -> None:
        self.__dict__["_head_stats_value"] = value

    @property
    def _last_sparse_state(self) -> Optional[dict]:
        self._materialize()
        return self.__dict__.get("_sparse_state_value")

    @_last_sparse_state.setter
    def _last_sparse_state(self, value: Optional[dict]) -> None:
        self.__dict__["_sparse_state_value"] = value

    def _materialize(self) -> None:
        """Turn the pending host record of the last call into the telemetry dictionaries (waits for its copy)."""
        ctx = self.__dict__.get("_pending")
        if ctx is None:
            return
        self.__dict__["_pending"] = None
        if ctx["event"] is not None:
            ctx["event"].synchronize()
        else:
            torch.cuda.synchronize(ctx["device"])
        info = self._decode_record(ctx)
        self._publish(ctx, info, force_dense=False, dense_reason=None, exec_mode=ctx["exec_mode"])

    def check_previous_call(self) -> None:
        """A call that runs without waiting for the host (lazy telemetry, graph replay) cannot report an expired
        device-side wait of its own router; the pinned record it left behind can.  Called at the start of the next
        call and by ``CapturedLayerCall``: reads one word of pinned memory, never waits; raises ``DeviceWaitTimeout``
        (after clearing the device word) if the previous call's router gave up, because what that call returned was
        built on unwritten gate probabilities."""
        ctx = self.__dict__.get("_pending")
        if ctx is None or ctx.get("pin") is None or torch.cuda.is_current_stream_capturing():
            return
        if ctx["event"] is not None and not ctx["event"].query():
            return
        slot = ctx["B"] * self.h_total + 1 + ctx["B"] + 7
        if slot < ctx["pin"].numel() and int(ctx["pin"][slot]) != 0:
            ops.check_router_status(ctx["device"])

    def _decode_record(self, ctx: dict) -> dict:
        rec = ctx["pin"].tolist()
        B, T, H = ctx["B"], ctx["T"], self.h_total
        nbh = B * H
        offs = [int(v) for v in rec[: nbh + 1]]
        kept = [int(v) for v in rec[nbh + 1: nbh + 1 + B]]
        p0 = nbh + 1 + B
        counts = [offs[i + 1] - offs[i] for i in range(nbh)]
        if int(rec[p0 + 7]) != 0:
            ops.check_router_status(ctx["device"])   # raises DeviceWaitTimeout and clears the device word
            raise RuntimeError("the tensor-core router reported an expired device-side wait; its outputs are invalid")
        return {"offs": offs, "kept": kept, "topk": int(rec[p0]), "adaptive": int(rec[p0 + 1]), "score_sum": rec[p0 + 2],
                "entropy_sum": rec[p0 + 3], "sim_sum": rec[p0 + 4], "bs_sum": rec[p0 + 5], "bs_pos": rec[p0 + 6],
                "counts": counts, "total_rows": offs[-1], "max_rows": max(counts) if counts else 0,
                "active_heads": sum(1 for c in counts if c > 0),
                "keep_fraction": float(sum(kept)) / float(B * T) if self.token_sparse else 1.0}

    def _publish(self, ctx: dict, info: dict, *, force_dense: bool, dense_reason: Optional[str], exec_mode: str) -> None:
        """Build ``last_head_stats`` / ``_last_sparse_state`` exactly as the reference fills them (aspa.py:1688-1915)."""
        B, T, H = ctx["B"], ctx["T"], self.h_total
        nbh, alpha, dev = B * H, ctx["alpha"], ctx["device"]
        topk, counts, total_rows, max_rows = info["topk"], info["counts"], info["total_rows"], info["max_rows"]
        density = float(max_rows) / float(max(1, T))
        thr = self._density_threshold()
        if ctx.get("lazy"):
            self._last_target_k = topk
            self._update_density(density)
            if ctx["use_proto"]:
                n_tok = float(B * T)
                self._last_proto_stats = {"max_sim_mean": info["sim_sum"] / n_tok, "blend_mean": info["bs_sum"] / n_tok,
                                          "active_tokens": int(round(info["bs_pos"]))}
        common = {"density": density, "target_k": int(topk), "force_dense_threshold": None if thr is None else float(thr),
                  "quantized": False, "token_keep_fraction": float(info["keep_fraction"]),
                  "mode_setting": self.mode_setting, "mode_selected": f"cvt(alpha={alpha:.2f})",
                  "shortlist_alpha": float(alpha)}
        if force_dense:
            mode_str = "dense_alpha" if dense_reason == "alpha" else ("dense" if info["active_heads"] == nbh else "dense_auto")
            exec_mode = mode_str
            state = dict(common, mode=mode_str, backend=BACKEND_NAME, max_rows=max_rows, dense_reason=dense_reason)
        elif total_rows == 0:
            state = dict(common, mode="dense", backend="not_invoked", max_rows=max_rows, dense_reason=None)
        else:
            active = [i for i, c in enumerate(counts) if c > 0]
            offs = info["offs"]
            state = dict(common, mode="shortlist", backend=BACKEND_NAME, max_rows=int(max_rows), cache_hit=False,
                         token_idx=ctx["token_idx"][:total_rows], row_offsets_all=ctx["row_offsets"],
                         active_head_indices=torch.tensor(active, dtype=torch.long, device=dev),
                         row_offsets=torch.tensor([offs[i] for i in active] + [total_rows], dtype=torch.int32, device=dev),
                         linear_L=int(self.linear_L), linear_window=int(self.linear_window),
                         linear_anchor_stride=int(self.linear_anchor_stride), linear_shortlist_backend=BACKEND_NAME)
        n_tok = float(B * T)
        stats = {
            "top_k": int(topk), "mean_gate_prob": float(info["score_sum"] / max(float(total_rows), 1.0)),
            "router_entropy": float(info["entropy_sum"] / n_tok), "mean_active_per_token": float(total_rows / n_tok),
            "unique_heads": len({i % H for i, c in enumerate(counts) if c > 0}),
            "active_fraction": float(total_rows / (n_tok * H)), "max_active_rows": int(max_rows),
            "max_active_density": float(density), "target_k": int(topk), "seq_len": int(T),
            "active_min": int(self.h_active_min), "active_max": int(self.h_active_max),
            "force_dense_threshold": None if thr is None else float(thr), "active_curve": float(self.h_active_curve),
            "token_keep_fraction": float(info["keep_fraction"]), "mode": exec_mode,
            "mode_selected": ctx.get("label") or f"cvt(alpha={alpha:.2f})", "shortlist_alpha": float(alpha),
            "router_top_p": float(self.router_top_p), "nucleus_k": int(info["adaptive"]), "top_a_consensus": True,
            "mode_setting": self.mode_setting}
        if dense_reason is not None:
            stats["dense_reason"] = dense_reason
        if alpha > 0.0:
            stats.update(linear_L=int(self.linear_L), linear_window=int(self.linear_window),
                         linear_anchor_stride=int(self.linear_anchor_stride), linear_shortlist_backend=BACKEND_NAME)
        if self._last_proto_stats:
            stats["proto"] = dict(self._last_proto_stats)
            stats["dna"] = dict(self._last_proto_stats)
        if ctx.get("label"):
            state["mode_selected"] = ctx["label"]
        self.__dict__["_head_stats_value"] = stats
        self.__dict__["_sparse_state_value"] = state

    # ---- forward ------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self._check_input(x)
        x = x.contiguous()
        B, T, C = x.shape
        dev = x.device
        H, D, G = self.h_total, self.d_head, self.attn_gates
        self.check_previous_call()
        self.__dict__["_pending"] = None
        self.last_aux_loss = None
        self._last_token_importance = self._last_token_mask = self._last_token_blend = None
        if not self.proto_enabled:
            self._last_token_similarity = None
        t_start = ev0 = None
        if self.track_latency:
            ev0 = torch.cuda.Event(enable_timing=True)
            ev0.record()
            t_start = time.perf_counter()
        self._last_batch_size = B

        if self.small_seq_dense and T <= self.small_seq_dense:
            y = self._forward_dense_fastpath(x)
            self._finalize_latency("dense_fastpath", ev0, t_start)
            return y

        alpha = self._compute_cvt_alpha(T)
        self._current_alpha = alpha
        if self.token_sparse:
            ratio = (1.0 - alpha) * float(self.token_keep_ratio_base) + alpha * float(self._linear_token_keep_ratio(T))
            self._token_keep_ratio_runtime = float(max(0.0, min(1.0, ratio)))
        else:
            self._token_keep_ratio_runtime = None

        # host-side arithmetic of the token keep (aspa.py:806-829): how many tokens can survive is known before any
        # kernel runs, which lets the K/V projection start on a second stream beside the routing chain
        keep_all = need = guard = 0
        kept_bound = T          # upper bound on kept tokens per batch element
        bound_known = True
        if self.token_sparse:
            ratio = float(self._token_keep_ratio_runtime)
            keep_all = ratio >= 0.999 and self.token_keep_threshold <= 0.0
            if not keep_all:
                guard = min(max(0, self.token_keep_guard), T)
                min_keep = max(min(max(0, self.token_keep_min), T), guard)
                need = _py_round_f32(ratio * T)
                if min_keep > 0:
                    need = max(need, min_keep)
                need = max(1, min(need, T))
                kept_bound = min(T, max(need, guard) + guard)
                bound_known = self.token_keep_threshold <= 0.0
        use_quant = bool(self.quantize_sparse_int8 and not self.training)
        # Queries and outputs only exist for kept tokens (every path below computes rows of kept tokens only, and
        # the rows of dropped tokens reach the output projection as zeros): with a known bound on the kept count
        # the query projection, the attention output and the output projection run on the kept rows alone.
        # INT8 scales are taken over the queries of every token (aspa.py:1328), so that mode projects them all.
        will_compact = (self.compact_projection and self.token_sparse and not keep_all and bound_known
                        and not use_quant and 4 * kept_bound <= 3 * T and not self.training)
        # Started before the router: launched after it, the projection's CTAs starve the cluster launches of the token
        # keep (158 us instead of 40 us per call).
        kv_fork = self._fork_kv_projection(x) if will_compact else None
        # INT8 shortlist that can never turn dense (alpha >= 0.95): the fused projection and its rotate / split /
        # quantise passes do not depend on the routing either, so they take the second stream the same way
        fuse_quant = (use_quant and not will_compact and alpha >= 0.95 and x.dtype == torch.bfloat16 and D % 8 == 0
                      and not self.memory_enabled
                      and (self.quantize_sparse_int8_mode == "max" or self.quantize_sparse_int8_percentile >= 1.0))
        quant_fork = self._fork_qkv_quantize(x) if fuse_quant else None

        # 1. router
        x2d = x.view(B * T, C)
        proto_hat = conf_eps = usage_bias = None
        use_proto = self.proto_enabled and self.routing_prototypes is not None
        if use_proto:
            proto_hat = ops.normalize_rows(self.routing_prototypes)
            if self.routing_confidence is not None:
                conf_eps = (self.routing_confidence + 1e-6).to(torch.float32)
            if self.proto_usage_boost > 0.0 and self.routing_usage_ema is not None:
                usage_bias = torch.softmax(-(self.routing_usage_ema + 1e-6), dim=0).to(torch.float32)
        gate, imp, sim, bs, proto_sums = ops.router_fwd(
            x2d, self.head_router.linear.weight.contiguous(), proto_hat, conf_eps, usage_bias, temp=self.proto_temp,
            threshold=self.proto_threshold, span=max(1e-6, 1.0 - self.proto_threshold), blend=self.proto_blend,
            usage_boost=self.proto_usage_boost, raw_stats=True)
        self._last_token_similarity = sim.view(B, T) if sim is not None else None
        self._last_token_blend = bs.view(B, T) if bs is not None else None
        self._last_token_importance = imp.view(B, T)
        # 2. token keep
        token_mask_u8 = kept = compact = None
        if self.token_sparse:
            if keep_all:
                token_mask_u8 = torch.ones((B, T), dtype=torch.uint8, device=dev)
            elif will_compact and T <= ops.TOKEN_COMPACT_MAX_T:
                # the keep also emits the ordered list of kept tokens (row b owns slots [b*kept_bound, ...), -1 padded)
                token_mask_u8, kept, kept_idx, slot_of = ops.token_select_compact(
                    self._last_token_importance, need, self.token_keep_threshold, guard, kept_bound)
                compact = {"idx": kept_idx, "slot_of": slot_of, "count": None, "slots": B * kept_bound,
                           "mask": token_mask_u8.view(-1)}
            else:
                token_mask_u8, kept = ops.token_select(self._last_token_importance, need, self.token_keep_threshold, guard)
            self._last_token_mask = token_mask_u8.view(torch.bool)
        if self.after_token_keep is not None:  # importance and mask are final: work that only needs them can fork here
            self.after_token_keep(self)

        # 3. head budget and per-token head choice
        dense_k = self._choose_active_k(T)
        k_dev = None
        if self.router_top_p > 0.0 and dense_k > self.h_active_min and dense_k > 1:
            k_dev = ops.head_budget(gate, self._gate_to_head_i32, H, top_p=self.router_top_p, dense_k=dense_k,
                                    h_min=self.h_active_min, linear_head_k=self.linear_head_k, alpha=alpha)
        k_host = adaptive_host = 0
        if k_dev is None:
            adaptive_host = dense_k
            lin_k = max(1, min(adaptive_host, self.linear_head_k))
            k_host = min(adaptive_host, max(1, int(round((1.0 - alpha) * float(adaptive_host) + alpha * float(lin_k)))))
        k_bound = k_host if k_dev is None else dense_k
        if k_dev is None:
            self._last_target_k = k_host
        capacity = B * T * dense_k
        head_bits, top_idx, top_score, head_partials, row_offsets, token_idx = ops.head_select_pack(
            gate, self._gate_to_head_i32, B, T, H, k_host=k_host, k_dev=k_dev, kmax=dense_k,
            token_mask=token_mask_u8.view(-1) if token_mask_u8 is not None else None, capacity=capacity)

        # 4. one statistics record to the host: [row offsets | kept per batch | k, adaptive | score, entropy sums |
        #    prototype sums | router status], built by one kernel, copied asynchronously and read when (and if) needed
        rec_dev = ops.stats_record(row_offsets, kept, B, float(T), k_dev, float(k_host), head_partials, proto_sums,
                                   ops.router_status(dev))
        if self._pin is None or self._pin.numel() != rec_dev.numel():
            self._pin = torch.empty(rec_dev.numel(), dtype=torch.float64, pin_memory=True)
        self._pin.copy_(rec_dev, non_blocking=True)
        capturing = torch.cuda.is_current_stream_capturing()
        ev_rec = None
        if not capturing:  # inside a CUDA-graph capture the record is read after the replay's stream has drained
            ev_rec = torch.cuda.Event()
            ev_rec.record()
        ctx = {"B": B, "T": T, "alpha": alpha, "device": dev, "pin": self._pin, "event": ev_rec, "use_proto": use_proto,
               "token_idx": token_idx, "row_offsets": row_offsets, "exec_mode": "shortlist"}

        # Work that needs neither q, k, v nor the record goes first: while the projection is still running on the
        # second stream this stream would otherwise only wait for it.  The prototype EMA (runs in eval mode too,
        # aspa.py:1917; a decay of exactly 1 leaves the state untouched; the router has read the prototypes already),
        # the block lists of the prototype picks, the zero fill of the attention output.
        if use_proto and self.routing_usage_ema is not None and self.routing_confidence is not None \
                and self.proto_decay != 1.0:
            self._last_proto_updated = ops.proto_ema_update(x2d, gate, self.proto_decay, self.routing_prototypes,
                                                            self.routing_usage_ema, self.routing_confidence)
        runtime = self._prepare_linear_runtime(T, B, alpha)
        plan_args = self._plan_shape(runtime, T, sim is not None)
        # Can this call turn dense at all?  Not at alpha >= 0.95 (aspa.py:1636-1639); below that the reference goes
        # dense on alpha <= cutoff (without INT8), on a row density at or above the threshold, or when every
        # (head, token) row is active (aspa.py:1625-1635) - and with host-side bounds on the kept tokens and on k
        # all three can often be ruled out before any kernel has run.  Then the call needs no row counts on the host:
        # it sizes its grids from the bounds and can be captured into a CUDA graph.
        thr = self._density_threshold()
        never_dense = alpha >= 0.95 or (
            (alpha > self.dense_alpha_cutoff or self.quantize_sparse_int8)
            and (thr is None or float(kept_bound) / float(max(1, T)) < thr)
            and (kept_bound < T or k_bound < H or not self.force_dense_when_full))
        lazy = never_dense and bound_known and plan_args is not None
        early_lists = None
        if plan_args is not None and plan_args[2] > 0:
            early_lists = ops.proto_plan(self._last_token_similarity.contiguous(), plan_args[2])
        out_early = None if will_compact else torch.zeros((B, T, C), dtype=x.dtype, device=dev)
        early_plan = early_regroup = None
        if plan_args is not None:
            early_plan = ops.make_plan(plan_args[0], plan_args[1], runtime["anchor_stride"], plan_args[2],
                                       *(early_lists if early_lists is not None else (None, None)))
            if lazy:   # row counts are host-side bounds: the anchor regrouping can go now too
                early_regroup = ops.regroup_rows(early_plan, torch.int8 if use_quant else x.dtype, B * H, T, D,
                                                 row_offsets, token_idx, B * kept_bound * k_bound)

        # 5. projection + RoPE + head-major relayout (does not depend on the record)
        kv_layout = quant_pack = None
        if will_compact:
            if compact is None:  # rows too long for the fused keep: compact the mask separately
                n_slots = B * kept_bound
                kept_idx, slot_of, kept_cnt = ops.compact_mask(token_mask_u8.view(-1), n_slots)
                compact = {"idx": kept_idx, "slot_of": slot_of, "count": kept_cnt, "slots": n_slots,
                           "mask": token_mask_u8.view(-1)}
            q = self._project_compact_q(x, compact)
            k, v, kv_layout = kv_fork["k"], kv_fork["v"], kv_fork["layout"]
            torch.cuda.current_stream().wait_event(kv_fork["done"])
            amax = None
        elif quant_fork is not None:
            # rotate, split and quantise straight from the fused projection; the bf16 head-major q, k, v are never
            # materialised
            quant_pack = quant_fork["pack"]
            torch.cuda.current_stream().wait_event(quant_fork["done"])
            q = k = v = amax = None
        else:
            # queries of dropped tokens are never used: skip their relayout
            q, k, v, amax = self._project_qkv(x, want_amax=use_quant and self.quantize_sparse_int8_mode == "max",
                                              q_keep=None if use_quant else token_mask_u8)

        # The mode decision needs row counts — unless alpha >= 0.95, where the reference never goes dense
        # (aspa.py:1636-1639): then the call runs without waiting for the record, on host-side bounds.
        if compact is not None:
            out = torch.zeros((compact["slots"], C), dtype=x.dtype, device=dev)
            row_map = compact["slot_of"]
        else:
            out = out_early
            row_map = None
        info = None
        force_dense, dense_reason, exec_mode = False, None, "shortlist"
        if lazy:
            total_rows, max_rows = B * kept_bound * k_bound, kept_bound
        else:
            if capturing:
                raise RuntimeError("this call needs row counts on the host (alpha < 0.95, a keep threshold, or candidate "
                                   "pieces that may exceed L) and cannot be captured into a CUDA graph")
            ev_rec.synchronize()
            info = self._decode_record(ctx)
            total_rows, max_rows = info["total_rows"], info["max_rows"]
            self._last_target_k = info["topk"]
            if info["topk"] <= 0:
                raise RuntimeError("ASPA requires at least one active head per token")
            density_est = float(max_rows) / float(max(1, T))
            self._update_density(density_est)
            density_threshold = self._density_threshold()
            if alpha <= self.dense_alpha_cutoff and not self.quantize_sparse_int8:
                force_dense, dense_reason = True, "alpha"
            if density_threshold is not None and density_est >= density_threshold:
                force_dense, dense_reason = True, dense_reason or "density"
            elif info["total_rows"] == B * H * T and self.force_dense_when_full:
                force_dense, dense_reason = True, dense_reason or "full"
            if alpha >= 0.95:
                dense_reason = None if dense_reason == "alpha" else dense_reason
                force_dense = False
            if use_proto:
                n_tok = float(B * T)
                self._last_proto_stats = {"max_sim_mean": info["sim_sum"] / n_tok, "blend_mean": info["bs_sum"] / n_tok,
                                          "active_tokens": int(round(info["bs_pos"]))}
            else:
                self._last_proto_stats = None

        # 6. attention
        if force_dense:
            nbh = B * H
            if token_mask_u8 is None:
                d_offs, d_tok = self._identity_rows(B, T, dev)
                d_total, d_max = nbh * T, T
            else:  # every head, kept tokens only: rows of dropped tokens are zero either way (aspa.py:1841-1842)
                full = (1 << H) - 1 if H < 64 else -1
                all_bits = torch.where(token_mask_u8.view(-1) != 0, torch.full((), full, dtype=torch.int64, device=dev),
                                       torch.zeros((), dtype=torch.int64, device=dev))
                d_offs, d_tok = ops.pack_rows(all_bits, B, T, H, B * T * H)
                d_total, d_max = H * sum(info["kept"]), max(info["kept"])
            if d_total > 0:
                attention_packed(q, k, v, row_offsets=d_offs, token_idx=d_tok, max_rows=d_max, total_rows=d_total, H=H,
                                 out=out, out_layout=N.OUT_TOKEN_MAJOR, out_row_map=row_map, kv_layout=kv_layout)
            _record_backend(BACKEND_NAME, device=str(dev), heads=nbh, tokens=T, max_rows=int(d_max))
        elif total_rows == 0:
            exec_mode = "sparse"
        else:
            dense_reason = None
            scales = None
            qa, ka, va = q, k, v
            if self.memory_enabled:   # aspa.py:1220-1225: the bank takes this call's mean keys / values first
                ops.memory_update(k, v, kv_layout, B, H, T, D, row_offsets, token_idx, self.memory_decay,
                                  self.memory_keys, self.memory_values, self.memory_counts, self.memory_ptr)
            if quant_pack is not None:
                qa, ka, va, sc3 = quant_pack
                scales = (sc3[0], sc3[1], sc3[2])
            elif use_quant:
                if amax is None:
                    amax = torch.stack([ops.head_amax(t_) for t_ in (q, k, v)])
                if self.quantize_sparse_int8_mode != "max":
                    if self.memory_enabled:
                        raise NotImplementedError("INT8 percentile scaling together with the key/value memory bank is not "
                                                  "built in the sm_100a path")
                    amax = self._percentile_bases((q, k, v), amax)
                if self.memory_enabled:   # k and v are quantised with the ring appended (aspa.py:1226-1272)
                    amax = amax.clone()
                    ops.memory_fold_amax(self.memory_keys, self.memory_values, self.memory_counts, self.memory_ptr, B,
                                         x.dtype, row_offsets, amax[1], amax[2])
                qa, s_q = ops.quantize_int8(q, amax[0].contiguous())
                ka, s_k = ops.quantize_int8(k, amax[1].contiguous())
                va, s_v = ops.quantize_int8(v, amax[2].contiguous())
                scales = (s_q, s_k, s_v)
            if plan_args is not None:
                attention_packed(qa, ka, va, row_offsets=row_offsets, token_idx=token_idx, max_rows=max_rows,
                                 total_rows=total_rows, H=H, scales=scales, plan=early_plan, out=out,
                                 out_layout=N.OUT_TOKEN_MAJOR, out_row_map=row_map, kv_layout=kv_layout,
                                 regroup=early_regroup if lazy else None)
                path = "planned"
            else:  # the candidate pieces can overflow L: use the exact table builder (needs exact row counts)
                L = runtime["effective_L"]
                tok_used = token_idx[:total_rows]
                counts_t = (row_offsets[1:] - row_offsets[:-1]).long()
                use_p = self.linear_use_proto and sim is not None and runtime["proto_cap"] > 0
                bids = None
                if use_p:
                    bids = torch.repeat_interleave(torch.arange(B * H, device=dev) // H, counts_t, output_size=total_rows)
                cand, lens = ops.build_candidates(
                    tok_used.to(torch.int64), bids, T, L, linear_window=runtime["window"],
                    anchor_stride=runtime["anchor_stride"], use_local=self.linear_use_local,
                    use_anchors=self.linear_use_anchors,
                    proto_scores=self._last_token_similarity.contiguous() if use_p else None,
                    local_cap=runtime["local_cap"], anchor_cap=runtime["anchor_cap"], proto_cap=runtime["proto_cap"])
                attention_packed(qa, ka, va, row_offsets=row_offsets, token_idx=tok_used, max_rows=max_rows,
                                 total_rows=total_rows, H=H, scales=scales, cand=cand, cand_len=lens, out=out,
                                 out_layout=N.OUT_TOKEN_MAJOR, out_row_map=row_map, kv_layout=kv_layout)
                path = "table"
            _record_backend(BACKEND_NAME, device=str(dev), heads=B * H, tokens=T, max_rows=int(max_rows),
                            quantized=bool(use_quant), candidates=path)
            self._last_shortlist_backend_info = get_last_backend_info()

        if compact is not None:
            # rows of dropped tokens are zero before the projection, so they leave it as the bias (aspa.py:1854)
            y_rows = self.proj(out)
            y = ops.scatter_rows_fill(y_rows, compact["slot_of"], compact["mask"], self.proj.bias, B * T).view(B, T, C)
            self.__dict__["_consensus_value"] = None
            self.__dict__["_consensus_pending"] = (out, compact["slot_of"], compact["mask"], (B, T, C))
        else:
            self.last_head_consensus = None if self.training else out
            y = self.dropout(self.proj(out))

        # 7. telemetry
        if lazy:
            ctx["lazy"] = True
            self.__dict__["_head_stats_value"] = None
            self.__dict__["_sparse_state_value"] = None
            self.__dict__["_pending"] = ctx
        else:
            self._publish(ctx, info, force_dense=force_dense, dense_reason=dense_reason, exec_mode=exec_mode)
        self.last_router_reg = self._router_regulariser(gate, B, T) if self.router_reg_lambda > 0.0 else None
        self._top_head_indices, self._top_head_scores = top_idx.view(B, T, -1), top_score.view(B, T, -1)
        self._last_gate_probs = gate.view(B, T, G)

        mode_now = self.__dict__["_sparse_state_value"]["mode"] if not lazy else "shortlist"
        self._finalize_latency(f"cvt(alpha={alpha:.2f})::{mode_now if force_dense else exec_mode}", ev0, t_start, ctx if lazy else None)
        return y

    def _plan_shape(self, runtime: dict, T: int, have_sim: bool) -> Optional[Tuple[int, int, int]]:
        """(window, anchor slots, prototype cap) of the structural plan, or None when the candidate pieces could
        exceed L — then only the explicit table reproduces the reference's "keep the L smallest" cut."""
        L = runtime["effective_L"]
        win = min(runtime["window"], L, runtime["local_cap"]) if (self.linear_use_local and runtime["local_cap"] > 0) else 0
        slots = 0
        if self.linear_use_anchors and runtime["anchor_stride"] > 0 and runtime["anchor_cap"] > 0:
            slots = min(runtime["anchor_cap"], L, max(1, T))
        pcap = 0
        if self.linear_use_proto and have_sim and runtime["proto_cap"] > 0:
            pcap = min(L, runtime["proto_cap"], T)
        return (win, slots, pcap) if max(win, 1) + slots + pcap <= L else None

    def _router_regulariser(self, gate: torch.Tensor, B: int, T: int) -> Optional[torch.Tensor]:
        parts = {p.strip() for p in str(self.router_reg_mode or "").lower().replace("|", ",").replace("+", ",").split(",")
                 if p.strip()} or {"entropy"}
        terms = []
        if parts & {"entropy", "ent"}:
            terms.append((gate.clamp_min(1e-9).log() * gate).sum(dim=-1).mean())
        if parts & {"l1", "l_1"}:
            terms.append((gate.sum(dim=-1) ** self.router_reg_beta).mean())
        if not terms:
            return None
        total = terms[0]
        for t_ in terms[1:]:
            total = total + t_
        return self.router_reg_lambda * total

    def _finalize_latency(self, label: str, ev0, t_start, lazy_ctx: Optional[dict] = None) -> Optional[float]:
        latency = None
        if self.track_latency and ev0 is not None:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            ev1.synchronize()
            latency = float(ev0.elapsed_time(ev1))
            self._latency_ema = latency if self._latency_ema is None else 0.8 * self._latency_ema + 0.2 * latency
        if lazy_ctx is not None:
            lazy_ctx["label"] = label
            if latency is None:
                return None
            self._materialize()
        for d in (self.__dict__.get("_head_stats_value"), self.__dict__.get("_sparse_state_value")):
            if d is not None:
                if latency is not None:
                    d["latency_ms"] = latency
                d["mode_selected"] = label
        hs = self.__dict__.get("_head_stats_value")
        if hs is not None:
            hs["mode_setting"] = self.mode_setting
        return latency


class AdaptiveSparseProtoAttention(AdaptiveSparseAttention):
    """The layer with prototype-guided routing switched on (reference aspa.py:1935-1944)."""

    def __init__(self, config: ModelConfig):
        if not getattr(config, "attn_proto_enable", False):
            try:
                setattr(config, "attn_proto_enable", True)
            except Exception:
                pass
        super().__init__(config)


class AdaptiveSparseAttentionBlock(nn.Module):
    """Pre-norm transformer block around the layer (reference aspa.py:1947-1990)."""

    def __init__(self, config: ModelConfig):
        super().__init__()
        self.ln1 = _build_norm(config)
        cls = AdaptiveSparseProtoAttention if bool(getattr(config, "attn_proto_enable", False)) else AdaptiveSparseAttention
        self.attn = cls(config)
        self.ln2 = _build_norm(config)
        self.mlp = MLP(config)
        self._is_moe = False
        self.last_aux_loss = self.last_moe_stats = self.last_router_reg = None
        self.last_head_stats = self.last_sparse_state = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.ln1(x))
        x = x + self.mlp(self.ln2(x))
        self.last_aux_loss = getattr(self.mlp, "last_aux_loss", None)
        self.last_router_reg = getattr(self.attn, "last_router_reg", None)
        self.last_moe_stats = None
        self.last_head_stats = getattr(self.attn, "last_head_stats", None)
        self.last_sparse_state = getattr(self.attn, "_last_sparse_state", None)
        return x
