"""``nn.MultiheadAttention``-shaped wrapper around the ASPA layer.

Mirrors ``CausalASPAMultiheadAttention`` of the reference
(src/proteus_attention/modules/aspa_multihead.py:14-252): same constructor
arguments and config defaults, the same fallback rule (cross-attention,
non-causal calls and non-causal masks go to an internal ``nn.MultiheadAttention``
with its own weights), padding handling, optional zero attention weights and the
runtime statistics record."""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn

from .aspa import AdaptiveSparseProtoAttention, ModelConfig
from .sparse_attn import get_last_backend_info
from .sparse_ctl import SparseCtlSnapshot, SparseHeadController

_WRAPPER_DEFAULTS = {  # aspa_multihead.py:43-67
    "attn_h_active_min": 2, "attn_mode": "auto", "attn_linear_L": 512, "attn_linear_window": 512,
    "attn_linear_anchor_stride": 256, "attn_linear_head_k": 2, "attn_small_seq_dense": 0,
    "attn_force_dense_threshold": 0.6, "attn_quantize_int8": False, "attn_quantize_int8_mode": "max",
    "attn_quantize_int8_percentile": 1.0, "attn_quantize_int8_ema_decay": 0.9, "attn_router_top_p": 0.9,
}


class CausalASPAMultiheadAttention(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, *, dropout: float = 0.0, bias: bool = True,
                 batch_first: bool = True, device: torch.device | None = None, dtype: torch.dtype | None = None,
                 max_seq_len: int | None = None, return_stats_default: bool = False,
                 sparse_ctl_config: Optional[Dict[str, Any]] = None, **config_overrides: Any) -> None:
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError("embed_dim must be divisible by num_heads.")
        self.embed_dim, self.num_heads = int(embed_dim), int(num_heads)
        self.batch_first = bool(batch_first)
        self._return_stats_default = bool(return_stats_default)
        self._last_runtime_stats: Optional[Dict[str, Any]] = None
        self._sparse_ctl: Optional[SparseHeadController] = None
        cfg: Dict[str, Any] = {"d_model": self.embed_dim, "attn_h_total": self.num_heads, "n_head": self.num_heads,
                               "p_dropout": float(dropout), "bias": bool(bias), "attn_variant": "aspa"}
        cfg["attn_h_active"] = config_overrides.pop("attn_h_active", min(self.num_heads, 8))
        cfg["attn_h_active_max"] = config_overrides.pop("attn_h_active_max", self.num_heads)
        cfg["attn_proto_enable"] = bool(config_overrides.pop("attn_proto_enable", True))
        cfg["n_ctx"] = int(max_seq_len or config_overrides.pop("n_ctx", 0))
        for key, default in _WRAPPER_DEFAULTS.items():
            cfg[key] = config_overrides.pop(key, default)
        cfg.update(config_overrides)
        self.attention = AdaptiveSparseProtoAttention(ModelConfig(**cfg))
        self.fallback_attention = nn.MultiheadAttention(embed_dim=self.embed_dim, num_heads=self.num_heads,
                                                        dropout=float(dropout), bias=bool(bias),
                                                        batch_first=self.batch_first)
        if device is not None or dtype is not None:
            self.attention.to(device=device, dtype=dtype)
            self.fallback_attention.to(device=device, dtype=dtype)
        if sparse_ctl_config:
            self._sparse_ctl = SparseHeadController(self.attention, **sparse_ctl_config)

    @staticmethod
    def _is_supported_attn_mask(attn_mask: Optional[torch.Tensor], seq_len: int, device: torch.device) -> bool:
        """True for ``None`` or exactly the strict upper-triangular (causal) pattern."""
        if attn_mask is None:
            return True
        mask = attn_mask.squeeze(0) if (attn_mask.dim() == 3 and attn_mask.size(0) == 1) else attn_mask
        if mask.dim() != 2 or mask.size(0) != seq_len or mask.size(1) != seq_len:
            return False
        blocked = mask if mask.dtype == torch.bool else torch.isinf(mask)
        # blocked[i, j] must equal (j > i)
        cols = torch.arange(seq_len, device=mask.device)
        return bool((blocked == (cols.unsqueeze(0) > cols.unsqueeze(1))).all())

    def forward(self, query: torch.Tensor, key: Optional[torch.Tensor] = None, value: Optional[torch.Tensor] = None,
                key_padding_mask: Optional[torch.Tensor] = None, need_weights: bool = True,
                attn_mask: Optional[torch.Tensor] = None, average_attn_weights: bool = True,
                is_causal: Optional[bool] = None, *, return_stats: Optional[bool] = None
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        reason: Optional[str] = None
        if (key is not None and key is not query) or (value is not None and value is not query):
            reason = "cross_attention"
        if is_causal is not None and not is_causal:
            reason = reason or "non_causal"
        seq_len = query.shape[1] if self.batch_first else query.shape[0]
        if not self._is_supported_attn_mask(attn_mask, seq_len, query.device):
            reason = reason or "custom_attn_mask"
        want_stats = self._return_stats_default if return_stats is None else bool(return_stats)

        if reason is not None:
            fb = self.fallback_attention.to(device=query.device, dtype=query.dtype)
            out, weights = fb(query, query if key is None else key, query if value is None else value,
                              key_padding_mask=key_padding_mask, need_weights=need_weights, attn_mask=attn_mask,
                              average_attn_weights=average_attn_weights,
                              is_causal=bool(is_causal) if is_causal is not None else False)
            self._last_runtime_stats = None
            if want_stats:
                self._last_runtime_stats = {"head_stats": None, "sparse_state": None,
                                            "shortlist_backend": {"name": "torch.nn.MultiheadAttention",
                                                                  "details": {"reason": reason}}}
                if self._sparse_ctl is not None:
                    self._last_runtime_stats["sparse_ctl"] = None
            return out, weights

        x = query if self.batch_first else query.transpose(0, 1)
        x = x if x.is_contiguous() else x.contiguous()
        batch, seq_len, _ = x.shape
        padding = None
        if key_padding_mask is not None:
            if key_padding_mask.dim() != 2 or key_padding_mask.size(1) != seq_len:
                raise ValueError("key_padding_mask must have shape (batch, seq_len).")
            padding = key_padding_mask.to(device=x.device).unsqueeze(-1)
            x = x.masked_fill(padding, 0.0)
        out = self.attention(x)
        if padding is not None:
            out = out.masked_fill(padding, 0.0)
        if not self.batch_first:
            out = out.transpose(0, 1)
        weights: Optional[torch.Tensor] = None
        if need_weights:
            rows = batch if average_attn_weights else batch * self.num_heads
            weights = out.new_zeros(rows, seq_len, seq_len)
        head_stats = getattr(self.attention, "last_head_stats", None)
        snap: Optional[SparseCtlSnapshot] = self._sparse_ctl.observe(head_stats) if self._sparse_ctl is not None else None
        self._last_runtime_stats = None
        if want_stats:
            stats: Dict[str, Any] = {"head_stats": head_stats,
                                     "sparse_state": getattr(self.attention, "_last_sparse_state", None),
                                     "shortlist_backend": get_last_backend_info()}
            if snap is not None:
                stats["sparse_ctl"] = {"density": snap.density, "action": snap.action, "min_heads": snap.min_heads,
                                       "max_heads": snap.max_heads, "step": snap.step}
            elif self._sparse_ctl is not None:
                stats["sparse_ctl"] = None
            self._last_runtime_stats = stats
        return out, weights

    @property
    def last_runtime_stats(self) -> Optional[Dict[str, Any]]:
        return self._last_runtime_stats

    @property
    def sparse_controller(self) -> Optional[SparseHeadController]:
        return self._sparse_ctl
