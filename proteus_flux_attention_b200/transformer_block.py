"""Encoder-layer-shaped block around :class:`CausalASPAMultiheadAttention`
(reference src/proteus_attention/modules/transformer_block.py:31-117)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .multihead import CausalASPAMultiheadAttention

_ACTIVATIONS = {"relu": F.relu, "gelu": F.gelu, "silu": F.silu}


class CausalASPATransformerBlock(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, *, dim_feedforward: int = 2048, dropout: float = 0.1,
                 activation: str = "gelu", layer_norm_eps: float = 1e-5, norm_first: bool = False,
                 attention_kwargs: Optional[dict] = None) -> None:
        super().__init__()
        if activation.lower() not in _ACTIVATIONS:
            raise ValueError(f"Unsupported activation '{activation}'.")
        kw = dict(attention_kwargs or {})
        kw.setdefault("batch_first", True)
        kw.setdefault("dropout", dropout)
        self.self_attn = CausalASPAMultiheadAttention(embed_dim=embed_dim, num_heads=num_heads, **kw)
        self.linear1 = nn.Linear(embed_dim, dim_feedforward)
        self.activation = _ACTIVATIONS[activation.lower()]
        self.dropout = nn.Dropout(dropout)
        self.linear2 = nn.Linear(dim_feedforward, embed_dim)
        self.norm_first = bool(norm_first)
        self.norm1 = nn.LayerNorm(embed_dim, eps=layer_norm_eps)
        self.norm2 = nn.LayerNorm(embed_dim, eps=layer_norm_eps)
        self.dropout1 = nn.Dropout(dropout)
        self.dropout2 = nn.Dropout(dropout)

    def forward(self, src: torch.Tensor, *, src_mask: Optional[torch.Tensor] = None,
                src_key_padding_mask: Optional[torch.Tensor] = None, return_attn: bool = False, **kwargs):
        h = self.norm1(src) if self.norm_first else src
        attn_out, weights = self.self_attn(h, attn_mask=src_mask, key_padding_mask=src_key_padding_mask,
                                           need_weights=return_attn, **kwargs)
        src = src + self.dropout1(attn_out)
        if not self.norm_first:
            src = self.norm1(src)
        h = self.norm2(src) if self.norm_first else src
        src = src + self.dropout2(self.linear2(self.dropout(self.activation(self.linear1(h)))))
        if not self.norm_first:
            src = self.norm2(src)
        return (src, weights) if return_attn else src
