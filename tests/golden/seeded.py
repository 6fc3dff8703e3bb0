"""Seeded weights and inputs shared by the golden generator and the tests that replay a fixture from its seeds
(fixtures of full-size configurations store seeds and outputs only, not the multi-megabyte weights and inputs)."""
from __future__ import annotations

import torch


def xavier_state(d_model: int, gates: int, dtype: torch.dtype, seed: int) -> dict:
    """Xavier-uniform ``qkv``, ``proj``, router and prototype matrices drawn from one seeded CPU generator, in this
    order; prototypes stay fp32 like the layer's buffer."""
    g = torch.Generator().manual_seed(seed)

    def xav(rows, cols):
        bound = (6.0 / (rows + cols)) ** 0.5
        return (torch.rand(rows, cols, generator=g) * 2 - 1) * bound

    return {"qkv.weight": xav(3 * d_model, d_model).to(dtype), "proj.weight": xav(d_model, d_model).to(dtype),
            "head_router.linear.weight": xav(gates, d_model).to(dtype), "routing_prototypes": xav(gates, d_model)}


def normal_input(B: int, T: int, C: int, dtype: torch.dtype, seed: int, outliers: int = 0,
                 outlier_seed: int = 1) -> torch.Tensor:
    """x ~ N(0, 1); with ``outliers`` that many rows (positions from a second seeded permutation) are scaled by 4."""
    x = torch.randn(B, T, C, generator=torch.Generator().manual_seed(seed))
    if outliers:
        pos = torch.randperm(T, generator=torch.Generator().manual_seed(outlier_seed))[:outliers]
        x[:, pos] *= 4.0
    return x.to(dtype)


# BASELINE configuration 1: one sparse layer, fp32, 1 x 4096 x 512, 8 heads, 8 gates, top-2 heads, keep 0.25
CONFIG1 = dict(d_model=512, n_head=8, attn_h_total=8, attn_h_active=2, attn_h_active_min=2, attn_h_active_max=2,
               attn_gates=8, attn_token_sparse=True, attn_token_keep_ratio=0.25, attn_mode="auto",
               attn_small_seq_dense=0, attn_router_top_p=0.0, n_ctx=4096, attn_track_latency=False,
               attn_proto_enable=True)
