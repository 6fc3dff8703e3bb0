"""Functional ASPA attention op and shortlist builders on the sm_100a kernels.

Same call signatures, argument meaning and validation errors as the reference
module ``src/proteus_attention/kernels/sparse_attn.py`` (``aspa_sparse_attention``
:1373-1646, ``build_shortlist_candidates`` :376-454,
``build_packed_shortlist_candidates`` :457-596, ``get_last_backend[_info]``
:72-85, ``_pack_active_rows`` :924-947).  There is one back-end: the CUDA
library.  CPU tensors, or a missing library, raise.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _native as N
from . import ops

BACKEND_NAME = "b200_cuda"
_LAST_BACKEND_INFO: Dict[str, object] = {"name": "uninitialized", "details": {}}


def _record_backend(name: str, **details: object) -> None:
    global _LAST_BACKEND_INFO
    _LAST_BACKEND_INFO = {"name": name, "details": details}


def get_last_backend() -> str:
    """Name of the back-end used by the most recent attention call."""
    return str(_LAST_BACKEND_INFO.get("name", "uninitialized"))


def get_last_backend_info() -> Dict[str, object]:
    """Copy of the most recent back-end record ``{"name", "details"}``."""
    info = dict(_LAST_BACKEND_INFO)
    if isinstance(info.get("details"), dict):
        info["details"] = dict(info["details"])
    return info


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("proteus_flux_attention_b200 has no CPU path: tensors must live on a CUDA device")


def _pack_active_rows(active_mask: torch.Tensor):
    """(heads, T) bool mask -> (head_idx, token_idx, row_offsets int32, max_rows) or None.

    Device-side packing; reading ``max_rows`` is the one host synchronisation."""
    if active_mask.dim() != 2:
        raise ValueError("active_mask must have rank 2 after squeeze")
    _require_cuda(active_mask)
    heads, T = active_mask.shape
    m8 = active_mask.to(torch.uint8).contiguous() if active_mask.dtype != torch.uint8 else active_mask.contiguous()
    offs, tok = ops.pack_mask(m8)
    counts = (offs[1:] - offs[:-1])
    host = torch.stack([counts.max(), offs[-1]]).tolist()
    max_rows, total = int(host[0]), int(host[1])
    if total == 0:
        return None
    tok = tok[:total]
    head_idx = torch.repeat_interleave(torch.arange(heads, device=tok.device), counts.long(), output_size=total)
    return head_idx.to(torch.int64), tok.to(torch.int64), offs, max_rows


def build_shortlist_candidates(rows: torch.Tensor, seq_len: int, *, max_candidates: int, linear_window: int,
                               anchor_stride: int, use_local: bool, use_anchors: bool,
                               proto_scores: Optional[torch.Tensor] = None, local_cap: Optional[int] = None,
                               anchor_cap: Optional[int] = None, proto_cap: Optional[int] = None
                               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row candidate table for one head (reference sa.py:376-454)."""
    return build_packed_shortlist_candidates(
        rows, None, seq_len, max_candidates=max_candidates, linear_window=linear_window,
        anchor_stride=anchor_stride, use_local=use_local, use_anchors=use_anchors, proto_scores=proto_scores,
        local_cap=local_cap, anchor_cap=anchor_cap, proto_cap=proto_cap)


def build_packed_shortlist_candidates(rows: torch.Tensor, row_batch_ids: Optional[torch.Tensor], seq_len: int, *,
                                      max_candidates: int, linear_window: int, anchor_stride: int, use_local: bool,
                                      use_anchors: bool, proto_scores: Optional[torch.Tensor] = None,
                                      local_cap: Optional[int] = None, anchor_cap: Optional[int] = None,
                                      proto_cap: Optional[int] = None, chunk_size: int = 4096,
                                      extra_candidates: Optional[torch.Tensor] = None,
                                      extra_lengths: Optional[torch.Tensor] = None
                                      ) -> Tuple[torch.Tensor, torch.Tensor]:
    """(N, L) int64 ascending unique candidate ids padded with the row id, and lengths (N,) int64
    (reference sa.py:457-596).  ``chunk_size`` is accepted for signature compatibility; the kernel
    handles one row per CTA and needs no chunking."""
    if rows.numel() == 0 or max_candidates <= 0:
        return rows.new_empty(rows.shape + (0,)), rows.new_zeros(rows.shape, dtype=torch.long)
    if extra_candidates is not None:
        raise NotImplementedError("extra (memory-bank) candidates are not supported by the sm_100a builder")
    _require_cuda(rows, proto_scores)
    rows64 = rows.to(torch.int64).contiguous()
    rb = row_batch_ids.to(device=rows.device, dtype=torch.int64).contiguous() if row_batch_ids is not None else None
    ps = None
    if proto_scores is not None and proto_scores.numel() > 0:
        ps = proto_scores.detach().to(device=rows.device, dtype=torch.float32)
        ps = ps.unsqueeze(0) if ps.dim() == 1 else ps
        ps = ps[:, :seq_len].contiguous()
        if ps.size(1) < seq_len:
            raise ValueError("proto_scores must cover seq_len positions")
    cand, lens = ops.build_candidates(rows64, rb if ps is not None else None, seq_len, int(max_candidates),
                                      linear_window=linear_window, anchor_stride=anchor_stride, use_local=use_local,
                                      use_anchors=use_anchors, proto_scores=ps, local_cap=local_cap,
                                      anchor_cap=anchor_cap, proto_cap=proto_cap)
    return cand.to(rows.dtype), lens


def attention_packed(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, row_offsets: torch.Tensor,
                     token_idx: torch.Tensor, max_rows: int, total_rows: int, H: int,
                     scales=None, cand=None, cand_len=None, plan=None, add_mask=None,
                     out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                     out_layout: int = N.OUT_HEAD_MAJOR, out_row_map: Optional[torch.Tensor] = None,
                     kv_layout=None, regroup=None) -> torch.Tensor:
    """Internal entry used by the layer: rows already packed on the device."""
    heads, T, D = q.shape
    if out is None:
        out = torch.zeros((heads, T, D), dtype=out_dtype or q.dtype, device=q.device)
    ops.gather_attn(q, k, v, scales=scales, H=H, row_offsets=row_offsets, token_idx=token_idx, max_rows=max_rows,
                    total_rows=total_rows, cand=cand, cand_len=cand_len, plan=plan, add_mask=add_mask, out=out,
                    out_layout=out_layout, out_row_map=out_row_map, kv_layout=kv_layout, regroup=regroup)
    return out


def aspa_sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
                          active_mask: Optional[torch.Tensor] = None, causal_mask: Optional[torch.Tensor] = None,
                          dropout_p: float = 0.0, training: bool = False,
                          prepacked: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]] = None,
                          q_scale: Optional[torch.Tensor] = None, k_scale: Optional[torch.Tensor] = None,
                          v_scale: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                          shortlist_candidates: Optional[torch.Tensor] = None,
                          shortlist_lengths: Optional[torch.Tensor] = None) -> torch.Tensor:
    """ASPA attention over the active (head, token) rows.  q, k, v: (B*H, T, D).

    Rows marked inactive come back as zeros.  With a candidate table each active row attends to its own
    candidate keys; without one it attends to keys ``<= t`` (or as ``causal_mask`` says).  Argument
    checks and their messages follow the reference (sa.py:1415-1508)."""
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise ValueError("q, k, v must be rank-3 tensors of shape (B*H, T, D)")
    if q.shape != k.shape or q.shape != v.shape:
        raise ValueError("q, k, v must have matching shapes")
    heads, T, D = q.shape
    dropout_p = float(dropout_p)
    if dropout_p < 0.0 or dropout_p >= 1.0:
        raise ValueError("dropout_p must satisfy 0.0 <= dropout_p < 1.0")
    if bool(training) and dropout_p > 0.0:
        raise NotImplementedError("attention dropout is not implemented in the sm_100a kernels (forward-only build)")
    _require_cuda(q, k, v)
    _record_backend("uninitialized")
    quant = q.dtype == torch.int8 or k.dtype == torch.int8 or v.dtype == torch.int8
    if out_dtype is None:
        out_dtype = q.dtype if q.dtype.is_floating_point else torch.float32
    scales = None
    if quant:
        if q.dtype != torch.int8 or k.dtype != torch.int8 or v.dtype != torch.int8:
            raise ValueError("Quantized path expects int8 q, k, v tensors")
        if q_scale is None or k_scale is None or v_scale is None:
            raise ValueError("Quantized path requires q_scale, k_scale, and v_scale tensors")
        scales = tuple(s.to(device=q.device, dtype=torch.float32).contiguous().view(-1) for s in (q_scale, k_scale, v_scale))
        if any(s.numel() != heads for s in scales):
            raise ValueError("Scale tensors must have length equal to the number of heads in q/k/v")
    add_mask = None
    if causal_mask is not None:
        if causal_mask.dim() != 2 or causal_mask.size(0) != T or causal_mask.size(1) != T:
            raise ValueError("causal_mask must have shape (T, T)")
        add_mask = causal_mask.to(device=q.device, dtype=torch.float32).contiguous()
    mask_bool = None
    if active_mask is not None:
        if active_mask.dim() == 3 and active_mask.size(2) == 1:
            active_mask = active_mask.squeeze(-1)
        if active_mask.dim() != 2 or active_mask.size(0) != heads or active_mask.size(1) != T:
            raise ValueError("active_mask must have shape (B*H, T)")
        active_mask = active_mask.to(device=q.device)
        mask_bool = active_mask if active_mask.dtype == torch.bool else (active_mask > 0.0)

    if prepacked is not None:
        _, token_idx, row_offsets, max_rows = prepacked
        token_idx = token_idx.to(device=q.device, dtype=torch.int32).contiguous()
        row_offsets = row_offsets.to(device=q.device, dtype=torch.int32).contiguous()
        total = int(token_idx.numel())
        max_rows = int(max_rows)
    elif mask_bool is None:
        token_idx = torch.arange(T, device=q.device, dtype=torch.int32).repeat(heads)
        row_offsets = torch.arange(0, (heads + 1) * T, T, device=q.device, dtype=torch.int32)
        total, max_rows = heads * T, T
    else:
        packed = _pack_active_rows(mask_bool)
        if packed is None:
            _record_backend("empty", device=str(q.device), heads=heads, quantized=bool(quant))
            return torch.zeros(q.shape, device=q.device, dtype=out_dtype)
        _, token_idx64, row_offsets, max_rows = packed
        token_idx = token_idx64.to(torch.int32)
        total = int(token_idx.numel())

    cand = lens = None
    if shortlist_candidates is not None or shortlist_lengths is not None:
        if shortlist_candidates is None or shortlist_lengths is None:
            raise ValueError("shortlist_candidates and shortlist_lengths must be provided together.")
        if shortlist_candidates.dim() != 2:
            raise ValueError("shortlist_candidates must have shape (N_active, L_max)")
        if shortlist_lengths.dim() != 1:
            raise ValueError("shortlist_lengths must have shape (N_active,)")
        if shortlist_candidates.size(0) != shortlist_lengths.size(0):
            raise ValueError("shortlist_lengths must align with shortlist_candidate rows")
        cand = shortlist_candidates.to(device=q.device, dtype=torch.long).contiguous()
        lens = shortlist_lengths.to(device=q.device, dtype=torch.long).contiguous()
        if cand.size(0) != total:
            raise ValueError("Shortlist candidates must match the number of active rows")
        if cand.numel() == 0:
            cand = lens = None

    out = attention_packed(q.contiguous(), k.contiguous(), v.contiguous(), row_offsets=row_offsets,
                           token_idx=token_idx, max_rows=max_rows, total_rows=total, H=heads, scales=scales,
                           cand=cand, cand_len=lens, add_mask=add_mask, out_dtype=out_dtype)
    _record_backend(BACKEND_NAME, device=str(q.device), heads=heads, tokens=T, max_rows=int(max_rows),
                    quantized=bool(quant))
    return out


__all__ = ["aspa_sparse_attention", "get_last_backend", "get_last_backend_info", "build_shortlist_candidates",
           "build_packed_shortlist_candidates"]
