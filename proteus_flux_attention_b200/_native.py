"""ctypes binding of libaspa_b200.so (the C ABI declared in include/aspa_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  Tensors cross the boundary as raw device pointers plus sizes; the
current torch CUDA stream is passed as the ``stream`` argument of every call.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent / "libaspa_b200.so"
_lib: Optional[C.CDLL] = None

F32, BF16, I8 = 0, 1, 2
OUT_HEAD_MAJOR, OUT_TOKEN_MAJOR = 0, 1

_p, _i, _l, _f, _d = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_double


class ShortlistPlan(C.Structure):
    """Mirror of ``aspa_shortlist_plan``."""
    _fields_ = [("window", C.c_int32), ("anchor_slots", C.c_int32), ("anchor_stride", C.c_int32),
                ("proto_cap", C.c_int32), ("proto_block", C.c_int32), ("proto_list_stride", C.c_int32),
                ("proto_lists", C.c_void_p), ("proto_limit", C.c_void_p)]


class KVLayout(C.Structure):
    """Mirror of ``aspa_kv_layout``: element strides (batch, head, token) of k and of v."""
    _fields_ = [("k_batch", C.c_int64), ("k_head", C.c_int64), ("k_token", C.c_int64),
                ("v_batch", C.c_int64), ("v_head", C.c_int64), ("v_token", C.c_int64)]


# name -> (restype, argtypes); must list every symbol of include/aspa_b200.h
SIGNATURES = {
    "aspa_last_error_string": (C.c_char_p, []),
    "aspa_version": (_i, []),
    "aspa_router_fwd": (_i, [_p, _i, _l, _i, _p, _i, _p, _p, _p, _f, _f, _f, _f, _f, _p, _p, _p, _p, _p, _p]),
    "aspa_router_tc_scratch_bytes": (_l, [_i, _i, _i]),
    "aspa_router_fwd_tc": (_i, [_p, _l, _i, _p, _i, _p, _p, _p, _f, _f, _f, _f, _f, _p, _p, _p, _p, _p, _p, _p, _p]),
    "aspa_read_status": (_i, [_p, _i, _p]),
    "aspa_router_fwd_tc_probe": (_i, [_p, _l, _i, _p, _i, _p, _p, _p, _p, _p, _p, _p, _p, C.c_uint32, _l, _p]),
    "aspa_normalize_rows": (_i, [_p, _i, _i, _f, _p, _p]),
    "aspa_token_select": (_i, [_p, _i, _i, _i, _f, _i, _p, _p, _p]),
    "aspa_head_budget": (_i, [_p, _l, _i, _p, _i, _d, _i, _i, _i, _d, _p, _p, _p]),
    "aspa_head_select": (_i, [_p, _l, _i, _p, _i, _i, _p, _i, _p, _p, _p, _p, _p, _p]),
    "aspa_pack_rows_scratch": (_l, [_i, _i, _i]),
    "aspa_pack_rows": (_i, [_p, _i, _i, _i, _p, _p, _p, _l, _p]),
    "aspa_pack_rows_static_capacity": (_l, []),
    "aspa_pack_rows_static": (_i, [_p, _i, _i, _i, _p, _p, _l, _p]),
    "aspa_pack_mask": (_i, [_p, _i, _i, _p, _p, _p, _l, _p]),
    "aspa_rope_table": (_i, [_p, _i, _i, _i, _p, _p, _p]),
    "aspa_rope_relayout": (_i, [_p, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p]),
    "aspa_rope_quantize": (_i, [_p, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p]),
    "aspa_head_amax": (_i, [_p, _i, _i, _l, _p, _p]),
    "aspa_quantize_int8": (_i, [_p, _i, _i, _l, _p, _p, _p, _p]),
    "aspa_head_abs_quantile_scratch": (_l, [_i]),
    "aspa_head_abs_quantile": (_i, [_p, _i, _i, _l, _d, _p, _p, _p, _p]),
    "aspa_proto_plan_scratch": (_l, [_i, _i, _i]),
    "aspa_proto_plan": (_i, [_p, _i, _i, _i, _p, _p, _p, _p]),
    "aspa_build_candidates": (_i, [_p, _p, _l, _i, _i, _i, _i, _i, _i, _p, _i, _i, _i, _p, _p, _p]),
    "aspa_attn_workspace_bytes": (_l, [_l, _i]),
    "aspa_gather_attn_fwd": (_i, [_p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _p, _p, _i, _l, _p, _p, _i,
                                  C.POINTER(ShortlistPlan), _p, _p, _i, _i, _p, _p]),
    "aspa_proto_ema_scratch": (_l, [_l, _i, _i]),
    "aspa_proto_ema_update": (_i, [_p, _i, _l, _i, _p, _i, _d, _p, _p, _p, _p, _p, _p]),
    "aspa_chunk_select": (_i, [_p, _p, _i, _i, _f, _l, _p, _p, _p, _p]),
    "aspa_chunk_select_slot": (_i, [_p, _p, _i, _i, _f, _p, _p, _p, _p, _p, _p]),
    "aspa_merge_finalise_scratch": (_l, [_l]),
    "aspa_merge_finalise": (_i, [_p, _p, _l, _l, _i, _p, _p, _p, _p, _p, _p]),
    "aspa_gather_attn_fwd_ex": (_i, [_p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _p, _p, _i, _l, _p, _p, _i,
                                     C.POINTER(ShortlistPlan), _p, _p, _i, _i, _p, C.POINTER(KVLayout), _p, _p, _p]),
    "aspa_attn_regroup_bytes": (_l, [_l, _i, _i]),
    "aspa_attn_tc_mode": (_i, [_i]),
    "aspa_attn_picks_mode": (_i, [_i]),
    "aspa_attn_tc_status": (_i, [_i, _p]),
    "aspa_gather_attn_fwd_prepared": (_i, [_p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _p, _p, _i, _l, _p, _p, _i,
                                           C.POINTER(ShortlistPlan), _p, _p, _i, _i, _p, C.POINTER(KVLayout), _p, _p, _i,
                                           _p]),
    "aspa_attn_regroup_rows": (_i, [_i, _i, _i, _i, _p, _p, _l, C.POINTER(ShortlistPlan), _p, C.POINTER(C.c_int32), _p]),
    "aspa_rope_inplace": (_i, [_p, _i, _l, _i, _l, _i, _i, _p, _p, _p]),
    "aspa_rope_rows_to_heads": (_i, [_p, _i, _l, _i, _l, _i, _i, _p, _p, _p, _p]),
    "aspa_memory_update": (_i, [_p, _p, _i, _p, _i, _i, _i, _i, _p, _p, _f, _p, _p, _p, _p, _i, _p]),
    "aspa_memory_fold_amax": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _p, _p, _p]),
    "aspa_rope_relayout_kv": (_i, [_p, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p]),
    "aspa_rope_rows_q": (_i, [_p, _i, _p, _p, _l, _i, _i, _i, _i, _p, _p, _p, _p]),
    "aspa_compact_mask_scratch": (_l, [_l]),
    "aspa_compact_mask": (_i, [_p, _l, _l, _p, _p, _p, _p, _p]),
    "aspa_scatter_rows_fill": (_i, [_p, _p, _p, _p, _l, _l, _p, _p]),
    "aspa_gather_rows": (_i, [_p, _p, _p, _l, _l, _p, _p]),
    "aspa_reduce_partials": (_i, [_p, _i, _l, _p, _p]),
    "aspa_stats_record": (_i, [_p, _i, _p, _i, _d, _p, _d, _p, _l, _p, _l, _p, _p, _p]),
    "aspa_token_select_compact": (_i, [_p, _i, _i, _i, _f, _i, _p, _p, _p, _p, _i, _p]),
    "aspa_head_select_pack": (_i, [_p, _i, _i, _i, _p, _i, _i, _p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _l, _p]),
}


def library_path() -> Path:
    return _LIB_PATH


def lib() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(
                f"{_LIB_PATH} is missing: build it with `python -m proteus_flux_attention_b200.build` "
                "(there is no CPU or PyTorch fallback for the ASPA kernels)")
        handle = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        # kernel-choice switches for A/B measurements: ASPA_ATTN_TC_MODE=0|1|2, ASPA_ATTN_PICKS_MODE=0|1
        import os
        for var, setter in (("ASPA_ATTN_TC_MODE", handle.aspa_attn_tc_mode), ("ASPA_ATTN_PICKS_MODE", handle.aspa_attn_picks_mode)):
            if os.environ.get(var, "").strip().isdigit():
                setter(int(os.environ[var]))
        _lib = handle
    return _lib


def last_error() -> str:
    return lib().aspa_last_error_string().decode("utf-8", "replace")


ERR_TIMEOUT = -4


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait ran out (status ASPA_ERR_TIMEOUT); the outputs of that call are invalid."""


def check(rc: int, what: str) -> None:
    if rc == ERR_TIMEOUT:
        raise DeviceWaitTimeout(f"{what}: {last_error()}")
    if rc != 0:
        raise RuntimeError(f"{what} failed with status {rc}: {last_error()}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    if dt == torch.int8:
        return I8
    raise TypeError(f"unsupported dtype {dt}: the ASPA kernels take float32, bfloat16 or int8")


def ptr(t: Optional[torch.Tensor]):
    """Device pointer of a contiguous CUDA tensor (None -> NULL)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("the ASPA kernels need CUDA tensors; there is no CPU path")
    if not t.is_contiguous():
        raise RuntimeError("internal error: non-contiguous tensor handed to a kernel")
    return C.c_void_p(t.data_ptr())


def stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)
