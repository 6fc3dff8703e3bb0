"""Generate the golden vectors under tests/golden/ by running the reference.

Run in the development container, where the reference source tree is
mounted read-only:

    PROTEUS_REF_SRC=<reference>/src python tests/golden/make_golden.py [--memory-only | --config1-only | --quant-only]

The reference is imported unmodified from PROTEUS_REF_SRC.  Every case stores
the seeded inputs, the module weights and the outputs the reference produced,
as plain tensors in ``tests/golden/<case>.pt``.  Nothing here is needed (or
present) on the GPU machine; tests only read the ``.pt`` files.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import torch

REF = os.environ.get("PROTEUS_REF_SRC")
if not REF:
    raise SystemExit("set PROTEUS_REF_SRC to the src directory of the reference project")
sys.path.insert(0, REF)

import proteus_attention.kernels.sparse_attn as sa  # noqa: E402
import proteus_attention.tools.chunked_shortlist as cs  # noqa: E402
from proteus_attention.models.aspa import AdaptiveSparseAttention, AdaptiveSparseProtoAttention, ModelConfig  # noqa: E402

OUT = Path(__file__).resolve().parent
sa.TRITON_AVAILABLE = False


def _state(mod):
    return {k: v.detach().clone() for k, v in mod.state_dict().items()}


def _build(cfg: dict, dtype: torch.dtype, seed: int):
    """Build the reference layer the way its own benchmark does: default dtype
    set before construction so float buffers stay fp32, then Xavier weights."""
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        torch.manual_seed(seed)
        mod = AdaptiveSparseProtoAttention(ModelConfig(**cfg)).eval()
        with torch.no_grad():
            for name in ("qkv", "proj"):
                torch.nn.init.xavier_uniform_(getattr(mod, name).weight)
            torch.nn.init.xavier_uniform_(mod.head_router.linear.weight)
            torch.nn.init.xavier_uniform_(mod.routing_prototypes)
    finally:
        torch.set_default_dtype(old)
    return mod


def layer_case(name: str, cfg: dict, *, B: int, T: int, dtype=torch.float32, seed: int = 0,
               calls: int = 1, outliers: int = 0, proto_scale: float = 1.0, conf: float = 0.0):
    cfg = dict(cfg)
    cfg.setdefault("attn_track_latency", False)
    cfg.setdefault("attn_proto_enable", True)  # what AdaptiveSparseProtoAttention switches on (aspa.py:1938-1944)
    mod = _build(cfg, dtype, seed)
    if proto_scale != 1.0 or conf:
        with torch.no_grad():
            mod.routing_prototypes.mul_(proto_scale)
            mod.routing_confidence.fill_(conf)
    weights = _state(mod)
    g = torch.Generator().manual_seed(seed + 100)
    xs, rec = [], []
    captured = {}
    orig_builder = sa.build_packed_shortlist_candidates

    def spy(*a, **k):
        out = orig_builder(*a, **k)
        captured["cand"], captured["len"] = out[0].clone(), out[1].clone()
        return out

    import proteus_attention.models.aspa as aspa_mod
    aspa_mod.build_packed_shortlist_candidates = spy
    try:
        for _ in range(calls):
            x = torch.randn(B, T, cfg["d_model"], generator=g)
            if outliers:
                pos = torch.randperm(T, generator=g)[:outliers]
                x[:, pos] *= 4.0
            x = x.to(dtype)
            captured.clear()
            with torch.no_grad():
                y = mod(x)
            st = mod._last_sparse_state or {}
            r = {
                "y": y.clone(),
                "importance": mod._last_token_importance.clone() if mod._last_token_importance is not None else None,
                "token_mask": mod._last_token_mask.clone() if mod._last_token_mask is not None else None,
                "proto_sim": mod._last_token_similarity.clone() if mod._last_token_similarity is not None else None,
                "blend": mod._last_token_blend.clone() if mod._last_token_blend is not None else None,
                "consensus": mod.last_head_consensus.clone() if mod.last_head_consensus is not None else None,
                "mode": st.get("mode"),
                "stats": {k: v for k, v in (mod.last_head_stats or {}).items()
                          if isinstance(v, (int, float, str, bool)) or v is None},
                "token_idx": st["token_idx"].clone() if "token_idx" in st else None,
                "row_offsets": st["row_offsets"].clone() if "row_offsets" in st else None,
                "active_head_indices": st["active_head_indices"].clone() if "active_head_indices" in st else None,
                "candidates": captured.get("cand"),
                "lengths": captured.get("len"),
                "protos_after": mod.routing_prototypes.clone(),
                "usage_after": mod.routing_usage_ema.clone(),
                "conf_after": mod.routing_confidence.clone(),
                "linear_L": int(mod.linear_L), "linear_window": int(mod.linear_window),
            }
            if getattr(mod, "memory_enabled", False):
                r["memory_after"] = {"keys": mod.memory_keys.clone(), "values": mod.memory_values.clone(),
                                     "counts": mod.memory_counts.clone(), "ptr": mod.memory_ptr.clone()}
            xs.append(x)
            rec.append(r)
    finally:
        aspa_mod.build_packed_shortlist_candidates = orig_builder
    torch.save({"cfg": cfg, "dtype": str(dtype), "weights": weights, "x": xs, "out": rec}, OUT / f"{name}.pt")
    print(name, [r["mode"] for r in rec], "rows", [None if r["token_idx"] is None else r["token_idx"].numel() for r in rec])


def schedule_case():
    """Known answers for the host-side schedules (aspa.py:731-747, 879-923, 862-877, 1037-1145)."""
    rows = []
    grids = [
        dict(d_model=512, n_head=8, attn_h_total=8, attn_h_active=2, attn_h_active_min=2, attn_h_active_max=2,
             attn_gates=8, attn_token_sparse=True, attn_token_keep_ratio=0.25, n_ctx=4096, attn_small_seq_dense=0),
        dict(d_model=1024, n_head=16, attn_h_total=16, attn_h_active=4, attn_h_active_min=4, attn_h_active_max=4,
             attn_linear_head_k=4, attn_gates=16, attn_token_sparse=True, attn_token_keep_ratio=0.2, n_ctx=16384),
        dict(d_model=1024, n_head=16, attn_h_total=16, attn_mode="linear", attn_linear_L=4096,
             attn_linear_L_base=4096, attn_linear_L_max=4096, attn_linear_window=4096,
             attn_linear_anchor_stride=128, attn_linear_policy="local+anchors+proto", attn_h_active=2,
             attn_h_active_min=2, attn_h_active_max=2, attn_token_sparse=True, attn_token_keep_ratio=0.2,
             n_ctx=262144),
        dict(d_model=768, n_head=12, attn_h_total=12, attn_h_active=8, attn_h_active_min=2, attn_h_active_max=12,
             n_ctx=32768, attn_small_seq_dense=1024, attn_active_seq_low=1024, attn_linear_switch_ctx=16384,
             attn_force_dense_threshold=0.6),
        dict(d_model=256, n_head=8, attn_h_total=8, attn_h_active=6, attn_h_active_min=2, attn_h_active_max=8,
             n_ctx=2048, attn_linear_L_schedule="sqrt", attn_linear_L_base=8, attn_linear_L_max=1024,
             attn_linear_policy="anchors+proto", attn_token_sparse=True, attn_token_keep_ratio=0.6,
             attn_linear_token_keep_schedule="log"),
        cs._build_model_config(65536, 1024, heads=16, sparse_ratio=0.05, shortlist_alpha=1.0, router_top_p=0.9).to_dict(),
        cs._build_model_config(32768, 1024, heads=16, sparse_ratio=0.5, shortlist_alpha=1.0, router_top_p=0.9).to_dict(),
    ]
    for cfg in grids:
        mod = AdaptiveSparseAttention(ModelConfig(**cfg))
        for T in (1, 17, 64, 65, 500, 1024, 1025, 2048, 4096, 8192, 16384, 20000, 32768, 65536, 262144):
            mod._current_alpha = 0.0
            alpha = mod._compute_cvt_alpha(T)
            k = mod._choose_active_k(T)
            ratio = mod._linear_token_keep_ratio(T)
            for a in (alpha, 0.0, 0.5, 1.0):
                p = mod._compute_effective_linear_params(T, 2, a)
                rows.append({"cfg": cfg, "T": T, "alpha_in": a, "alpha": alpha, "k": k, "ratio": ratio, "params": p})
    torch.save(rows, OUT / "schedules.pt")
    print("schedules", len(rows))


def candidate_case():
    """Exact candidate tables from the reference builders (sa.py:376-596)."""
    g = torch.Generator().manual_seed(42)
    cases = []
    for (seq_len, n, L, win, stride, ul, ua, up, caps) in [
        (64, 16, 16, 12, 4, True, False, False, None),
        (64, 16, 16, 12, 4, True, True, False, None),
        (64, 16, 16, 12, 4, True, False, True, None),
        (64, 16, 16, 12, 4, False, True, True, None),
        (32, 12, 8, 6, 3, True, True, True, (5, 6, 6)),
        (300, 40, 24, 16, 7, True, True, True, (14, 7, 3)),
        (300, 40, 24, 16, 7, False, True, False, (0, 24, 0)),
        (1, 1, 4, 4, 2, True, True, False, None),
        (513, 64, 64, 40, 32, True, True, True, (38, 19, 7)),
    ]:
        rows = torch.randint(0, seq_len, (n,), generator=g)
        bids = torch.randint(0, 2, (n,), generator=g)
        proto = torch.rand(2, seq_len, generator=g) if up else None
        kw = dict(max_candidates=L, linear_window=win, anchor_stride=stride, use_local=ul, use_anchors=ua,
                  proto_scores=proto)
        if caps is not None:
            kw.update(local_cap=caps[0], anchor_cap=caps[1], proto_cap=caps[2])
        c, l = sa.build_packed_shortlist_candidates(rows, bids if up else None, seq_len, **kw)
        cases.append({"rows": rows, "bids": bids if up else None, "seq_len": seq_len, "kw": kw, "cand": c, "len": l})
    torch.save(cases, OUT / "candidates.pt")
    print("candidates", len(cases))


def attention_case():
    """aspa_sparse_attention known answers (sa.py:1373-1646): masked-dense, shortlist, int8."""
    torch.manual_seed(0)
    out = []
    heads, T, D = 5, 37, 16
    q, k, v = (torch.randn(heads, T, D) for _ in range(3))
    am = torch.rand(heads, T) > 0.4
    am[0] = False
    cm = torch.triu(torch.full((T, T), float("-inf")), diagonal=1)
    out.append({"kind": "dense_masked", "q": q, "k": k, "v": v, "active": am, "causal": cm,
                "y": sa.aspa_sparse_attention(q, k, v, active_mask=am.unsqueeze(-1).float(), causal_mask=cm)})
    out.append({"kind": "dense_nomask_rows", "q": q, "k": k, "v": v, "active": am, "causal": None,
                "y": sa.aspa_sparse_attention(q, k, v, active_mask=am.unsqueeze(-1).float())})
    out.append({"kind": "dense_all", "q": q, "k": k, "v": v, "active": None, "causal": cm,
                "y": sa.aspa_sparse_attention(q, k, v, causal_mask=cm)})
    packed = sa._pack_active_rows(am)
    cand, lens = sa.build_packed_shortlist_candidates(packed[1], None, T, max_candidates=12, linear_window=8,
                                                      anchor_stride=5, use_local=True, use_anchors=True,
                                                      local_cap=8, anchor_cap=4)
    out.append({"kind": "shortlist", "q": q, "k": k, "v": v, "active": am, "cand": cand, "len": lens,
                "packed": packed,
                "y": sa.aspa_sparse_attention(q, k, v, active_mask=am.unsqueeze(-1), prepacked=packed,
                                              shortlist_candidates=cand, shortlist_lengths=lens)})
    mod = AdaptiveSparseAttention(ModelConfig(d_model=64, n_head=4))
    qi, qs = mod._quantize_per_head_int8(q, "_quant_ema_q")
    ki, ks = mod._quantize_per_head_int8(k, "_quant_ema_k")
    vi, vs = mod._quantize_per_head_int8(v, "_quant_ema_v")
    out.append({"kind": "shortlist_int8", "q": q, "k": k, "v": v, "qi": qi, "ki": ki, "vi": vi,
                "qs": qs, "ks": ks, "vs": vs, "active": am, "cand": cand, "len": lens, "packed": packed,
                "y": sa.aspa_sparse_attention(qi, ki, vi, active_mask=am.unsqueeze(-1), prepacked=packed,
                                              shortlist_candidates=cand, shortlist_lengths=lens,
                                              q_scale=qs, k_scale=ks, v_scale=vs, out_dtype=torch.float32)})
    torch.save(out, OUT / "attention.pt")
    print("attention", len(out))


def chunk_select_case():
    """_nucleus_select / _select_top_tokens (CPU twin) / _finalise_indices (cs.py:140-254)."""
    g = torch.Generator().manual_seed(3)
    out = []
    for n, budget, top_p in [(64, 8, 0.9), (500, 64, 0.5), (500, 600, 0.9), (256, 16, 1.0), (1000, 100, 0.2)]:
        # distinct scores so the reference's unstable ordering has a single answer
        sc = torch.rand(n, generator=g) * 4 + torch.arange(n) * 1e-5
        mask = torch.rand(n, generator=g) > 0.3
        masked = torch.where(mask, sc, torch.full_like(sc, float("-inf")))
        vals, idx = cs._nucleus_select(masked, budget, top_p)
        fin = torch.isfinite(vals)
        out.append({"scores": sc, "mask": mask, "budget": budget, "top_p": top_p,
                    "vals": vals[fin], "idx": idx[fin] + 1000})
    fins = []
    for n, mt in [(50, 10), (400, 64), (64, 100)]:
        sc = torch.rand(n, generator=g) + torch.arange(n) * 1e-6
        ix = torch.randint(0, max(4, n // 2), (n,), generator=g)
        ki, ks_ = cs._finalise_indices(sc, ix, max_tokens=mt)
        fins.append({"scores": sc, "indices": ix, "max_tokens": mt, "keep_idx": ki, "keep_sc": ks_})
    torch.save({"select": out, "finalise": fins}, OUT / "chunk_select.pt")
    print("chunk_select", len(out), len(fins))


def chunked_pipeline_case():
    """Whole ChunkedShortlistRunner.run with router-importance scoring on CPU.

    The stock run scores by L2 norm when the importance tensor is not on a CUDA
    device (cs.py:149-154).  The generator swaps in the importance-based CPU
    twin the reference ships in scripts/chunked_shortlist_tests.py:58-84 so the
    GPU semantics are what gets recorded."""
    created, inputs = [], []

    class Spy(AdaptiveSparseAttention):
        def __init__(self, config):
            super().__init__(config)
            created.append(self)
            self._init_state = _state(self)

        def forward(self, x):
            inputs.append((len(created) - 1, x.detach().clone()))
            return super().forward(x)

    def select_cpu(model, global_offset, *, per_chunk_budget, nucleus_top_p):
        imp = model._last_token_importance
        scores = imp.squeeze(0).to(torch.float32)
        m = model._last_token_mask
        if m is not None:
            scores = torch.where(m.squeeze(0).bool(), scores, torch.full_like(scores, float("-inf")))
        sel = cs._nucleus_select(scores, per_chunk_budget, nucleus_top_p)
        if sel is None:
            return None
        vals, idx = sel
        f = torch.isfinite(vals)
        return vals[f], idx[f] + int(global_offset)

    old_cls, old_sel = cs.AdaptiveSparseAttention, cs._select_top_tokens
    cs.AdaptiveSparseAttention, cs._select_top_tokens = Spy, select_cpu
    try:
        cases = []
        for seq_len, d, heads, chunk, budget, buf, seed in [(2048, 64, 4, 512, 48, 160, 11), (1536, 128, 8, 512, 64, 192, 5)]:
            created.clear()
            inputs.clear()
            g = torch.Generator().manual_seed(seed)
            seq = torch.randn(1, seq_len, d, generator=g)
            torch.manual_seed(seed)
            cfg = cs.ChunkedShortlistConfig(seq_len=seq_len, d_model=d, chunk_len=chunk, buffer_tokens=buf,
                                            per_chunk_budget=budget, device=torch.device("cpu"), heads=heads,
                                            storage="cpu")
            res = cs.ChunkedShortlistRunner(cfg).run(seq)
            cases.append({
                "seq": seq, "seq_len": seq_len, "d_model": d, "heads": heads, "chunk_len": chunk,
                "budget": budget, "buffer": buf,
                "chunk_weights": created[0]._init_state, "final_weights": created[1]._init_state,
                "warmup": inputs[0][1],
                "keep_indices": res.keep_indices, "keep_scores": res.keep_scores,
                "final_output": res.final_output, "used_fallback": res.metrics.used_fallback,
                "chunk_idx": [torch.tensor(c.promoted) for c in res.chunks],
                "chunk_scores": [torch.tensor(c.scores) for c in res.chunks],
            })
            print("chunked", seq_len, res.keep_indices.numel(), res.metrics.used_fallback)
    finally:
        cs.AdaptiveSparseAttention, cs._select_top_tokens = old_cls, old_sel
    torch.save(cases, OUT / "chunked.pt")


BASE = dict(d_model=64, n_head=4, attn_h_total=4, attn_gates=8, attn_h_active=2, attn_h_active_min=2,
            attn_h_active_max=2, attn_token_sparse=True, attn_token_keep_ratio=0.5, attn_mode="auto",
            attn_small_seq_dense=0, attn_router_top_p=0.0, n_ctx=256, attn_linear_L=32, attn_linear_window=24,
            attn_linear_anchor_stride=8, attn_use_rope=True)


def memory_cases():
    # the key/value memory bank (aspa.py:932-1035): state after every call, ring of 3 slots wrapping with B = 2
    layer_case("layer_fp32_memory", dict(BASE, attn_mode="linear", attn_memory_enable=True, attn_memory_slots=3,
                                         attn_memory_decay=0.75), B=2, T=160, calls=3)
    layer_case("layer_bf16_int8_memory", dict(BASE, attn_mode="linear", attn_quantize_int8=True, attn_linear_L=40,
                                              attn_linear_L_max=40, attn_linear_window=40, attn_memory_enable=True,
                                              attn_memory_slots=2, attn_memory_decay=0.9),
               B=2, T=192, dtype=torch.bfloat16, calls=3, outliers=8)


def quant_cases():
    # percentile and running-percentile INT8 bases (aspa.py:1329-1356): three calls, so the running base moves twice
    q = dict(BASE, attn_mode="linear", attn_quantize_int8=True, attn_linear_L=40, attn_linear_L_max=40,
             attn_linear_window=40, attn_linear_policy="local+anchors+proto", attn_gates=8)
    layer_case("layer_bf16_int8_percentile", dict(q, attn_quantize_int8_mode="percentile", attn_quantize_int8_percentile=0.98),
               B=1, T=224, dtype=torch.bfloat16, outliers=8, calls=2)
    layer_case("layer_bf16_int8_ema", dict(q, attn_quantize_int8_mode="ema_percentile", attn_quantize_int8_percentile=0.995,
                                           attn_quantize_int8_ema_decay=0.8),
               B=2, T=192, dtype=torch.bfloat16, outliers=6, calls=3)


def config1_case():
    """BASELINE configuration 1 at full size (1 x 4096 x 512 fp32, 8 heads, 8 gates, top-2, keep 0.25).  Weights and
    input come from seeds (``seeded.py``), so only what the reference produced is stored: token mask, packed rows,
    head choice, and the output rows of the kept tokens (the other rows are exactly zero: no projection bias)."""
    sys.path.insert(0, str(OUT))
    import seeded
    cfg = dict(seeded.CONFIG1)
    mod = AdaptiveSparseProtoAttention(ModelConfig(**cfg)).eval()
    w = seeded.xavier_state(cfg["d_model"], cfg["attn_gates"], torch.float32, 0)
    sd = mod.state_dict()
    sd.update(w)
    mod.load_state_dict(sd)
    x = seeded.normal_input(1, 4096, cfg["d_model"], torch.float32, 0)
    with torch.no_grad():
        y = mod(x)
    st = mod._last_sparse_state
    mask = mod._last_token_mask.clone()
    kept = mask[0].nonzero().flatten()
    assert float(y[0][~mask[0]].abs().max()) == 0.0
    stats = {k: v for k, v in mod.last_head_stats.items() if isinstance(v, (int, float, str, bool)) or v is None}
    torch.save({"seed": 0, "mode": st["mode"], "token_mask": mask, "token_idx": st["token_idx"].to(torch.int32),
                "row_offsets": st["row_offsets"].clone(), "active_head_indices": st["active_head_indices"].clone(),
                "head_idx": mod._top_head_indices[0][kept].to(torch.int8) if hasattr(mod, "_top_head_indices") else None,
                "importance": mod._last_token_importance.clone(), "y_kept": y[0][kept].clone(),
                "y_abs_sum": float(y.double().abs().sum()), "stats": stats,
                "linear_L": int(mod.linear_L), "linear_window": int(mod.linear_window)}, OUT / "layer_cfg1_full.pt")
    print("layer_cfg1_full", st["mode"], "rows", st["token_idx"].numel(), "kept", int(mask.sum()))


def main():
    import sys
    if "--memory-only" in sys.argv:
        memory_cases()
        return
    if "--config1-only" in sys.argv:
        config1_case()
        return
    if "--quant-only" in sys.argv:
        quant_cases()
        return
    config1_case()
    quant_cases()
    schedule_case()
    candidate_case()
    attention_case()
    chunk_select_case()
    memory_cases()
    layer_case("layer_fp32_auto", dict(BASE, attn_linear_switch_ctx=400), B=2, T=192, calls=2)
    layer_case("layer_fp32_proto", dict(BASE, attn_mode="linear", attn_linear_policy="local+anchors+proto",
                                        attn_linear_L=48, attn_linear_L_max=48, attn_linear_window=20,
                                        attn_proto_threshold=0.05),
               B=2, T=160, proto_scale=1.0, conf=0.3, outliers=6)
    layer_case("layer_bf16_rope", dict(BASE, d_model=128, attn_h_total=8, n_head=8, attn_gates=8, attn_h_active=4,
                                       attn_h_active_min=4, attn_h_active_max=4, attn_linear_head_k=4,
                                       attn_token_keep_ratio=0.3, attn_linear_switch_ctx=300),
               B=2, T=256, dtype=torch.bfloat16)
    layer_case("layer_bf16_int8", dict(BASE, attn_mode="linear", attn_quantize_int8=True, attn_linear_L=40,
                                       attn_linear_L_max=40, attn_linear_window=40,
                                       attn_linear_policy="local+anchors+proto", attn_gates=8),
               B=1, T=224, dtype=torch.bfloat16, outliers=8)
    layer_case("layer_fp32_dense_fastpath", dict(BASE, attn_small_seq_dense=128), B=2, T=96)
    layer_case("layer_fp32_dense_density", dict(BASE, attn_token_sparse=False, attn_force_dense_threshold=0.3,
                                                attn_linear_switch_ctx=4000), B=1, T=128)
    layer_case("layer_fp32_nucleus", dict(BASE, attn_router_top_p=0.7, attn_h_active=4, attn_h_active_min=1,
                                          attn_h_active_max=4, attn_linear_switch_ctx=1000, attn_token_sparse=False),
               B=2, T=200)
    chunked_pipeline_case()


if __name__ == "__main__":
    main()
