"""Pins the CPU oracle to vectors produced by the reference implementation itself
(tests/golden/make_golden.py).  Runs without a GPU."""
import math

import pytest
import torch

from oracle import aspa_oracle as O


def _load(golden_dir, name):
    return torch.load(golden_dir / name, weights_only=False)


def test_schedules_match_reference(golden_dir):
    rows = _load(golden_dir, "schedules.pt")
    for r in rows:
        s = O.derive_config(**r["cfg"])
        st = O.SimpleNamespace(latency_ema=None, current_alpha=0.0, L_scale=s.linear_L_scale_init,
                               alpha_override=None, last_target_k=None)
        assert O.cvt_alpha(s, r["T"], st) == r["alpha"]
        k = O.choose_active_k(s, r["T"])
        assert k == r["k"]
        assert O.linear_token_keep_ratio(s, r["T"]) == r["ratio"]
        # the reference evaluates the params right after _choose_active_k, whose result it remembers
        p = O.effective_linear_params(s, r["T"], 2, r["alpha_in"], s.linear_L_scale_init, k)
        assert p == r["params"], (r["cfg"], r["T"], r["alpha_in"])


def test_choose_active_k_known_answers():
    # tests/test_aspa.py:718-747 of the reference pins 1024 -> 7 and 2048 -> 4
    s = O.derive_config(d_model=64, n_head=8, attn_h_total=8, attn_h_active=8, attn_h_active_min=4,
                        attn_h_active_max=8, attn_active_seq_low=512, attn_active_seq_high=2048,
                        attn_active_curve=0.5)
    assert O.choose_active_k(s, 256) == 8
    assert O.choose_active_k(s, 4096) == 4


def test_candidates_match_reference(golden_dir):
    for c in _load(golden_dir, "candidates.pt"):
        cand, ln = O.build_candidates(c["rows"], c["bids"], c["seq_len"], **c["kw"])
        assert torch.equal(cand, c["cand"])
        assert torch.equal(ln, c["len"])


def test_attention_matches_reference(golden_dir):
    for c in _load(golden_dir, "attention.pt"):
        q, k, v = c["q"], c["k"], c["v"]
        heads, T, _ = q.shape
        if c["kind"].startswith("dense"):
            am = c["active"] if c["active"] is not None else torch.ones(heads, T, dtype=torch.bool)
            packed = O.pack_active_rows(am)
            y = O.sparse_attention(q, k, v, packed=packed, causal_mask=c["causal"])
        elif c["kind"] == "shortlist":
            packed = O.pack_active_rows(c["active"])
            assert torch.equal(packed[1], c["packed"][1]) and torch.equal(packed[2], c["packed"][2])
            y = O.sparse_attention(q, k, v, packed=packed, candidates=c["cand"], lengths=c["len"])
        else:
            qi, qs = O.quantize_per_head_int8(q)
            ki, ks = O.quantize_per_head_int8(k)
            vi, vs = O.quantize_per_head_int8(v)
            assert torch.equal(qi, c["qi"]) and torch.equal(ki, c["ki"]) and torch.equal(vi, c["vi"])
            assert torch.equal(qs, c["qs"])
            y = O.sparse_attention(qi, ki, vi, packed=O.pack_active_rows(c["active"]), candidates=c["cand"],
                                   lengths=c["len"], q_scale=qs, k_scale=ks, v_scale=vs, out_dtype=torch.float32)
        assert torch.allclose(y, c["y"], atol=1e-6, rtol=1e-5), c["kind"]


def test_chunk_selection_matches_reference(golden_dir):
    g = _load(golden_dir, "chunk_select.pt")
    for c in g["select"]:
        vals, idx = O.select_top_tokens(c["scores"], c["mask"], 1000, budget=c["budget"], top_p=c["top_p"])
        assert torch.equal(idx, c["idx"])
        assert torch.equal(vals, c["vals"])
    for c in g["finalise"]:
        ki, ks = O.finalise_indices(c["scores"], c["indices"], max_tokens=c["max_tokens"])
        assert torch.equal(ki, c["keep_idx"])
        assert torch.equal(ks, c["keep_sc"])


LAYER_CASES = ["layer_fp32_auto", "layer_fp32_proto", "layer_bf16_rope", "layer_bf16_int8",
               "layer_fp32_dense_fastpath", "layer_fp32_dense_density", "layer_fp32_nucleus",
               "layer_fp32_memory", "layer_bf16_int8_memory", "layer_bf16_int8_percentile", "layer_bf16_int8_ema"]


def _tie_only(imp_row, a, b):
    """True when masks a and b differ only on tokens whose importance equals the cut value."""
    diff = a ^ b
    if not diff.any():
        return True
    cut = imp_row[a].min()
    return bool((imp_row[diff] - cut).abs().max() < 1e-6)


def _rows_to_mask(rec, B, H, T):
    """(B, H, T) bool mask of computed (head, token) rows from a packed row list."""
    m = torch.zeros(B * H, T, dtype=torch.bool)
    offs = rec["row_offsets"].long()
    for i, h in enumerate(rec["active_head_indices"].tolist()):
        m[h, rec["token_idx"][offs[i]:offs[i + 1]]] = True
    return m.view(B, H, T)


@pytest.mark.parametrize("name", LAYER_CASES)
def test_layer_matches_reference(golden_dir, name):
    g = _load(golden_dir, name + ".pt")
    bf16 = "bfloat16" in g["dtype"]
    layer = O.OracleLayer(g["weights"], **g["cfg"])
    for x, ref in zip(g["x"], g["out"]):
        y = layer.forward(x)
        tr = layer.trace
        assert tr["mode"] == ref["mode"]
        if ref["mode"] != "dense_fastpath":
            assert torch.allclose(tr["importance"], ref["importance"], atol=2e-6 if not bf16 else 1e-5)
            if ref["token_mask"] is not None:
                for b in range(x.size(0)):
                    assert _tie_only(ref["importance"][b], tr["token_mask"][b], ref["token_mask"][b])
            same_mask = ref["token_mask"] is None or torch.equal(tr["token_mask"], ref["token_mask"])
            assert tr["topk"] == ref["stats"]["top_k"]
            ok_tok = torch.ones(x.shape[:2], dtype=torch.bool)
            if ref["token_idx"] is not None and same_mask:
                H = layer.s.h_total
                ref_rows = _rows_to_mask(ref, x.size(0), H, x.size(1))
                got_rows = _rows_to_mask({"token_idx": tr["packed"][1], "row_offsets": tr["packed"][2],
                                          "active_head_indices": torch.arange(x.size(0) * H)}, x.size(0), H, x.size(1))
                ok_tok = ~(ref_rows ^ got_rows).any(dim=1)  # (B,T): same head set
                hp = tr["gate_probs"] @ layer.onehot
                for b, t in (~ok_tok).nonzero().tolist():
                    srt = torch.sort(hp[b, t], descending=True).values
                    assert float(srt[tr["topk"] - 1] - srt[tr["topk"]]) < 1e-6  # a genuine tie at the cut
                assert int((~ok_tok).sum()) <= 2
                if bool(ok_tok.all()):
                    assert torch.equal(tr["packed"][1], ref["token_idx"])
                    assert torch.equal(tr["candidates"], ref["candidates"])
                    assert torch.equal(tr["lengths"], ref["lengths"])
            if same_mask:
                tol = dict(atol=2e-2, rtol=1e-2) if bf16 else dict(atol=1e-5, rtol=1e-4)
                assert torch.allclose(y.float()[ok_tok], ref["y"].float()[ok_tok], **tol)
            assert torch.allclose(layer.protos, ref["protos_after"], atol=1e-5, rtol=1e-4)
            assert torch.allclose(layer.usage, ref["usage_after"], atol=1e-3, rtol=1e-4)
            assert torch.allclose(layer.conf, ref["conf_after"], atol=1e-6)
            if "memory_after" in ref and same_mask and bool(ok_tok.all()):   # the bank after this call (aspa.py:932-969)
                m, want = layer.memory, ref["memory_after"]
                mtol = dict(atol=2e-2, rtol=2e-2) if bf16 else dict(atol=1e-5, rtol=1e-4)
                assert torch.equal(m.ptr, want["ptr"])
                assert torch.allclose(m.counts, want["counts"], atol=1e-5, rtol=1e-6)
                assert torch.allclose(m.keys, want["keys"], **mtol) and torch.allclose(m.values, want["values"], **mtol)
        else:
            assert torch.allclose(y.float(), ref["y"].float(), atol=1e-5, rtol=1e-4)


def test_chunked_pipeline_matches_reference(golden_dir):
    for c in _load(golden_dir, "chunked.pt"):
        assert c["used_fallback"] is False
        r = O.chunked_run(c["seq"], chunk_len=c["chunk_len"], buffer_tokens=c["buffer"],
                          per_chunk_budget=c["budget"], heads=c["heads"], chunk_weights=c["chunk_weights"],
                          final_weights=c["final_weights"], warmup_input=c["warmup"])
        assert torch.equal(r["keep_indices"], c["keep_indices"])
        assert torch.allclose(r["keep_scores"], c["keep_scores"], atol=1e-6)
        assert torch.allclose(r["final_output"], c["final_output"], atol=1e-5, rtol=1e-4)


def test_oracle_matches_reference_at_baseline_config1_full_size(golden_dir):
    """1 x 4096 x 512 fp32, 8 heads, top-2, keep 0.25 (the reference's own CPU-runnable headline configuration): the
    oracle reproduces the token mask, the packed rows and the output rows the reference produced.  Weights and input
    are rebuilt from the seeds the fixture was generated with."""
    import sys
    sys.path.insert(0, str(golden_dir))
    import seeded
    g = _load(golden_dir, "layer_cfg1_full.pt")
    cfg = dict(seeded.CONFIG1)
    w = seeded.xavier_state(cfg["d_model"], cfg["attn_gates"], torch.float32, g["seed"])
    x = seeded.normal_input(1, 4096, cfg["d_model"], torch.float32, g["seed"])
    lay = O.OracleLayer(w, **cfg)
    y = lay.forward(x)
    tr = lay.trace
    assert tr["mode"] == g["mode"]
    assert torch.equal(tr["token_mask"], g["token_mask"])
    assert torch.equal(tr["packed"][1].to(torch.int32), g["token_idx"])
    assert torch.equal(tr["packed"][2].to(torch.int32), g["row_offsets"])
    assert float((tr["importance"] - g["importance"]).abs().max()) < 1e-6
    kept = g["token_mask"][0].nonzero().flatten()
    assert torch.allclose(y[0][kept], g["y_kept"], atol=1e-6, rtol=1e-5)
    assert float(y[0][~g["token_mask"][0]].abs().max()) == 0.0
