"""Layer-, wrapper- and pipeline-level parity: the CUDA path against the golden vectors recorded from
the reference and against the CPU oracle, stage by stage.  All tests need a CUDA device."""
import pytest
import torch

from oracle import aspa_oracle as O

pytestmark = pytest.mark.gpu

LAYER_CASES = ["layer_fp32_auto", "layer_fp32_proto", "layer_bf16_rope", "layer_bf16_int8",
               "layer_fp32_dense_fastpath", "layer_fp32_dense_density", "layer_fp32_nucleus",
               "layer_fp32_memory", "layer_bf16_int8_memory", "layer_bf16_int8_percentile", "layer_bf16_int8_ema"]


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _build(cfg, weights, dtype, dev):
    import proteus_flux_attention_b200 as P
    mod = P.AdaptiveSparseProtoAttention(P.ModelConfig(**cfg)).to(dtype)
    mod.load_state_dict(weights)
    return mod.to(dev).eval()


def _rows_mask(token_idx, row_offsets, heads, T):
    m = torch.zeros(heads, T, dtype=torch.bool)
    offs = row_offsets.long().tolist()
    for h in range(heads):
        m[h, token_idx[offs[h]:offs[h + 1]].long()] = True
    return m


def check_layer(mod, ora, x, dev, bf16):
    """Run both sides on x; check every stage of the CUDA path against the oracle fed with the CUDA
    path's own upstream results (exact where the stage is integer work), then end to end."""
    B, T, C = x.shape
    s = ora.s
    protos0 = ora.protos.clone() if ora.protos is not None else None
    y = mod(x.to(dev))
    st = mod._last_sparse_state
    y_o = ora.forward(x)
    tr = ora.trace
    report = {"mode": st["mode"]}
    if tr["mode"] == "dense_fastpath":
        assert st["mode"] == "dense_fastpath"
        tol = dict(atol=2e-2, rtol=1e-2) if bf16 else dict(atol=1e-5, rtol=1e-4)
        assert torch.allclose(y.cpu().float(), y_o.float(), **tol)
        return report
    # -- router ------------------------------------------------------------------------------
    imp = mod._last_token_importance.cpu()
    gate = mod._last_gate_probs.cpu()
    d_imp = (imp - tr["importance"]).abs()
    if bf16:
        assert (d_imp > 1e-5).float().mean() < 1e-2
    else:
        assert d_imp.max() < 2e-6, float(d_imp.max())
        assert (gate - tr["gate_probs"]).abs().max() < 2e-6
    # -- token keep: exact on the device's own importance ------------------------------------------
    if s.token_sparse:
        want_mask = O.select_active_tokens(s, imp, tr["keep_ratio"])
        assert torch.equal(mod._last_token_mask.cpu(), want_mask)
        report["mask_equal_e2e"] = bool(torch.equal(want_mask, tr["token_mask"]))
    else:
        want_mask = None
    # -- head choice: exact on the device's own gate probabilities (up to last-bit ties) -----------
    hp = gate @ ora.onehot
    topk = mod.last_head_stats["top_k"]
    assert topk == tr["topk"]
    _, hidx = O.head_topk(hp, topk)
    hm = torch.zeros(B, T, s.h_total, dtype=torch.bool).scatter_(2, hidx, True)
    if want_mask is not None:
        hm &= want_mask.unsqueeze(-1)
    flat = hm.permute(0, 2, 1).reshape(B * s.h_total, T)
    assert mod.last_head_stats["max_active_rows"] == int(flat.sum(1).max()) or bf16
    if st["mode"] == "shortlist":
        got_rows = _rows_mask(st["token_idx"].cpu(), st["row_offsets_all"].cpu(), B * s.h_total, T)
        assert (got_rows != flat).any(dim=0).float().mean() < 5e-3
    # percentile INT8 bases carry state from call to call: those cases are checked end to end (and in test_gpu_kernels)
    if st["mode"] == "shortlist" and not (s.quantize_int8 and s.quantize_mode != "max"):
        # -- attention on the device's own rows: consensus vs oracle attention over the same rows ---
        q, k, v, _ = mod._project_qkv(x.to(dev))
        packed = O.pack_active_rows(got_rows)
        rt = mod._linear_runtime
        sim = mod._last_token_similarity.cpu() if (s.linear_use_proto and mod._last_token_similarity is not None) else None
        cand, lens = O.build_candidates(packed[1], (packed[0] // s.h_total) if sim is not None else None, T,
                                        max_candidates=rt["effective_L"], linear_window=rt["window"],
                                        anchor_stride=s.linear_anchor_stride, use_local=s.linear_use_local,
                                        use_anchors=s.linear_use_anchors, proto_scores=sim, local_cap=rt["local_cap"],
                                        anchor_cap=rt["anchor_cap"], proto_cap=rt["proto_cap"])
        qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
        if s.quantize_int8:
            (qq, sq), (kq, sk), (vq, sv) = (O.quantize_per_head_int8(t) for t in (qc, kc, vc))
            att = O.sparse_attention(qq, kq, vq, packed=packed, candidates=cand, lengths=lens, q_scale=sq, k_scale=sk,
                                     v_scale=sv, out_dtype=qc.dtype)
        else:
            att = O.sparse_attention(qc, kc, vc, packed=packed, candidates=cand, lengths=lens)
        to_btc = lambda a: a.view(B, s.h_total, T, s.d_head).permute(0, 2, 1, 3).reshape(B, T, C).float()  # noqa: E731
        got_cons = mod.last_head_consensus.cpu().float()
        if bf16 and not s.quantize_int8:
            # The reference evaluates scores and softmax in bf16, which costs it several percent on rows with large
            # logits; the kernel accumulates in fp32.  So: the stated tolerance must hold everywhere against the same
            # algorithm evaluated in fp32, and on all but a sliver of elements against the bf16 evaluation.
            att32 = O.sparse_attention(qc.float(), kc.float(), vc.float(), packed=packed, candidates=cand, lengths=lens)
            assert torch.allclose(got_cons, to_btc(att32), atol=2e-2, rtol=1e-2)
            off = ~torch.isclose(got_cons, to_btc(att), atol=2e-2, rtol=1e-2)
            report["bf16_eval_outliers"] = float(off.float().mean())
            assert off.float().mean() < 1e-3
        else:
            tol = dict(atol=2e-2, rtol=1e-2) if bf16 else dict(atol=1e-5, rtol=1e-4)
            assert torch.allclose(got_cons, to_btc(att), **tol)
        report["rows"] = int(packed[1].numel())
    # -- end to end --------------------------------------------------------------------------------
    tol = dict(atol=2e-2, rtol=1e-2) if bf16 else dict(atol=1e-5, rtol=1e-4)
    same_tok = torch.ones(B, T, dtype=torch.bool)
    if st["mode"] == "shortlist" and tr["mode"] == "shortlist":
        ref_rows = _rows_mask(tr["packed"][1], tr["packed"][2], B * s.h_total, T)
        same_tok = ~(ref_rows != got_rows).view(B, s.h_total, T).any(dim=1)
    frac = float(same_tok.float().mean())
    report["same_routing_fraction"] = frac
    assert frac > (0.97 if bf16 else 0.999)
    off = ~torch.isclose(y.cpu().float(), y_o.float(), **tol)
    off &= same_tok.unsqueeze(-1)
    report["e2e_outliers"] = float(off.float().mean())
    assert off.float().mean() < (1e-3 if bf16 else 1e-12)
    # -- prototype EMA -------------------------------------------------------------------------------
    if protos0 is not None and s.proto_decay != 1.0:
        assert torch.allclose(mod.routing_prototypes.cpu(), ora.protos, atol=1e-4, rtol=1e-3)
        assert torch.allclose(mod.routing_confidence.cpu(), ora.conf, atol=1e-6)
    return report


@pytest.mark.parametrize("name", LAYER_CASES)
def test_layer_matches_golden_and_oracle(dev, golden_dir, name):
    g = torch.load(golden_dir / f"{name}.pt", weights_only=False)
    bf16 = "bfloat16" in g["dtype"]
    dtype = torch.bfloat16 if bf16 else torch.float32
    mod = _build(g["cfg"], g["weights"], dtype, dev)
    ora = O.OracleLayer(g["weights"], **g["cfg"])
    for x, ref in zip(g["x"], g["out"]):
        rep = check_layer(mod, ora, x, dev, bf16)
        assert rep["mode"] == ref["mode"]
        # and directly against what the reference produced
        y = mod.last_head_consensus  # noqa: F841  (kept for debugging)
        if ref["token_mask"] is not None and not bf16:
            assert torch.equal(mod._last_token_mask.cpu(), ref["token_mask"])
        if not bf16 and ref["mode"] != "dense_fastpath":
            assert mod.last_head_stats["top_k"] == ref["stats"]["top_k"]
            for key in ("mean_gate_prob", "router_entropy", "mean_active_per_token", "active_fraction",
                        "max_active_density", "token_keep_fraction"):
                assert abs(mod.last_head_stats[key] - ref["stats"][key]) < 1e-4, key
            assert mod.last_head_stats["unique_heads"] == ref["stats"]["unique_heads"]
            assert mod.last_head_stats["max_active_rows"] == ref["stats"]["max_active_rows"]
        if "memory_after" in ref:   # the key/value memory bank after this call, against the reference's and the oracle's
            want = ref["memory_after"]
            mtol = dict(atol=5e-2, rtol=5e-2) if bf16 else dict(atol=1e-5, rtol=1e-4)
            assert torch.equal(mod.memory_ptr.cpu(), want["ptr"]) and torch.equal(ora.memory.ptr, want["ptr"])
            assert mod.memory_keys.dtype == torch.float32
            assert torch.allclose(mod.memory_counts.cpu(), want["counts"], atol=(3.0 if bf16 else 1e-5))
            assert torch.allclose(mod.memory_keys.cpu(), want["keys"], **mtol)
            assert torch.allclose(mod.memory_values.cpu(), want["values"], **mtol)
            assert float(want["keys"].abs().max()) > 0.05


def test_layer_state_dict_roundtrip_and_fp32_buffers(dev):
    import proteus_flux_attention_b200 as P
    cfg = dict(d_model=128, n_head=8, attn_h_total=8, attn_proto_enable=True, n_ctx=512)
    a = P.AdaptiveSparseProtoAttention(P.ModelConfig(**cfg))
    keys = set(a.state_dict().keys())
    assert keys == {"qkv.weight", "proj.weight", "head_router.linear.weight", "routing_prototypes",
                    "routing_usage_ema", "routing_confidence"}
    b = P.AdaptiveSparseProtoAttention(P.ModelConfig(**cfg))
    b.load_state_dict(a.state_dict())
    b = b.to(device=dev, dtype=torch.bfloat16)
    assert b.qkv.weight.dtype == torch.bfloat16
    assert b._rope_inv_freq.dtype == torch.float32 and b.routing_prototypes.dtype == torch.float32
    assert not b._rope_cache
    x = torch.randn(1, 300, 128, device=dev, dtype=torch.bfloat16)
    y = b(x)
    assert y.shape == x.shape and torch.isfinite(y.float()).all()
    assert b._rope_cache


def test_layer_rejects_cpu_and_wrong_dtype(dev):
    import proteus_flux_attention_b200 as P
    m = P.AdaptiveSparseProtoAttention(P.ModelConfig(d_model=64, n_head=4, attn_h_total=4))
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(torch.randn(1, 16, 64))
    m = m.to(dev)
    with pytest.raises(TypeError):
        m(torch.randn(1, 16, 64, device=dev, dtype=torch.float16))


def test_layer_is_deterministic_and_mutates_prototypes(dev):
    import proteus_flux_attention_b200 as P
    torch.manual_seed(0)
    cfg = dict(d_model=128, n_head=8, attn_h_total=8, attn_gates=8, attn_token_sparse=True, attn_token_keep_ratio=0.4,
               n_ctx=2048, attn_router_top_p=0.0, attn_track_latency=False)
    m = P.AdaptiveSparseProtoAttention(P.ModelConfig(**cfg)).to(dev).eval()
    state = {k: v.clone() for k, v in m.state_dict().items()}
    x = torch.randn(2, 1024, 128, device=dev)
    y1 = m(x)
    p1 = m.routing_prototypes.clone()
    assert not torch.equal(p1, state["routing_prototypes"])  # eval-mode forward updates the EMA, like the reference
    m.load_state_dict(state)
    y2 = m(x)
    assert torch.equal(y1, y2) and torch.equal(p1, m.routing_prototypes)


def test_random_layers_against_oracle(dev):
    import proteus_flux_attention_b200 as P
    cases = [
        (dict(d_model=128, n_head=8, attn_h_total=8, attn_gates=16, attn_h_active=3, attn_h_active_min=3,
              attn_h_active_max=3, attn_linear_head_k=3, attn_token_sparse=True, attn_token_keep_ratio=0.3, n_ctx=1024,
              attn_router_top_p=0.0, attn_linear_L=64, attn_linear_window=48, attn_linear_anchor_stride=16,
              attn_linear_switch_ctx=700, attn_track_latency=False, attn_proto_enable=True), 2, 600, torch.float32),
        (dict(d_model=256, n_head=4, attn_h_total=4, attn_gates=8, attn_h_active=2, attn_h_active_min=2,
              attn_h_active_max=2, attn_token_sparse=True, attn_token_keep_ratio=0.2, n_ctx=2048, attn_mode="linear",
              attn_linear_policy="local+anchors+proto", attn_linear_L=128, attn_linear_L_max=128,
              attn_linear_window=128, attn_linear_anchor_stride=32, attn_router_top_p=0.0,
              attn_track_latency=False, attn_proto_enable=True, attn_proto_threshold=0.02), 1, 1500, torch.bfloat16),
    ]
    for cfg, B, T, dtype in cases:
        torch.manual_seed(3)
        old = torch.get_default_dtype()
        torch.set_default_dtype(dtype)
        try:
            mod = P.AdaptiveSparseProtoAttention(P.ModelConfig(**cfg))
        finally:
            torch.set_default_dtype(old)
        with torch.no_grad():
            for w in (mod.qkv.weight, mod.proj.weight, mod.head_router.linear.weight, mod.routing_prototypes):
                torch.nn.init.xavier_uniform_(w)
        weights = {k: v.clone() for k, v in mod.state_dict().items()}
        ora = O.OracleLayer(weights, **cfg)
        mod = mod.to(dev).eval()
        g = torch.Generator().manual_seed(4)
        x = torch.randn(B, T, cfg["d_model"], generator=g)
        x[:, ::97] *= 4.0
        rep = check_layer(mod, ora, x.to(dtype), dev, dtype == torch.bfloat16)
        assert rep["mode"] == "shortlist"


# ------------------------------------------------------------------------------------------ drop-in wrapper
def test_multihead_wrapper_contract(dev):
    import proteus_flux_attention_b200 as P
    torch.manual_seed(0)
    m = P.CausalASPAMultiheadAttention(64, 4, batch_first=True, max_seq_len=256, return_stats_default=True).to(dev).eval()
    x = torch.randn(2, 96, 64, device=dev)
    state0 = {k: v.clone() for k, v in m.state_dict().items()}  # every forward moves the prototype EMA
    out, w = m(x)
    assert out.shape == x.shape and w.shape == (2, 96, 96) and float(w.abs().sum()) == 0.0
    assert m.last_runtime_stats["head_stats"]["seq_len"] == 96
    out2, w2 = m(x, need_weights=False)
    assert w2 is None
    # key padding: padded positions are zeroed on the way in and out
    pad = torch.zeros(2, 96, dtype=torch.bool, device=dev)
    pad[:, 80:] = True
    out3, _ = m(x, key_padding_mask=pad, need_weights=False)
    assert float(out3[:, 80:].abs().sum()) == 0.0
    with pytest.raises(ValueError, match="key_padding_mask"):
        m(x, key_padding_mask=pad[:, :10])
    # sequence-first layout
    m2 = P.CausalASPAMultiheadAttention(64, 4, batch_first=False).to(dev).eval()
    o, _ = m2(x.transpose(0, 1).contiguous(), need_weights=False)
    assert o.shape == (96, 2, 64)
    # fallbacks equal nn.MultiheadAttention with the fallback weights
    kv = torch.randn(2, 50, 64, device=dev)
    got, _ = m(x, kv, kv, need_weights=False)
    want, _ = m.fallback_attention(x, kv, kv, need_weights=False)
    assert torch.allclose(got, want, atol=1e-6)
    assert m.last_runtime_stats["shortlist_backend"]["details"]["reason"] == "cross_attention"
    band = torch.zeros(96, 96, device=dev)
    band[0, 5] = float("-inf")
    got, _ = m(x, attn_mask=band, need_weights=False)
    want, _ = m.fallback_attention(x, x, x, attn_mask=band, need_weights=False)
    assert torch.allclose(got, want, atol=1e-6)
    causal = torch.triu(torch.full((96, 96), float("-inf"), device=dev), diagonal=1)
    m.load_state_dict(state0)
    got, _ = m(x, attn_mask=causal, need_weights=False)
    assert torch.equal(got, out)
    with pytest.raises(ValueError, match="divisible"):
        P.CausalASPAMultiheadAttention(65, 4)


def test_controller_and_block(dev):
    import proteus_flux_attention_b200 as P
    m = P.CausalASPAMultiheadAttention(64, 4, sparse_ctl_config=dict(target_density=0.01, tolerance=0.0, cooldown=2),
                                       attn_h_active=4, attn_h_active_min=1).to(dev).eval()
    x = torch.randn(1, 128, 64, device=dev)
    before = m.attention.h_active_max
    for _ in range(2):
        m(x, need_weights=False, return_stats=True)
    assert m.sparse_controller.last_snapshot.action == "decrease"
    assert m.attention.h_active_max == before - 1
    blk = P.CausalASPATransformerBlock(64, 4, dim_feedforward=128, dropout=0.0).to(dev).eval()
    y = blk(x)
    assert y.shape == x.shape and torch.isfinite(y).all()
    y2, w = blk(x, return_attn=True)
    assert w.shape == (1, 128, 128)


# ------------------------------------------------------------------------------------------ chunked pipeline
def test_chunked_pipeline_matches_golden(dev, golden_dir):
    import proteus_flux_attention_b200 as P
    for c in torch.load(golden_dir / "chunked.pt", weights_only=False):
        cfg = P.ChunkedShortlistConfig(seq_len=c["seq_len"], d_model=c["d_model"], chunk_len=c["chunk_len"],
                                       buffer_tokens=c["buffer"], per_chunk_budget=c["budget"], device=dev,
                                       heads=c["heads"], storage="cpu")
        for seq in (c["seq"], c["seq"].to(dev)):  # host-streamed and HBM-resident input
            res = P.ChunkedShortlistRunner(cfg).run(seq, chunk_state=c["chunk_weights"], final_state=c["final_weights"],
                                                    warmup_input=c["warmup"])
            assert res.keep_indices.device.type == "cpu"
            assert torch.equal(res.keep_indices, c["keep_indices"])
            assert torch.allclose(res.keep_scores, c["keep_scores"], atol=1e-6)
            assert torch.equal(res.reduced_sequence.cpu(), c["seq"][:, c["keep_indices"]])
            assert torch.allclose(res.final_output.cpu(), c["final_output"], atol=1e-5, rtol=1e-4)
            assert res.metrics.used_fallback is False and res.metrics.retained_tokens == c["keep_indices"].numel()
            assert [s.promoted for s in res.chunks] == [t.tolist() for t in c["chunk_idx"]]


def test_chunked_scoring_only_equals_full_forward(dev):
    import proteus_flux_attention_b200 as P
    torch.manual_seed(1)
    seq = torch.randn(1, 4096, 128, device=dev)
    base = dict(seq_len=4096, d_model=128, chunk_len=1024, buffer_tokens=300, per_chunk_budget=100, device=dev, heads=8,
                freeze_prototypes=False, warmup=False)
    ref_layer = P.AdaptiveSparseAttention(P.chunked_shortlist._build_model_config(
        1024, 128, heads=8, sparse_ratio=0.05, shortlist_alpha=1.0, router_top_p=0.9))
    st = ref_layer.state_dict()
    fin_layer = P.AdaptiveSparseAttention(P.chunked_shortlist._build_model_config(
        300, 128, heads=8, sparse_ratio=0.5, shortlist_alpha=1.0, router_top_p=0.9))
    fs = fin_layer.state_dict()
    a = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**base, pass1_full_forward=True)).run(seq, chunk_state=st, final_state=fs)
    b = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**base, pass1_full_forward=False)).run(seq, chunk_state=st, final_state=fs)
    assert torch.equal(a.keep_indices, b.keep_indices) and torch.equal(a.final_output, b.final_output)
    ora = O.chunked_run(seq.cpu(), chunk_len=1024, buffer_tokens=300, per_chunk_budget=100, heads=8, chunk_weights=st,
                        final_weights=fs)
    assert torch.equal(a.keep_indices, ora["keep_indices"])
    assert torch.allclose(a.final_output.cpu(), ora["final_output"], atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_projection_on_kept_rows_equals_full_projection(dev, dtype):
    """Projecting q / the output for kept tokens only must give what projecting every token gives."""
    import proteus_flux_attention_b200 as P
    cfg = dict(d_model=128, n_head=8, attn_h_total=8, attn_gates=8, attn_h_active=2, attn_h_active_min=2, attn_h_active_max=2,
               attn_token_sparse=True, attn_token_keep_ratio=0.3, attn_mode="auto", attn_small_seq_dense=0,
               attn_router_top_p=0.0, attn_use_rope=True, n_ctx=1024, attn_proto_enable=True, bias=True)
    torch.manual_seed(3)
    layer = P.AdaptiveSparseProtoAttention(P.ModelConfig(**cfg)).to(dtype).to(dev).eval()
    with torch.no_grad():
        layer.proj.bias.normal_()
        layer.qkv.bias.normal_()
    state = {k: v.clone() for k, v in layer.state_dict().items()}
    x = torch.randn(2, 700, 128, device=dev).to(dtype)
    outs, cons = [], []
    for flag in (True, False):
        layer.load_state_dict(state)
        layer.compact_projection = flag
        outs.append(layer(x).float())
        cons.append(layer.last_head_consensus.float())
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert float((outs[0] - outs[1]).abs().max()) <= tol
    assert float((cons[0] - cons[1]).abs().max()) <= tol
    kept = layer._last_token_mask
    assert 0 < int(kept.sum()) < kept.numel()
    # rows of dropped tokens are exactly the projection bias
    assert torch.equal(outs[0][~kept], layer.proj.bias.float().expand_as(outs[0])[~kept])


def test_chunked_pipeline_graph_replay_equals_eager(dev):
    """Pass 1 replayed from captured graphs (promotion forked inside, double-buffered inputs) and pass 2 from its own
    graph must give what the eager pipeline gives, run after run, for resident and host-streamed sequences."""
    import proteus_flux_attention_b200 as P
    from proteus_flux_attention_b200.chunked_shortlist import _build_model_config
    torch.manual_seed(11)
    mk = lambda n, r: P.AdaptiveSparseAttention(_build_model_config(n, 256, heads=4, sparse_ratio=r, shortlist_alpha=1.0,  # noqa: E731
                                                                   router_top_p=0.9))
    cast = lambda sd: {k: v.to(torch.bfloat16) if v.dtype == torch.float32 and "routing" not in k else v for k, v in sd.items()}  # noqa: E731
    cs, fs = cast(mk(2048, 0.05).state_dict()), cast(mk(512, 0.5).state_dict())
    seq = torch.randn(1, 5 * 2048 + 300, 256, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    base = dict(seq_len=seq.size(1), d_model=256, chunk_len=2048, buffer_tokens=512, per_chunk_budget=128, device=dev, heads=4,
                freeze_prototypes=True, warmup=False)
    want = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**base)).run(seq.to(dev), chunk_state=cs, final_state=fs)
    runner = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**base, use_cuda_graph=True), cache_layers=True)
    for source in (seq.to(dev), seq.pin_memory(), seq.to(dev)):
        got = runner.run(source, chunk_state=cs, final_state=fs)
        assert torch.equal(got.keep_indices, want.keep_indices)
        assert torch.equal(got.keep_scores, want.keep_scores)
        assert torch.equal(got.reduced_sequence.cpu(), want.reduced_sequence.cpu())
        assert torch.equal(got.final_output.cpu(), want.final_output.cpu())
        assert got.final_stats["sparse_state"]["mode"] == want.final_stats["sparse_state"]["mode"]
        assert [c.promoted for c in got.chunks] == [c.promoted for c in want.chunks]
    # a buffer the promotions cannot fill: the graph path enqueues pass 2 for min(buffer, chunks * budget) kept tokens
    # before the real count is known, finds fewer (the short last chunk promotes only what it kept) and repeats it
    wide = dict(base, buffer_tokens=1024)
    want = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**wide)).run(seq.to(dev), chunk_state=cs, final_state=fs)
    assert want.keep_indices.numel() < 6 * 128
    runner = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**wide, use_cuda_graph=True), cache_layers=True)
    for source in (seq.to(dev), seq.pin_memory()):
        got = runner.run(source, chunk_state=cs, final_state=fs)
        assert torch.equal(got.keep_indices, want.keep_indices)
        assert torch.equal(got.reduced_sequence.cpu(), want.reduced_sequence.cpu())
        assert torch.equal(got.final_output.cpu(), want.final_output.cpu())
    with pytest.raises(ValueError, match="freeze_prototypes"):
        P.ChunkedShortlistConfig(**{**base, "freeze_prototypes": False}, use_cuda_graph=True).validate()


def test_chunked_pipeline_whole_run_graph_equals_eager(dev):
    """The whole run replayed from ONE captured graph (reset, pass 1 on two lanes, merge, gather, pass 2, read-backs)
    gives what the eager pipeline gives, replay after replay; a sequence at another address is captured afresh, a
    buffer the promotions cannot fill falls back to the chunk-by-chunk path, and so does a ragged last chunk."""
    import proteus_flux_attention_b200 as P
    from proteus_flux_attention_b200.chunked_shortlist import _build_model_config
    torch.manual_seed(12)
    mk = lambda n, r: P.AdaptiveSparseAttention(_build_model_config(n, 256, heads=4, sparse_ratio=r, shortlist_alpha=1.0,  # noqa: E731
                                                                   router_top_p=0.9))
    cast = lambda sd: {k: v.to(torch.bfloat16) if v.dtype == torch.float32 and "routing" not in k else v for k, v in sd.items()}  # noqa: E731
    cs, fs = cast(mk(2048, 0.05).state_dict()), cast(mk(512, 0.5).state_dict())
    seq = torch.randn(1, 6 * 2048, 256, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    base = dict(seq_len=seq.size(1), d_model=256, chunk_len=2048, buffer_tokens=512, per_chunk_budget=128, device=dev, heads=4,
                freeze_prototypes=True, warmup=False)
    want = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**base)).run(seq.to(dev), chunk_state=cs, final_state=fs)
    cfg = P.ChunkedShortlistConfig(**base, use_cuda_graph=True, whole_run_graph=True, collect_summaries=False)
    runner = P.ChunkedShortlistRunner(cfg, cache_layers=True)
    a, b = seq.to(dev), seq.to(dev).clone()
    for source in (a, a, b, a):
        got = runner.run(source, chunk_state=cs, final_state=fs)
        assert "whole_run_graph" in runner.last_phase_ms
        assert torch.equal(got.keep_indices, want.keep_indices)
        assert torch.equal(got.keep_scores, want.keep_scores)
        assert torch.equal(got.reduced_sequence.cpu(), want.reduced_sequence.cpu())
        assert torch.equal(got.final_output.cpu(), want.final_output.cpu())
    # a host sequence, a ragged last chunk and an unfillable buffer take the chunk-by-chunk path and still agree
    got = runner.run(seq.pin_memory(), chunk_state=cs, final_state=fs)
    assert "whole_run_graph" not in runner.last_phase_ms and torch.equal(got.keep_indices, want.keep_indices)
    wide = dict(base, buffer_tokens=1024)
    ragged = {**wide, "seq_len": seq.size(1) - 100}
    want = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**ragged)).run(seq[:, :-100].to(dev), chunk_state=cs, final_state=fs)
    cfgw = P.ChunkedShortlistConfig(**ragged, use_cuda_graph=True, whole_run_graph=True, collect_summaries=False)
    got = P.ChunkedShortlistRunner(cfgw, cache_layers=True).run(seq[:, :-100].to(dev), chunk_state=cs, final_state=fs)
    assert torch.equal(got.keep_indices, want.keep_indices) and torch.equal(got.final_output.cpu(), want.final_output.cpu())
    want = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**wide)).run(seq.to(dev), chunk_state=cs, final_state=fs)
    runner = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**wide, use_cuda_graph=True, whole_run_graph=True,
                                                               collect_summaries=False), cache_layers=True)
    for _ in range(2):
        got = runner.run(a, chunk_state=cs, final_state=fs)
        assert torch.equal(got.keep_indices, want.keep_indices) and torch.equal(got.final_output.cpu(), want.final_output.cpu())


def test_captured_layer_call_equals_eager(dev):
    """A layer call replayed from a captured graph gives what the eager call gives, state updates included (the
    prototype EMA moves with every replay); a call that must wait for the host refuses to be captured."""
    import proteus_flux_attention_b200 as P
    cfg = dict(d_model=256, n_head=4, attn_h_total=4, attn_gates=8, attn_h_active=2, attn_h_active_min=2,
               attn_h_active_max=2, attn_token_sparse=True, attn_token_keep_ratio=0.3, attn_router_top_p=0.0,
               attn_mode="linear", attn_linear_L=96, attn_linear_window=64, attn_linear_anchor_stride=16, n_ctx=2048,
               attn_track_latency=False, attn_proto_enable=True, attn_quantize_int8=True)
    torch.manual_seed(5)
    make = lambda c: P.AdaptiveSparseProtoAttention(P.ModelConfig(**c)).to(torch.bfloat16).to(dev).eval()  # noqa: E731
    a = make(cfg)
    b = make(cfg)
    b.load_state_dict(a.state_dict())
    g = torch.Generator().manual_seed(6)
    xs = [torch.randn(2, 1536, 256, generator=g).to(torch.bfloat16).to(dev) for _ in range(3)]
    call = P.CapturedLayerCall(b, xs[0])
    assert all(torch.equal(v, b.state_dict()[k]) for k, v in a.state_dict().items())   # capture left the state alone
    for x in xs:
        want = a(x)
        got = call(x).clone()
        assert torch.equal(got, want)
        assert torch.equal(a.routing_prototypes, b.routing_prototypes)
        assert a.last_head_stats["top_k"] == b.last_head_stats["top_k"]
        assert a._last_sparse_state["mode"] == b._last_sparse_state["mode"] == "shortlist"
    with pytest.raises(ValueError):
        call(xs[0][:, :100])
    # alpha < 0.95 alone does not stop a capture (a kept-token bound below the density threshold rules dense out) ...
    auto = make(dict(cfg, attn_mode="auto", attn_linear_switch_ctx=4000, attn_quantize_int8=False))
    ref_auto = make(dict(cfg, attn_mode="auto", attn_linear_switch_ctx=4000, attn_quantize_int8=False))
    ref_auto.load_state_dict(auto.state_dict())
    call_auto = P.CapturedLayerCall(auto, xs[0])
    assert torch.equal(call_auto(xs[1]), ref_auto(xs[1])) and 0.0 < auto._current_alpha < 0.95
    # ... a keep threshold does: how many tokens survive is then only known on the device
    slow = make(dict(cfg, attn_token_keep_threshold=0.5))
    with pytest.raises(RuntimeError, match="cannot be captured"):
        P.CapturedLayerCall(slow, xs[0])


def test_chunked_graphs_do_not_outlive_their_layers(dev):
    """Without ``cache_layers`` every ``run`` builds fresh layers; graphs captured in one call must not be replayed
    by the next, whose layers (and weights) are different objects.  Two graph runs with different weights must each
    equal the eager run with the same weights."""
    import proteus_flux_attention_b200 as P
    from proteus_flux_attention_b200.chunked_shortlist import _build_model_config
    T, C, chunk = 4 * 2048, 256, 2048
    seq = torch.randn(1, T, C, generator=torch.Generator().manual_seed(21)).to(torch.bfloat16).to(dev)

    def states(seed):
        torch.manual_seed(seed)
        a = P.AdaptiveSparseAttention(_build_model_config(chunk, C, heads=4, sparse_ratio=0.05, shortlist_alpha=1.0, router_top_p=0.9))
        b = P.AdaptiveSparseAttention(_build_model_config(256, C, heads=4, sparse_ratio=0.5, shortlist_alpha=1.0, router_top_p=0.9))
        return tuple({k: (v.to(torch.bfloat16) if v.dtype == torch.float32 and "routing" not in k else v)
                      for k, v in m.state_dict().items()} for m in (a, b))

    def cfg(graph):
        return P.ChunkedShortlistConfig(seq_len=T, d_model=C, chunk_len=chunk, buffer_tokens=256, per_chunk_budget=64,
                                        device=dev, heads=4, freeze_prototypes=True, warmup=False, use_cuda_graph=graph)

    graph_runner = P.ChunkedShortlistRunner(cfg(True))            # cache_layers=False
    for seed in (31, 32):
        cs, fs = states(seed)
        got = graph_runner.run(seq, chunk_state=cs, final_state=fs)
        want = P.ChunkedShortlistRunner(cfg(False)).run(seq, chunk_state=cs, final_state=fs)
        assert torch.equal(got.keep_indices, want.keep_indices)
        assert torch.equal(got.final_output, want.final_output)
    assert "_graph_tmp" not in graph_runner.__dict__


def test_rope_table_survives_a_longer_eager_call_between_replays(dev):
    """A captured call keeps the address of the RoPE table it was captured with; an eager call at a larger length on
    the same layer must not free or move that table."""
    import proteus_flux_attention_b200 as P
    cfg = dict(d_model=128, n_head=4, attn_h_total=4, attn_gates=8, attn_h_active=2, attn_h_active_min=2,
               attn_h_active_max=2, attn_token_sparse=True, attn_token_keep_ratio=0.3, attn_mode="linear",
               attn_router_top_p=0.0, attn_linear_L=64, attn_linear_window=48, attn_linear_anchor_stride=16,
               attn_use_rope=True, n_ctx=512, attn_track_latency=False, attn_proto_enable=True, attn_proto_decay=1.0)
    torch.manual_seed(2)
    layer = P.AdaptiveSparseProtoAttention(P.ModelConfig(**cfg)).to(torch.bfloat16).to(dev).eval()
    x = torch.randn(1, 512, 128, device=dev).to(torch.bfloat16)
    want = layer(x).clone()
    call = P.CapturedLayerCall(layer, x)
    assert torch.equal(call(x), want)
    big = torch.randn(1, 2048, 128, device=dev).to(torch.bfloat16)
    layer(big)                                    # grows the table past n_ctx
    junk = [torch.full((1 << 16,), 7.0, device=dev) for _ in range(64)]   # would land in freed table memory
    torch.cuda.synchronize()
    assert torch.equal(call(x), want)
    del junk


def test_captured_model_call_equals_eager(dev):
    """A model with two ASPA layers inside replayed from one captured graph gives what the eager model gives, state
    updates included; a model with a layer that must wait for the host refuses to be captured and is left untouched."""
    import proteus_flux_attention_b200 as P
    cfg = dict(d_model=256, n_head=4, attn_h_total=4, attn_gates=8, attn_h_active=2, attn_h_active_min=2,
               attn_h_active_max=2, attn_token_sparse=True, attn_token_keep_ratio=0.3, attn_router_top_p=0.0,
               attn_mode="linear", attn_linear_L=96, attn_linear_window=64, attn_linear_anchor_stride=16, n_ctx=2048,
               attn_track_latency=False, attn_proto_enable=True)

    class Two(torch.nn.Module):
        def __init__(self, **over):
            super().__init__()
            self.a = P.AdaptiveSparseProtoAttention(P.ModelConfig(**{**cfg, **over}))
            self.b = P.AdaptiveSparseProtoAttention(P.ModelConfig(**cfg))
            self.norm = torch.nn.LayerNorm(256)

        def forward(self, x):
            return x + self.b(self.norm(x + self.a(x)))

    torch.manual_seed(21)
    eager = Two().to(torch.bfloat16).to(dev).eval()
    twin = Two().to(torch.bfloat16).to(dev).eval()
    twin.load_state_dict(eager.state_dict())
    x = torch.randn(2, 1024, 256, device=dev).to(torch.bfloat16)
    call = P.CapturedModelCall(twin, x)
    for step in range(3):
        xs = torch.randn(2, 1024, 256, generator=torch.Generator().manual_seed(step)).to(dev).to(torch.bfloat16)
        with torch.no_grad():
            want = eager(xs)
        got = call(xs)
        assert torch.equal(got, want)
        for (n, p_e), (_, p_t) in zip(eager.named_buffers(), twin.named_buffers()):
            assert torch.equal(p_e, p_t), n   # prototype EMAs moved alike
    assert twin.b.last_head_stats is not None   # telemetry of the replayed call decodes
    needs_host = Two(attn_token_keep_threshold=0.5).to(torch.bfloat16).to(dev).eval()   # a keep threshold: counts on the host
    before = {n: b.clone() for n, b in needs_host.named_buffers()}
    with pytest.raises(RuntimeError, match="cannot be captured"):
        P.CapturedModelCall(needs_host, torch.randn(1, 256, 256, device=dev).to(torch.bfloat16))
    assert all(torch.equal(b, before[n]) for n, b in needs_host.named_buffers())


# ------------------------------------------------------------------------------------------ command lines
def test_chunked_cli_flags_and_report_layout(dev, tmp_path):
    """The chunk tool's command line takes the reference's flags and writes the reference's report layout."""
    from proteus_flux_attention_b200 import chunked_cli
    rep_path, idx_path = tmp_path / "r" / "report.json", tmp_path / "keep.pt"
    report = chunked_cli.main(["--seq-len", "8192", "--d-model", "128", "--chunk-len", "2048", "--buffer-tokens", "256",
                               "--per-chunk-budget", "64", "--heads", "4", "--chunk-sparse-ratio", "0.05",
                               "--final-sparse-ratio", "0.5", "--seed", "3", "--shortlist-alpha", "1.0", "--nucleus-top-p", "0.9",
                               "--device", "cuda:0", "--storage", "cpu", "--dtype", "fp32", "--save-report", str(rep_path),
                               "--save-indices", str(idx_path), "--log-level", "ERROR"])
    import json
    on_disk = json.loads(rep_path.read_text())
    assert set(on_disk) == {"metrics", "keep_indices", "keep_scores", "chunks", "backend_info", "final_stats"}
    assert on_disk["metrics"]["original_tokens"] == 8192 and on_disk["metrics"]["retained_tokens"] == len(on_disk["keep_indices"])
    assert on_disk["metrics"]["used_fallback"] is False and 0 < len(on_disk["keep_indices"]) <= 256
    assert on_disk["keep_indices"] == sorted(on_disk["keep_indices"]) == report["keep_indices"]
    assert {"index", "start", "end", "promoted", "scores"} <= set(on_disk["chunks"][0])
    assert torch.load(idx_path).tolist() == on_disk["keep_indices"]


def test_chunked_pipeline_disk_staging(dev, tmp_path):
    """storage="disk" stages the sequence in a float32 memory-mapped file (the reference's layout) and streams it from
    there: same kept tokens and outputs as the host-memory run, the reference's storage metrics, the file gone afterwards;
    "auto" and "cpu" fall back to disk when the sequence exceeds ram_limit_bytes."""
    import proteus_flux_attention_b200 as P
    from proteus_flux_attention_b200 import chunked_cli
    from proteus_flux_attention_b200.chunked_shortlist import _build_model_config
    torch.manual_seed(14)
    mk = lambda n, r: P.AdaptiveSparseAttention(_build_model_config(n, 128, heads=4, sparse_ratio=r, shortlist_alpha=1.0,  # noqa: E731
                                                                   router_top_p=0.9))
    cast = lambda sd: {k: v.to(torch.bfloat16) if v.dtype == torch.float32 and "routing" not in k else v for k, v in sd.items()}  # noqa: E731
    cs, fs = cast(mk(2048, 0.05).state_dict()), cast(mk(256, 0.5).state_dict())
    seq = torch.randn(1, 4 * 2048 + 500, 128, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    base = dict(seq_len=seq.size(1), d_model=128, chunk_len=2048, buffer_tokens=256, per_chunk_budget=64, device=dev, heads=4,
                freeze_prototypes=True, warmup=False)
    want = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**base, storage="cpu")).run(seq, chunk_state=cs, final_state=fs)
    assert want.metrics.storage_mode == "cpu" and want.metrics.host_allocated_mb > 0
    stage = tmp_path / "stage"
    for kw in (dict(storage="disk"), dict(storage="auto", ram_limit_bytes=1 << 16), dict(storage="cpu", ram_limit_bytes=1 << 16),
               dict(storage="disk", use_cuda_graph=True)):
        got = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**base, temp_dir=stage, **kw)).run(seq, chunk_state=cs, final_state=fs)
        assert got.metrics.storage_mode == "disk"
        assert got.metrics.host_required_mb == pytest.approx(seq.size(1) * 128 * 4 / (1024 * 1024))
        assert got.metrics.host_allocated_mb == pytest.approx(2048 * 128 * 4 / (1024 * 1024))
        if "ram_limit_bytes" in kw:
            assert "staging on disk" in got.metrics.storage_reason and got.metrics.host_limit_mb == pytest.approx(1 / 16)
        assert torch.equal(got.keep_indices, want.keep_indices) and torch.equal(got.keep_scores, want.keep_scores)
        assert torch.equal(got.reduced_sequence.cpu(), want.reduced_sequence.cpu())
        assert torch.equal(got.final_output.cpu(), want.final_output.cpu())
        assert list(stage.glob("*.mmap")) == []
    # a device-resident sequence asked onto disk goes there too; generated noise is staged block by block
    got = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**base, temp_dir=stage, storage="disk")).run(seq.to(dev), chunk_state=cs, final_state=fs)
    assert got.metrics.storage_mode == "disk" and torch.equal(got.keep_indices, want.keep_indices)
    report = chunked_cli.main(["--seq-len", "8192", "--d-model", "128", "--chunk-len", "2048", "--buffer-tokens", "256",
                               "--per-chunk-budget", "64", "--heads", "4", "--seed", "3", "--device", "cuda:0", "--storage", "disk",
                               "--temp-dir", str(stage), "--dtype", "bf16", "--log-level", "ERROR"])
    assert report["metrics"]["storage_mode"] == "disk" and 0 < len(report["keep_indices"]) <= 256
    assert list(stage.glob("*.mmap")) == []


def test_tinytoy_sweep_report_layout(dev, tmp_path):
    from proteus_flux_attention_b200 import tinytoy
    rec = tinytoy.main(["--max-seq-len", "1024", "--num-runs", "2", "--report-dir", str(tmp_path)])
    assert {"device", "safe_standard", "safe_aspa", "last_safe_standard", "last_safe_variants", "sequence_lengths",
            "base_batch_size", "d_model", "variant_labels", "runs", "auto_logs", "scaling_alpha"} <= set(rec)
    assert rec["sequence_lengths"] == [128, 256, 512, 1024] and rec["d_model"] == 512
    models = {r["model"] for r in rec["runs"]}
    assert models == {"standard", "aspa_bf16", "aspa_int8"}
    assert all(r["status"] == "ok" and r["latency_ms"] > 0 for r in rec["runs"])
    assert len(list(tmp_path.glob("tinytoy_summary_*.json"))) == 1
