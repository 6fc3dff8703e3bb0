"""CPU-side tests of the product: the C-ABI library loads and exports what the header declares, the
host-side schedules of the layer reproduce the reference's known answers, the drop-in wrapper's
argument handling, and the failure behaviour when no GPU is present (no silent fallback)."""
import ctypes
import re

import pytest
import torch

import proteus_flux_attention_b200 as P
from proteus_flux_attention_b200 import _native

ROOT = __import__("pathlib").Path(__file__).resolve().parents[1]


def _declared_symbols():
    text = (ROOT / "include" / "aspa_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aspa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared_symbols()
    assert len(names) >= 25
    handle = ctypes.CDLL(str(_native.library_path()))
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in include/aspa_b200.h but not exported"
    assert set(names) == set(_native.SIGNATURES), "ctypes table and header disagree"
    assert _native.lib().aspa_version() == 1


def test_argument_errors_come_back_as_status_codes():
    lib = _native.lib()
    rc = lib.aspa_normalize_rows(None, 4, 4, 1e-6, None, None)
    assert rc == -1 and "normalize_rows" in _native.last_error()
    assert lib.aspa_pack_rows_scratch(2, 4, 1000) == 2 * 4 * 4 + 1
    assert lib.aspa_attn_workspace_bytes(10, 64) == 4 * 10 * 66


def test_host_schedules_match_reference(golden_dir):
    rows = torch.load(golden_dir / "schedules.pt", weights_only=False)
    layers = {}
    for r in rows:
        key = id(r["cfg"])
        if key not in layers:
            layers[key] = P.AdaptiveSparseAttention(P.ModelConfig(**r["cfg"]))
        m = layers[key]
        m._current_alpha = 0.0
        assert m._compute_cvt_alpha(r["T"]) == r["alpha"]
        assert m._choose_active_k(r["T"]) == r["k"]
        assert m._linear_token_keep_ratio(r["T"]) == r["ratio"]
        assert m._compute_effective_linear_params(r["T"], 2, r["alpha_in"]) == r["params"]


def test_layer_knobs_follow_reference_defaults():
    m = P.AdaptiveSparseAttention(P.ModelConfig(d_model=512, n_head=8))
    assert (m.h_total, m.h_active, m.h_active_min, m.h_active_max, m.attn_gates) == (8, 4, 2, 8, 16)
    assert (m.seq_low, m.seq_high, m.small_seq_dense) == (64, 256, 32)
    assert m.gate_to_head.tolist() == [0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5, 6, 6, 7, 7]
    assert m.linear_use_local and m.linear_use_anchors and not m.linear_use_proto
    assert m.routing_prototypes is None
    w = P.CausalASPAMultiheadAttention(64, 4)
    a = w.attention
    assert a.proto_enabled and a._dense_threshold == 0.6 and a.small_seq_dense == 0 and a.router_top_p == 0.9
    assert a.h_active == 4 and a.h_active_min == 2 and a.h_active_max == 4
    with pytest.raises(ValueError):
        P.AdaptiveSparseAttention(P.ModelConfig(d_model=10, n_head=4))


def test_no_cpu_fallback():
    m = P.CausalASPAMultiheadAttention(64, 4)
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(torch.randn(1, 8, 64))
    q = torch.randn(2, 4, 8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        P.aspa_sparse_attention(q, q, q)
    with pytest.raises(RuntimeError, match="no CPU path"):
        P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(seq_len=64, d_model=8, chunk_len=32, buffer_tokens=8,
                                                          per_chunk_budget=4, device=torch.device("cpu"))).run()


def test_wrapper_fallback_paths_on_cpu():
    """Cross-attention and custom masks are served by nn.MultiheadAttention exactly as in the reference."""
    torch.manual_seed(0)
    m = P.CausalASPAMultiheadAttention(32, 4, return_stats_default=True).eval()
    x, kv = torch.randn(2, 6, 32), torch.randn(2, 5, 32)
    got, _ = m(x, kv, kv, need_weights=False)
    want, _ = m.fallback_attention(x, kv, kv, need_weights=False)
    assert torch.allclose(got, want, atol=1e-6)
    assert m.last_runtime_stats["shortlist_backend"]["name"] == "torch.nn.MultiheadAttention"
    got, _ = m(x, is_causal=False, need_weights=False)
    assert m.last_runtime_stats["shortlist_backend"]["details"]["reason"] == "non_causal"
    assert m._is_supported_attn_mask(None, 6, x.device)
    assert m._is_supported_attn_mask(torch.triu(torch.ones(6, 6, dtype=torch.bool), 1), 6, x.device)
    assert not m._is_supported_attn_mask(torch.zeros(6, 6), 6, x.device)
    assert not m._is_supported_attn_mask(torch.zeros(5, 6), 6, x.device)


def test_controller_logic():
    class Layer:
        h_total, h_active, h_active_min, h_active_max, _dense_threshold = 8, 4, 2, 6, None
    lay = Layer()
    c = P.SparseHeadController(lay, target_density=0.3, tolerance=0.05, cooldown=2, dense_threshold=0.7)
    assert lay._dense_threshold == 0.7
    assert c.observe({"max_active_density": 0.9}) is None
    snap = c.observe({"max_active_density": 0.9})
    assert snap.action == "decrease" and lay.h_active_max == 5
    c.observe({"max_active_density": 0.1})
    assert c.observe({"max_active_density": 0.1}).action == "increase" and lay.h_active_max == 6
    c.observe({"max_active_density": 0.3})
    assert c.observe({"max_active_density": 0.3}).action == "steady"
    assert c.observe(None) is None


def test_chunk_config_validation():
    ok = dict(seq_len=64, d_model=8, chunk_len=32, buffer_tokens=8, per_chunk_budget=4, device=torch.device("cuda"))
    P.ChunkedShortlistConfig(**ok).validate()
    for bad in (dict(seq_len=0), dict(chunk_len=70000), dict(nucleus_top_p=0.0), dict(shortlist_alpha=1.5),
                dict(storage="tape"), dict(per_chunk_budget=0)):
        with pytest.raises(ValueError):
            P.ChunkedShortlistConfig(**{**ok, **bad}).validate()


def test_storage_rules_and_disk_stage(tmp_path):
    """Where a host sequence is staged follows the reference's rules (tools/chunked_shortlist.py:420-451), and the
    memory-mapped stage holds the sequence as float32, written block by block, and disappears with the call."""
    base = dict(seq_len=5000, d_model=32, chunk_len=2048, buffer_tokens=64, per_chunk_budget=16, device=torch.device("cuda"),
                temp_dir=tmp_path)
    need = 5000 * 32 * 2
    mode = lambda on_device=False, **kw: P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**base, **kw))._resolve_storage(need, on_device)  # noqa: E731
    assert mode(storage="auto", ram_limit_bytes=1000)[0] == "disk" and "exceeds limit=1,000B" in mode(storage="auto", ram_limit_bytes=1000)[1]
    assert mode(storage="auto", ram_limit_bytes=10 ** 9)[:2] == ("cpu", f"limit=1,000,000,000B, required={need:,}B")
    assert mode(storage="cpu", ram_limit_bytes=1000)[0] == "disk" and mode(storage="cpu")[0] == "cpu"
    assert mode(storage="disk")[0] == "disk" and mode(True, storage="disk")[0] == "disk"
    assert mode(True, storage="auto")[0] == "device" and mode(True, storage="cpu")[0] == "device" and mode(storage="device")[0] == "device"
    runner = P.ChunkedShortlistRunner(P.ChunkedShortlistConfig(**base, storage="disk", seed=5))
    x = torch.randn(1, 5000, 32).to(torch.bfloat16)
    staged, block_bytes = runner._stage_on_disk(x, 5000)
    assert staged.dtype == torch.float32 and staged.shape == (1, 5000, 32) and block_bytes == 2048 * 32 * 4
    assert torch.equal(staged.to(torch.bfloat16), x)
    noise, _ = runner._stage_on_disk(None, 5000)     # seeded noise, generated block by block as the reference does
    gen = torch.Generator().manual_seed(5)
    want = torch.cat([torch.randn(n, 32, generator=gen) for n in (2048, 2048, 904)])
    assert torch.equal(noise[0], want)
    assert len(list(tmp_path.glob("chunked_shortlist_*.mmap"))) == 2
    del staged, noise
    runner._drop_disk_stage()
    assert list(tmp_path.glob("*.mmap")) == []
