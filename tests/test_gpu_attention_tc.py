"""The tcgen05 / tensor-memory window attention kernel against the oracle (and against the warp-MMA tile kernel it
replaces where rows are dense): plans with a local window, anchors, prototype picks; INT8 inputs; dense causal
attention; strided key/value layouts; sizes that wrap the three-stage key ring, leave ragged row and key tiles, and
give a CTA several row tiles.  Every call goes through the C ABI with the kernel choice forced; the status word of
the kernel's bounded waits must stay clear."""
import pytest
import torch

from oracle import aspa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


class forced_mode:
    """Kernel choice for the window passes: 0 warp-MMA only, 2 tcgen05 whenever the shape allows."""

    def __init__(self, mode):
        self.mode = mode

    def __enter__(self):
        from proteus_flux_attention_b200 import _native as N
        self.old = N.lib().aspa_attn_tc_mode(self.mode)
        N.lib().aspa_attn_tc_status(1, N.stream())

    def __exit__(self, *exc):
        from proteus_flux_attention_b200 import _native as N
        N.lib().aspa_attn_tc_mode(self.old)
        if exc[0] is None:
            assert N.lib().aspa_attn_tc_status(1, N.stream()) == 0, N.last_error()
        return False


def _planned(dev, **kw):
    import test_gpu_kernels as K
    return K._planned_vs_table(dev, **kw)


CASES = [
    # window only; 333 rows per head in three row tiles, 24 key tiles (the ring wraps eight times)
    dict(heads=4, T=3000, L=512, window=400, stride=0, local_cap=400, anchor_cap=0, proto_cap=0, H=2, seed=3),
    # ragged: T not a multiple of 128, window wider than the sequence start
    dict(heads=2, T=1111, L=1024, window=700, stride=0, local_cap=700, anchor_cap=0, proto_cap=0, H=2, seed=4),
    # window + gathered anchors + prototype picks (partial state handed to the row kernel)
    dict(heads=4, T=1500, L=384, window=256, stride=32, local_cap=256, anchor_cap=40, proto_cap=24, H=4, seed=5),
    # tiny: fewer rows than one tile, one key tile
    dict(heads=2, T=100, L=64, window=50, stride=0, local_cap=50, anchor_cap=0, proto_cap=0, H=1, seed=6),
    # window of one key (every row sees only itself)
    dict(heads=2, T=600, L=8, window=1, stride=0, local_cap=1, anchor_cap=0, proto_cap=0, H=2, seed=7),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("quant", [False, True])
def test_tcgen05_window_pass_matches_oracle_and_warp_mma(dev, case, quant):
    with forced_mode(2):
        a = _planned(dev, dtype=torch.bfloat16, D=64, quant=quant, **case)
    with forced_mode(0):
        b = _planned(dev, dtype=torch.bfloat16, D=64, quant=quant, **case)
    assert float((a - b).abs().max()) < 2e-2 and float((a - b).abs().mean()) < 1e-3


@pytest.mark.parametrize("case", [
    dict(T=3000, L=400, window=40, stride=8, local_cap=40, anchor_cap=200, proto_cap=20),
    dict(T=2500, L=300, window=33, stride=16, local_cap=33, anchor_cap=140, proto_cap=0),
    dict(T=2048, L=256, window=0, stride=4, local_cap=0, anchor_cap=120, proto_cap=8),
])
@pytest.mark.parametrize("quant", [False, True])
def test_tcgen05_anchor_pass_over_regrouped_rows(dev, case, quant):
    """The anchors of a residue class are a window over every stride-th key: the tcgen05 kernel reads that strided view,
    starts from the partial softmax state of the window pass and hands its own state on."""
    with forced_mode(2):
        a = _planned(dev, dtype=torch.bfloat16, heads=4, D=64, H=2, seed=17, quant=quant, **case)
    with forced_mode(0):
        b = _planned(dev, dtype=torch.bfloat16, heads=4, D=64, H=2, seed=17, quant=quant, **case)
    assert float((a - b).abs().max()) < 2e-2 and float((a - b).abs().mean()) < 1e-3


@pytest.mark.parametrize("T", [333, 2048, 4500])
def test_tcgen05_dense_causal_attention(dev, T):
    from proteus_flux_attention_b200 import aspa_sparse_attention
    g = torch.Generator().manual_seed(T)
    q, k, v = (torch.randn(3, T, 64, generator=g).to(torch.bfloat16) for _ in range(3))
    q[:, ::50] *= 3.0   # rows with large logits
    want = torch.nn.functional.scaled_dot_product_attention(q.float()[None], k.float()[None], v.float()[None], is_causal=True)[0]
    with forced_mode(2):
        got = aspa_sparse_attention(q.to(dev), k.to(dev), v.to(dev)).cpu().float()
    assert torch.allclose(got, want, atol=2e-2, rtol=1e-2), float((got - want).abs().max())
    assert float((got - want).abs().mean()) < 2e-3


def test_tcgen05_reads_strided_keys_and_values(dev):
    """Keys and values where a fused (B*T, 2, H, D) projection leaves them, token-major output through a row map."""
    from proteus_flux_attention_b200 import _native as N
    from proteus_flux_attention_b200 import ops
    from proteus_flux_attention_b200.sparse_attn import attention_packed
    B, H, T, D = 2, 4, 900, 64
    C = H * D
    g = torch.Generator().manual_seed(8)
    q = torch.randn(B * H, T, D, generator=g).to(torch.bfloat16)
    kv = torch.randn(B * T, 2, H, D, generator=g).to(torch.bfloat16)
    k = kv[:, 0].view(B, T, H, D).permute(0, 2, 1, 3).reshape(B * H, T, D)
    v = kv[:, 1].view(B, T, H, D).permute(0, 2, 1, 3).reshape(B * H, T, D)
    active = torch.rand(B * H, T, generator=g) > 0.5
    active[:, 0] = True
    packed = O.pack_active_rows(active)
    window = 300
    cand, lens = O.build_candidates(packed[1], None, T, max_candidates=512, linear_window=window, anchor_stride=0,
                                    use_local=True, use_anchors=False, proto_scores=None, local_cap=window,
                                    anchor_cap=0, proto_cap=0)
    want = O.sparse_attention(q.float(), k.float(), v.float(), packed=packed, candidates=cand, lengths=lens)
    want = want.view(B, H, T, D).permute(0, 2, 1, 3).reshape(B, T, C)
    flat = kv.to(dev).view(-1)
    layout = N.KVLayout(k_batch=T * 2 * C, k_head=D, k_token=2 * C, v_batch=T * 2 * C, v_head=D, v_token=2 * C)
    out = torch.zeros(B, T, C, dtype=torch.float32, device=dev)
    with forced_mode(2):
        attention_packed(q.to(dev), flat, flat[C:], row_offsets=packed[2].to(dev), token_idx=packed[1].to(torch.int32).to(dev),
                         max_rows=packed[3], total_rows=packed[1].numel(), H=H, plan=ops.make_plan(window, 0, 0, 0, None, None),
                         out=out, out_layout=N.OUT_TOKEN_MAJOR, kv_layout=layout)
    assert torch.allclose(out.cpu(), want, atol=2e-2, rtol=1e-2), float((out.cpu() - want).abs().max())
