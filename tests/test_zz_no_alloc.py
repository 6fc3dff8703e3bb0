"""The allocation-free packing entry point, called through the C ABI.

`aspa_pack_rows_static` serves hosts that may not allocate when they call the library (a serving loop
with a fixed device arena, a binding without a CUDA allocator): its scratch is a fixed array inside the
library.  The test calls it twice in a row on different inputs — the second call finds the first call's
leftovers in the shared scratch — and requires exactly what `aspa_pack_rows` returns with caller scratch.
Collected last on purpose, so a run that stops at the first failure has already run everything else."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bits(B, T, H, k, seed, dev):
    g = torch.Generator().manual_seed(seed)
    pick = torch.rand(B * T, H, generator=g).topk(k, dim=-1).indices
    bits = torch.zeros(B * T, dtype=torch.int64)
    for j in range(k):
        bits |= torch.ones(B * T, dtype=torch.int64) << pick[:, j]
    bits[torch.rand(B * T, generator=g) > 0.3] = 0  # most tokens dropped
    return bits.to(dev)


def test_static_scratch_packing_equals_caller_scratch_packing():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from proteus_flux_attention_b200 import _native as N
    from proteus_flux_attention_b200 import ops
    dev = torch.device("cuda:0")
    lib = N.lib()
    assert lib.aspa_pack_rows_static_capacity() == 262144
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (B, T, H, k) in enumerate([(2, 5000, 16, 4), (1, 70000, 8, 2)]):
        bits = _bits(B, T, H, k, 100 + call, dev)
        cap = B * T * k
        want_offs, want_tok = ops.pack_rows(bits, B, T, H, cap)
        offs = torch.full((B * H + 1,), -7, dtype=torch.int32, device=dev)
        tok = torch.full((cap,), -7, dtype=torch.int32, device=dev)
        rc = lib.aspa_pack_rows_static(N.ptr(bits), B, T, H, N.ptr(offs), N.ptr(tok), cap, stream)
        assert rc == 0, N.last_error()
        torch.cuda.synchronize()
        n = int(want_offs[-1])
        assert n > 0
        assert torch.equal(offs, want_offs)
        assert torch.equal(tok[:n], want_tok[:n])
    # beyond the built-in scratch: refused with a message, nothing launched
    rc = lib.aspa_pack_rows_static(N.ptr(bits), 64, 1 << 20, 64, N.ptr(offs), N.ptr(tok), cap, stream)
    assert rc == -1 and "exceed" in N.last_error()
