"""GPU: the allocation-free cross-entropy entry point against the regular one.

Some hosts of this library cannot hand it a scratch buffer -- their device memory is fully
owned by a pool, or they run where cudaMalloc's device-wide synchronisation is not
acceptable -- so ``pe_ce_loss_sums_static`` works out of an array built into the library.
This test calls it through the C ABI twice in a row (the array is shared between calls and
keeps old contents) and checks both results against ``pe_ce_loss_sums`` with a caller-owned
scratch.  The two run the same kernel, so the sums must agree to the tolerance the other
cross-entropy tests use (2e-6 relative); the counts must be equal.

Collected last on purpose: a failure here must not hide any other test from a run that
stops at the first failure.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(L, logits, tgt, out):
    dt = L.BF16 if logits.dtype == torch.bfloat16 else L.FP32
    stream = torch.cuda.current_stream().cuda_stream
    return L.lib.pe_ce_loss_sums_static(logits.data_ptr(), dt, logits.stride(0), tgt.data_ptr(), logits.shape[0],
                                        logits.shape[1], -100, out.data_ptr(), C.c_void_p(stream))


def _call_regular(L, logits, tgt, out, scratch):
    dt = L.BF16 if logits.dtype == torch.bfloat16 else L.FP32
    stream = torch.cuda.current_stream().cuda_stream
    return L.lib.pe_ce_loss_sums(logits.data_ptr(), dt, logits.stride(0), tgt.data_ptr(), logits.shape[0],
                                 logits.shape[1], -100, scratch.data_ptr(), out.data_ptr(), C.c_void_p(stream))


def test_static_scratch_entry_point_matches_regular_one_twice():
    from pe_ablations_b200 import _lib as L

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    assert L.lib.pe_ce_static_max_rows() == 16384
    g = torch.Generator().manual_seed(99)
    # two different chunks back to back, the second smaller than the first so that stale
    # row losses from the first call sit beyond its end in the shared array
    chunks = []
    for n, vocab, dtype in ((4096, 32000, torch.bfloat16), (1000, 4099, torch.float32)):
        logits = (torch.randn(n, vocab, generator=g) * 2.5).to(dtype).to(dev)
        tgt = torch.randint(0, vocab, (n,), generator=g).to(dev)
        tgt[::5] = -100
        chunks.append((logits, tgt))
    for logits, tgt in chunks:
        n = logits.shape[0]
        want = torch.zeros(2, dtype=torch.float64, device=dev)
        scratch = torch.zeros(L.lib.pe_ce_scratch_bytes(n), dtype=torch.uint8, device=dev)
        assert _call_regular(L, logits, tgt, want, scratch) == 0, L.lib.pe_attn_last_error()
        got = torch.zeros(2, dtype=torch.float64, device=dev)
        assert _call_static(L, logits, tgt, got) == 0, L.lib.pe_attn_last_error()
        torch.cuda.synchronize()
        assert got[1].item() == want[1].item() == float((tgt != -100).sum().item())
        assert abs(got[0].item() - want[0].item()) <= 2e-6 * abs(want[0].item())
        # and against torch, like the other cross-entropy tests
        ref = torch.nn.functional.cross_entropy(logits.double(), tgt, ignore_index=-100, reduction="sum").item()
        assert abs(got[0].item() - ref) <= 2e-6 * abs(ref)


def test_static_scratch_entry_point_rejects_oversized_chunks():
    from pe_ablations_b200 import _lib as L

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n = L.lib.pe_ce_static_max_rows() + 1
    logits = torch.zeros(n, 8, dtype=torch.float32, device=dev)
    tgt = torch.zeros(n, dtype=torch.int64, device=dev)
    out = torch.zeros(2, dtype=torch.float64, device=dev)
    assert _call_static(L, logits, tgt, out) == 7  # PE_ATTN_ERR_TOO_LARGE
    assert b"16384" in L.lib.pe_attn_last_error()
    torch.cuda.synchronize()
    assert out.abs().sum().item() == 0.0
