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


def test_static_scratch_entry_point_allocates_nothing():
    """What the entry point is for: once the first call on the device has looked up the array's
    address, a call changes neither the driver's free-memory figure nor torch's allocator
    counters (a cudaMalloc anywhere below the C ABI would show in the first, a torch
    allocation in the second)."""
    from pe_ablations_b200 import _lib as L

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(98)
    logits = (torch.randn(2048, 8192, generator=g) * 2).to(torch.bfloat16).to(dev)
    tgt = torch.randint(0, 8192, (2048,), generator=g).to(dev)
    out = torch.zeros(2, dtype=torch.float64, device=dev)
    assert _call_static(L, logits, tgt, out) == 0, L.lib.pe_attn_last_error()      # the set-up call
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(dev)
    stats0 = torch.cuda.memory_stats(dev)
    for _ in range(3):
        assert _call_static(L, logits, tgt, out) == 0, L.lib.pe_attn_last_error()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(dev)
    stats1 = torch.cuda.memory_stats(dev)
    assert free1 == free0
    for key in ("allocation.all.allocated", "segment.all.allocated", "allocated_bytes.all.allocated"):
        assert stats1[key] == stats0[key], key
    assert int(out[1].item()) == 4 * 2048


def test_static_scratch_entry_point_refused_call_leaves_the_array_alone():
    """A call with bad arguments is refused before the shared array is touched."""
    from pe_ablations_b200 import _lib as L

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    logits = torch.zeros(4, 8, dtype=torch.float32, device=dev)
    tgt = torch.zeros(4, dtype=torch.int64, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    rc = L.lib.pe_ce_loss_sums_static(logits.data_ptr(), L.FP32, 8, tgt.data_ptr(), 4, 8, -100, None, C.c_void_p(stream))
    assert rc == 1                          # PE_ATTN_ERR_NULL: no output pointer
    rc = L.lib.pe_ce_loss_sums_static(logits.data_ptr(), 9, 8, tgt.data_ptr(), 4, 8, -100, logits.data_ptr(),
                                      C.c_void_p(stream))
    assert rc != 0                          # unknown dtype


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
