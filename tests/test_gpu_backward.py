"""GPU parity of the attention backward (C ABI ``pe_attn_backward``) against autograd.

The checker is PyTorch's autograd over an explicit fp32 softmax attention on the CPU, run on
the same bf16-rounded operands -- the gradient the reference's training step takes through
``F.scaled_dot_product_attention`` (src/model/attention.py:91-96,
src/model/fpope_attention.py:171-177) and through the explicit ALiBi softmax
(src/model/alibi.py:145-160).  Tolerance: rtol = atol = 1e-2, the reference's own bound for
its fused backward (debug_backward.py:120-124).
"""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = dict(rtol=1e-2, atol=1e-2)


def autograd_core(q, k, v, dout, scale, slopes=None):
    """out, lse and (dq, dk, dv) of causal softmax attention in fp32; tensors are [B, S, H, d]."""
    q, k, v = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    B, Sq, H, _ = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    g = H // Hkv
    kk = k.repeat_interleave(g, dim=2)
    vv = v.repeat_interleave(g, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) * scale
    rows = torch.arange(Sq).view(-1, 1) + (Sk - Sq)
    cols = torch.arange(Sk).view(1, -1)
    if slopes is not None:
        s = s - slopes.float().view(1, H, 1, 1) * (rows - cols).clamp(min=0).float()
    s = s.masked_fill(cols > rows, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    out = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), vv)
    out.backward(dout.float())
    return out.detach(), lse.detach(), q.grad, k.grad, v.grad


CASES = [
    # name, B, H, Hkv, Sq, Sk, d_qk, d_v, alibi
    ("d64_gqa_ragged", 2, 4, 2, 300, 300, 64, 64, False),
    ("pope_shape_128_64", 1, 2, 2, 512, 512, 128, 64, False),
    ("d128_mqa_257", 1, 4, 1, 257, 257, 128, 128, False),
    ("alibi_d64", 1, 4, 4, 384, 384, 64, 64, True),
    ("cached_prefix_sq_lt_sk", 1, 2, 1, 200, 328, 128, 64, False),
    ("one_block", 2, 2, 2, 96, 96, 64, 64, False),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_backward_matches_autograd(case):
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200.ops import attention_backward

    _, B, H, Hkv, Sq, Sk, dqk, dv, alibi = case
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(1234)
    mk = lambda s, h, d: torch.randn(B, s, h, d, generator=g).to(torch.bfloat16)
    q, k, v, dout = mk(Sq, H, dqk), mk(Sk, Hkv, dqk), mk(Sk, Hkv, dv), mk(Sq, H, dv)
    scale = dqk ** -0.5
    slopes = torch.tensor([2.0 ** (-(i + 1) * 8.0 / H) for i in range(H)]) if alibi else None
    out, lse, dq_w, dk_w, dv_w = autograd_core(q, k, v, dout, scale, slopes)
    c = lambda t: t.to(dev)
    dq, dk, dv_ = attention_backward(c(q), c(k), c(v), c(out.to(torch.bfloat16)), c(dout),
                                     c(lse.contiguous()), scale=scale, alibi_slopes=slopes)
    torch.cuda.synchronize()
    check_device_status()
    assert dq.shape == q.shape and dk.shape == k.shape and dv_.shape == v.shape
    torch.testing.assert_close(dv_.float().cpu(), dv_w, **TOL)
    torch.testing.assert_close(dk.float().cpu(), dk_w, **TOL)
    torch.testing.assert_close(dq.float().cpu(), dq_w, **TOL)


@pytest.mark.parametrize("variant,dims", [("nope", (64, 0, 64)), ("nope", (128, 0, 128)), ("pope", (64, 32, 64)),
                                          ("pope", (128, 64, 128))])
@pytest.mark.parametrize("S", [200, 1024])
def test_forward_logsumexp_output(variant, dims, S):
    """The forward's optional ``lse`` output against the oracle's logits (both tcgen05 kernels)."""
    from pe_ablations_b200 import check_device_status, pe_attention
    from oracle import pe_attention_oracle as O

    dc, dr, dv = dims
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(5)
    B, H, Hkv = 1, 4, 2
    mk = lambda h, d: torch.randn(B, S, h, d, generator=g).to(torch.bfloat16)
    q, k, v = mk(H, dc), mk(Hkv, dc), mk(Hkv, dv)
    kw, okw = {}, {}
    if variant == "pope":
        q_r, k_r = mk(H, dr), mk(Hkv, dr)
        freqs, delta = O.pope_base_freqs(dr), -torch.rand(dr, generator=g) * 3
        kw = dict(q_r=q_r.to(dev), k_r=k_r.to(dev), freqs=freqs, delta=delta)
        okw = dict(q_r=q_r.float(), k_r=k_r.float(), freqs=freqs, delta=delta)
    lse = torch.full((B, H, S), float("nan"), device=dev)
    pe_attention(variant, q.to(dev), k.to(dev), v.to(dev), lse=lse, **kw)
    torch.cuda.synchronize()
    check_device_status()
    want = O.attention_core(variant, q.float(), k.float(), v.float(), dtype=torch.bfloat16, return_lse=True, **okw)[1]
    assert torch.isfinite(lse).all()
    assert (lse.cpu() - want).abs().max().item() <= 2e-2
