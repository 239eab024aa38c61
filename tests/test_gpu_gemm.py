"""GPU: the tensor-core GEMM with fused epilogues (language-model head + cross-entropy, SwiGLU
feed-forward input, plain store) against fp32 torch references on the same bf16 operands.

bf16 outputs are compared at one bf16 rounding step of the largest result (2^-7 relative);
loss sums at 2e-5 relative against ``F.cross_entropy`` on the bf16-rounded logits, the rounding
the head's autocast output has.
"""

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(BF16).cuda()


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (1, 8, 64), (300, 520, 128), (129, 264, 72), (1000, 2048, 2048),
                                   (4096, 5632, 512), (16384, 1024, 256)])
def test_gemm_nt_matches_fp32_matmul(m, n, k):
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200.ops import gemm_nt

    a, b = _rand((m, k), 1), _rand((n, k), 2)
    c = gemm_nt(a, b)
    check_device_status()
    want = a.float() @ b.float().T
    assert c.shape == (m, n) and c.dtype == BF16
    assert (c.float() - want).abs().max().item() <= want.abs().max().item() * 2 ** -7


@pytest.mark.parametrize("m,n,k", [(300, 520, 128), (2048, 2048, 512), (129, 264, 72)])
def test_gemm_nt_adds_a_residual_like_a_bf16_add(m, n, k):
    """cast(cast(a b^T) + residual): the projection's bf16 output added to a bf16 residual."""
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200.ops import gemm_nt

    a, b, r = _rand((m, k), 31, 0.3), _rand((n, k), 32, 0.3), _rand((m, n), 33, 3.0)
    c = gemm_nt(a, b, residual=r)
    check_device_status()
    want = ((a.float() @ b.float().T).to(BF16) + r).float()
    assert (c.float() - want).abs().max().item() <= max(want.abs().max().item(), 1.0) * 2 ** -6
    # in place on the residual stream: c may be the residual's own memory
    same = gemm_nt(a, b)
    assert torch.equal(gemm_nt(a, b, residual=torch.zeros_like(same)), same)


def test_gemm_nt_reads_strided_views_in_place():
    """Operands that are column slices of wider buffers (row stride > k) and a leading batch dim."""
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200.ops import gemm_nt

    wide_a, wide_b = _rand((2, 150, 384), 3), _rand((200, 512), 4)
    a, b = wide_a[..., 128:256], wide_b[:, 256:384]
    c = gemm_nt(a, b)
    check_device_status()
    want = a.float() @ b.float().T
    assert c.shape == (2, 150, 200)
    assert (c.float() - want).abs().max().item() <= want.abs().max().item() * 2 ** -7


@pytest.mark.parametrize("m,ffn,k", [(300, 264, 128), (16, 8, 64), (2048, 5632, 2048), (777, 1000, 320)])
def test_swiglu_gemm_matches_the_two_projections_and_swiglu(m, ffn, k):
    """Against the unfused data flow: two bf16 projections, then cast(cast(silu(g)) * u)."""
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200.ops import swiglu_gemm

    x, wg, wu = _rand((m, k), 5), _rand((ffn, k), 6, k ** -0.5), _rand((ffn, k), 7, k ** -0.5)
    y = swiglu_gemm(x, wg, wu)
    check_device_status()
    g = (x.float() @ wg.float().T).to(BF16).float()
    u = (x.float() @ wu.float().T).to(BF16).float()
    want = (F.silu(g).to(BF16).float() * u).to(BF16).float()
    assert y.shape == (m, ffn) and y.dtype == BF16
    # a gate or up value that rounds the other way in the fp32 accumulation moves the product by
    # one bf16 step of that factor
    assert (y.float() - want).abs().max().item() <= max(want.abs().max().item(), 1.0) * 2 ** -6


@pytest.mark.parametrize("m,vocab,k", [(100, 1000, 128), (777, 32000, 512), (4096, 32000, 2048), (500, 50257, 256),
                                       (1, 300, 64), (257, 256, 64)])
def test_lm_head_ce_loss_sums_matches_cross_entropy(m, vocab, k):
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200.ops import lm_head_ce_loss_sums

    h, w = _rand((m, k), 8), _rand((vocab, k), 9, 2.0 * k ** -0.5)
    g = torch.Generator().manual_seed(10)
    t = torch.randint(0, vocab, (m,), generator=g)
    t[::7] = -100
    t[-1] = vocab - 1                       # a target in the last, possibly ragged, vocabulary tile
    t = t.cuda()
    out = lm_head_ce_loss_sums(h, w, t)
    check_device_status()
    logits = (h.float() @ w.float().T).to(BF16).float()
    want = F.cross_entropy(logits.double(), t, ignore_index=-100, reduction="sum").item()
    assert out[1].item() == (t != -100).sum().item()
    assert abs(out[0].item() - want) <= 2e-5 * abs(want) + 1e-4
    # accumulates into a given ``out``; a second call doubles both sums
    lm_head_ce_loss_sums(h, w, t, out=out)
    assert abs(out[0].item() - 2 * want) <= 4e-5 * abs(want) + 2e-4 and out[1].item() == 2 * (t != -100).sum().item()


def test_lm_head_ce_is_deterministic_and_flags_bad_targets():
    from pe_ablations_b200.ops import lm_head_ce_loss_sums

    h, w = _rand((600, 256), 11), _rand((5000, 256), 12, 0.1)
    t = torch.randint(0, 5000, (600,), generator=torch.Generator().manual_seed(13)).cuda()
    a = lm_head_ce_loss_sums(h, w, t)
    b = lm_head_ce_loss_sums(h, w, t)
    assert torch.equal(a, b)
    t[5] = 5000                              # out of range and not the ignore index: NaN, still counted
    c = lm_head_ce_loss_sums(h, w, t)
    assert torch.isnan(c[0]).item() and c[1].item() == 600
    t[:] = -100                              # nothing scored
    d = lm_head_ce_loss_sums(h, w, t)
    assert d[0].item() == 0.0 and d[1].item() == 0.0


def test_model_takes_the_fused_paths_for_bf16_inference_and_agrees_with_the_unfused_ones():
    """FeedForward and Transformer.loss_sums with bf16 weights: fused kernels against the library
    GEMM + stand-alone kernels the same modules use when the weights are fp32 under autocast."""
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200 import model as M
    from pe_ablations_b200.eval import cast_matmul_weights
    from pe_ablations_b200.ops import fused_gemm_ok

    torch.manual_seed(21)
    cfg = M.TransformerConfig(vocab_size=1000, hidden_dim=128, num_layers=2, num_heads=2, num_kv_heads=1, head_dim=64,
                              ffn_dim=264, max_seq_len=512, pe_mode="fpope", fpope_d_rope=32, fpope_num_fourier_terms=8,
                              fpope_training_length=64)
    with torch.device("cuda"):
        m32 = M.Transformer(cfg).eval()
        m16 = M.Transformer(cfg).eval()
    m16.load_state_dict(m32.state_dict())
    cast_matmul_weights(m16)
    ids = torch.randint(0, 1000, (2, 300), generator=torch.Generator().manual_seed(22)).cuda()
    x = _rand((2, 300, 128), 23)
    with torch.no_grad(), torch.autocast("cuda", dtype=BF16):
        ff16, ff32 = m16.layers[0].feed_forward, m32.layers[0].feed_forward
        assert fused_gemm_ok(x, ff16.w3.weight, ff16.w1.weight) and not fused_gemm_ok(x, ff32.w3.weight)
        y16, y32 = ff16(x), ff32(x)
        r16, r32 = ff16(x, residual=x), ff32(x, residual=x)          # w2 with the block's residual add
        b16, b32 = m16.layers[1](x), m32.layers[1](x)                # a whole block: wo and w2 add their residuals
        nll16, cnt16 = m16.loss_sums(ids)
        nll32, cnt32 = m32.loss_sums(ids)
    check_device_status()
    assert (y16.float() - y32.float()).abs().max().item() <= max(y32.float().abs().max().item(), 1.0) * 2 ** -6
    for got, want in ((r16, r32), (b16, b32)):
        assert got.dtype == want.dtype == BF16
        assert (got.float() - want.float()).abs().max().item() <= max(want.float().abs().max().item(), 1.0) * 2 ** -6
    assert cnt16.item() == cnt32.item() == 2 * 299
    assert abs(nll16.item() - nll32.item()) <= 2e-3 * abs(nll32.item())


def test_attention_input_projections_run_as_one_gemm_and_follow_weight_updates():
    """bf16 inference: q_c | k_c | q_r | k_r | v come out of one GEMM against the concatenated
    weights (column slices read in place by the norm and attention kernels); the concatenation
    is rebuilt when a weight changes, and the state_dict does not contain it."""
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200 import model as M
    from pe_ablations_b200.eval import cast_matmul_weights
    from pe_ablations_b200.ops import projections

    torch.manual_seed(41)
    cfg = M.TransformerConfig(vocab_size=512, hidden_dim=128, num_layers=1, num_heads=2, num_kv_heads=1, head_dim=64,
                              ffn_dim=264, max_seq_len=512, pe_mode="fpope", fpope_d_rope=32, fpope_num_fourier_terms=8,
                              fpope_training_length=64)
    with torch.device("cuda"):
        m = cast_matmul_weights(M.Transformer(cfg).eval())
    att = m.layers[0].attention
    x = _rand((2, 200, 128), 42)
    lins = (att.wq_c, att.wk_c, att.wq_r, att.wk_r, att.wv)
    with torch.no_grad(), torch.autocast("cuda", dtype=BF16):
        outs = projections(att, x, *lins)
        assert outs[1].stride(-2) == sum(l.weight.shape[0] for l in lins)      # slices of one wide result
        for o, lin in zip(outs, lins):
            want = lin(x)
            assert (o.float() - want.float()).abs().max().item() <= max(want.float().abs().max().item(), 1.0) * 2 ** -7
        y0 = att(x)
        att.wv.weight.mul_(2.0)                  # in place: same storage, new version
        y1 = att(x)
    check_device_status()
    assert "_wcat" not in m.state_dict() and not any("_wcat" in k for k in m.state_dict())
    # doubling v doubles the attention output before wo, hence the module output
    assert (y1.float() - 2.0 * y0.float()).abs().max().item() <= max(y0.float().abs().max().item(), 1.0) * 2 ** -5


@pytest.mark.parametrize("bad", [float("nan"), float("inf")])
def test_lm_head_ce_non_finite_logits_make_the_sum_non_finite(bad):
    """A NaN or +inf logit is scored and makes the loss sum non-finite, as F.cross_entropy does
    (and as pe_ce_loss_sums does on stored logits); the count is unaffected."""
    from pe_ablations_b200.ops import lm_head_ce_loss_sums

    h, w = _rand((300, 128), 51), _rand((700, 128), 52, 0.1)
    w[13, 5] = bad                               # every row's logit 13 becomes non-finite
    t = torch.randint(0, 700, (300,), generator=torch.Generator().manual_seed(53)).cuda()
    out = lm_head_ce_loss_sums(h, w, t)
    want = F.cross_entropy((h.float() @ w.float().T), t, reduction="sum")
    assert not torch.isfinite(want).item()
    assert not torch.isfinite(out[0]).item() and out[1].item() == 300
