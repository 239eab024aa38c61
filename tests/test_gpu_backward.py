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


def autograd_core(q, k, v, dout, scale, slopes=None, dtype=torch.float32):
    """out, lse and (dq, dk, dv) of causal softmax attention in ``dtype``; tensors are [B, S, H, d]."""
    q, k, v = (t.detach().to(dtype).requires_grad_(True) for t in (q, k, v))
    B, Sq, H, _ = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    g = H // Hkv
    kk = k.repeat_interleave(g, dim=2)
    vv = v.repeat_interleave(g, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) * scale
    rows = torch.arange(Sq).view(-1, 1) + (Sk - Sq)
    cols = torch.arange(Sk).view(1, -1)
    if slopes is not None:
        s = s - slopes.to(dtype).view(1, H, 1, 1) * (rows - cols).clamp(min=0).to(dtype)
    s = s.masked_fill(cols > rows, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    out = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), vv)
    out.backward(dout.to(dtype))
    return out.detach(), lse.detach(), q.grad, k.grad, v.grad


CASES = [
    # name, B, H, Hkv, Sq, Sk, d_qk, d_v, alibi
    ("d64_gqa_ragged", 2, 4, 2, 300, 300, 64, 64, False),
    ("pope_shape_128_64", 1, 2, 2, 512, 512, 128, 64, False),
    ("d128_mqa_257", 1, 4, 1, 257, 257, 128, 128, False),
    ("alibi_d64", 1, 4, 4, 384, 384, 64, 64, True),
    ("cached_prefix_sq_lt_sk", 1, 2, 1, 200, 328, 128, 64, False),
    ("one_block", 2, 2, 2, 96, 96, 64, 64, False),
    ("single_row", 1, 2, 2, 1, 1, 64, 64, False),
    ("gqa_8_to_1_s129", 1, 8, 1, 129, 129, 128, 64, False),
    ("alibi_d128_cached", 2, 4, 2, 131, 400, 128, 128, True),
    ("many_blocks_1153", 1, 2, 2, 1153, 1153, 64, 64, False),
    ("many_blocks_2100_d128", 1, 2, 1, 2100, 2100, 128, 128, False),
    # head dimensions the tensor-core kernel lacks: the FFMA backward
    ("ffma_1b_shape_256_128", 1, 2, 2, 600, 600, 256, 128, False),
    ("ffma_192_128_gqa_cached", 2, 4, 2, 130, 333, 192, 128, False),
    ("ffma_alibi_d32", 1, 4, 2, 200, 200, 32, 32, True),
    ("ffma_256_128_ragged_1100", 1, 2, 1, 1100, 1100, 256, 128, False),
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
    # P and dS enter the products rounded to bf16; a gradient entry sums up to Sk of them, so the
    # absolute floor grows like the square root of the sequence length beyond the 512 the
    # reference's own comparison ran at
    tol = dict(rtol=TOL["rtol"], atol=TOL["atol"] * max(1.0, math.sqrt(Sk / 512)))
    torch.testing.assert_close(dv_.float().cpu(), dv_w, **tol)
    torch.testing.assert_close(dk.float().cpu(), dk_w, **tol)
    torch.testing.assert_close(dq.float().cpu(), dq_w, **tol)


FP32_CASES = [
    # name, B, H, Hkv, Sq, Sk, d_qk, d_v, alibi
    ("fp32_config1_128_64", 1, 8, 8, 512, 512, 128, 64, False),
    ("fp32_d64_gqa_ragged", 2, 4, 2, 300, 300, 64, 64, False),
    ("fp32_alibi_d64_cached", 1, 4, 2, 131, 264, 64, 64, True),
    ("fp32_192_128_mqa", 1, 4, 1, 200, 200, 192, 128, False),
    ("fp32_1b_shape_256_128", 1, 2, 2, 330, 330, 256, 128, False),      # one P / dS tile in shared memory
    ("fp32_d24_d40", 1, 2, 2, 70, 70, 24, 40, False),
    ("fp32_single_row", 1, 2, 2, 1, 1, 64, 64, False),
]


@pytest.mark.parametrize("case", FP32_CASES, ids=lambda c: c[0])
def test_fp32_backward_matches_autograd(case):
    """fp32 operands through the FFMA backward kernels against autograd in fp64 (tolerance 1e-4 of
    each gradient's largest entry: fp32 products and sums in a different order than the checker's)."""
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200.ops import attention_backward

    _, B, H, Hkv, Sq, Sk, dqk, dv, alibi = case
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(4321)
    mk = lambda s, h, d: torch.randn(B, s, h, d, generator=g)
    q, k, v, dout = mk(Sq, H, dqk), mk(Sk, Hkv, dqk), mk(Sk, Hkv, dv), mk(Sq, H, dv)
    scale = dqk ** -0.5
    slopes = torch.tensor([2.0 ** (-(i + 1) * 8.0 / H) for i in range(H)]) if alibi else None
    out, lse, dq_w, dk_w, dv_w = autograd_core(q, k, v, dout, scale, slopes, dtype=torch.float64)
    c = lambda t: t.float().contiguous().to(dev)
    dq, dk, dv_ = attention_backward(c(q), c(k), c(v), c(out), c(dout), c(lse), scale=scale, alibi_slopes=slopes)
    torch.cuda.synchronize()
    check_device_status()
    assert dk.dtype == torch.float32 and dv_.dtype == torch.float32
    for have, want, name in ((dq, dq_w, "dq"), (dk, dk_w, "dk"), (dv_, dv_w, "dv")):
        err = (have.double().cpu() - want).abs().max().item()
        bound = 1e-4 * max(want.abs().max().item(), 1e-1)    # single row: dq is exactly 0, operands are O(1)
        assert err <= bound, f"{name}: |diff| {err:.3e} > {bound:.3e}"


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


@pytest.fixture(scope="module")
def grads(golden_dir):
    import os

    import numpy as np

    return np.load(os.path.join(golden_dir, "module_grads.npz"))


def _train_cases():
    from oracle import golden_cases as G

    return list(enumerate(G.TRAIN_CASES))


def _train_model_cases_early():
    from oracle import golden_cases as G

    return list(enumerate(G.TRAIN_MODEL_CASES))


@pytest.mark.parametrize("i,spec", _train_cases(), ids=lambda s: s["name"] if isinstance(s, dict) else str(s))
def test_module_gradients_match_reference_autograd(grads, i, spec):
    """Drop-in module under bf16 autocast, forward + backward, against the reference module's
    autograd under bf16 autocast (fixture generated by tests/golden/make_golden_grad.py).

    Two bf16 runs of the same step differ by rounding alone; the fixture records how far the
    reference's own bf16 step sits from its fp32 step for each tensor (about 1e-2 of the
    tensor's largest gradient).  Bound per tensor: 1e-2 * max|g| + 2 * that distance.
    """
    from oracle import golden_cases as G
    from pe_ablations_b200 import check_device_status
    from tests.test_modules_cpu import build_module

    torch.manual_seed(7000 + i)
    m = build_module(spec).train()
    G.fill_parameters(m, 8000 + i)
    m = m.cuda()
    g = torch.Generator().manual_seed(9000 + i)
    x = torch.randn(spec["B"], spec["S"], spec["hidden"], generator=g).cuda().requires_grad_(True)
    dy = torch.randn(spec["B"], spec["S"], spec["hidden"], generator=g).cuda()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m(x)
    y.float().backward(dy)
    torch.cuda.synchronize()
    check_device_status()
    name = spec["name"]
    want_y = torch.from_numpy(grads[f"{name}/y"])
    assert (y.detach().float().cpu() - want_y).abs().max().item() <= 2e-2 * max(1.0, want_y.abs().max().item())
    got = {"x": x.grad}
    got.update({n: p.grad for n, p in m.named_parameters() if p.grad is not None})
    names = [str(n) for n in grads[f"{name}/grad_names"]]
    assert sorted(got) == names
    for n in names:
        want = torch.from_numpy(grads[f"{name}/grad/{n}"])
        have = got[n].float().cpu()
        if have.dim() == 2:
            have = have[::G.TRAIN_ROW_STRIDE]
        bound = 1e-2 * float(grads[f"{name}/fp32_max/{n}"]) + 2.0 * float(grads[f"{name}/bf16_noise/{n}"])
        err = (have - want).abs().max().item()
        assert err <= bound, f"{name} grad {n}: |diff| {err:.3e} > {bound:.3e}"


@pytest.mark.parametrize("i,spec", _train_cases(), ids=lambda s: s["name"] if isinstance(s, dict) else str(s))
def test_fp32_module_gradients_match_reference_autograd(grads, i, spec):
    """Drop-in module in fp32, forward + backward, against the reference module's fp32 autograd
    (``y_fp32`` / ``grad_fp32`` of the fixture): fp32 forward kernel, fp32 FFMA backward kernels,
    the transform's gradient by autograd over its torch restatement.  Bound per tensor: 2e-4 of
    its largest entry (parameter gradients sum over every token of the batch)."""
    from oracle import golden_cases as G
    from pe_ablations_b200 import check_device_status
    from tests.test_modules_cpu import build_module

    torch.manual_seed(7000 + i)
    m = build_module(spec).train()
    G.fill_parameters(m, 8000 + i)
    m = m.cuda()
    g = torch.Generator().manual_seed(9000 + i)
    x = torch.randn(spec["B"], spec["S"], spec["hidden"], generator=g).cuda().requires_grad_(True)
    dy = torch.randn(spec["B"], spec["S"], spec["hidden"], generator=g).cuda()
    y = m(x)
    assert y.dtype == torch.float32
    y.backward(dy)
    torch.cuda.synchronize()
    check_device_status()
    name = spec["name"]
    want_y = torch.from_numpy(grads[f"{name}/y_fp32"])
    assert (y.detach().cpu() - want_y).abs().max().item() <= 1e-4 * max(1.0, want_y.abs().max().item())
    got = {"x": x.grad}
    got.update({n: p.grad for n, p in m.named_parameters() if p.grad is not None})
    names = [str(n) for n in grads[f"{name}/grad_names"]]
    assert sorted(got) == names
    for n in names:
        want = torch.from_numpy(grads[f"{name}/grad_fp32/{n}"])
        have = got[n].float().cpu()
        if have.dim() == 2:
            have = have[::G.TRAIN_ROW_STRIDE]
        bound = 2e-4 * max(float(grads[f"{name}/fp32_max/{n}"]), 1e-3)
        err = (have - want).abs().max().item()
        assert err <= bound, f"{name} fp32 grad {n}: |diff| {err:.3e} > {bound:.3e}"


@pytest.mark.parametrize("i,spec", _train_model_cases_early(), ids=lambda s: s["name"] if isinstance(s, dict) else str(s))
def test_fp32_transformer_training_step(grads, i, spec):
    """The Transformer host in fp32: the loss against the reference's fp32 loss, every parameter
    with a finite gradient whose sample sits within the bf16 noise of the reference's bf16 one."""
    from oracle import golden_cases as G
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200.model import Transformer, TransformerConfig

    kw = dict(G.TRAIN_MODEL_BASE)
    kw.update({k: v for k, v in spec.items() if k != "name"})
    torch.manual_seed(7500 + i)
    model = Transformer(TransformerConfig(**kw)).train()
    G.fill_parameters(model, 8500 + i)
    model = model.cuda()
    ids = torch.randint(0, kw["vocab_size"], (G.TRAIN_MODEL_BATCH, G.TRAIN_MODEL_SEQ),
                        generator=torch.Generator().manual_seed(9500 + i)).cuda()
    out = model(ids, labels=ids)
    out["loss"].backward()
    torch.cuda.synchronize()
    check_device_status()
    name = spec["name"]
    assert abs(out["loss"].item() - float(grads[f"{name}/loss_fp32"])) <= 1e-4 * float(grads[f"{name}/loss_fp32"])
    got = {n: p.grad for n, p in model.named_parameters() if p.grad is not None}
    assert sorted(got) == [str(n) for n in grads[f"{name}/grad_names"]]
    for n, gr in got.items():
        assert torch.isfinite(gr).all(), n
        want = torch.from_numpy(grads[f"{name}/grad_sample/{n}"])            # the reference's bf16 step
        have = gr.float().cpu().flatten()[::G.TRAIN_MODEL_SAMPLE_STRIDE]
        bound = 1e-3 * float(grads[f"{name}/fp32_max/{n}"]) + 1.5 * float(grads[f"{name}/bf16_noise/{n}"])
        err = (have - want).abs().max().item()
        assert err <= bound, f"{name} fp32 grad {n}: |diff| {err:.3e} > {bound:.3e}"


def test_training_call_refuses_what_the_backward_does_not_cover():
    from pe_ablations_b200 import pe_attention

    dev = torch.device("cuda", 0)
    mk = lambda d, dt: torch.randn(1, 64, 2, d, device=dev, dtype=dt, requires_grad=True)
    with pytest.raises(NotImplementedError):     # bf16 head dims outside the forward's
        pe_attention("nope", mk(96, torch.bfloat16), mk(96, torch.bfloat16), mk(64, torch.bfloat16))
    with pytest.raises(NotImplementedError):     # a caller-owned output
        pe_attention("nope", mk(64, torch.bfloat16), mk(64, torch.bfloat16), mk(64, torch.bfloat16),
                     out=torch.empty(1, 64, 2, 64, device=dev, dtype=torch.bfloat16))
    with torch.no_grad():                        # the same calls without gradients are fine
        pe_attention("nope", mk(64, torch.bfloat16), mk(64, torch.bfloat16), mk(64, torch.bfloat16),
                     out=torch.empty(1, 64, 2, 64, device=dev, dtype=torch.bfloat16))


@pytest.mark.parametrize("dc,dr", [(128, 64), (128, 32)], ids=["d_qk256", "d_qk192"])
def test_1b_head_dims_train_through_the_ffma_backward(dc, dr):
    """FoPE+PoPE attention at the 1B shape's head dims (d_qk 256 / d_v 128, which the tensor-core
    backward does not have) with gradients: output and every gradient against autograd over the
    torch restatement of the transform and an explicit fp32 attention."""
    from pe_ablations_b200 import autograd as A
    from pe_ablations_b200 import check_device_status, pe_attention

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(77)
    B, S, H, Hkv, dv = 1, 330, 4, 2, 128
    mk = lambda h, d: torch.randn(B, S, h, d, generator=g).to(torch.bfloat16)
    host = dict(q=mk(H, dc), k=mk(Hkv, dc), v=mk(Hkv, dv), q_r=mk(H, dr), k_r=mk(Hkv, dr))
    freqs = 10000.0 ** (-(torch.arange(dr, dtype=torch.float32) / dr))
    coeffs = torch.randn(dr, 8, generator=g) * 0.3
    delta = -torch.rand(dr, generator=g) * 3
    dout = torch.randn(B, S, H, dv, generator=g).to(torch.bfloat16)
    floor = 2 * math.pi / 4096
    scale = (dc + 2 * dr) ** -0.5

    leaf = {n: t.to(dev).requires_grad_(True) for n, t in host.items()}
    pl = {n: t.to(dev).requires_grad_(True) for n, t in dict(freqs=freqs, coeffs=coeffs, delta=delta).items()}
    out = pe_attention("pope", leaf["q"], leaf["k"], leaf["v"], q_r=leaf["q_r"], k_r=leaf["k_r"], freqs=pl["freqs"],
                       fourier_coeffs=pl["coeffs"], delta=pl["delta"], floor_freq=floor)
    out.backward(dout.to(dev))
    torch.cuda.synchronize()
    check_device_status()

    ref = {n: t.float().requires_grad_(True) for n, t in host.items()}
    rp = {n: t.clone().requires_grad_(True) for n, t in dict(freqs=freqs, coeffs=coeffs, delta=delta).items()}
    o = dict(start_pos=0, k_start_pos=0, normalize_coeffs=True, floor_freq=floor, ceil_freq=None)
    qt, kt = A.transformed_operands("pope", ref["q"], ref["k"], ref["q_r"], ref["k_r"], o, rp["freqs"], rp["delta"], rp["coeffs"])
    kk, vv = kt.repeat_interleave(H // Hkv, dim=2), ref["v"].repeat_interleave(H // Hkv, dim=2)
    sc = torch.einsum("bqhd,bkhd->bhqk", qt, kk) * scale
    sc = sc.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), diagonal=1), float("-inf"))
    want = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, dim=-1), vv)
    want.backward(dout.float())
    assert (out.detach().float().cpu() - want.detach()).abs().max().item() <= 2e-2
    pairs = [(leaf[n].grad, ref[n].grad, n) for n in host] + [(pl[n].grad, rp[n].grad, n) for n in pl]
    for have, ref_g, name in pairs:
        bound = 3e-2 * max(ref_g.abs().max().item(), 1e-3)
        err = (have.float().cpu() - ref_g).abs().max().item()
        assert err <= bound, f"{name}: |diff| {err:.3e} > {bound:.3e}"


def _train_model_cases():
    from oracle import golden_cases as G

    return list(enumerate(G.TRAIN_MODEL_CASES))


@pytest.mark.parametrize("i,spec", _train_model_cases(), ids=lambda s: s["name"] if isinstance(s, dict) else str(s))
def test_transformer_training_step_matches_reference(grads, i, spec):
    """loss.backward() of the Transformer host under bf16 autocast against the reference's
    Transformer under bf16 autocast: the loss, and a strided sample of every parameter's
    gradient (bound as in the module test, scaled by the reference's own bf16 noise)."""
    from oracle import golden_cases as G
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200.model import Transformer, TransformerConfig

    kw = dict(G.TRAIN_MODEL_BASE)
    kw.update({k: v for k, v in spec.items() if k != "name"})
    torch.manual_seed(7500 + i)
    model = Transformer(TransformerConfig(**kw)).train()
    G.fill_parameters(model, 8500 + i)
    model = model.cuda()
    ids = torch.randint(0, kw["vocab_size"], (G.TRAIN_MODEL_BATCH, G.TRAIN_MODEL_SEQ),
                        generator=torch.Generator().manual_seed(9500 + i)).cuda()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = model(ids, labels=ids)
    out["loss"].backward()
    torch.cuda.synchronize()
    check_device_status()
    name = spec["name"]
    assert abs(out["loss"].item() - float(grads[f"{name}/loss"])) <= 2e-3 * float(grads[f"{name}/loss"])
    got = {n: p.grad for n, p in model.named_parameters() if p.grad is not None}
    names = [str(n) for n in grads[f"{name}/grad_names"]]
    assert sorted(got) == names
    for n in names:
        want = torch.from_numpy(grads[f"{name}/grad_sample/{n}"])
        have = got[n].float().cpu().flatten()[::G.TRAIN_MODEL_SAMPLE_STRIDE]
        bound = 1e-2 * float(grads[f"{name}/fp32_max/{n}"]) + 2.0 * float(grads[f"{name}/bf16_noise/{n}"])
        err = (have - want).abs().max().item()
        assert err <= bound, f"{name} grad {n}: |diff| {err:.3e} > {bound:.3e}"


@pytest.mark.parametrize("dc,dr", [(64, 32), (128, 64), (0, 32)])
def test_pope_transform_kernels_match_autograd(dc, dr):
    """pe_pope_expand / pe_pope_expand_backward against the torch restatement of the transform
    (autograd.transformed_operands, itself tied to the oracle in tests/test_modules_cpu.py)."""
    from pe_ablations_b200 import autograd as A
    from pe_ablations_b200.ops import pope_expand, pope_expand_backward

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(21)
    B, S, H = 2, 193, 3
    mk = lambda d: torch.randn(B, S, H, d, generator=g).to(torch.bfloat16).to(dev)
    x_c = mk(dc) if dc else None
    x_r = mk(dr)
    omega = (10000.0 ** (-(torch.arange(dr, dtype=torch.float32) / dr))).to(dev)
    delta = ((torch.rand(dr, generator=g) * 2 - 1) * math.pi).to(dev)
    grad = torch.randn(B, S, H, dc + 2 * dr, generator=g).to(dev)
    for key_side in (False, True):
        dl = delta if key_side else None
        xr_leaf = x_r.clone().requires_grad_(True)
        xc_leaf = None if x_c is None else x_c.clone().requires_grad_(True)
        om_leaf, dl_leaf = omega.clone().requires_grad_(True), delta.clone().requires_grad_(True)
        want = A._pope_rows(xc_leaf, xr_leaf, 7, om_leaf, dl_leaf if key_side else None)
        got = pope_expand(x_c, x_r, 7, omega, dl)
        assert (got.float() - want.detach()).abs().max().item() <= 2e-2
        want.backward(grad)
        sums = torch.zeros(2, dr, dtype=torch.float64, device=dev)
        for gdt in (torch.float32, torch.bfloat16):
            sums.zero_()
            dxc, dxr = pope_expand_backward(grad.to(gdt), x_r, dc, 7, omega, dl, sums[0], sums[1] if key_side else None)
            tol = 2e-2 if gdt == torch.bfloat16 else 1e-2
            torch.testing.assert_close(dxr.float(), xr_leaf.grad.float(), rtol=tol, atol=tol)
            if dc:
                torch.testing.assert_close(dxc.float(), xc_leaf.grad.float(), rtol=tol, atol=tol)
            ref_w = om_leaf.grad.double()
            assert (sums[0] - ref_w).abs().max().item() <= 2e-2 * ref_w.abs().max().item()
            if key_side:
                # gradient of the raw bias: zero where the clamp to [-2 pi, 0] is active, as torch's
                ref_d = dl_leaf.grad.double()
                assert (ref_d == 0).any().item() and (ref_d != 0).any().item()   # both sides of the clamp occur
                assert (sums[1] - ref_d).abs().max().item() <= 2e-2 * max(ref_d.abs().max().item(), 1.0)


@pytest.mark.parametrize("D,rotate,norm,mscale", [(64, True, True, 1.0), (128, True, False, 1.07), (64, False, True, 1.0),
                                                  (128, True, True, 1.07)])
def test_rotary_norm_transform_kernels_match_autograd(D, rotate, norm, mscale):
    """pe_rotary_norm_expand / ..._backward against the torch restatement (rotation, mscale,
    QKNorm) and its autograd."""
    from oracle import pe_attention_oracle as O
    from pe_ablations_b200 import autograd as A
    from pe_ablations_b200.ops import rotary_norm_expand

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(33)
    B, S, H = 2, 171, 3            # 2 * 171 * 3 rows: the last warp is partly idle
    x = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16).to(dev)
    table = O.rotary_table(O.rope_inv_freq(D), 256).to(dev) if rotate else None
    grad = torch.randn(B, S, H, D, generator=g).to(dev)
    leaf = x.clone().requires_grad_(True)
    o = dict(start_pos=9, k_start_pos=9, table_pos0=0, mscale=mscale, qk_norm=norm, qk_norm_eps=1e-6, rotary_table=table)
    want, _ = A.transformed_operands("rotary" if rotate else "nope", leaf, leaf, None, None, o, None, None, None)
    got = rotary_norm_expand(x, table, 9, mscale, norm, 1e-6)
    assert (got.float() - want.detach()).abs().max().item() <= 2e-2 * max(1.0, want.detach().abs().max().item())
    want.backward(grad)
    for gdt in (torch.float32, torch.bfloat16):
        dx = rotary_norm_expand(x, table, 9, mscale, norm, 1e-6, grad=grad.to(gdt))
        tol = 3e-2 if gdt == torch.bfloat16 else 2e-2
        torch.testing.assert_close(dx.float(), leaf.grad.float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("normalize,ceiling", [(True, False), (False, False), (True, True)])
def test_fope_frequency_mix_kernels_match_autograd(normalize, ceiling):
    """pe_fope_effective_freqs / ..._backward against the torch restatement and its autograd
    (floor clip and ceiling clamp both active on some dimensions)."""
    from pe_ablations_b200 import autograd as A
    from pe_ablations_b200.ops import fope_effective_freqs

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(17)
    d_r, n_f = 32, 8
    base = (10000.0 ** (-(torch.arange(d_r, dtype=torch.float32) / d_r)) * 3.0).to(dev)
    coeffs = (torch.randn(d_r, n_f, generator=g) * (0.4 if normalize else 0.05)).to(dev)
    coeffs[3, 2] = 0.0                                   # |a| is not differentiable here: torch uses 0
    floor, ceil = 2 * math.pi / 64, (2.0 if ceiling else None)
    b_leaf, c_leaf = base.clone().requires_grad_(True), coeffs.clone().requires_grad_(True)
    want = A.effective_freqs(b_leaf, c_leaf, normalize, floor, ceil)
    got = fope_effective_freqs(base, coeffs, normalize, floor, ceil)
    assert (got == 0).any() and (got != 0).any()
    torch.testing.assert_close(got, want.detach(), rtol=1e-6, atol=1e-7)
    d_omega = torch.randn(d_r, generator=g, dtype=torch.float64).to(dev)
    want.backward(d_omega.float())
    d_coeffs, d_base = fope_effective_freqs(base, coeffs, normalize, floor, ceil, d_omega=d_omega, want_d_base=True)
    torch.testing.assert_close(d_coeffs, c_leaf.grad, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(d_base, b_leaf.grad, rtol=1e-4, atol=1e-6)


def test_logsumexp_output_of_the_fp32_kernel():
    from pe_ablations_b200 import pe_attention
    from oracle import pe_attention_oracle as O

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(8)
    B, S, H, Hkv, d = 1, 150, 4, 2, 48
    mk = lambda h: torch.randn(B, S, h, d, generator=g)
    q, k, v = mk(H), mk(Hkv), mk(Hkv)
    slopes = O.alibi_slopes(H)
    lse = torch.full((B, H, S), float("nan"), device=dev)
    pe_attention("alibi", q.to(dev), k.to(dev), v.to(dev), alibi_slopes=slopes, lse=lse)
    want = O.attention_core("alibi", q, k, v, slopes=slopes, return_lse=True)[1]
    assert (lse.cpu() - want).abs().max().item() <= 1e-4


def test_backward_accepts_a_strided_upstream_gradient():
    """dout as autograd hands it over after a transpose: not contiguous, copied before the TMA loads."""
    from pe_ablations_b200 import pe_attention

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(9)
    B, S, H, d = 1, 260, 2, 64
    mk = lambda: torch.randn(B, S, H, d, generator=g).to(torch.bfloat16).to(dev).requires_grad_(True)
    q, k, v = mk(), mk(), mk()
    w = torch.randn(B, H, S, d, generator=g).to(torch.bfloat16).to(dev)
    out = pe_attention("nope", q, k, v)
    (out.transpose(1, 2) * w).sum().backward()            # upstream gradient arrives as a transposed view
    g1 = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    out = pe_attention("nope", q, k, v)
    out.backward(w.transpose(1, 2).contiguous())
    for a, b_ in zip(g1, (q.grad, k.grad, v.grad)):
        torch.testing.assert_close(a.float(), b_.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("shape", [(2, 8, 8, 2048, 128, 128), (8, 8, 4, 512, 128, 64), (2, 12, 12, 1024, 64, 64)],
                         ids=["d128_128", "d128_64_gqa", "d64_64"])
def test_repeated_backward_launches_give_the_same_dk_dv(shape):
    """dK and dV are written once per key block in a fixed order of MMAs (P^T / dS^T handed over in
    parts, the next block's products issued early): bitwise the same on every launch.  dQ is a sum
    of TMA reductions in an order that is not fixed: equal up to fp32 rounding."""
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200.ops import attention_backward

    B, H, Hkv, S, dqk, dv = shape
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    mk = lambda h, d: torch.randn(B, S, h, d, device=dev, generator=g).to(torch.bfloat16)
    q, k, v, do, o = mk(H, dqk), mk(Hkv, dqk), mk(Hkv, dv), mk(H, dv), mk(H, dv)
    lse = torch.full((B, H, S), 5.0, device=dev) + torch.log(torch.arange(1, S + 1, device=dev).float())
    first = [t.clone() for t in attention_backward(q, k, v, o, do, lse, scale=dqk ** -0.5)]
    for _ in range(10):
        dq, dk, dv_ = attention_backward(q, k, v, o, do, lse, scale=dqk ** -0.5)
        assert torch.equal(dk, first[1]) and torch.equal(dv_, first[2])
        assert (dq - first[0]).abs().max().item() <= 1e-5 * max(first[0].abs().max().item(), 1.0)
    torch.cuda.synchronize()
    check_device_status()
