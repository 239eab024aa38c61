"""Training path of the fused attention: ``torch.autograd.Function`` around the two kernels.

Forward: the fused forward kernel, unchanged (positional transform in-kernel), plus its
logsumexp output.  Backward: the tensor-core backward kernel (``pe_attn_backward``) gives the
gradients with respect to the TRANSFORMED operands and V; the positional transform itself is
re-evaluated here with differentiable torch operations and autograd carries those gradients
back to the projections and to the encoding's parameters (phase bias, frequencies, Fourier
coefficients).  The transforms and their gradients are kernels too (``pe_pope_expand`` /
``pe_pope_expand_backward`` for the PoPE family, ``pe_rotary_norm_expand`` /
``..._backward`` for rotation, mscale and QKNorm, ``pe_fope_effective_freqs`` / ``..._backward``
for the FoPE frequency mix).  ``transformed_operands`` is the same transform as differentiable torch
code: the tests check the kernels against it, and it against the oracle.  It is the gradient the reference's training step obtains by autograd through
its eager modules (src/model/attention.py:77-96, src/model/alibi.py:137-160,
src/model/fpope_attention.py:145-177 with src/model/pope.py:124-183 /
src/model/fpope.py:107-146,266-338, src/model/rope.py:35-57, src/model/normalization.py:44-56).

bf16 (the modules under bf16 autocast, the precision of the reference's training loop): (d_qk, d_v)
in {(64, 64), (128, 64), (128, 128)} -- every YAML configuration of the reference -- take the
tensor-core backward kernel; the other head dimensions of the bf16 forward, d_qk = 192 / 256 with
d_v = 128 (the 1B shape), take the FFMA backward kernels.

fp32 (the reference's CPU-runnable configuration and its own tests): the forward is the fp32 FFMA
kernel with the transform in-kernel, the attention core's gradients come from the fp32
instantiation of the FFMA backward kernels, and the transform's gradient from autograd over
``transformed_operands`` (ATen operations on the GPU, fp32 throughout: the transform kernels store
bf16 operands and would throw the precision away).  A parity path, not a throughput path.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

_TWO_PI = 2 * math.pi


def effective_freqs(freqs: torch.Tensor, fourier_coeffs: torch.Tensor | None, normalize_coeffs: bool,
                    floor_freq: float, ceil_freq: float | None) -> torch.Tensor:
    """FoPE's collapse of base frequencies and Fourier coefficients (src/model/fpope.py:116-146)."""
    if fourier_coeffs is None:
        return freqs
    a = fourier_coeffs
    if normalize_coeffs:
        a = a / (a.abs().sum(dim=-1, keepdim=True) + 1e-8)
    j = torch.arange(1, a.shape[-1] + 1, device=a.device, dtype=a.dtype)
    eff = (a * (freqs.unsqueeze(1) * j.unsqueeze(0))).sum(dim=1) + freqs   # the reference's operation order
    eff = torch.where(eff.abs() < floor_freq, torch.zeros_like(eff), eff)
    if ceil_freq is not None:
        eff = eff.clamp(-ceil_freq, ceil_freq)
    return eff


def _f32c(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(torch.float32).contiguous()


def _rotate(x: torch.Tensor, table: torch.Tensor, row0: int, mscale: float) -> torch.Tensor:
    """Interleaved-pair rotation of x [B,S,H,D] by table rows row0.. (src/model/rope.py:35-57)."""
    S = x.shape[1]
    t = table[row0:row0 + S]
    cos, sin = t[..., 0].view(1, S, 1, -1), t[..., 1].view(1, S, 1, -1)
    x2 = x.float().reshape(*x.shape[:-1], -1, 2)
    a, b = x2[..., 0], x2[..., 1]
    out = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(-2)
    return out * mscale if mscale != 1.0 else out


def _l2_normalise(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / (x.norm(dim=-1, keepdim=True) + eps)


def _pope_rows(x_c, x_r, pos0: int, omega: torch.Tensor, delta: torch.Tensor | None) -> torch.Tensor:
    """[x_c | softplus(x_r) cos(phase) | softplus(x_r) sin(phase)], phase = pos * omega (+ clamped delta)."""
    S = x_r.shape[1]
    mu = F.softplus(x_r.float())
    pos = torch.arange(pos0, pos0 + S, device=x_r.device, dtype=torch.float32).view(1, S, 1, 1)
    phase = pos * omega.view(1, 1, 1, -1)
    if delta is not None:
        phase = phase + delta.clamp(-_TWO_PI, 0.0).view(1, 1, 1, -1)
    parts = [] if x_c is None else [x_c.float()]
    parts += [mu * torch.cos(phase), mu * torch.sin(phase)]
    return torch.cat(parts, dim=-1)


def transformed_operands(variant: str, q, k, q_r, k_r, o: dict, freqs, delta, fourier_coeffs):
    """The MMA operands the forward kernel builds in shared memory, as differentiable torch, in
    fp32 (the kernel's operands are these rounded to bf16)."""
    if variant == "pope":
        omega = effective_freqs(freqs.float(), None if fourier_coeffs is None else fourier_coeffs.float(),
                                o["normalize_coeffs"], o["floor_freq"], o["ceil_freq"])
        qt = _pope_rows(q, q_r, o["start_pos"], omega, None)
        kt = _pope_rows(k, k_r, o["k_start_pos"], omega, None if delta is None else delta.float())
    else:
        qt, kt = q.float(), k.float()
        if variant == "rotary":
            tab = o["rotary_table"]
            qt = _rotate(qt, tab, o["start_pos"] - o["table_pos0"], o["mscale"])
            kt = _rotate(kt, tab, o["k_start_pos"] - o["table_pos0"], o["mscale"])
        if o["qk_norm"]:
            qt, kt = _l2_normalise(qt, o["qk_norm_eps"]), _l2_normalise(kt, o["qk_norm_eps"])
    return qt, kt


class FusedAttentionFunction(torch.autograd.Function):
    """out = pe_attention(...) with gradients for q, k, v, q_r, k_r, freqs, delta, fourier_coeffs."""

    @staticmethod
    def forward(ctx, variant, o, q, k, v, q_r, k_r, freqs, delta, fourier_coeffs):
        from .ops import _forward_impl

        B, Sq, H = (q if q is not None else q_r).shape[:3]
        lse = torch.empty(B, H, Sq, dtype=torch.float32, device=v.device)
        out = _forward_impl(variant, q, k, v, q_r=q_r, k_r=k_r, freqs=freqs, delta=delta,
                            fourier_coeffs=fourier_coeffs, lse=lse, **o["forward_kwargs"])
        ctx.variant, ctx.o = variant, o
        ctx.save_for_backward(q, k, v, q_r, k_r, freqs, delta, fourier_coeffs, out, lse)
        return out

    @staticmethod
    def backward(ctx, dout):
        from .ops import attention_backward

        q, k, v, q_r, k_r, freqs, delta, fourier_coeffs, out, lse = ctx.saved_tensors
        variant, o = ctx.variant, ctx.o
        dout = dout.to(v.dtype)
        if v.dtype == torch.float32:
            return FusedAttentionFunction._backward_fp32(ctx, dout)
        if variant == "pope":
            return FusedAttentionFunction._backward_pope(ctx, dout)
        from .ops import rotary_norm_expand

        tab = o["rotary_table"] if variant == "rotary" else None
        plain = tab is None and not o["qk_norm"]
        args_q = (tab, o["start_pos"] - o["table_pos0"], o["mscale"], o["qk_norm"], o["qk_norm_eps"])
        args_k = (tab, o["k_start_pos"] - o["table_pos0"], o["mscale"], o["qk_norm"], o["qk_norm_eps"])
        qt = q if plain else rotary_norm_expand(q, *args_q)
        kt = k if plain else rotary_norm_expand(k, *args_k)
        dqt, dkt, dv = attention_backward(qt, kt, v, out, dout, lse, scale=o["scale"], alibi_slopes=o["alibi_slopes"])
        if plain:
            dq, dk = dqt.to(q.dtype), dkt
        else:
            dq = rotary_norm_expand(q, *args_q, grad=dqt)
            dk = rotary_norm_expand(k, *args_k, grad=dkt)
        return (None, None, dq, dk, dv if ctx.needs_input_grad[4] else None, None, None, None, None, None)

    @staticmethod
    def _backward_fp32(ctx, dout):
        """fp32: kernel for the attention core, autograd over the torch restatement for the transform."""
        from .ops import attention_backward

        q, k, v, q_r, k_r, freqs, delta, fourier_coeffs, out, lse = ctx.saved_tensors
        variant, o = ctx.variant, ctx.o
        need = ctx.needs_input_grad[2:]          # q, k, v, q_r, k_r, freqs, delta, fourier_coeffs
        plain = variant in ("nope", "alibi") and not o["qk_norm"]
        leaves = [None] * 8
        if plain:
            qt, kt = q, k
        else:
            with torch.enable_grad():
                given = (q, k, None, q_r, k_r, freqs, delta, fourier_coeffs)
                for i, t in enumerate(given):
                    if t is not None:
                        leaves[i] = t.detach().requires_grad_(bool(need[i]))
                qt, kt = transformed_operands(variant, leaves[0], leaves[1], leaves[3], leaves[4], o, leaves[5],
                                              leaves[6], leaves[7])
        dqt, dkt, dv = attention_backward(qt.detach().contiguous(), kt.detach().contiguous(), v, out, dout, lse,
                                          scale=o["scale"], alibi_slopes=o["alibi_slopes"])
        grads = [None] * 8
        if plain:
            grads[0], grads[1] = dqt, dkt
        else:
            wanted = [i for i in range(8) if leaves[i] is not None and leaves[i].requires_grad]
            pairs = [(t, g) for t, g in ((qt, dqt), (kt, dkt)) if t.requires_grad]
            if wanted and pairs:
                got = torch.autograd.grad([t for t, _ in pairs], [leaves[i] for i in wanted], [g for _, g in pairs],
                                          allow_unused=True)
                for i, g in zip(wanted, got):
                    grads[i] = g
        grads[2] = dv if need[2] else None
        return (None, None, *grads)

    @staticmethod
    def _backward_pope(ctx, dout):
        """PoPE family: frequency mix, transform and both gradients as kernels."""
        from .ops import attention_backward, fope_effective_freqs, pope_expand, pope_expand_backward

        q, k, v, q_r, k_r, freqs, delta, fourier_coeffs, out, lse = ctx.saved_tensors
        o = ctx.o
        dev = v.device
        base = _f32c(freqs)
        coeffs = None if fourier_coeffs is None else _f32c(fourier_coeffs)
        om = base if coeffs is None else fope_effective_freqs(base, coeffs, o["normalize_coeffs"], o["floor_freq"],
                                                              o["ceil_freq"])
        qt = pope_expand(q, q_r, o["start_pos"], om, None)
        kt = pope_expand(k, k_r, o["k_start_pos"], om, delta)
        dqt, dkt, dv = attention_backward(qt, kt, v, out, dout, lse, scale=o["scale"], alibi_slopes=None)
        d_r = q_r.shape[-1]
        d_c = 0 if q is None else q.shape[-1]
        sums = torch.zeros(2, d_r, dtype=torch.float64, device=dev)      # d omega, d clamped delta
        dq, dq_r = pope_expand_backward(dqt, q_r, d_c, o["start_pos"], om, None, sums[0], None)
        dk, dk_r = pope_expand_backward(dkt, k_r, d_c, o["k_start_pos"], om, delta, sums[0], sums[1])
        d_freqs = d_coeffs = d_delta = None
        if coeffs is None:
            if ctx.needs_input_grad[7]:
                d_freqs = sums[0].float()
        elif ctx.needs_input_grad[7] or ctx.needs_input_grad[9]:
            d_coeffs, d_freqs = fope_effective_freqs(base, coeffs, o["normalize_coeffs"], o["floor_freq"], o["ceil_freq"],
                                                     d_omega=sums[0], want_d_base=bool(ctx.needs_input_grad[7]))
        if delta is not None and ctx.needs_input_grad[8]:
            d_delta = sums[1].to(delta.dtype)      # the kernel already zeroes it where the clamp is active
        cast = lambda grad, like: None if grad is None or like is None else grad.to(like.dtype)
        return (None, None, dq, dk, dv if ctx.needs_input_grad[4] else None, dq_r, dk_r,
                cast(d_freqs, freqs), d_delta, cast(d_coeffs, fourier_coeffs))
