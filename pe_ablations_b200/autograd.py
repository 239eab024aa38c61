"""Training path of the fused attention: ``torch.autograd.Function`` around the two kernels.

Forward: the fused forward kernel, unchanged (positional transform in-kernel), plus its
logsumexp output.  Backward: the tensor-core backward kernel (``pe_attn_backward``) gives the
gradients with respect to the TRANSFORMED operands and V; the positional transform itself is
re-evaluated here with differentiable torch operations and autograd carries those gradients
back to the projections and to the encoding's parameters (phase bias, frequencies, Fourier
coefficients).  It is the gradient the reference's training step obtains by autograd through
its eager modules (src/model/attention.py:77-96, src/model/alibi.py:137-160,
src/model/fpope_attention.py:145-177 with src/model/pope.py:124-183 /
src/model/fpope.py:107-146,266-338, src/model/rope.py:35-57, src/model/normalization.py:44-56).

bf16 only, and only the head dimensions the backward kernel has: (d_qk, d_v) in
{(64, 64), (128, 64), (128, 128)}.  Anything else raises; there is no eager fallback.
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
        # differentiable re-evaluation of the transform on detached leaves
        srcs = [q, k, q_r, k_r, freqs, delta, fourier_coeffs]
        need = [ctx.needs_input_grad[i] for i in (2, 3, 5, 6, 7, 8, 9)]
        leaves = [None if t is None else t.detach().requires_grad_(n) for t, n in zip(srcs, need)]
        with torch.enable_grad():
            qt, kt = transformed_operands(variant, leaves[0], leaves[1], leaves[2], leaves[3], o, leaves[4], leaves[5],
                                          leaves[6])
        dqt, dkt, dv = attention_backward(qt.detach().to(torch.bfloat16), kt.detach().to(torch.bfloat16), v, out,
                                          dout.to(torch.bfloat16), lse, scale=o["scale"],
                                          alibi_slopes=o["alibi_slopes"])
        wanted = [t for t in leaves if t is not None and t.requires_grad]
        # the cast to bf16 is treated as the identity, as autograd treats the reference's own cast
        grads = iter(torch.autograd.grad([qt, kt], wanted, [dqt, dkt.float()], allow_unused=True) if wanted else ())
        g = [next(grads) if (t is not None and t.requires_grad) else None for t in leaves]
        cast = lambda grad, like: None if grad is None else grad.to(like.dtype)
        return (None, None, cast(g[0], q) if q is not None else None, cast(g[1], k) if k is not None else None,
                dv if ctx.needs_input_grad[4] else None,
                cast(g[2], q_r) if q_r is not None else None, cast(g[3], k_r) if k_r is not None else None,
                cast(g[4], freqs) if freqs is not None else None, cast(g[5], delta) if delta is not None else None,
                cast(g[6], fourier_coeffs) if fourier_coeffs is not None else None)
