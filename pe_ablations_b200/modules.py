"""Drop-in replacements for the reference's three attention modules.

Same constructor signatures, same ``forward(x, mask=None, start_pos=0)``, same
parameter and buffer names (so the reference's checkpoints load with
``strict=True``).  Projections stay ``nn.Linear``; everything between "projected
Q/K/V" and "attention output before ``wo``" is one fused kernel call.

Reference classes mirrored (paths inside the reference project):
  GroupedQueryAttention       src/model/attention.py:12-100
  ALiBiAttention              src/model/alibi.py:47-163
  FPoPEGroupedQueryAttention  src/model/fpope_attention.py:29-181
  RMSNorm                     src/model/normalization.py:7-27

The fused path is causal-only: a ``mask`` raises.  The modules also train: a call that needs
gradients goes through ``autograd.FusedAttentionFunction`` -- under bf16 autocast the fused
forward and the tensor-core (or, at the 1B head dims, FFMA) backward kernel, in fp32 the fp32
FFMA forward and backward kernels; at head dimensions no backward kernel has, such a call
raises -- there is no eager fallback.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .ops import linear_residual, pe_attention, projections
from .pe import alibi_slopes


class RMSNorm(nn.Module):
    """x * rsqrt(mean(x^2) + eps) in fp32, cast back, times a learned weight."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda and not (torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad)):
            fused_bf16 = x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and (
                self.weight.dtype == torch.bfloat16
                or (torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16))
            if fused_bf16 or (x.dtype == torch.float32 and self.weight.dtype == torch.float32 and x.shape[-1] % 8 == 0):
                # one pass; for bf16 the result already carries the cast the next linear applies
                from .ops import rmsnorm

                return rmsnorm(x, self.weight, self.eps)
        xf = x.float()
        y = xf * torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + self.eps)
        return y.type_as(x) * self.weight


class QKNorm(nn.Module):
    """Marker for per-row L2 normalisation of q and k; the kernel applies it (eps as here)."""

    def __init__(self, head_dim: int, eps: float = 1e-6):
        super().__init__()
        self.head_dim, self.eps = head_dim, eps


def _check_call(x: torch.Tensor, mask) -> None:
    if mask is not None:
        raise NotImplementedError("the fused attention is causal-only; an explicit mask is not supported")


def _kernel_dtype(t: torch.Tensor) -> torch.dtype:
    # under bf16 autocast the projections are bf16; anything else runs the fp32 path
    return torch.bfloat16 if t.dtype == torch.bfloat16 else torch.float32


class GroupedQueryAttention(nn.Module):
    """GQA with RoPE (plain / NTK / YaRN tables) or no positional encoding, optional QKNorm."""

    def __init__(self, hidden_dim: int, num_heads: int, num_kv_heads: int, head_dim: int | None = None,
                 use_qk_norm: bool = True, rope: nn.Module | None = None):
        super().__init__()
        assert num_heads % num_kv_heads == 0, "num_heads must be divisible by num_kv_heads"
        self.hidden_dim, self.num_heads, self.num_kv_heads = hidden_dim, num_heads, num_kv_heads
        self.head_dim = head_dim or (hidden_dim // num_heads)
        self.num_groups = num_heads // num_kv_heads
        self.wq = nn.Linear(hidden_dim, num_heads * self.head_dim, bias=False)
        self.wk = nn.Linear(hidden_dim, num_kv_heads * self.head_dim, bias=False)
        self.wv = nn.Linear(hidden_dim, num_kv_heads * self.head_dim, bias=False)
        self.wo = nn.Linear(num_heads * self.head_dim, hidden_dim, bias=False)
        self.qk_norm = QKNorm(self.head_dim) if use_qk_norm else None
        self.rope = rope

    def forward(self, x: torch.Tensor, mask: torch.Tensor | None = None, start_pos: int = 0,
                residual: torch.Tensor | None = None) -> torch.Tensor:
        _check_call(x, mask)
        B, S, _ = x.shape
        q, k, v = projections(self, x, self.wq, self.wk, self.wv)
        q = q.view(B, S, self.num_heads, self.head_dim)
        k = k.view(B, S, self.num_kv_heads, self.head_dim)
        v = v.view(B, S, self.num_kv_heads, self.head_dim)
        dt = _kernel_dtype(q)
        kw = {}
        variant = "nope"
        if self.rope is not None:
            variant = "rotary"
            kw["rotary_table"] = self.rope.freqs_cis
            # every table of the reference's rope classes is angle = position x inverse frequency
            kw["table_geometric"] = bool(getattr(self.rope, "table_geometric", True))
            scale_qk = getattr(self.rope, "attention_scale", None)
            if scale_qk is None and hasattr(self.rope, "mscale"):
                scale_qk = float(self.rope.mscale)
            kw["mscale"] = 1.0 if scale_qk is None else scale_qk
        out = pe_attention(variant, q.to(dt), k.to(dt), v.to(dt), start_pos=start_pos,
                           scale=1.0 / (self.head_dim ** 0.5), qk_norm=self.qk_norm is not None,
                           qk_norm_eps=self.qk_norm.eps if self.qk_norm is not None else 1e-6, **kw)
        return linear_residual(self.wo, out.view(B, S, self.num_heads * self.head_dim).to(x.dtype), residual)


class ALiBiAttention(nn.Module):
    """GQA with ALiBi: logits - slope_h |t - s| (bias not scaled), optional QKNorm."""

    def __init__(self, hidden_dim: int, num_heads: int, num_kv_heads: int, head_dim: int | None = None,
                 use_qk_norm: bool = True):
        super().__init__()
        assert num_heads % num_kv_heads == 0, "num_heads must be divisible by num_kv_heads"
        self.hidden_dim, self.num_heads, self.num_kv_heads = hidden_dim, num_heads, num_kv_heads
        self.head_dim = head_dim or (hidden_dim // num_heads)
        self.num_groups = num_heads // num_kv_heads
        self.wq = nn.Linear(hidden_dim, num_heads * self.head_dim, bias=False)
        self.wk = nn.Linear(hidden_dim, num_kv_heads * self.head_dim, bias=False)
        self.wv = nn.Linear(hidden_dim, num_kv_heads * self.head_dim, bias=False)
        self.wo = nn.Linear(num_heads * self.head_dim, hidden_dim, bias=False)
        self.qk_norm = QKNorm(self.head_dim) if use_qk_norm else None
        self.register_buffer("alibi_slopes", alibi_slopes(num_heads).view(1, num_heads, 1, 1))

    def forward(self, x: torch.Tensor, mask: torch.Tensor | None = None, start_pos: int = 0,
                residual: torch.Tensor | None = None) -> torch.Tensor:
        _check_call(x, mask)
        B, S, _ = x.shape
        q, k, v = projections(self, x, self.wq, self.wk, self.wv)
        q = q.view(B, S, self.num_heads, self.head_dim)
        k = k.view(B, S, self.num_kv_heads, self.head_dim)
        v = v.view(B, S, self.num_kv_heads, self.head_dim)
        dt = _kernel_dtype(q)
        out = pe_attention("alibi", q.to(dt), k.to(dt), v.to(dt), scale=self.head_dim ** -0.5,
                           qk_norm=self.qk_norm is not None,
                           qk_norm_eps=self.qk_norm.eps if self.qk_norm is not None else 1e-6,
                           alibi_slopes=self.alibi_slopes)
        return linear_residual(self.wo, out.view(B, S, self.num_heads * self.head_dim).to(x.dtype), residual)


class FPoPEGroupedQueryAttention(nn.Module):
    """Content + position split attention for PoPE, PoPE-floor and FoPE+PoPE.

    q = [q_c, mu_q cos(t w), mu_q sin(t w)], k = [k_c, mu_k cos(s w + d), mu_k sin(s w + d)] with
    mu = softplus of the RMS-normalised position projections; the expansion happens in the
    kernel, so only the un-expanded d_rope columns are ever read from memory.
    """

    def __init__(self, hidden_dim: int, num_heads: int, num_kv_heads: int, head_dim: int = 64, d_rope: int = 32,
                 use_qk_norm: bool = True, fpope: nn.Module | None = None):
        super().__init__()
        assert num_heads % num_kv_heads == 0, "num_heads must be divisible by num_kv_heads"
        self.hidden_dim, self.num_heads, self.num_kv_heads = hidden_dim, num_heads, num_kv_heads
        self.head_dim, self.d_rope, self.d_content = head_dim, d_rope, head_dim
        self.num_groups = num_heads // num_kv_heads
        self.wq_c = nn.Linear(hidden_dim, num_heads * self.d_content, bias=False)
        self.wk_c = nn.Linear(hidden_dim, num_kv_heads * self.d_content, bias=False)
        self.wq_r = nn.Linear(hidden_dim, num_heads * d_rope, bias=False)
        self.wk_r = nn.Linear(hidden_dim, num_kv_heads * d_rope, bias=False)
        self.qr_norm = RMSNorm(num_heads * d_rope) if use_qk_norm else None
        self.kr_norm = RMSNorm(num_kv_heads * d_rope) if use_qk_norm else None
        self.wv = nn.Linear(hidden_dim, num_kv_heads * head_dim, bias=False)
        self.wo = nn.Linear(num_heads * head_dim, hidden_dim, bias=False)
        self.fpope = fpope
        self.scale = (self.d_content + 2 * d_rope) ** -0.5

    def _pe_args(self) -> dict:
        pe = self.fpope
        if pe is None:
            raise NotImplementedError("FPoPEGroupedQueryAttention needs a PoPE / FoPE+PoPE embedding")
        if hasattr(pe, "kernel_args"):
            return pe.kernel_args()
        # the reference's own embedding objects
        if hasattr(pe, "fourier_coeffs"):
            return dict(freqs=pe.base_freqs, fourier_coeffs=pe.fourier_coeffs, delta=pe.phase_bias,
                        floor_freq=pe.floor_freq, normalize_coeffs=pe.normalize_coeffs,
                        ceil_freq=pe.ceiling_freq if pe.use_ceiling else None)
        return dict(freqs=pe.effective_freqs, delta=pe.phase_bias)

    def forward(self, x: torch.Tensor, mask: torch.Tensor | None = None, start_pos: int = 0,
                residual: torch.Tensor | None = None) -> torch.Tensor:
        _check_call(x, mask)
        B, S, _ = x.shape
        q_c, k_c, q_r, k_r, v = projections(self, x, self.wq_c, self.wk_c, self.wq_r, self.wk_r, self.wv)
        q_c = q_c.view(B, S, self.num_heads, self.d_content)
        k_c = k_c.view(B, S, self.num_kv_heads, self.d_content)
        if self.qr_norm is not None:
            q_r, k_r = self.qr_norm(q_r), self.kr_norm(k_r)
        dt = _kernel_dtype(q_c)
        q_r = q_r.to(dt).view(B, S, self.num_heads, self.d_rope)
        k_r = k_r.to(dt).view(B, S, self.num_kv_heads, self.d_rope)
        v = v.view(B, S, self.num_kv_heads, self.head_dim)
        out = pe_attention("pope", q_c.to(dt), k_c.to(dt), v.to(dt), q_r=q_r, k_r=k_r, start_pos=start_pos,
                           scale=self.scale, **self._pe_args())
        return linear_residual(self.wo, out.view(B, S, self.num_heads * self.head_dim).to(x.dtype), residual)


class FPoPEGroupedQueryAttentionWithCache(FPoPEGroupedQueryAttention):
    """FPoPEGroupedQueryAttention with a KV cache for autoregressive decoding
    (src/model/fpope_attention.py:184-327).

    The reference caches the already-transformed keys; here the cache holds the RAW content
    and position halves of K (and V), [B, max_cache_len, Hkv, d], and the kernel transforms
    the cached keys at use with their absolute positions -- same output, and the phase bias /
    frequencies stay live.  ``forward(..., use_cache=True)`` appends the new tokens at
    ``start_pos`` and attends over everything cached so far (key s visible to the new token
    at position t iff s <= t).
    """

    def __init__(self, hidden_dim: int, num_heads: int, num_kv_heads: int, head_dim: int = 64, d_rope: int = 32,
                 use_qk_norm: bool = True, fpope: nn.Module | None = None, max_cache_len: int = 2048):
        super().__init__(hidden_dim, num_heads, num_kv_heads, head_dim, d_rope, use_qk_norm, fpope)
        self.max_cache_len = max_cache_len
        self.k_cache = self.kr_cache = self.v_cache = None
        self.cache_len = 0

    def reset_cache(self) -> None:
        self.k_cache = self.kr_cache = self.v_cache = None
        self.cache_len = 0

    def forward(self, x: torch.Tensor, mask: torch.Tensor | None = None, start_pos: int = 0,
                use_cache: bool = False) -> torch.Tensor:
        if not use_cache:
            return super().forward(x, mask, start_pos)
        _check_call(x, mask)
        B, S, _ = x.shape
        if start_pos + S > self.max_cache_len:
            raise ValueError(f"start_pos + seq_len = {start_pos + S} exceeds max_cache_len = {self.max_cache_len}")
        q_c = self.wq_c(x).view(B, S, self.num_heads, self.d_content)
        k_c = self.wk_c(x).view(B, S, self.num_kv_heads, self.d_content)
        q_r, k_r = self.wq_r(x), self.wk_r(x)
        if self.qr_norm is not None:
            q_r, k_r = self.qr_norm(q_r), self.kr_norm(k_r)
        dt = _kernel_dtype(q_c)
        q_r = q_r.to(dt).view(B, S, self.num_heads, self.d_rope)
        k_r = k_r.to(dt).view(B, S, self.num_kv_heads, self.d_rope)
        v = self.wv(x).view(B, S, self.num_kv_heads, self.head_dim)
        if self.k_cache is None or self.k_cache.shape[0] != B or self.k_cache.dtype != dt or self.k_cache.device != x.device:
            mk = lambda d: torch.zeros(B, self.max_cache_len, self.num_kv_heads, d, dtype=dt, device=x.device)
            self.k_cache, self.kr_cache, self.v_cache = mk(self.d_content), mk(self.d_rope), mk(self.head_dim)
        self.k_cache[:, start_pos:start_pos + S] = k_c.to(dt)
        self.kr_cache[:, start_pos:start_pos + S] = k_r
        self.v_cache[:, start_pos:start_pos + S] = v.to(dt)
        self.cache_len = start_pos + S
        n = self.cache_len
        out = pe_attention("pope", q_c.to(dt), self.k_cache[:, :n], self.v_cache[:, :n], q_r=q_r,
                           k_r=self.kr_cache[:, :n], start_pos=start_pos, k_start_pos=0, scale=self.scale,
                           **self._pe_args())
        return self.wo(out.view(B, S, self.num_heads * self.head_dim).to(x.dtype))


def install(namespace=None) -> None:
    """Rebind the reference's attention classes to the fused ones.

    With the reference importable (``src.model``), its ``Transformer`` builds the drop-in
    modules from unchanged YAML configs afterwards.  ``namespace`` defaults to
    ``src.model.transformer``.
    """
    if namespace is None:
        import importlib

        namespace = importlib.import_module("src.model.transformer")
    namespace.GroupedQueryAttention = GroupedQueryAttention
    namespace.ALiBiAttention = ALiBiAttention
    namespace.FPoPEGroupedQueryAttention = FPoPEGroupedQueryAttention
