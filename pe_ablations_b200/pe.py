"""Positional-encoding parameter holders with the reference's names and state_dict keys.

These modules own the constants and learnable parameters of each encoding
(frequency tables, Fourier coefficients, key phase bias) exactly as the
reference's do, so its checkpoints load unchanged.  They do NOT apply the
transform: that happens inside the fused attention kernel, which reads the
parameters from here.  Calling them as functions raises.

Reference classes mirrored (paths inside the reference project):
  RotaryEmbedding / NTKAwareRotaryEmbedding / YaRNRotaryEmbedding  src/model/rope.py:60-217
  PoPEEmbedding                                                    src/model/pope.py:25-122
  FoPEPoPEEmbedding                                                src/model/fpope.py:22-146,246-264
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

_FUSED_MSG = ("the positional transform is fused into the attention kernel; "
              "use the attention modules of pe_ablations_b200.modules")


def _cis_table(inv_freq: torch.Tensor, n_pos: int, device=None) -> torch.Tensor:
    """complex64 [n_pos, len(inv_freq)]: exp(i * t * inv_freq), angles formed in fp32."""
    t = torch.arange(n_pos, device=device)
    ang = torch.outer(t, inv_freq.to(device=device, dtype=torch.float32))
    return torch.polar(torch.ones_like(ang), ang)


class RotaryEmbedding(nn.Module):
    """RoPE table holder: ``freqs_cis`` [max_seq_len, dim/2] complex64 (non-persistent)."""

    def __init__(self, dim: int, max_seq_len: int = 2048, theta: float = 10000.0):
        super().__init__()
        self.dim, self.max_seq_len, self.theta = dim, max_seq_len, theta
        self.register_buffer("freqs_cis", _cis_table(self._inv_freq(), max_seq_len), persistent=False)

    def _inv_freq(self) -> torch.Tensor:
        return 1.0 / (self.theta ** (torch.arange(0, self.dim, 2).float() / self.dim))

    @property
    def attention_scale(self) -> float:
        """Factor applied to q and k after rotation (1 except for YaRN)."""
        return 1.0

    def table(self) -> torch.Tensor:
        """[max_seq_len, dim/2, 2] fp32 (cos, sin) view of ``freqs_cis`` for the kernel."""
        return torch.view_as_real(self.freqs_cis)

    def extend_seq_len(self, new_max_seq_len: int) -> None:
        """Grow the table; like the reference this always rebuilds PLAIN RoPE frequencies from
        ``theta`` (so a YaRN table loses its blend once extended, rope.py:103-119)."""
        if new_max_seq_len <= self.max_seq_len:
            return
        inv = 1.0 / (self.theta ** (torch.arange(0, self.dim, 2).float() / self.dim))
        self.register_buffer("freqs_cis", _cis_table(inv, new_max_seq_len, self.freqs_cis.device), persistent=False)
        self.max_seq_len = new_max_seq_len

    def forward(self, *args, **kwargs):
        raise NotImplementedError(_FUSED_MSG)


class NTKAwareRotaryEmbedding(RotaryEmbedding):
    """RoPE with the NTK-aware base theta * scale^(dim / (dim - 2))."""

    def __init__(self, dim: int, max_seq_len: int = 2048, theta: float = 10000.0, scale: float = 1.0):
        self.scale = scale
        super().__init__(dim, max_seq_len, theta * (scale ** (dim / (dim - 2))))


class YaRNRotaryEmbedding(RotaryEmbedding):
    """YaRN: interpolated / extrapolated frequency blend plus ``mscale`` on q and k."""

    def __init__(self, dim: int, max_seq_len: int = 2048, theta: float = 10000.0, scale: float = 1.0,
                 original_max_seq_len: int = 512, beta_fast: float = 32.0, beta_slow: float = 1.0):
        self.scale = scale
        self.original_max_seq_len = original_max_seq_len
        self.beta_fast, self.beta_slow = beta_fast, beta_slow
        super().__init__(dim, max_seq_len, theta)
        self.register_buffer("freqs_cis", _cis_table(self._yarn_inv_freq(), max_seq_len), persistent=False)
        mscale = 0.1 * torch.log(torch.tensor(scale)) + 1.0
        self.register_buffer("mscale", mscale, persistent=False)
        self._mscale_value = float(mscale)

    def _ramp_bounds(self) -> tuple[int, int]:
        # the reference derives both indices from ``dim`` although the table has dim/2 entries
        def idx(beta: float) -> torch.Tensor:
            return self.dim * torch.log(torch.tensor(self.original_max_seq_len / (beta * 2 * torch.pi))) / \
                torch.log(torch.tensor(self.theta))
        low = max(int(torch.floor(idx(self.beta_fast))), 0)
        high = min(int(torch.ceil(idx(self.beta_slow))), self.dim - 1)
        return low, high

    def _yarn_inv_freq(self) -> torch.Tensor:
        wavelen = self.theta ** (torch.arange(0, self.dim, 2).float() / self.dim)
        keep, stretch = 1.0 / wavelen, 1.0 / (self.scale * wavelen)
        low, high = self._ramp_bounds()
        inv = stretch.clone()
        inv[:low] = keep[:low]
        if low < high:
            w = (torch.arange(low, high + 1).float() - low) / (high - low)
            inv[low:high + 1] = (1 - w) * keep[low:high + 1] + w * stretch[low:high + 1]
        return inv

    @property
    def attention_scale(self) -> float:
        return self._mscale_value


class PoPEEmbedding(nn.Module):
    """Pure PoPE parameters: fixed frequencies theta^(-c/dim), optional floor clip, phase bias."""

    def __init__(self, dim: int, max_seq_len: int = 2048, theta: float = 10000.0, training_length: int = 512,
                 use_floor: bool = False, delta_init: str = "zero"):
        super().__init__()
        self.dim = self.n_freq = dim
        self.max_seq_len, self.theta_base = max_seq_len, theta
        self.training_length, self.use_floor, self.delta_init = training_length, use_floor, delta_init
        self.floor_freq = 2 * math.pi / training_length
        freqs = theta ** (-(torch.arange(0, dim, dtype=torch.float32) / dim))
        self.register_buffer("freqs", freqs)
        eff = torch.where(freqs < self.floor_freq, torch.zeros_like(freqs), freqs) if use_floor else freqs
        self.register_buffer("effective_freqs", eff)
        # kept only so that the reference's checkpoints (which hold it) load strictly
        self.register_buffer("base_angles", torch.outer(torch.arange(max_seq_len, dtype=torch.float32), eff))
        if delta_init == "zero":
            bias = torch.zeros(dim)
        else:
            bias = torch.rand(dim) * 2 * math.pi - 2 * math.pi
        self.phase_bias = nn.Parameter(bias)

    def extend_seq_len(self, new_max_seq_len: int) -> None:
        if new_max_seq_len <= self.max_seq_len:
            return
        pos = torch.arange(new_max_seq_len, dtype=torch.float32, device=self.freqs.device)
        self.register_buffer("base_angles", torch.outer(pos, self.effective_freqs), persistent=False)
        self.max_seq_len = new_max_seq_len

    def kernel_args(self) -> dict:
        """Keyword arguments of ``pe_attention`` that carry this encoding's parameters."""
        return dict(freqs=self.effective_freqs, delta=self.phase_bias)

    def forward(self, *args, **kwargs):
        raise NotImplementedError(_FUSED_MSG)

    forward_query = forward_key = forward


class FoPEPoPEEmbedding(nn.Module):
    """FoPE + PoPE parameters: base frequencies, Fourier coefficients, phase bias.

    The effective frequency of dimension c is base_c * (1 + sum_j a^_{c,j} j) with
    L1-normalised coefficients, clipped to 0 below 2 pi / training_length (and optionally
    clamped to +-2 pi).  The kernel evaluates this from the raw parameters at every call,
    so learnable coefficients stay live; ``effective_freqs()`` is the same formula on the
    host for logging.
    """

    def __init__(self, dim: int, max_seq_len: int = 2048, theta: float = 10000.0, num_fourier_terms: int = 64,
                 fourier_sigma: float = 0.4, training_length: int = 512, delta_init: str = "zero",
                 freeze_coeffs: bool = False, use_ceiling: bool = False, normalize_coeffs: bool = True):
        super().__init__()
        self.dim, self.max_seq_len, self.theta = dim, max_seq_len, theta
        self.num_fourier_terms, self.fourier_sigma = num_fourier_terms, fourier_sigma
        self.training_length, self.delta_init = training_length, delta_init
        self.floor_freq = 2 * math.pi / training_length
        self.use_ceiling, self.ceiling_freq = use_ceiling, 2 * math.pi
        self.normalize_coeffs = normalize_coeffs
        self.register_buffer("base_freqs", theta ** (-torch.arange(0, dim, dtype=torch.float32) / dim))
        self.fourier_coeffs = nn.Parameter(torch.randn(dim, num_fourier_terms) * fourier_sigma,
                                           requires_grad=not freeze_coeffs)
        self.register_buffer("fourier_indices", torch.arange(1, num_fourier_terms + 1, dtype=torch.float32))
        bias = torch.zeros(dim) if delta_init == "zero" else torch.rand(dim) * 2 * math.pi - math.pi
        self.phase_bias = nn.Parameter(bias)
        self.register_buffer("positions", torch.arange(max_seq_len, dtype=torch.float32))

    def extend_seq_len(self, new_max_seq_len: int) -> None:
        if new_max_seq_len <= self.max_seq_len:
            return
        pos = torch.arange(new_max_seq_len, dtype=torch.float32, device=self.positions.device)
        self.register_buffer("positions", pos, persistent=False)
        self.max_seq_len = new_max_seq_len

    @torch.no_grad()
    def effective_freqs(self) -> torch.Tensor:
        a = self.fourier_coeffs
        if self.normalize_coeffs:
            a = a / (a.abs().sum(dim=1, keepdim=True) + 1e-8)
        eff = (a * (self.base_freqs[:, None] * self.fourier_indices[None, :])).sum(dim=1) + self.base_freqs
        eff = torch.where(eff.abs() < self.floor_freq, torch.zeros_like(eff), eff)
        return eff.clamp(-self.ceiling_freq, self.ceiling_freq) if self.use_ceiling else eff

    _compute_effective_freqs = effective_freqs

    def kernel_args(self) -> dict:
        return dict(freqs=self.base_freqs, fourier_coeffs=self.fourier_coeffs, delta=self.phase_bias,
                    floor_freq=self.floor_freq, normalize_coeffs=self.normalize_coeffs,
                    ceil_freq=self.ceiling_freq if self.use_ceiling else None)

    def forward(self, *args, **kwargs):
        raise NotImplementedError(_FUSED_MSG)

    forward_query = forward_key = forward


def alibi_slopes(num_heads: int) -> torch.Tensor:
    """Per-head ALiBi slopes (src/model/alibi.py:20-44): a geometric sequence for power-of-two
    head counts, otherwise the closest lower power of two plus every other slope of the next."""

    def geometric(n: int) -> list[float]:
        first = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [first ** (i + 1) for i in range(n)]

    if math.log2(num_heads).is_integer():
        return torch.tensor(geometric(num_heads))
    base = 2 ** math.floor(math.log2(num_heads))
    return torch.tensor(geometric(base) + geometric(2 * base)[0::2][: num_heads - base])
