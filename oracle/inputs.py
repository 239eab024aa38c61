"""Seeded synthetic inputs for the PE-attention cases.  TEST INFRASTRUCTURE ONLY.

One CPU ``torch.Generator`` per case, draws in a fixed order (q, k, [q_r, k_r],
v, delta, fourier coefficients), so the same case name and seed give the same
tensors on every machine.  Tensors are in the projection layout [B, S, H, d].
The named cases follow the benchmark configurations (shapes, dtypes, value
distributions); no public dataset stands behind any of them.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from . import pe_attention_oracle as O


@dataclass
class Case:
    name: str
    variant: str              # nope | rotary | alibi | pope
    dtype: torch.dtype
    B: int
    H: int
    Hkv: int
    S: int
    d_c: int                  # content / plain head dim (0 = position-only PoPE)
    d_r: int = 0              # PoPE position dim before the cos/sin expansion
    d_v: int = 0
    seed: int = 0
    pos0: int = 0
    qk_norm: bool = False
    # rotary
    rope_kind: str = "standard"     # standard | ntk | yarn | fope
    rope_theta: float = 10000.0
    rope_scale: float = 1.0
    # pope family
    pope_kind: str = "pope"         # pope | pope_floor | fpope
    pope_theta: float = 10000.0
    training_length: int = 512
    n_fourier: int = 16
    fourier_sigma: float = 0.3
    delta_init: str = "uniform_pm_pi"   # uniform_pm_pi | zero | uniform_neg
    extra: dict = field(default_factory=dict)

    @property
    def d_qk(self) -> int:
        return self.d_c + 2 * self.d_r

    @property
    def flops(self) -> float:
        """Algorithmic causal attention FLOPs: B*H*S^2*(d_qk + d_v)."""
        return float(self.B) * self.H * self.S * self.S * (self.d_qk + self.d_v)


def _randn(g, *shape):
    return torch.randn(*shape, generator=g, dtype=torch.float32)


def make_inputs(case: Case) -> dict:
    """Draw the tensors and PE parameters for ``case`` (all fp32 on CPU)."""
    g = torch.Generator().manual_seed(case.seed)
    B, S, H, Hkv = case.B, case.S, case.H, case.Hkv
    out: dict = {}
    if case.d_c > 0:
        out["q"] = _randn(g, B, S, H, case.d_c)
        out["k"] = _randn(g, B, S, Hkv, case.d_c)
    else:
        out["q"] = out["k"] = None
    if case.variant == "pope":
        out["q_r"] = _randn(g, B, S, H, case.d_r)
        out["k_r"] = _randn(g, B, S, Hkv, case.d_r)
    out["v"] = _randn(g, B, S, Hkv, case.d_v)

    if case.variant == "pope":
        u = torch.rand(case.d_r, generator=g)
        if case.delta_init == "uniform_pm_pi":
            out["delta"] = (u * 2.0 - 1.0) * math.pi
        elif case.delta_init == "uniform_neg":
            out["delta"] = u * 2 * math.pi - 2 * math.pi
        else:
            out["delta"] = torch.zeros(case.d_r)
        base = O.pope_base_freqs(case.d_r, case.pope_theta)
        out["base_freqs"] = base
        if case.pope_kind == "fpope":
            coeffs = _randn(g, case.d_r, case.n_fourier) * case.fourier_sigma
            out["fourier_coeffs"] = coeffs
            out["freqs"] = O.fope_effective_freqs(base, coeffs, case.training_length)
        elif case.pope_kind == "pope_floor":
            out["freqs"] = O.pope_floor_clip(base, case.training_length)
        else:
            out["freqs"] = base
    elif case.variant == "rotary":
        D = case.d_c
        mscale = 1.0
        if case.rope_kind == "standard":
            inv = O.rope_inv_freq(D, case.rope_theta)
        elif case.rope_kind == "ntk":
            inv = O.rope_inv_freq(D, O.ntk_theta(D, case.rope_theta, case.rope_scale))
        elif case.rope_kind == "yarn":
            inv, mscale = O.yarn_inv_freq(D, case.rope_theta, case.rope_scale)
        elif case.rope_kind == "fope":
            base = O.pope_base_freqs(D // 2, case.rope_theta)
            coeffs = _randn(g, D // 2, case.n_fourier) * case.fourier_sigma
            out["fourier_coeffs"] = coeffs
            out["base_freqs"] = base
            inv = O.fope_effective_freqs(base, coeffs, case.training_length)
        else:
            raise ValueError(case.rope_kind)
        out["inv_freq"] = inv
        out["mscale"] = mscale
        out["table"] = O.rotary_table(inv, case.pos0 + S)[case.pos0:]
    elif case.variant == "alibi":
        out["slopes"] = O.alibi_slopes(H)
    return out


def oracle_output(case: Case, inp: dict, acc: torch.dtype = torch.float32) -> torch.Tensor:
    """Run the oracle for ``case`` on ``inp`` -> [B, S, H, d_v] in ``acc``."""
    return O.attention_core(
        case.variant, inp.get("q"), inp.get("k"), inp["v"],
        dtype=case.dtype, q_r=inp.get("q_r"), k_r=inp.get("k_r"), pos0=case.pos0,
        table=inp.get("table"), mscale=inp.get("mscale", 1.0), qk_norm=case.qk_norm,
        freqs=inp.get("freqs"), delta=inp.get("delta"), slopes=inp.get("slopes"), acc=acc,
    )


# ---- the five benchmark configurations -----------------------------------
BF16, FP32 = torch.bfloat16, torch.float32

CONFIGS = {
    # PoPE fp32, the CPU-runnable case: attention shapes of an 8-head, head_dim 64,
    # d_rope 32, seq 512 model; theta_c = 10000^(-c/32); delta ~ U(-pi, pi)
    "cfg1_pope_fp32": Case("cfg1_pope_fp32", "pope", FP32, 1, 8, 8, 512, 64, 32, 64,
                           pope_kind="pope", training_length=512),
    "cfg1_pope_fp32_posonly": Case("cfg1_pope_fp32_posonly", "pope", FP32, 1, 8, 8, 512, 0, 32, 64,
                                   pope_kind="pope", training_length=512),
    "cfg2_rope_bf16": Case("cfg2_rope_bf16", "rotary", BF16, 8, 12, 12, 2048, 64, 0, 64),
    "cfg2_ntk4_bf16": Case("cfg2_ntk4_bf16", "rotary", BF16, 8, 12, 12, 2048, 64, 0, 64,
                           rope_kind="ntk", rope_scale=4.0),
    "cfg3_fope_bf16": Case("cfg3_fope_bf16", "rotary", BF16, 4, 16, 16, 4096, 128, 0, 128,
                           rope_kind="fope", training_length=4096, n_fourier=16, fourier_sigma=0.3),
    "cfg4_fpope_bf16": Case("cfg4_fpope_bf16", "pope", BF16, 2, 16, 16, 16384, 128, 64, 128,
                            pope_kind="fpope", training_length=16384, n_fourier=16, fourier_sigma=0.3),
}
