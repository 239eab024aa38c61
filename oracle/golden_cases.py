"""The small cases whose reference outputs are frozen under tests/golden/.

TEST INFRASTRUCTURE ONLY.  Shared by the script that generates the fixtures
(which imports the reference) and by the tests that read them (which do not).
"""

from __future__ import annotations

import torch

from .inputs import BF16, FP32, CONFIGS, Case

CORE_CASES = [
    # PoPE family --------------------------------------------------------------
    Case("g_pope_fp32", "pope", FP32, 1, 4, 2, 160, 32, 16, 32, seed=11, training_length=64),
    Case("g_pope_posonly_fp32", "pope", FP32, 2, 2, 2, 97, 0, 32, 64, seed=12),
    Case("g_popefloor_fp32", "pope", FP32, 1, 4, 4, 130, 64, 32, 64, seed=13,
         pope_kind="pope_floor", training_length=64),
    Case("g_fpope_fp32", "pope", FP32, 1, 4, 1, 128, 64, 32, 64, seed=14,
         pope_kind="fpope", training_length=128, n_fourier=16, fourier_sigma=0.3),
    Case("g_fpope_pos0_fp32", "pope", FP32, 1, 2, 2, 70, 32, 16, 32, seed=15, pos0=37,
         pope_kind="fpope", training_length=64, n_fourier=8, fourier_sigma=0.4),
    Case("g_pope_bf16", "pope", BF16, 1, 4, 2, 200, 64, 32, 64, seed=16),
    Case("g_fpope_bf16", "pope", BF16, 1, 2, 2, 320, 128, 64, 128, seed=17,
         pope_kind="fpope", training_length=256, n_fourier=16, fourier_sigma=0.3),
    # rotary family --------------------------------------------------------------
    Case("g_rope_fp32", "rotary", FP32, 1, 4, 2, 150, 64, 0, 64, seed=21),
    Case("g_rope_qknorm_fp32", "rotary", FP32, 2, 4, 4, 77, 32, 0, 32, seed=22, qk_norm=True),
    Case("g_rope_pos0_fp32", "rotary", FP32, 1, 2, 2, 64, 64, 0, 64, seed=23, pos0=100),
    Case("g_ntk_fp32", "rotary", FP32, 1, 4, 4, 128, 64, 0, 64, seed=24, rope_kind="ntk", rope_scale=4.0),
    Case("g_yarn_fp32", "rotary", FP32, 1, 4, 4, 128, 64, 0, 64, seed=25, rope_kind="yarn", rope_scale=2.0),
    Case("g_fope_rotary_fp32", "rotary", FP32, 1, 2, 2, 128, 128, 0, 128, seed=26,
         rope_kind="fope", training_length=128, n_fourier=16, fourier_sigma=0.3),
    Case("g_rope_bf16", "rotary", BF16, 2, 4, 2, 256, 64, 0, 64, seed=27),
    Case("g_ntk_qknorm_bf16", "rotary", BF16, 1, 4, 4, 200, 64, 0, 64, seed=28,
         rope_kind="ntk", rope_scale=4.0, qk_norm=True),
    Case("g_fope_rotary_bf16", "rotary", BF16, 1, 2, 2, 300, 128, 0, 128, seed=29,
         rope_kind="fope", training_length=256, n_fourier=16, fourier_sigma=0.3),
    # NoPE / ALiBi ---------------------------------------------------------------
    Case("g_nope_fp32", "nope", FP32, 1, 4, 2, 100, 64, 0, 64, seed=31),
    Case("g_nope_qknorm_bf16", "nope", BF16, 1, 4, 4, 260, 64, 0, 64, seed=32, qk_norm=True),
    Case("g_alibi_fp32", "alibi", FP32, 1, 12, 4, 90, 64, 0, 64, seed=33, qk_norm=True),
    Case("g_alibi_bf16", "alibi", BF16, 1, 4, 4, 257, 64, 0, 64, seed=34, qk_norm=True),
]

# position-only cases run through the reference's explicit cosine-sum attention
# (src/model/fpope.py:208-244,341-418); fixtures in tests/golden/cos_sum.npz
COS_SUM_CASES = [
    Case("cs_fpope_fp32", "pope", FP32, 1, 4, 1, 128, 0, 32, 64, seed=14, pope_kind="fpope",
         training_length=128, n_fourier=16, fourier_sigma=0.3),
    Case("cs_pope_fp32", "pope", FP32, 1, 4, 2, 160, 0, 16, 32, seed=11, training_length=64),
    Case("cs_fpope_pos0_fp32", "pope", FP32, 2, 2, 2, 70, 0, 16, 32, seed=15, pos0=37, pope_kind="fpope",
         training_length=64, n_fourier=8, fourier_sigma=0.4),
]

# the CPU-runnable benchmark configuration at full size; rows are subsampled in the fixture
FULL_CASES = [(CONFIGS["cfg1_pope_fp32"], 8), (CONFIGS["cfg1_pope_fp32_posonly"], 8)]
TABLE_ROW_STRIDE = 8   # rotary tables are stored every 8th row

# attention-module level: reference module classes with deterministic weights
MODULE_CASES = [
    # name, kind, hidden, H, Hkv, head_dim, d_rope, S, B, pe kwargs
    dict(name="m_gqa_rope", kind="rope", hidden=128, H=4, Hkv=2, head_dim=32, S=48, B=2, use_qk_norm=True),
    dict(name="m_gqa_yarn", kind="yarn", hidden=128, H=4, Hkv=2, head_dim=64, S=40, B=1, use_qk_norm=False,
         rope_scale=2.0),
    dict(name="m_gqa_nope", kind="nope", hidden=128, H=4, Hkv=4, head_dim=32, S=33, B=1, use_qk_norm=True),
    dict(name="m_alibi", kind="alibi", hidden=96, H=6, Hkv=2, head_dim=16, S=50, B=2, use_qk_norm=True),
    dict(name="m_pope", kind="pope", hidden=128, H=4, Hkv=2, head_dim=32, d_rope=16, S=48, B=2,
         use_qk_norm=True, delta_init="uniform"),
    dict(name="m_pope_floor", kind="pope_floor", hidden=128, H=4, Hkv=4, head_dim=32, d_rope=16, S=48, B=1,
         use_qk_norm=True, delta_init="zero", training_length=16),
    dict(name="m_fpope", kind="fpope", hidden=128, H=4, Hkv=1, head_dim=32, d_rope=16, S=48, B=2,
         use_qk_norm=True, delta_init="uniform", n_fourier=8, sigma=0.4, training_length=32),
]

# gradients through the reference's attention modules under bf16 autocast (its training
# precision), at the head dimensions the tensor-core backward covers
TRAIN_CASES = [
    dict(name="g_rope", kind="rope", hidden=64, H=4, Hkv=2, head_dim=64, S=160, B=2, use_qk_norm=True),
    dict(name="g_yarn", kind="yarn", hidden=64, H=2, Hkv=2, head_dim=64, S=144, B=1, use_qk_norm=False,
         rope_scale=2.0),
    dict(name="g_nope_d128", kind="nope", hidden=64, H=2, Hkv=1, head_dim=128, S=130, B=2, use_qk_norm=True),
    dict(name="g_alibi", kind="alibi", hidden=64, H=4, Hkv=2, head_dim=64, S=160, B=2, use_qk_norm=True),
    dict(name="g_pope", kind="pope", hidden=64, H=4, Hkv=2, head_dim=64, d_rope=32, S=160, B=2,
         use_qk_norm=True, delta_init="uniform"),
    dict(name="g_pope_floor", kind="pope_floor", hidden=64, H=2, Hkv=2, head_dim=64, d_rope=32, S=136, B=1,
         use_qk_norm=True, delta_init="zero", training_length=16),
    dict(name="g_fpope", kind="fpope", hidden=64, H=4, Hkv=1, head_dim=64, d_rope=32, S=160, B=2,
         use_qk_norm=True, delta_init="uniform", n_fourier=8, sigma=0.4, training_length=32),
]

# one training step of a small Transformer (loss + gradients) per positional-encoding family
TRAIN_MODEL_BASE = dict(vocab_size=256, hidden_dim=128, num_layers=2, num_heads=2, num_kv_heads=1, head_dim=64,
                        max_seq_len=192, pope_d_rope=32, fpope_d_rope=32)
TRAIN_MODEL_CASES = [
    dict(name="tt_rope", pe_mode="rope"),
    dict(name="tt_alibi", pe_mode="alibi"),
    dict(name="tt_fpope", pe_mode="fpope", fpope_delta_init="uniform", fpope_num_fourier_terms=8,
         fpope_training_length=32),
]
TRAIN_MODEL_BATCH, TRAIN_MODEL_SEQ = 2, 192
TRAIN_MODEL_SAMPLE_STRIDE = 17     # every 17th entry of each flattened gradient is stored

# 2-D parameter gradients are stored for every TRAIN_ROW_STRIDE-th row
TRAIN_ROW_STRIDE = 2

# cached decoding through the reference's FPoPEGroupedQueryAttentionWithCache: a prefill of
# CACHE_PREFILL tokens, then steps of the listed lengths, all with use_cache=True
CACHE_CASE = dict(name="m_fpope_cache", hidden=128, H=4, Hkv=2, head_dim=32, d_rope=16, B=2, use_qk_norm=True,
                  n_fourier=8, sigma=0.4, training_length=32, delta_init="uniform", max_cache_len=64)
CACHE_PREFILL, CACHE_STEPS = 40, (1, 1, 5, 1)

# whole-model level: tiny Transformer per pe_mode, deterministic weights, loss + logits sample
MODEL_CASES = [
    dict(name="t_rope", pe_mode="rope"),
    dict(name="t_ntk", pe_mode="rope", rope_type="ntk", rope_scale=2.0),
    dict(name="t_yarn", pe_mode="rope", rope_type="yarn", rope_scale=2.0, head_dim=64),
    dict(name="t_nope", pe_mode="nope"),
    dict(name="t_alibi", pe_mode="alibi"),
    dict(name="t_pope", pe_mode="pope", pope_delta_init="uniform"),
    dict(name="t_pope_floor", pe_mode="pope_floor", pope_training_length=16),
    dict(name="t_fpope", pe_mode="fpope", fpope_delta_init="uniform", fpope_num_fourier_terms=8,
         fpope_training_length=32),
]
MODEL_BASE = dict(vocab_size=256, hidden_dim=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
                  max_seq_len=64, pope_d_rope=16, fpope_d_rope=16)
MODEL_BATCH, MODEL_SEQ = 2, 64


# the 1B-shape FoPE+PoPE decoder of the benchmark configuration list (d_model 2048, 16 layers,
# 16 heads x head_dim 128, SwiGLU 5632, vocab 32000); MHA and d_rope 64 (d_qk 256)
MODEL_1B = dict(vocab_size=32000, hidden_dim=2048, num_layers=16, num_heads=16, num_kv_heads=16, head_dim=128,
                ffn_dim=5632, max_seq_len=16384, pe_mode="fpope", fpope_d_rope=64, fpope_num_fourier_terms=16,
                fpope_sigma=0.3, fpope_training_length=16384, fpope_delta_init="uniform")
MODEL_1B_SEQ, MODEL_1B_SEED, MODEL_1B_IDS_SEED = 16384, 7000, 7001


def fill_parameters(module: torch.nn.Module, seed: int, std: float = 0.02, linear_gain: float = 4.0) -> None:
    """Overwrite every parameter from one seeded generator, in sorted-name order.

    Independent of construction order, so the reference's modules and the
    drop-in ones get identical weights from the same seed.  Norm weights get
    1 + noise, phase biases U(-pi, pi), everything else N(0, std^2).
    Shared (tied) parameters are written once, under their first sorted name.
    """
    import math

    g = torch.Generator().manual_seed(seed)
    seen: set[int] = set()
    with torch.no_grad():
        for name, p in sorted(module.named_parameters(remove_duplicate=False), key=lambda kv: kv[0]):
            if id(p) in seen:
                continue
            seen.add(id(p))
            if name.endswith("phase_bias"):
                p.copy_((torch.rand(p.shape, generator=g) * 2 - 1) * math.pi)
            elif name.endswith("fourier_coeffs"):
                p.copy_(torch.randn(p.shape, generator=g) * 0.4)
            elif "norm" in name and p.dim() == 1:
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
            else:
                p.copy_(torch.randn(p.shape, generator=g) * std * (linear_gain if p.dim() == 2 and "norm" not in name else 1.0))
