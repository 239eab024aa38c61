"""Decoder-only Transformer host for the fused attention, with the reference's interface.

``TransformerConfig`` has the reference's fields, ``Transformer(config)`` its module tree
and state_dict keys (including the shared positional-encoding module registered both on
the model and under every block's attention), so reference checkpoints load with
``strict=True`` and ``model(input_ids, labels=..., start_pos=...)`` returns the same dict.
Everything except attention is plain torch (cuBLAS linears, elementwise ops); attention is
the fused kernel.  Under bf16 autocast ``loss.backward()`` works too (tensor-core backward
kernel, see ``autograd.py``).

Reference mirrored (paths inside the reference project): src/model/transformer.py:21-387,
src/model/ffn.py:30-68, src/model/embeddings.py:7-34.

``loss_sums`` is the evaluation entry point: it returns (sum of token NLLs, token count)
without materialising the full logits, which is what a sharded perplexity run reduces.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .modules import ALiBiAttention, FPoPEGroupedQueryAttention, GroupedQueryAttention, RMSNorm
from .pe import (FoPEPoPEEmbedding, NTKAwareRotaryEmbedding, PoPEEmbedding, RotaryEmbedding,
                 YaRNRotaryEmbedding)


@dataclass
class TransformerConfig:
    vocab_size: int = 50257
    hidden_dim: int = 512
    num_layers: int = 24
    num_heads: int = 8
    num_kv_heads: int = 4
    head_dim: int = 64
    ffn_dim: int | None = None
    ffn_multiple_of: int = 256
    pe_mode: str = "rope"            # rope | fpope | pope | pope_floor | alibi | nope
    max_seq_len: int = 512
    rope_theta: float = 10000.0
    rope_type: str = "standard"      # standard | ntk | yarn
    rope_scale: float = 1.0
    fpope_theta: float = 10000.0
    fpope_num_fourier_terms: int = 64
    fpope_sigma: float = 0.4
    fpope_training_length: int = 512
    fpope_delta_init: str = "zero"
    fpope_d_rope: int = 32
    fpope_freeze_coeffs: bool = False
    fpope_use_ceiling: bool = False
    fpope_normalize_coeffs: bool = True
    pope_theta: float = 10000.0
    pope_training_length: int = 512
    pope_delta_init: str = "zero"
    pope_d_rope: int = 32
    norm_eps: float = 1e-6
    use_qk_norm: bool = True
    dropout: float = 0.0
    tie_embeddings: bool = True
    gradient_checkpointing: bool = False

    def __post_init__(self) -> None:
        if self.head_dim is None:
            self.head_dim = self.hidden_dim // self.num_heads

    def resolved_ffn_dim(self) -> int:
        if self.ffn_dim is not None:
            return self.ffn_dim
        d = int(4 * self.hidden_dim * 2 / 3)
        m = self.ffn_multiple_of
        return m * ((d + m - 1) // m)


class TokenEmbedding(nn.Module):
    def __init__(self, vocab_size: int, embed_dim: int):
        super().__init__()
        self.vocab_size, self.embed_dim = vocab_size, embed_dim
        self.embedding = nn.Embedding(vocab_size, embed_dim)

    @property
    def weight(self) -> torch.Tensor:
        return self.embedding.weight

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return self.embedding(ids)


class FeedForward(nn.Module):
    """SwiGLU: w2(silu(w3 x) * w1 x)."""

    def __init__(self, hidden_dim: int, ffn_dim: int):
        super().__init__()
        self.w1 = nn.Linear(hidden_dim, ffn_dim, bias=False)
        self.w2 = nn.Linear(ffn_dim, hidden_dim, bias=False)
        self.w3 = nn.Linear(hidden_dim, ffn_dim, bias=False)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``w2(silu(w3 x) * w1 x)``, plus ``residual`` when the block passes its stream in."""
        from .ops import fused_gemm_ok, linear_residual, swiglu, swiglu_gemm

        if fused_gemm_ok(x, self.w3.weight, self.w1.weight):
            # both input projections and SwiGLU in one tensor-core kernel: gate and up never exist
            return linear_residual(self.w2, swiglu_gemm(x, self.w3.weight, self.w1.weight), residual)
        gate, up = self.w3(x), self.w1(x)
        if gate.is_cuda and not (torch.is_grad_enabled() and gate.requires_grad) and gate.numel() % 8 == 0 \
                and gate.dtype in (torch.bfloat16, torch.float32):
            return linear_residual(self.w2, swiglu(gate, up), residual)
        return linear_residual(self.w2, F.silu(gate) * up, residual)


def _build_pe(cfg: TransformerConfig):
    """(rope, fpope, pope) shared positional-encoding modules for ``cfg.pe_mode``."""
    rope = fpope = pope = None
    mode = cfg.pe_mode
    if mode == "rope":
        if cfg.rope_type == "standard":
            rope = RotaryEmbedding(cfg.head_dim, cfg.max_seq_len, cfg.rope_theta)
        elif cfg.rope_type == "ntk":
            rope = NTKAwareRotaryEmbedding(cfg.head_dim, cfg.max_seq_len, cfg.rope_theta, cfg.rope_scale)
        elif cfg.rope_type == "yarn":
            rope = YaRNRotaryEmbedding(cfg.head_dim, cfg.max_seq_len, cfg.rope_theta, cfg.rope_scale,
                                       original_max_seq_len=512)
        else:
            raise ValueError(f"Unknown rope_type: {cfg.rope_type}")
    elif mode == "fpope":
        fpope = FoPEPoPEEmbedding(dim=cfg.fpope_d_rope, max_seq_len=cfg.max_seq_len, theta=cfg.fpope_theta,
                                  num_fourier_terms=cfg.fpope_num_fourier_terms, fourier_sigma=cfg.fpope_sigma,
                                  training_length=cfg.fpope_training_length, delta_init=cfg.fpope_delta_init,
                                  freeze_coeffs=cfg.fpope_freeze_coeffs, use_ceiling=cfg.fpope_use_ceiling,
                                  normalize_coeffs=cfg.fpope_normalize_coeffs)
    elif mode in ("pope", "pope_floor"):
        pope = PoPEEmbedding(dim=cfg.pope_d_rope, max_seq_len=cfg.max_seq_len, theta=cfg.pope_theta,
                             training_length=cfg.pope_training_length, use_floor=(mode == "pope_floor"),
                             delta_init=cfg.pope_delta_init)
    elif mode not in ("alibi", "nope"):
        raise ValueError(f"Unknown pe_mode: {mode}")
    return rope, fpope, pope


class TransformerBlock(nn.Module):
    """Pre-RMSNorm block: x + attn(norm(x)); x + ffn(norm(x))."""

    def __init__(self, cfg: TransformerConfig, rope=None, fpope=None, pope=None):
        super().__init__()
        self.attention_norm = RMSNorm(cfg.hidden_dim, eps=cfg.norm_eps)
        common = dict(hidden_dim=cfg.hidden_dim, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads,
                      head_dim=cfg.head_dim, use_qk_norm=cfg.use_qk_norm)
        if cfg.pe_mode == "fpope":
            self.attention = FPoPEGroupedQueryAttention(d_rope=cfg.fpope_d_rope, fpope=fpope, **common)
        elif cfg.pe_mode in ("pope", "pope_floor"):
            self.attention = FPoPEGroupedQueryAttention(d_rope=cfg.pope_d_rope, fpope=pope, **common)
        elif cfg.pe_mode == "alibi":
            self.attention = ALiBiAttention(**common)
        else:
            self.attention = GroupedQueryAttention(rope=rope if cfg.pe_mode == "rope" else None, **common)
        self.ffn_norm = RMSNorm(cfg.hidden_dim, eps=cfg.norm_eps)
        self.feed_forward = FeedForward(cfg.hidden_dim, cfg.resolved_ffn_dim())

    def forward(self, x: torch.Tensor, mask=None, start_pos: int = 0) -> torch.Tensor:
        # each block hands its residual stream to the output projection, which adds it (in the
        # GEMM's epilogue for bf16 inference, as a separate add otherwise)
        x = self.attention(self.attention_norm(x), mask, start_pos, residual=x)
        return self.feed_forward(self.ffn_norm(x), residual=x)


class Transformer(nn.Module):
    def __init__(self, config: TransformerConfig):
        super().__init__()
        self.config = config
        self.token_embedding = TokenEmbedding(config.vocab_size, config.hidden_dim)
        self.rope, self.fpope, self.pope = _build_pe(config)
        self.layers = nn.ModuleList(
            [TransformerBlock(config, rope=self.rope, fpope=self.fpope, pope=self.pope)
             for _ in range(config.num_layers)])
        self.norm = RMSNorm(config.hidden_dim, eps=config.norm_eps)
        self.output = nn.Linear(config.hidden_dim, config.vocab_size, bias=False)
        if config.tie_embeddings:
            self.output.weight = self.token_embedding.weight
        self.gradient_checkpointing = config.gradient_checkpointing
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=0.02)

    def hidden_states(self, input_ids: torch.Tensor, start_pos: int = 0) -> torch.Tensor:
        x = self.token_embedding(input_ids)
        for layer in self.layers:
            x = layer(x, mask=None, start_pos=start_pos)
        return self.norm(x)

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None, start_pos: int = 0) -> dict:
        logits = self.output(self.hidden_states(input_ids, start_pos))
        out = {"logits": logits}
        if labels is not None:
            out["loss"] = F.cross_entropy(logits[..., :-1, :].reshape(-1, self.config.vocab_size).float(),
                                          labels[..., 1:].reshape(-1), ignore_index=-100)
        return out

    @torch.no_grad()
    def loss_sums(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None, start_pos: int = 0,
                  chunk_tokens: int = 8192) -> tuple[torch.Tensor, torch.Tensor]:
        """(sum of next-token NLLs, number of scored tokens) for a batch, both fp64 scalars on device.

        bf16 inference with bf16 weights: one tensor-core kernel computes the head's logits tile by
        tile and reduces them to the loss in its epilogue (``ops.lm_head_ce_loss_sums``).  Otherwise
        the head and the cross-entropy kernel run over ``chunk_tokens`` positions at a time, so the
        [tokens, vocab] logits never exist in full (1 GB per 16k sequence at the 1B shape).
        mean loss = nll_sum / count, perplexity = exp of it.
        """
        from .ops import ce_loss_sums, lm_head_ce_loss_sums

        labels = input_ids if labels is None else labels
        h = self.hidden_states(input_ids, start_pos)[:, :-1].reshape(-1, self.config.hidden_dim)
        tgt = labels[:, 1:].reshape(-1)
        sums = torch.zeros(2, dtype=torch.float64, device=h.device)
        from .ops import fused_gemm_ok

        if fused_gemm_ok(h, self.output.weight):
            # head GEMM with the cross-entropy in its epilogue: no logits at all
            for i in range(0, h.shape[0], 65536):
                lm_head_ce_loss_sums(h[i:i + 65536], self.output.weight, tgt[i:i + 65536], out=sums)
            return sums[0], sums[1]
        for i in range(0, h.shape[0], chunk_tokens):
            # logits stay in the head's output dtype (bf16 under autocast); the loss kernel
            # reads them once and accumulates in fp32 / fp64
            ce_loss_sums(self.output(h[i:i + chunk_tokens]), tgt[i:i + chunk_tokens], out=sums)
        return sums[0], sums[1]

    def extend_context_length(self, new_max_seq_len: int) -> None:
        for pe in (self.rope, self.fpope, self.pope):
            if pe is not None:
                pe.extend_seq_len(new_max_seq_len)
        self.config.max_seq_len = new_max_seq_len
