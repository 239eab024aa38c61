"""CPU timing leg of the benchmark.  TEST / MEASUREMENT INFRASTRUCTURE ONLY.

Times the reference's eager data flow for the PoPE-family attention core on the host:
fp32 positional transform (softplus, position x frequency phases, clamped key phase bias,
cos/sin expansion, concat with the content half), operands cast to bf16, GQA repeat, then
``F.scaled_dot_product_attention(is_causal=True)`` -- the composition of
src/model/fpope_attention.py:145-177 (paths inside the reference project), restated by
``oracle.pe_attention_oracle``.  When ``oracle/_ref`` holds the reference's own modules (put
there by ``oracle/make_ref.py``), the transform is the reference's real
``FoPEPoPEEmbedding.forward_query`` / ``forward_key`` instead of the restatement
(``kind = "reference"``; ``"port"`` otherwise).  Only ``bench.py`` (its cpu_baseline leg and
its ``--impl reference`` arm) calls this; it is never part of the GPU path.
"""

from __future__ import annotations

import os
import time

import torch
import torch.nn.functional as F

from . import pe_attention_oracle as O


_REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_ref_cache: dict = {}


def reference_modules():
    """The reference's ``src.model.fpope`` module imported from ``oracle/_ref``, or None."""
    if "fpope" not in _ref_cache:
        mod = None
        if os.path.exists(os.path.join(_REF_DIR, "src", "model", "fpope.py")):
            import importlib
            import sys

            sys.path.insert(0, _REF_DIR)
            try:
                mod = importlib.import_module("src.model.fpope")
            except Exception:
                mod = None
            finally:
                sys.path.remove(_REF_DIR)
        _ref_cache["fpope"] = mod
    return _ref_cache["fpope"]


def reference_attention_cpu(emb, q, k, v, q_r, k_r, dtype=torch.bfloat16):
    """src/model/fpope_attention.py:145-177 on CPU with the reference's own embedding module ``emb``:
    forward_query / forward_key on fp32 position halves (what the module sees under autocast
    with its fp32 RMSNorm in front), concat with the content halves, GQA repeat, operands cast to
    ``dtype`` as autocast does for SDPA."""
    qr = emb.forward_query(q_r.float(), 0).transpose(1, 2)
    kr = emb.forward_key(k_r.float(), 0).transpose(1, 2)
    vv = v.transpose(1, 2).to(dtype)
    kc = k.transpose(1, 2)
    g = q.shape[2] // k.shape[2]
    if g > 1:
        kc, kr, vv = (t.repeat_interleave(g, dim=1) for t in (kc, kr, vv))
    qq = torch.cat([q.transpose(1, 2), qr], dim=-1).to(dtype)
    kk = torch.cat([kc, kr], dim=-1).to(dtype)
    out = F.scaled_dot_product_attention(qq, kk, vv, attn_mask=None, dropout_p=0.0, is_causal=True,
                                         scale=qq.shape[-1] ** -0.5)
    return out.transpose(1, 2)


def pope_attention_cpu(q, k, v, q_r, k_r, freqs, delta, dtype=torch.bfloat16):
    """Eager-style forward on CPU tensors in [B, S, H, d] layout; returns [B, S, H, d_v]."""
    qr = O.pope_expand(q_r.float(), 0, freqs, None)
    kr = O.pope_expand(k_r.float(), 0, freqs, delta)
    qq = torch.cat([q.float(), qr], dim=-1).transpose(1, 2).to(dtype)
    kk = torch.cat([k.float(), kr], dim=-1).transpose(1, 2).to(dtype)
    vv = v.transpose(1, 2).to(dtype)
    g = qq.shape[1] // kk.shape[1]
    if g > 1:
        kk = kk.repeat_interleave(g, dim=1)
        vv = vv.repeat_interleave(g, dim=1)
    out = F.scaled_dot_product_attention(qq, kk, vv, is_causal=True, scale=qq.shape[-1] ** -0.5)
    return out.transpose(1, 2)


def time_cfg4_sample(seq_len: int, heads: int, batch: int = 1, d_c: int = 128, d_r: int = 64, d_v: int = 128,
                     repeats: int = 1, seed: int = 0) -> dict:
    """Time ``repeats`` passes over a [batch, seq_len, heads] slice of the configuration-4 workload.

    Returns seconds per pass, the algorithmic FLOPs of the slice (B H S^2 (d_qk + d_v)) and the
    thread count used.
    """
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    mk = lambda d: torch.randn(batch, seq_len, heads, d, generator=g).to(torch.bfloat16)
    q, k, q_r, k_r, v = mk(d_c), mk(d_c), mk(d_r), mk(d_r), mk(d_v)
    freqs = O.pope_base_freqs(d_r)
    delta = (torch.rand(d_r, generator=g) * 2 - 1) * torch.pi
    ref = reference_modules()
    emb = None
    if ref is not None:
        torch.manual_seed(seed)
        emb = ref.FoPEPoPEEmbedding(dim=d_r, max_seq_len=seq_len, num_fourier_terms=16, fourier_sigma=0.3,
                                    training_length=seq_len, delta_init="zero")
        with torch.no_grad():
            emb.phase_bias.copy_(delta)
    with torch.no_grad():
        best = float("inf")
        total = 0.0
        for _ in range(repeats):
            t0 = time.perf_counter()
            if emb is not None:
                reference_attention_cpu(emb, q, k, v, q_r, k_r)
            else:
                pope_attention_cpu(q, k, v, q_r, k_r, freqs, delta)
            dt = time.perf_counter() - t0
            total += dt
            best = min(best, dt)
    flops = float(batch) * heads * seq_len * seq_len * (d_c + 2 * d_r + d_v)
    return {"seconds": total / repeats, "best_seconds": best, "flops": flops, "threads": threads,
            "kind": "reference" if emb is not None else "port"}
