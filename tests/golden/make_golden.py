"""Generate the golden fixtures by running the reference's own live modules.

Usage (only where the reference checkout is available):

    python tests/golden/make_golden.py --reference /path/to/pe_ablations

Writes ``core.npz``, ``modules.npz`` and ``models.npz`` next to this file.  The
inputs come from ``oracle.inputs`` / ``oracle.golden_cases`` (seeded), so the
fixtures hold only what the reference produced: attention outputs, and the
positional-encoding constants its modules derive (frequencies, tables, slopes).
The tests read the fixtures and never import the reference.
"""

from __future__ import annotations

import argparse
import math
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import golden_cases as G  # noqa: E402
from oracle.inputs import make_inputs  # noqa: E402


def ref_core(case, inp, R):
    """Compose the reference's functions exactly as its attention classes do."""
    dt = case.dtype
    rnd = lambda t: None if t is None else t.to(dt)
    B, S, H, Hkv = case.B, case.S, case.H, case.Hkv
    g = H // Hkv
    consts = {}
    v = rnd(inp["v"]).transpose(1, 2)
    if case.variant == "pope":
        if case.pope_kind == "fpope":
            emb = R["FoPEPoPEEmbedding"](dim=case.d_r, max_seq_len=case.pos0 + S, theta=case.pope_theta,
                                         num_fourier_terms=case.n_fourier, fourier_sigma=case.fourier_sigma,
                                         training_length=case.training_length, delta_init="zero")
            with torch.no_grad():
                emb.fourier_coeffs.copy_(inp["fourier_coeffs"])
            consts["freqs"] = emb._compute_effective_freqs().detach()
            consts["base_freqs"] = emb.base_freqs.clone()
        else:
            emb = R["PoPEEmbedding"](dim=case.d_r, max_seq_len=case.pos0 + S, theta=case.pope_theta,
                                     training_length=case.training_length,
                                     use_floor=(case.pope_kind == "pope_floor"), delta_init="zero")
            consts["freqs"] = emb.effective_freqs.clone()
            consts["base_freqs"] = emb.freqs.clone()
        with torch.no_grad():
            emb.phase_bias.copy_(inp["delta"])
            # fp32 transform on (possibly bf16-rounded) inputs: the data flow under autocast
            q_r = emb.forward_query(rnd(inp["q_r"]).float(), case.pos0).transpose(1, 2)
            k_r = emb.forward_key(rnd(inp["k_r"]).float(), case.pos0).transpose(1, 2)
            if case.d_c > 0:
                q = torch.cat([rnd(inp["q"]).float().transpose(1, 2), q_r], dim=-1)
                k = torch.cat([rnd(inp["k"]).float().transpose(1, 2), k_r], dim=-1)
            else:
                q, k = q_r, k_r
            scale = (case.d_c + 2 * case.d_r) ** -0.5
            if g > 1:
                k = k.repeat_interleave(g, dim=1)
                v = v.repeat_interleave(g, dim=1)
            out = F.scaled_dot_product_attention(q.to(dt), k.to(dt), v, attn_mask=None, dropout_p=0.0,
                                                 is_causal=True, scale=scale)
    else:
        q, k = rnd(inp["q"]), rnd(inp["k"])
        D = case.d_c
        if case.variant == "rotary":
            n = case.pos0 + S
            if case.rope_kind == "standard":
                rope = R["RotaryEmbedding"](D, n, case.rope_theta)
            elif case.rope_kind == "ntk":
                rope = R["NTKAwareRotaryEmbedding"](D, n, case.rope_theta, case.rope_scale)
            elif case.rope_kind == "yarn":
                rope = R["YaRNRotaryEmbedding"](D, n, case.rope_theta, case.rope_scale)
                consts["mscale"] = rope.mscale.clone().reshape(1)
            if case.rope_kind == "fope":
                emb = R["FoPEPoPEEmbedding"](dim=D // 2, max_seq_len=n, theta=case.rope_theta,
                                             num_fourier_terms=case.n_fourier, fourier_sigma=case.fourier_sigma,
                                             training_length=case.training_length)
                with torch.no_grad():
                    emb.fourier_coeffs.copy_(inp["fourier_coeffs"])
                eff = emb._compute_effective_freqs().detach()
                consts["inv_freq"] = eff
                ang = torch.outer(torch.arange(n).float(), eff)
                cis = torch.polar(torch.ones_like(ang), ang)
                consts["table"] = torch.view_as_real(cis)[case.pos0:].clone()
                q, k = R["apply_rotary_emb"](q, k, cis[case.pos0:case.pos0 + S])
            else:
                consts["table"] = torch.view_as_real(rope.freqs_cis)[case.pos0:].clone()
                q, k = rope(q, k, case.pos0)
        q, k = q.transpose(1, 2), k.transpose(1, 2)
        if case.qk_norm:
            q, k = R["QKNorm"](D)(q, k)
        if g > 1:
            k = k.repeat_interleave(g, dim=1)
            v = v.repeat_interleave(g, dim=1)
        if case.variant == "alibi":
            slopes = R["get_alibi_slopes"](H)
            consts["slopes"] = slopes.clone()
            scores = torch.matmul(q, k.transpose(-2, -1)) * (D ** -0.5)
            pos = torch.arange(S)
            rel = pos.unsqueeze(0) - pos.unsqueeze(1)
            scores = scores + (-slopes.view(1, H, 1, 1) * rel.abs().float()).to(scores.dtype)
            mask = torch.triu(torch.ones(S, S, dtype=torch.bool), diagonal=1)
            scores = scores.masked_fill(mask, float("-inf"))
            out = torch.matmul(torch.softmax(scores, dim=-1), v)
        else:
            out = F.scaled_dot_product_attention(q, k, v, attn_mask=None, is_causal=True, scale=1.0 / (D ** 0.5))
    return out.transpose(1, 2).float().contiguous(), consts


def build_module(spec, R):
    kind = spec["kind"]
    hd, H, Hkv, hidden, S = spec["head_dim"], spec["H"], spec["Hkv"], spec["hidden"], spec["S"]
    if kind in ("rope", "yarn", "ntk", "nope"):
        rope = None
        if kind == "rope":
            rope = R["RotaryEmbedding"](hd, S, 10000.0)
        elif kind == "ntk":
            rope = R["NTKAwareRotaryEmbedding"](hd, S, 10000.0, spec["rope_scale"])
        elif kind == "yarn":
            rope = R["YaRNRotaryEmbedding"](hd, S, 10000.0, spec["rope_scale"], original_max_seq_len=512)
        return R["GroupedQueryAttention"](hidden, H, Hkv, hd, spec["use_qk_norm"], rope)
    if kind == "alibi":
        return R["ALiBiAttention"](hidden, H, Hkv, hd, spec["use_qk_norm"])
    if kind == "fpope":
        pe = R["FoPEPoPEEmbedding"](dim=spec["d_rope"], max_seq_len=S, num_fourier_terms=spec["n_fourier"],
                                    fourier_sigma=spec["sigma"], training_length=spec["training_length"],
                                    delta_init=spec["delta_init"])
    else:
        pe = R["PoPEEmbedding"](dim=spec["d_rope"], max_seq_len=S, training_length=spec.get("training_length", 512),
                                use_floor=(kind == "pope_floor"), delta_init=spec["delta_init"])
    return R["FPoPEGroupedQueryAttention"](hidden, H, Hkv, hd, spec["d_rope"], spec["use_qk_norm"], pe)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    from src.model.alibi import ALiBiAttention, get_alibi_slopes
    from src.model.attention import GroupedQueryAttention
    from src.model.fpope import FoPEPoPEEmbedding
    from src.model.fpope_attention import FPoPEGroupedQueryAttention
    from src.model.normalization import QKNorm
    from src.model.pope import PoPEEmbedding
    from src.model.rope import (NTKAwareRotaryEmbedding, RotaryEmbedding, YaRNRotaryEmbedding, apply_rotary_emb)
    from src.model.transformer import Transformer, TransformerConfig

    R = dict(ALiBiAttention=ALiBiAttention, get_alibi_slopes=get_alibi_slopes,
             GroupedQueryAttention=GroupedQueryAttention, FoPEPoPEEmbedding=FoPEPoPEEmbedding,
             FPoPEGroupedQueryAttention=FPoPEGroupedQueryAttention, QKNorm=QKNorm, PoPEEmbedding=PoPEEmbedding,
             NTKAwareRotaryEmbedding=NTKAwareRotaryEmbedding, RotaryEmbedding=RotaryEmbedding,
             YaRNRotaryEmbedding=YaRNRotaryEmbedding, apply_rotary_emb=apply_rotary_emb)

    core = {"torch_version": np.array(torch.__version__)}
    for case in G.CORE_CASES:
        inp = make_inputs(case)
        out, consts = ref_core(case, inp, R)
        if case.dtype == torch.bfloat16:
            # the reference's output is bf16: keep its bit pattern (half the bytes)
            core[f"{case.name}/out_bf16_bits"] = out.to(torch.bfloat16).view(torch.int16).numpy()
        else:
            core[f"{case.name}/out"] = out.numpy()
        for k, t in consts.items():
            if k == "table":
                t = t[::G.TABLE_ROW_STRIDE]
            core[f"{case.name}/{k}"] = t.float().numpy()
        print(case.name, tuple(out.shape), float(out.abs().mean()))
    for case, stride in G.FULL_CASES:
        inp = make_inputs(case)
        out, consts = ref_core(case, inp, R)
        core[f"{case.name}/out_rows"] = out[:, ::stride].contiguous().numpy()
        core[f"{case.name}/row_stride"] = np.array(stride)
        core[f"{case.name}/freqs"] = consts["freqs"].numpy()
        print(case.name, tuple(out.shape), "stride", stride)
    np.savez_compressed(os.path.join(HERE, "core.npz"), **core)

    mods = {}
    for i, spec in enumerate(G.MODULE_CASES):
        torch.manual_seed(1000 + i)
        m = build_module(spec, R).eval()
        G.fill_parameters(m, 2000 + i)
        g = torch.Generator().manual_seed(3000 + i)
        x = torch.randn(spec["B"], spec["S"], spec["hidden"], generator=g)
        with torch.no_grad():
            y = m(x)
        mods[f"{spec['name']}/y"] = y.numpy()
        # buffers the drop-in must reproduce (names as in the reference's state_dict)
        for bname, buf in m.named_buffers():
            if bname.endswith(("freqs", "effective_freqs", "base_freqs", "alibi_slopes", "mscale")):
                mods[f"{spec['name']}/buf/{bname}"] = buf.float().numpy()
        mods[f"{spec['name']}/state_keys"] = np.array(sorted(m.state_dict().keys()))
        print(spec["name"], tuple(y.shape), float(y.abs().mean()))
    # cached decoding (src/model/fpope_attention.py:184-327)
    from src.model.fpope_attention import FPoPEGroupedQueryAttentionWithCache
    cc = G.CACHE_CASE
    torch.manual_seed(1500)
    pe = FoPEPoPEEmbedding(dim=cc["d_rope"], max_seq_len=cc["max_cache_len"], num_fourier_terms=cc["n_fourier"],
                           fourier_sigma=cc["sigma"], training_length=cc["training_length"],
                           delta_init=cc["delta_init"])
    m = FPoPEGroupedQueryAttentionWithCache(cc["hidden"], cc["H"], cc["Hkv"], cc["head_dim"], cc["d_rope"],
                                            cc["use_qk_norm"], pe, max_cache_len=cc["max_cache_len"]).eval()
    G.fill_parameters(m, 2500)
    total = G.CACHE_PREFILL + sum(G.CACHE_STEPS)
    x = torch.randn(cc["B"], total, cc["hidden"], generator=torch.Generator().manual_seed(3500))
    outs, pos = [], 0
    with torch.no_grad():
        for n in (G.CACHE_PREFILL,) + tuple(G.CACHE_STEPS):
            outs.append(m(x[:, pos:pos + n], start_pos=pos, use_cache=True))
            pos += n
    mods[f"{cc['name']}/y"] = torch.cat(outs, dim=1).numpy()
    print(cc["name"], tuple(mods[f"{cc['name']}/y"].shape))
    np.savez_compressed(os.path.join(HERE, "modules.npz"), **mods)

    models = {}
    for i, spec in enumerate(G.MODEL_CASES):
        kw = dict(G.MODEL_BASE)
        kw.update({k: v for k, v in spec.items() if k != "name"})
        torch.manual_seed(4000 + i)
        model = Transformer(TransformerConfig(**kw)).eval()
        G.fill_parameters(model, 5000 + i)
        g = torch.Generator().manual_seed(6000 + i)
        ids = torch.randint(0, kw["vocab_size"], (G.MODEL_BATCH, G.MODEL_SEQ), generator=g)
        with torch.no_grad():
            o = model(ids, labels=ids)
        models[f"{spec['name']}/loss"] = o["loss"].numpy()
        models[f"{spec['name']}/logits_sample"] = o["logits"][:, ::8, ::16].contiguous().numpy()
        models[f"{spec['name']}/state_keys"] = np.array(sorted(model.state_dict().keys()))
        models[f"{spec['name']}/state_shapes"] = np.array(
            [",".join(map(str, model.state_dict()[k].shape)) for k in sorted(model.state_dict().keys())])
        print(spec["name"], float(o["loss"]))
    np.savez_compressed(os.path.join(HERE, "models.npz"), **models)


if __name__ == "__main__":
    main()
