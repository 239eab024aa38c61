"""Generate ``cos_sum.npz``: outputs of the reference's explicit cosine-sum PoPE attention.

Usage (only where the reference checkout is available):

    python tests/golden/make_golden_cos_sum.py --reference /path/to/pe_ablations

For every case of ``oracle.golden_cases.COS_SUM_CASES`` (position-only PoPE attention on
seeded inputs) this runs the reference's own ``FoPEPoPEEmbedding.forward`` (softplus
magnitudes), ``compute_attention_phases`` and ``pope_attention`` (src/model/fpope.py:169-244,
341-418) and stores the output.  That path shares no code with the concatenated
cos/sin form the live modules (and ``core.npz``) use, so it pins the second oracle,
``oracle.pe_attention_oracle.cos_sum_attention``, independently.

Two choices made here, both needed to describe the attention the live modules compute:
``compute_attention_phases`` adds the raw ``phase_bias`` while ``forward_key`` clamps it to
[-2 pi, 0] first, so the clamped vector is what is written into ``phase_bias``; and a plain
PoPE case (no Fourier mix) is a ``FoPEPoPEEmbedding`` with all coefficients zero and a
training length large enough that the floor clip removes nothing.
"""

from __future__ import annotations

import argparse
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import golden_cases as G  # noqa: E402
from oracle.inputs import make_inputs  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from src.model.fpope import FoPEPoPEEmbedding, pope_attention

    store = {"torch_version": np.array(torch.__version__)}
    for case in G.COS_SUM_CASES:
        inp = make_inputs(case)
        S, g = case.S, case.H // case.Hkv
        mixed = case.pope_kind == "fpope"
        emb = FoPEPoPEEmbedding(dim=case.d_r, max_seq_len=case.pos0 + S, theta=case.pope_theta,
                                num_fourier_terms=case.n_fourier, fourier_sigma=case.fourier_sigma,
                                training_length=case.training_length if mixed else 10 ** 12, delta_init="zero")
        with torch.no_grad():
            emb.fourier_coeffs.copy_(inp["fourier_coeffs"] if mixed else torch.zeros_like(emb.fourier_coeffs))
            emb.phase_bias.copy_(inp["delta"].clamp(-2 * math.pi, 0.0))
            mu_q, mu_k, freqs, _, _ = emb(inp["q_r"], inp["k_r"], case.pos0)
            phases = emb.compute_attention_phases(S, S, case.pos0)
            out = pope_attention(mu_q.transpose(1, 2), mu_k.transpose(1, 2).repeat_interleave(g, dim=1),
                                 inp["v"].transpose(1, 2).repeat_interleave(g, dim=1), phases, causal=True)
        store[f"{case.name}/out"] = out.transpose(1, 2).contiguous().numpy()
        store[f"{case.name}/freqs"] = freqs.detach().numpy()
        print(case.name, tuple(out.shape), float(out.abs().mean()))
    np.savez_compressed(os.path.join(HERE, "cos_sum.npz"), **store)


if __name__ == "__main__":
    main()
