"""Golden loss of the 1B-shape FoPE+PoPE model at 16k context, from the reference itself.

Runs the reference's own ``Transformer`` (fp32, CPU, eager) on ONE seeded sequence of
16384 uniform-random token ids with deterministic weights (``fill_parameters``), and stores
the mean next-token loss in ``model_1b.npz``.  Takes several minutes of CPU time.

    python tests/golden/make_golden_1b.py --reference /path/to/pe_ablations
"""

from __future__ import annotations

import argparse
import os
import sys
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import golden_cases as G  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    ap.add_argument("--seq-len", type=int, default=G.MODEL_1B_SEQ)
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    torch.set_num_threads(os.cpu_count() or 1)
    from src.model.transformer import Transformer, TransformerConfig

    torch.manual_seed(0)
    model = Transformer(TransformerConfig(**G.MODEL_1B)).eval()
    G.fill_parameters(model, G.MODEL_1B_SEED, std=0.02, linear_gain=1.0)
    ids = torch.randint(0, G.MODEL_1B["vocab_size"], (1, args.seq_len),
                        generator=torch.Generator().manual_seed(G.MODEL_1B_IDS_SEED))
    t0 = time.time()
    with torch.no_grad():
        out = model(ids, labels=ids)
    loss = float(out["loss"])
    print("loss", loss, "ppl", float(np.exp(loss)), "seconds", time.time() - t0)
    np.savez(os.path.join(HERE, "model_1b.npz"), loss=np.array(loss), seq_len=np.array(args.seq_len),
             logits_sample=out["logits"][0, ::1024, ::4000].contiguous().numpy())


if __name__ == "__main__":
    main()
