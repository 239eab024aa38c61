"""Generate tests/golden/module_grads.npz from the reference: gradients of its attention
modules under bf16 autocast.

For every case of oracle.golden_cases.TRAIN_CASES the reference module is built with seeded
parameters, run forward and backward under ``torch.autocast("cpu", dtype=torch.bfloat16)``
(the precision of its training loop, src/training/trainer.py) with a seeded upstream gradient,
and the output, the input gradient and every parameter gradient are stored.  The same run in
fp32 is stored beside it: the distance between the two is the noise floor of bf16 training,
which the parity test uses to scale its tolerance, and the fp32 output and gradients themselves
(``y_fp32``, ``grad_fp32/...``) pin the fp32 backward of the drop-in modules.

Run from the repository root:  python tests/golden/make_golden_grad.py --reference <checkout>
"""

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import golden_cases as G  # noqa: E402
from tests.golden.make_golden import build_module  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    from src.model.alibi import ALiBiAttention
    from src.model.attention import GroupedQueryAttention
    from src.model.fpope import FoPEPoPEEmbedding
    from src.model.fpope_attention import FPoPEGroupedQueryAttention
    from src.model.pope import PoPEEmbedding
    from src.model.rope import NTKAwareRotaryEmbedding, RotaryEmbedding, YaRNRotaryEmbedding

    R = dict(ALiBiAttention=ALiBiAttention, GroupedQueryAttention=GroupedQueryAttention,
             FoPEPoPEEmbedding=FoPEPoPEEmbedding, FPoPEGroupedQueryAttention=FPoPEGroupedQueryAttention,
             PoPEEmbedding=PoPEEmbedding, NTKAwareRotaryEmbedding=NTKAwareRotaryEmbedding,
             RotaryEmbedding=RotaryEmbedding, YaRNRotaryEmbedding=YaRNRotaryEmbedding)
    data = {"torch_version": np.array(torch.__version__)}
    for i, spec in enumerate(G.TRAIN_CASES):
        grads = {}
        for mode in ("bf16", "fp32"):
            torch.manual_seed(7000 + i)
            m = build_module(spec, R).train()
            G.fill_parameters(m, 8000 + i)
            g = torch.Generator().manual_seed(9000 + i)
            x = torch.randn(spec["B"], spec["S"], spec["hidden"], generator=g).requires_grad_(True)
            dy = torch.randn(spec["B"], spec["S"], spec["hidden"], generator=g)
            if mode == "bf16":
                with torch.autocast("cpu", dtype=torch.bfloat16):
                    y = m(x)
            else:
                y = m(x)
            y.float().backward(dy)
            grads[mode] = {"x": x.grad.clone()}
            grads[mode].update({n: p.grad.float().clone() for n, p in m.named_parameters() if p.grad is not None})
            data[f"{spec['name']}/y" + ("" if mode == "bf16" else "_fp32")] = y.detach().float().numpy()
        names = sorted(grads["bf16"])
        data[f"{spec['name']}/grad_names"] = np.array(names)
        worst = 0.0
        for n in names:
            gb, gf = grads["bf16"][n], grads["fp32"][n]
            keep = gb[::G.TRAIN_ROW_STRIDE] if gb.dim() == 2 else gb
            data[f"{spec['name']}/grad/{n}"] = keep.numpy()
            data[f"{spec['name']}/grad_fp32/{n}"] = (gf[::G.TRAIN_ROW_STRIDE] if gf.dim() == 2 else gf).numpy()
            # how far bf16 training itself sits from fp32: the scale for the parity tolerance
            data[f"{spec['name']}/bf16_noise/{n}"] = np.array(float((gb - gf).abs().max()))
            data[f"{spec['name']}/fp32_max/{n}"] = np.array(float(gf.abs().max()))
            worst = max(worst, float((gb - gf).abs().max() / (gf.abs().max() + 1e-12)))
        print(spec["name"], "tensors with grad:", len(names),
              "worst bf16-vs-fp32 relative gradient distance: %.3e" % worst)
    from src.model.transformer import Transformer, TransformerConfig

    for i, spec in enumerate(G.TRAIN_MODEL_CASES):
        kw = dict(G.TRAIN_MODEL_BASE)
        kw.update({k: v for k, v in spec.items() if k != "name"})
        grads, loss = {}, {}
        for mode in ("bf16", "fp32"):
            torch.manual_seed(7500 + i)
            model = Transformer(TransformerConfig(**kw)).train()
            G.fill_parameters(model, 8500 + i)
            ids = torch.randint(0, kw["vocab_size"], (G.TRAIN_MODEL_BATCH, G.TRAIN_MODEL_SEQ),
                                generator=torch.Generator().manual_seed(9500 + i))
            if mode == "bf16":
                with torch.autocast("cpu", dtype=torch.bfloat16):
                    out = model(ids, labels=ids)
            else:
                out = model(ids, labels=ids)
            out["loss"].backward()
            loss[mode] = float(out["loss"])
            grads[mode] = {n: p.grad.float().clone() for n, p in model.named_parameters() if p.grad is not None}
        name = spec["name"]
        data[f"{name}/loss"] = np.array(loss["bf16"])
        data[f"{name}/loss_fp32"] = np.array(loss["fp32"])
        names = sorted(grads["bf16"])
        data[f"{name}/grad_names"] = np.array(names)
        for n in names:
            gb, gf = grads["bf16"][n], grads["fp32"][n]
            # per tensor: its largest entry, its l2 norm, and a strided sample of its entries
            data[f"{name}/grad_norm/{n}"] = np.array(float(gb.norm()))
            data[f"{name}/grad_sample/{n}"] = gb.flatten()[::G.TRAIN_MODEL_SAMPLE_STRIDE].numpy()
            data[f"{name}/bf16_noise/{n}"] = np.array(float((gb - gf).abs().max()))
            data[f"{name}/fp32_max/{n}"] = np.array(float(gf.abs().max()))
        print(name, "loss bf16 %.6f fp32 %.6f" % (loss["bf16"], loss["fp32"]), "tensors:", len(names))
    np.savez_compressed(os.path.join(HERE, "module_grads.npz"), **data)
    print("wrote module_grads.npz", os.path.getsize(os.path.join(HERE, "module_grads.npz")), "bytes")


if __name__ == "__main__":
    main()
