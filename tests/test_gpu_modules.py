"""GPU: the drop-in attention modules and the Transformer host against the reference's outputs.

Weights come from ``fill_parameters`` (same seeds as the fixture generator), inputs from the
same seeded generators; the expected outputs were produced by the reference's own modules.
"""

import os

import numpy as np
import pytest
import torch

from oracle import golden_cases as G

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods(golden_dir):
    return np.load(os.path.join(golden_dir, "modules.npz"))


@pytest.fixture(scope="module")
def models(golden_dir):
    return np.load(os.path.join(golden_dir, "models.npz"))


@pytest.mark.parametrize("i,spec", list(enumerate(G.MODULE_CASES)), ids=lambda s: s["name"] if isinstance(s, dict) else str(s))
def test_attention_module_matches_reference_module(mods, i, spec):
    from tests.test_modules_cpu import build_module

    torch.manual_seed(1000 + i)
    m = build_module(spec).eval()
    G.fill_parameters(m, 2000 + i)
    m = m.cuda()
    g = torch.Generator().manual_seed(3000 + i)
    x = torch.randn(spec["B"], spec["S"], spec["hidden"], generator=g).cuda()
    with torch.no_grad():
        y = m(x)
    want = torch.from_numpy(mods[f"{spec['name']}/y"])
    assert (y.float().cpu() - want).abs().max().item() <= 1e-4


@pytest.mark.parametrize("i,spec", list(enumerate(G.MODEL_CASES)), ids=lambda s: s["name"] if isinstance(s, dict) else str(s))
def test_tiny_transformer_matches_reference(models, i, spec):
    from tests.test_modules_cpu import build_model

    torch.manual_seed(4000 + i)
    model = build_model(spec)
    G.fill_parameters(model, 5000 + i)
    model = model.cuda()
    g = torch.Generator().manual_seed(6000 + i)
    ids = torch.randint(0, G.MODEL_BASE["vocab_size"], (G.MODEL_BATCH, G.MODEL_SEQ), generator=g).cuda()
    with torch.no_grad():
        out = model(ids, labels=ids)
        nll, cnt = model.loss_sums(ids)
    want_loss = float(models[f"{spec['name']}/loss"])
    assert abs(out["loss"].item() - want_loss) <= 1e-4 * want_loss
    sample = out["logits"][:, ::8, ::16].float().cpu()
    assert (sample - torch.from_numpy(models[f"{spec['name']}/logits_sample"])).abs().max().item() <= 2e-4
    # the chunked evaluation path gives the same mean loss
    assert abs((nll / cnt).item() - want_loss) <= 1e-4 * want_loss
    assert int(cnt.item()) == G.MODEL_BATCH * (G.MODEL_SEQ - 1)


def test_bf16_autocast_model_close_to_fp32():
    """1B-shape building block at reduced width: bf16 autocast vs fp32 on the same weights."""
    from pe_ablations_b200.model import Transformer, TransformerConfig

    cfg = TransformerConfig(vocab_size=1024, hidden_dim=256, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=128,
                            ffn_dim=512, max_seq_len=1024, pe_mode="fpope", fpope_d_rope=64,
                            fpope_num_fourier_terms=16, fpope_sigma=0.3, fpope_training_length=1024,
                            fpope_delta_init="uniform")
    torch.manual_seed(0)
    model = Transformer(cfg).eval()
    G.fill_parameters(model, 77)
    model = model.cuda()
    ids = torch.randint(0, 1024, (2, 1024), generator=torch.Generator().manual_seed(1)).cuda()
    with torch.no_grad():
        a, c = model.loss_sums(ids)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            b, _ = model.loss_sums(ids)
    la, lb = (a / c).item(), (b / c).item()
    # a sanity bound: the bf16 linears around the kernel contribute most of this difference
    assert abs(la - lb) <= 5e-3, (la, lb)


@pytest.mark.parametrize("dtype,n,vocab", [(torch.float32, 300, 1000), (torch.bfloat16, 700, 32000),
                                           (torch.bfloat16, 64, 50257), (torch.float32, 5, 7)])
def test_ce_loss_sums_matches_torch(dtype, n, vocab):
    from pe_ablations_b200 import ce_loss_sums

    g = torch.Generator().manual_seed(n)
    logits = (torch.randn(n, vocab, generator=g) * 3).to(dtype).cuda()
    tgt = torch.randint(0, vocab, (n,), generator=g).cuda()
    tgt[::7] = -100
    out = ce_loss_sums(logits, tgt)
    out = ce_loss_sums(logits, tgt, out=out)          # accumulates
    want = torch.nn.functional.cross_entropy(logits.double(), tgt, ignore_index=-100, reduction="sum").item() * 2
    cnt = int((tgt != -100).sum().item()) * 2
    assert int(out[1].item()) == cnt
    assert abs(out[0].item() - want) <= 2e-6 * abs(want)
    # a strided view (the head's output sliced along vocab) works too
    out2 = ce_loss_sums(logits[:, : vocab - 1], tgt.clamp(max=vocab - 2))
    want2 = torch.nn.functional.cross_entropy(logits[:, : vocab - 1].double(), tgt.clamp(max=vocab - 2),
                                              ignore_index=-100, reduction="sum").item()
    assert abs(out2[0].item() - want2) <= 2e-6 * abs(want2)


def test_ce_loss_sums_non_finite_logits_behave_like_torch():
    """NaN logits give a NaN sum (the row is not dropped), -inf logits count as probability
    zero, an out-of-range target makes the sum NaN."""
    from pe_ablations_b200 import ce_loss_sums

    g = torch.Generator().manual_seed(5)
    n, vocab = 40, 4099
    logits = (torch.randn(n, vocab, generator=g) * 3).cuda()
    tgt = torch.randint(8, vocab, (n,), generator=g).cuda()
    masked = logits.clone()
    masked[:, :8] = float("-inf")               # a whole 16-byte vector of -inf at the start of every row
    masked[3, 100:2000] = float("-inf")
    for dtype in (torch.float32, torch.bfloat16):
        x = masked.to(dtype)
        want = torch.nn.functional.cross_entropy(x.double(), tgt, reduction="sum").item()
        out = ce_loss_sums(x, tgt)
        assert int(out[1].item()) == n
        assert abs(out[0].item() - want) <= 2e-6 * abs(want)
    bad = logits.clone()
    bad[7, 11] = float("nan")
    out = ce_loss_sums(bad, tgt)
    assert torch.isnan(out[0]).item() and int(out[1].item()) == n
    tgt2 = tgt.clone()
    tgt2[5] = vocab                             # outside the vocabulary and not ignore_index
    out = ce_loss_sums(logits, tgt2)
    assert torch.isnan(out[0]).item()
    out = ce_loss_sums(logits, tgt)             # the scratch counter is intact afterwards
    want = torch.nn.functional.cross_entropy(logits.double(), tgt, reduction="sum").item()
    assert abs(out[0].item() - want) <= 2e-6 * abs(want)


def test_1b_shape_16k_loss_matches_reference(golden_dir):
    """The 1B-shape FoPE+PoPE decoder on one 16k sequence against the loss the reference itself
    produced (fp32, CPU, eager) on the same weights and ids.

    fp32 fused path: same loss to fp32 noise.  bf16 fused path (bf16 weights + autocast, the
    benchmark's protocol): perplexity within 0.1 % relative, i.e. |delta loss| <= 1e-3.
    """
    path = os.path.join(golden_dir, "model_1b.npz")
    if not os.path.exists(path):
        pytest.skip("model_1b.npz has not been generated")
    from pe_ablations_b200 import eval as E
    from pe_ablations_b200.model import Transformer, TransformerConfig

    gold = np.load(path)
    want, seq = float(gold["loss"]), int(gold["seq_len"])
    assert G.MODEL_1B == E.MODEL_1B
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = Transformer(TransformerConfig(**G.MODEL_1B)).eval()
    G.fill_parameters(model, G.MODEL_1B_SEED, std=0.02, linear_gain=1.0)
    ids = torch.randint(0, G.MODEL_1B["vocab_size"], (1, seq),
                        generator=torch.Generator().manual_seed(G.MODEL_1B_IDS_SEED)).cuda()
    with torch.no_grad():
        nll, cnt = model.loss_sums(ids)
        h = model.hidden_states(ids)
        sample = model.output(h[0, ::1024])[:, ::4000].float().cpu()
    got32 = (nll / cnt).item()
    assert abs(got32 - want) <= 2e-5 * want, (got32, want)
    # logits of O(1) after 16 fp32 layers and 16k-long softmax sums: summation-order noise grows
    # with the position (5e-6 at the first rows, ~5e-4 at position 15360)
    assert (sample - torch.from_numpy(gold["logits_sample"])).abs().max().item() <= 3e-3
    E.cast_matmul_weights(model)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        nll, cnt = model.loss_sums(ids)
    got16 = (nll / cnt).item()
    assert abs(got16 - want) <= 1e-3, (got16, want)


@pytest.mark.parametrize("dtype,rows,dim", [(torch.float32, 37, 2048), (torch.bfloat16, 1000, 2048),
                                            (torch.bfloat16, 5, 1024), (torch.float32, 3, 64)])
def test_fused_rmsnorm_matches_reference_formula(dtype, rows, dim):
    from pe_ablations_b200.ops import rmsnorm

    g = torch.Generator().manual_seed(rows)
    x = (torch.randn(rows, dim, generator=g) * 2).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(dim, generator=g)).cuda()
    got = rmsnorm(x, w, 1e-6)
    xf = x.float()
    ref = (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + 1e-6)).type_as(x) * w   # normalization.py:22-27
    ref = ref.to(dtype)                                                                   # the next linear's autocast
    assert got.dtype == dtype and got.shape == x.shape
    if dtype == torch.float32:
        assert torch.allclose(got, ref, rtol=2e-6, atol=1e-7)
    else:
        d = (got.float() - ref.float()).abs()
        assert (d > 0).float().mean().item() < 0.02           # a different summation order flips few roundings
        assert (d <= ref.float().abs() * 2 ** -7 + 1e-6).all()  # and never by more than one bf16 ulp
    # a strided view (rows of a wider tensor) is read in place
    wide = torch.zeros(rows, dim + 64, dtype=dtype, device="cuda")
    wide[:, :dim] = x
    assert torch.equal(rmsnorm(wide[:, :dim], w, 1e-6), got)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_swiglu_matches_reference_formula(dtype):
    from pe_ablations_b200.ops import swiglu

    g = torch.Generator().manual_seed(3)
    a = (torch.randn(257, 5632, generator=g) * 3).to(dtype).cuda()
    b = torch.randn(257, 5632, generator=g).to(dtype).cuda()
    got = swiglu(a, b)
    ref = torch.nn.functional.silu(a) * b            # ffn.py:27,68
    if dtype == torch.float32:
        assert torch.allclose(got, ref, rtol=2e-6, atol=1e-7)
    else:
        d = (got.float() - ref.float()).abs()
        assert (d > 0).float().mean().item() < 0.01
        assert (d <= ref.float().abs() * 2 ** -7 + 1e-6).all()


def test_graphed_loss_sums_equal_eager():
    """eval.GraphedLossSums (one CUDA graph per batch shape) gives the eager loss sums."""
    from pe_ablations_b200 import eval as E
    from pe_ablations_b200.model import Transformer, TransformerConfig

    cfg = TransformerConfig(vocab_size=512, hidden_dim=256, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=128,
                            ffn_dim=512, max_seq_len=512, pe_mode="fpope", fpope_d_rope=64,
                            fpope_num_fourier_terms=8, fpope_training_length=512, fpope_delta_init="uniform")
    torch.manual_seed(0)
    model = Transformer(cfg).eval()
    G.fill_parameters(model, 91)
    model = model.cuda()
    ids = torch.randint(0, 512, (3, 512), generator=torch.Generator().manual_seed(2)).cuda()
    with torch.no_grad():
        want = E.evaluate_shard(model, ids)
        graphed = E.GraphedLossSums(model, ids[:1])
        got = E.evaluate_shard(model, ids, graphed=graphed)
    torch.cuda.synchronize()
    assert float(got[1]) == float(want[1]) == 3 * 511
    assert abs(float(got[0]) - float(want[0])) <= 1e-9 * abs(float(want[0]))
