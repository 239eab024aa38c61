"""GPU: more keys than queries (cached decoding) -- kernels against the oracle, module against the reference."""

import os

import numpy as np
import pytest
import torch

from oracle import golden_cases as G
from oracle import pe_attention_oracle as O

pytestmark = pytest.mark.gpu

BF16, FP32 = torch.bfloat16, torch.float32


def _run(variant, dtype, B, H, Hkv, Sq, Sk, d_c, d_r, d_v, seed, qk_norm=False, single_cta=False):
    from pe_ablations_b200 import check_device_status, pe_attention

    g = torch.Generator().manual_seed(seed)
    mk = lambda S, h, d: torch.randn(B, S, h, d, generator=g)
    q = mk(Sq, H, d_c) if d_c else None
    k = mk(Sk, Hkv, d_c) if d_c else None
    v = mk(Sk, Hkv, d_v)
    start = Sk - Sq
    kw_o, kw_g = {}, {}
    if variant == "pope":
        q_r, k_r = mk(Sq, H, d_r), mk(Sk, Hkv, d_r)
        freqs = O.pope_base_freqs(d_r)
        delta = (torch.rand(d_r, generator=g) * 2 - 1) * torch.pi
        kw_o = dict(q_r=q_r, k_r=k_r, freqs=freqs, delta=delta)
        kw_g = dict(freqs=freqs, delta=delta)
    elif variant == "rotary":
        table = O.rotary_table(O.rope_inv_freq(d_c), Sk)
        kw_o = dict(table=table, table_pos0=0)
        kw_g = dict(rotary_table=table, table_pos0=0)
    elif variant == "alibi":
        sl = O.alibi_slopes(H)
        kw_o = dict(slopes=sl)
        kw_g = dict(alibi_slopes=sl)
    want = O.attention_core(variant, q, k, v, dtype=dtype, pos0=start, k_pos0=0, qk_norm=qk_norm, **kw_o).float()
    dev = torch.device("cuda", 0)
    c = lambda t: None if t is None else t.to(dev, dtype)
    if variant == "pope":
        kw_g.update(q_r=c(kw_o["q_r"]), k_r=c(kw_o["k_r"]))
    got = pe_attention(variant, c(q), c(k), c(v), start_pos=start, k_start_pos=0, qk_norm=qk_norm,
                       single_cta=single_cta, **kw_g)
    torch.cuda.synchronize()
    check_device_status()
    return (got.float().cpu() - want).abs().max().item()


@pytest.mark.parametrize("args", [
    ("pope", FP32, 1, 4, 2, 1, 77, 32, 16, 32),
    ("pope", FP32, 2, 2, 2, 5, 130, 64, 32, 64),
    ("rotary", FP32, 1, 2, 1, 3, 100, 64, 0, 64),
    ("alibi", FP32, 1, 4, 4, 2, 65, 32, 0, 32),
], ids=lambda a: f"{a[0]}_fp32_q{a[5]}_k{a[6]}")
def test_decode_shapes_fp32(args):
    assert _run(*args, seed=101) <= 1e-4


@pytest.mark.parametrize("args", [
    ("pope", BF16, 1, 4, 2, 1, 700, 128, 64, 128),      # one new token
    ("pope", BF16, 2, 2, 2, 64, 200, 64, 32, 64),
    ("pope", BF16, 1, 2, 2, 300, 900, 128, 64, 128),     # chunked prefill, CTA-pair kernel
    ("pope", BF16, 1, 2, 1, 513, 1030, 128, 32, 128),
    ("rotary", BF16, 1, 4, 4, 1, 333, 128, 0, 128),
    ("rotary", BF16, 1, 2, 2, 400, 777, 128, 0, 128),
    ("nope", BF16, 1, 4, 2, 17, 257, 64, 0, 64),
    ("alibi", BF16, 1, 4, 4, 260, 600, 128, 0, 128),
], ids=lambda a: f"{a[0]}_bf16_q{a[5]}_k{a[6]}")
def test_decode_shapes_bf16(args):
    assert _run(*args, seed=102) <= 2e-2
    if args[9] == 128 and args[5] > 256:
        assert _run(*args, seed=102, single_cta=True) <= 2e-2


def test_cached_decoding_module_matches_reference(golden_dir):
    from pe_ablations_b200 import modules as M
    from pe_ablations_b200 import pe as P

    mods = np.load(os.path.join(golden_dir, "modules.npz"))
    cc = G.CACHE_CASE
    if f"{cc['name']}/y" not in mods.files:
        pytest.skip("fixture without the cached-decoding case")
    torch.manual_seed(1500)
    pe = P.FoPEPoPEEmbedding(dim=cc["d_rope"], max_seq_len=cc["max_cache_len"], num_fourier_terms=cc["n_fourier"],
                             fourier_sigma=cc["sigma"], training_length=cc["training_length"],
                             delta_init=cc["delta_init"])
    m = M.FPoPEGroupedQueryAttentionWithCache(cc["hidden"], cc["H"], cc["Hkv"], cc["head_dim"], cc["d_rope"],
                                              cc["use_qk_norm"], pe, max_cache_len=cc["max_cache_len"]).eval()
    G.fill_parameters(m, 2500)
    m = m.cuda()
    total = G.CACHE_PREFILL + sum(G.CACHE_STEPS)
    x = torch.randn(cc["B"], total, cc["hidden"], generator=torch.Generator().manual_seed(3500)).cuda()
    outs, pos = [], 0
    with torch.no_grad():
        for n in (G.CACHE_PREFILL,) + tuple(G.CACHE_STEPS):
            outs.append(m(x[:, pos:pos + n], start_pos=pos, use_cache=True))
            pos += n
        full = m(x)                      # the uncached forward over the same tokens
    got = torch.cat(outs, dim=1).float().cpu()
    want = torch.from_numpy(mods[f"{cc['name']}/y"])
    assert (got - want).abs().max().item() <= 1e-4
    assert (full.float().cpu() - want).abs().max().item() <= 1e-4
    m.reset_cache()
    assert m.cache_len == 0 and m.k_cache is None
