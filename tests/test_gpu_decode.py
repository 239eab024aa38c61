"""GPU: more keys than queries (cached decoding) -- kernels against the oracle, module against the reference."""

import os

import numpy as np
import pytest
import torch

from oracle import golden_cases as G
from oracle import pe_attention_oracle as O

pytestmark = pytest.mark.gpu

BF16, FP32 = torch.bfloat16, torch.float32


def _run(variant, dtype, B, H, Hkv, Sq, Sk, d_c, d_r, d_v, seed, qk_norm=False, single_cta=False, split_kv=None,
         fourier=False, with_lse=False):
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
        if fourier:
            coeffs = torch.randn(d_r, 8, generator=g) * 0.3
            kw_o.update(freqs=O.fope_effective_freqs(freqs, coeffs, training_length=4096))
            kw_g.update(fourier_coeffs=coeffs, floor_freq=2 * torch.pi / 4096)
    elif variant == "rotary":
        table = O.rotary_table(O.rope_inv_freq(d_c), Sk)
        kw_o = dict(table=table, table_pos0=0)
        kw_g = dict(rotary_table=table, table_pos0=0)
    elif variant == "alibi":
        sl = O.alibi_slopes(H)
        kw_o = dict(slopes=sl)
        kw_g = dict(alibi_slopes=sl)
    want = O.attention_core(variant, q, k, v, dtype=dtype, pos0=start, k_pos0=0, qk_norm=qk_norm, return_lse=with_lse,
                            **kw_o)
    want, want_lse = (want[0].float(), want[1]) if with_lse else (want.float(), None)
    dev = torch.device("cuda", 0)
    c = lambda t: None if t is None else t.to(dev, dtype)
    if variant == "pope":
        kw_g.update(q_r=c(kw_o["q_r"]), k_r=c(kw_o["k_r"]))
    lse = torch.full((B, H, Sq), float("nan"), device=dev) if with_lse else None
    got = pe_attention(variant, c(q), c(k), c(v), start_pos=start, k_start_pos=0, qk_norm=qk_norm,
                       single_cta=single_cta, split_kv=split_kv, lse=lse, **kw_g)
    torch.cuda.synchronize()
    check_device_status()
    err = (got.float().cpu() - want).abs().max().item()
    if with_lse:
        assert torch.isfinite(lse).all()
        err = max(err, (lse.cpu() - want_lse).abs().max().item())
    return err


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
    assert _run(*args, seed=102, split_kv=False) <= 2e-2
    if args[9] == 128 and args[5] > 256:
        assert _run(*args, seed=102, single_cta=True) <= 2e-2


SPLIT_CASES = [
    # variant, B, H, Hkv, Sq, Sk, d_c, d_r, d_v, qk_norm, fourier
    ("pope", 1, 4, 4, 1, 700, 128, 64, 128, False, False),      # one new token, the 1B attention shape
    ("pope", 2, 8, 2, 1, 1500, 128, 64, 128, False, True),      # 4:1 GQA, FoPE mix in-kernel
    ("pope", 1, 2, 2, 3, 333, 128, 32, 128, False, False),      # three new tokens: per-row causal limit
    ("pope", 2, 4, 2, 2, 257, 64, 32, 64, False, False),
    ("pope", 1, 8, 1, 1, 4100, 0, 32, 64, False, True),         # 8:1 GQA, position half only
    ("pope", 1, 2, 2, 4, 640, 0, 64, 128, False, False),
    ("rotary", 1, 4, 4, 1, 333, 128, 0, 128, False, False),
    ("rotary", 2, 4, 2, 2, 1000, 64, 0, 64, True, False),       # rotation + QKNorm
    ("nope", 1, 4, 2, 1, 129, 64, 0, 64, False, False),
    ("nope", 1, 2, 2, 8, 2048, 128, 0, 128, True, False),       # eight rows, QKNorm alone
    ("alibi", 1, 4, 4, 2, 600, 128, 0, 128, False, False),
    ("alibi", 3, 4, 1, 1, 64, 64, 0, 64, True, False),          # a single tile
    ("nope", 1, 2, 2, 1, 1, 64, 0, 64, False, False),           # first token: one key
]


@pytest.mark.parametrize("case", SPLIT_CASES, ids=lambda a: f"{a[0]}_h{a[2]}k{a[3]}_q{a[4]}_s{a[5]}_d{a[6]}_{a[7]}_{a[8]}")
def test_split_kv_matches_oracle(case):
    """The split-KV kernel (C ABI ``pe_attn_decode``) on every shape family, output and logsumexp."""
    variant, B, H, Hkv, Sq, Sk, d_c, d_r, d_v, qk_norm, fourier = case
    assert _run(variant, BF16, B, H, Hkv, Sq, Sk, d_c, d_r, d_v, seed=103, qk_norm=qk_norm, split_kv=True,
                fourier=fourier, with_lse=True) <= 2e-2


@pytest.mark.parametrize("fourier", [False, True], ids=["pope", "fope_mix"])
def test_split_kv_and_query_tiled_kernels_match_oracle_on_long_cache(fourier):
    """16384 cached keys, one new token at position 16383, 16 heads x batch 2: both kernels
    against the oracle on the same tensors, output and logsumexp."""
    from pe_ablations_b200 import check_device_status, pe_attention

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(104)
    B, H, Sk = 2, 16, 16384
    mk = lambda S, d: torch.randn(B, S, H, d, generator=g).to(BF16)
    q, k, v, q_r, k_r = mk(1, 128), mk(Sk, 128), mk(Sk, 128), mk(1, 64), mk(Sk, 64)
    base = O.pope_base_freqs(64)
    delta = (torch.rand(64, generator=g) * 2 - 1) * torch.pi
    kw, eff = dict(freqs=base), base
    if fourier:
        coeffs = torch.randn(64, 16, generator=g) * 0.3
        eff = O.fope_effective_freqs(base, coeffs, training_length=Sk)
        kw.update(fourier_coeffs=coeffs, floor_freq=2 * torch.pi / Sk)
    f = lambda t: t.float()
    want, want_lse = O.attention_core("pope", f(q), f(k), f(v), dtype=BF16, q_r=f(q_r), k_r=f(k_r), freqs=eff,
                                      delta=delta, pos0=Sk - 1, k_pos0=0, return_lse=True)
    c = lambda t: t.to(dev)
    for split in (True, False):
        lse = torch.full((B, H, 1), float("nan"), device=dev)
        got = pe_attention("pope", c(q), c(k), c(v), q_r=c(q_r), k_r=c(k_r), delta=delta, start_pos=Sk - 1,
                           k_start_pos=0, split_kv=split, lse=lse, **kw)
        torch.cuda.synchronize()
        check_device_status()
        assert (got.float().cpu() - want.float()).abs().max().item() <= 2e-2, f"split_kv={split}"
        assert (lse.cpu() - want_lse).abs().max().item() <= 2e-2, f"split_kv={split} (lse)"


@pytest.mark.parametrize("d,Hkv,qk_norm,Sk", [(64, 4, False, 16384), (64, 2, True, 9000), (128, 4, True, 16384),
                                              (128, 2, False, 4100)])
def test_split_kv_rotary_with_a_geometric_table(d, Hkv, qk_norm, Sk):
    """Rotary decode step with ``table_geometric``: the kernel fetches a key's (cos, sin) entries
    every 16 tiles and advances them by the rotation of one tile in between.  Against the oracle
    (which reads every table row) and against the same call without the flag."""
    from pe_ablations_b200 import check_device_status, pe_attention

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(105)
    B, H = 2, 8
    mk = lambda S, h: torch.randn(B, S, h, d, generator=g).to(BF16)
    q, k, v = mk(1, H), mk(Sk, Hkv), mk(Sk, Hkv)
    table = O.rotary_table(O.rope_inv_freq(d), Sk)
    f = lambda t: t.float()
    want, want_lse = O.attention_core("rotary", f(q), f(k), f(v), dtype=BF16, table=table, table_pos0=0, pos0=Sk - 1,
                                      k_pos0=0, qk_norm=qk_norm, return_lse=True)
    c = lambda t: t.to(dev)
    outs = []
    for geometric in (True, False):
        lse = torch.full((B, H, 1), float("nan"), device=dev)
        got = pe_attention("rotary", c(q), c(k), c(v), rotary_table=table, table_pos0=0, table_geometric=geometric,
                           start_pos=Sk - 1, k_start_pos=0, qk_norm=qk_norm, split_kv=True, lse=lse)
        torch.cuda.synchronize()
        check_device_status()
        assert (got.float().cpu() - want.float()).abs().max().item() <= 2e-2, f"geometric={geometric}"
        assert (lse.cpu() - want_lse).abs().max().item() <= 2e-2, f"geometric={geometric} (lse)"
        outs.append(got.float())
    assert (outs[0] - outs[1]).abs().max().item() <= 8e-3


def test_split_kv_refuses_wide_calls():
    from pe_ablations_b200 import pe_attention
    from pe_ablations_b200._lib import PeAttnError

    dev = torch.device("cuda", 0)
    x = torch.randn(1, 300, 4, 64, device=dev, dtype=BF16)
    with pytest.raises(PeAttnError, match="at most 8 query rows"):
        pe_attention("nope", x[:, :9], x, x, split_kv=True)


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


def test_cache_module_decode_steps_take_the_split_kv_kernel():
    """bf16 cache module: a prefill, then one-token steps (which go to the split-KV kernel once
    256 keys are cached) against the same module's uncached forward over all the tokens."""
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200 import modules as M
    from pe_ablations_b200 import pe as P

    torch.manual_seed(1600)
    hidden, H, Hkv, hd, dr = 256, 4, 2, 64, 32
    pe = P.FoPEPoPEEmbedding(dim=dr, max_seq_len=512, num_fourier_terms=8, fourier_sigma=0.3, training_length=512,
                             delta_init="uniform")
    m = M.FPoPEGroupedQueryAttentionWithCache(hidden, H, Hkv, hd, dr, False, pe, max_cache_len=512).eval()
    G.fill_parameters(m, 2600)
    m = m.cuda()
    x = torch.randn(2, 304, hidden, generator=torch.Generator().manual_seed(3600)).cuda()
    outs, pos = [], 0
    with torch.no_grad(), torch.autocast("cuda", dtype=BF16):
        for n in (300, 1, 1, 2):
            outs.append(m(x[:, pos:pos + n], start_pos=pos, use_cache=True))
            pos += n
        full = m(x)
    torch.cuda.synchronize()
    check_device_status()
    got, want = torch.cat(outs, dim=1).float(), full.float()
    assert (got - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item())
