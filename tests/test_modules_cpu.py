"""Host-side mirror of the reference's module interface: names, shapes, constants (CPU only)."""

import os

import numpy as np
import pytest
import torch

from oracle import golden_cases as G


@pytest.fixture(scope="module")
def mods(golden_dir):
    return np.load(os.path.join(golden_dir, "modules.npz"))


@pytest.fixture(scope="module")
def models(golden_dir):
    return np.load(os.path.join(golden_dir, "models.npz"))


def build_module(spec):
    from pe_ablations_b200 import modules as M
    from pe_ablations_b200 import pe as P

    kind = spec["kind"]
    hd, H, Hkv, hidden, S = spec["head_dim"], spec["H"], spec["Hkv"], spec["hidden"], spec["S"]
    if kind in ("rope", "yarn", "ntk", "nope"):
        rope = None
        if kind == "rope":
            rope = P.RotaryEmbedding(hd, S, 10000.0)
        elif kind == "ntk":
            rope = P.NTKAwareRotaryEmbedding(hd, S, 10000.0, spec["rope_scale"])
        elif kind == "yarn":
            rope = P.YaRNRotaryEmbedding(hd, S, 10000.0, spec["rope_scale"], original_max_seq_len=512)
        return M.GroupedQueryAttention(hidden, H, Hkv, hd, spec["use_qk_norm"], rope)
    if kind == "alibi":
        return M.ALiBiAttention(hidden, H, Hkv, hd, spec["use_qk_norm"])
    if kind == "fpope":
        pe = P.FoPEPoPEEmbedding(dim=spec["d_rope"], max_seq_len=S, num_fourier_terms=spec["n_fourier"],
                                 fourier_sigma=spec["sigma"], training_length=spec["training_length"],
                                 delta_init=spec["delta_init"])
    else:
        pe = P.PoPEEmbedding(dim=spec["d_rope"], max_seq_len=S, training_length=spec.get("training_length", 512),
                             use_floor=(kind == "pope_floor"), delta_init=spec["delta_init"])
    return M.FPoPEGroupedQueryAttention(hidden, H, Hkv, hd, spec["d_rope"], spec["use_qk_norm"], pe)


@pytest.mark.parametrize("spec", G.MODULE_CASES, ids=lambda s: s["name"])
def test_module_state_dict_keys_and_buffers_match_reference(mods, spec):
    m = build_module(spec)
    assert sorted(m.state_dict().keys()) == list(mods[f"{spec['name']}/state_keys"])
    bufs = dict(m.named_buffers())
    for key in mods.files:
        if key.startswith(f"{spec['name']}/buf/"):
            name = key.split("/buf/")[1]
            got = bufs[name].float().reshape(-1)
            want = torch.from_numpy(mods[key]).reshape(-1)
            assert torch.allclose(got, want, rtol=2e-6, atol=1e-9), name


def build_model(spec):
    from pe_ablations_b200.model import Transformer, TransformerConfig

    kw = dict(G.MODEL_BASE)
    kw.update({k: v for k, v in spec.items() if k != "name"})
    return Transformer(TransformerConfig(**kw)).eval()


@pytest.mark.parametrize("spec", G.MODEL_CASES, ids=lambda s: s["name"])
def test_model_state_dict_matches_reference(models, spec):
    model = build_model(spec)
    sd = model.state_dict()
    assert sorted(sd.keys()) == list(models[f"{spec['name']}/state_keys"])
    shapes = [",".join(map(str, sd[k].shape)) for k in sorted(sd.keys())]
    assert shapes == list(models[f"{spec['name']}/state_shapes"])


def test_yarn_extend_falls_back_to_plain_rope_like_the_reference():
    from pe_ablations_b200 import pe as P

    y = P.YaRNRotaryEmbedding(64, 128, 10000.0, 4.0)
    r = P.RotaryEmbedding(64, 256, 10000.0)
    assert not torch.allclose(y.freqs_cis, r.freqs_cis[:128])
    y.extend_seq_len(256)
    assert torch.allclose(torch.view_as_real(y.freqs_cis), torch.view_as_real(r.freqs_cis))
    assert abs(y.attention_scale - (0.1 * np.log(4.0) + 1.0)) < 1e-6


def test_pe_holders_do_not_compute():
    from pe_ablations_b200 import pe as P

    with pytest.raises(NotImplementedError):
        P.PoPEEmbedding(8).forward_query(torch.zeros(1, 1, 1, 8))
    with pytest.raises(NotImplementedError):
        P.RotaryEmbedding(8, 16)(torch.zeros(1), torch.zeros(1))


def test_modules_refuse_masks_and_cpu():
    from pe_ablations_b200 import modules as M

    m = M.GroupedQueryAttention(64, 2, 2, 32, True, None).eval()
    with torch.no_grad():
        with pytest.raises(NotImplementedError):
            m(torch.zeros(1, 4, 64), mask=torch.ones(1, 1, 4, 4))
        with pytest.raises(RuntimeError):
            m(torch.zeros(1, 4, 64))


def test_fope_effective_freqs_host_formula_matches_oracle():
    from oracle import pe_attention_oracle as O
    from pe_ablations_b200 import pe as P

    torch.manual_seed(3)
    e = P.FoPEPoPEEmbedding(dim=32, num_fourier_terms=16, fourier_sigma=0.3, training_length=128)
    want = O.fope_effective_freqs(e.base_freqs, e.fourier_coeffs.detach(), 128)
    assert torch.allclose(e.effective_freqs(), want, rtol=1e-6, atol=0)
    assert (want == 0).any()  # the floor clip is active at this size


def test_install_rebinds_the_three_attention_classes():
    import types

    from pe_ablations_b200 import modules as M

    ns = types.SimpleNamespace(GroupedQueryAttention=object, ALiBiAttention=object, FPoPEGroupedQueryAttention=object,
                               RMSNorm=object)
    M.install(ns)
    assert ns.GroupedQueryAttention is M.GroupedQueryAttention
    assert ns.ALiBiAttention is M.ALiBiAttention
    assert ns.FPoPEGroupedQueryAttention is M.FPoPEGroupedQueryAttention
    assert ns.RMSNorm is object      # only the attention classes are replaced


def test_cache_module_constructor_and_state_dict():
    from pe_ablations_b200 import modules as M
    from pe_ablations_b200 import pe as P

    pe = P.PoPEEmbedding(dim=16, max_seq_len=32)
    m = M.FPoPEGroupedQueryAttentionWithCache(64, 2, 1, 32, 16, True, pe, max_cache_len=128)
    base = M.FPoPEGroupedQueryAttention(64, 2, 1, 32, 16, True, pe)
    assert sorted(m.state_dict().keys()) == sorted(base.state_dict().keys())   # cache buffers are not persistent
    assert m.cache_len == 0 and m.max_cache_len == 128
    m.reset_cache()


def test_training_transform_equals_the_oracle_transform():
    """The differentiable restatement of the positional transform that the backward pass
    differentiates (autograd.transformed_operands) builds the same operands as the oracle."""
    import math

    from oracle import pe_attention_oracle as O
    from pe_ablations_b200 import autograd as A

    g = torch.Generator().manual_seed(3)
    B, S, H, Hkv, dc, dr = 2, 37, 4, 2, 64, 32
    mk = lambda h, d: torch.randn(B, S, h, d, generator=g).to(torch.bfloat16)
    q, k, q_r, k_r = mk(H, dc), mk(Hkv, dc), mk(H, dr), mk(Hkv, dr)
    base = O.pope_base_freqs(dr)
    coeffs = torch.randn(dr, 8, generator=g) * 0.4
    delta = (torch.rand(dr, generator=g) * 2 - 1) * math.pi
    o = dict(start_pos=5, k_start_pos=5, normalize_coeffs=True, floor_freq=2 * math.pi / 32, ceil_freq=None)
    qt, kt = A.transformed_operands("pope", q, k, q_r, k_r, o, base, delta, coeffs)
    eff = O.fope_effective_freqs(base, coeffs, 32)
    assert torch.equal(A.effective_freqs(base, coeffs, True, o["floor_freq"], None), eff)
    want_q = torch.cat([q.float(), O.pope_expand(q_r, 5, eff, None)], dim=-1).to(torch.bfloat16)
    want_k = torch.cat([k.float(), O.pope_expand(k_r, 5, eff, delta)], dim=-1).to(torch.bfloat16)
    assert torch.equal(qt.to(torch.bfloat16), want_q) and torch.equal(kt.to(torch.bfloat16), want_k)
    # rotary + mscale + QKNorm
    table = O.rotary_table(O.rope_inv_freq(dc), 64)
    o = dict(start_pos=3, k_start_pos=3, table_pos0=0, mscale=1.07, qk_norm=True, qk_norm_eps=1e-6, rotary_table=table)
    qt, kt = A.transformed_operands("rotary", q, k, None, None, o, None, None, None)
    want = O.qk_l2_norm(O.rotary_apply(q.float(), table[3:3 + S], 1.07)).to(torch.bfloat16)
    assert (qt.float() - want.float()).abs().max().item() <= 2 ** -8
    # gradients reach the encoding's parameters
    coeffs.requires_grad_(True)
    delta.requires_grad_(True)
    o = dict(start_pos=0, k_start_pos=0, normalize_coeffs=True, floor_freq=2 * math.pi / 32, ceil_freq=None)
    qt, kt = A.transformed_operands("pope", q, k, q_r, k_r, o, base, delta, coeffs)
    (qt.float().sum() + kt.float().square().sum()).backward()
    assert coeffs.grad.abs().sum() > 0 and delta.grad.abs().sum() > 0
    assert (delta.grad[delta.detach() > 0] == 0).all()          # clamped at use: no gradient above 0
