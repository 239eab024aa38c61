"""Pin the CPU oracle against outputs of the reference's own live modules.

The fixtures under tests/golden/ were produced by tests/golden/make_golden.py,
which imports the reference; these tests only read them.
"""

import os

import numpy as np
import pytest
import torch

from oracle import golden_cases as G
from oracle import pe_attention_oracle as O
from oracle.inputs import make_inputs, oracle_output


@pytest.fixture(scope="module")
def core(golden_dir):
    return np.load(os.path.join(golden_dir, "core.npz"))


def _golden_out(core, case):
    if case.dtype == torch.bfloat16:
        bits = torch.from_numpy(core[f"{case.name}/out_bf16_bits"])
        return bits.view(torch.bfloat16).float()
    return torch.from_numpy(core[f"{case.name}/out"])


@pytest.mark.parametrize("case", G.CORE_CASES, ids=lambda c: c.name)
def test_core_matches_reference(core, case):
    inp = make_inputs(case)
    got = oracle_output(case, inp)
    want = _golden_out(core, case)
    # fp32: two fp32 evaluations of the same math; bf16: the reference's SDPA also
    # rounds P and the output to bf16, the oracle keeps them in fp32
    tol = 2e-5 if case.dtype == torch.float32 else 1.2e-2
    assert got.shape == want.shape
    assert (got.float() - want).abs().max().item() <= tol


@pytest.mark.parametrize("case", G.CORE_CASES, ids=lambda c: c.name)
def test_pe_constants_match_reference(core, case):
    inp = make_inputs(case)
    for key in ("freqs", "base_freqs", "inv_freq", "slopes"):
        name = f"{case.name}/{key}"
        if name in core.files:
            want = torch.from_numpy(core[name])
            got = inp[key]
            # identical formulas in fp32; allow the last bit of a differently-ordered sum
            assert torch.allclose(got, want, rtol=3e-6, atol=1e-9), key
            # clipping must agree exactly: same zeros
            assert torch.equal(got == 0, want == 0), key
    if f"{case.name}/table" in core.files:
        want = torch.from_numpy(core[f"{case.name}/table"])
        got = inp["table"][::G.TABLE_ROW_STRIDE]
        assert (got - want).abs().max().item() <= 2e-6
    if f"{case.name}/mscale" in core.files:
        assert abs(float(core[f"{case.name}/mscale"][0]) - inp["mscale"]) < 1e-7


@pytest.mark.parametrize("case,stride", G.FULL_CASES, ids=lambda c: getattr(c, "name", str(c)))
def test_full_config1_matches_reference(core, case, stride):
    inp = make_inputs(case)
    got = oracle_output(case, inp)[:, ::stride]
    want = torch.from_numpy(core[f"{case.name}/out_rows"])
    assert int(core[f"{case.name}/row_stride"]) == stride
    assert (got - want).abs().max().item() <= 2e-5


def test_fp64_truth_bounds_fp32_oracle():
    case = G.CORE_CASES[0]
    inp = make_inputs(case)
    a = oracle_output(case, inp, acc=torch.float32)
    b = oracle_output(case, inp, acc=torch.float64)
    assert (a.double() - b).abs().max().item() < 1e-5


def test_structural_identities():
    # V = 0 gives 0; diagonal phase equals the clamped delta; clamp maps positive delta to 0
    case = G.CORE_CASES[0]
    inp = make_inputs(case)
    inp0 = dict(inp, v=torch.zeros_like(inp["v"]))
    assert oracle_output(case, inp0).abs().max().item() == 0.0
    d = torch.tensor([1.0, -1.0, -7.0])
    x = torch.zeros(1, 1, 1, 3)
    out = O.pope_expand(x, 0, torch.ones(3), d)
    mu = torch.nn.functional.softplus(torch.zeros(()))
    want_phase = torch.tensor([0.0, -1.0, -2 * torch.pi])
    assert torch.allclose(out[0, 0, 0, :3], mu * want_phase.cos(), atol=1e-6)
    assert torch.allclose(out[0, 0, 0, 3:], mu * want_phase.sin(), atol=1e-6)


def test_alibi_slopes_non_power_of_two():
    s = O.alibi_slopes(12)
    assert s.shape == (12,)
    assert torch.allclose(s[:8], torch.tensor([2.0 ** (-(i + 1)) for i in range(8)]))


# ---- the explicit cosine-sum formulation: an oracle that shares nothing with the GEMM form ----
@pytest.fixture(scope="module")
def cos_sum(golden_dir):
    return np.load(os.path.join(golden_dir, "cos_sum.npz"))


@pytest.mark.parametrize("case", G.COS_SUM_CASES, ids=lambda c: c.name)
def test_cos_sum_oracle_matches_reference(cos_sum, case):
    """``cos_sum_attention`` against the reference's own ``pope_attention`` output."""
    inp = make_inputs(case)
    want = torch.from_numpy(cos_sum[f"{case.name}/out"])
    assert torch.allclose(inp["freqs"], torch.from_numpy(cos_sum[f"{case.name}/freqs"]), rtol=3e-6, atol=1e-9)
    got = O.cos_sum_attention(inp["q_r"], inp["k_r"], inp["v"], inp["freqs"], inp["delta"], pos0=case.pos0)
    assert got.shape == want.shape
    assert (got - want).abs().max().item() <= 2e-5


@pytest.mark.parametrize("case", G.COS_SUM_CASES, ids=lambda c: c.name)
def test_gemm_form_oracle_agrees_with_cos_sum_reference(cos_sum, case):
    """The concatenated cos/sin restatement (what the kernels implement) gives the same attention
    as the reference's cosine-sum path: cos(a - b) = cos a cos b + sin a sin b, in fp32."""
    inp = make_inputs(case)
    want = torch.from_numpy(cos_sum[f"{case.name}/out"])
    got = O.attention_core("pope", None, None, inp["v"], q_r=inp["q_r"], k_r=inp["k_r"], pos0=case.pos0,
                           freqs=inp["freqs"], delta=inp["delta"], scale=case.d_r ** -0.5)
    # phases up to ~|pos| * freq: the two sides round pos * freq differently
    assert (got - want).abs().max().item() <= 5e-5


def test_cos_sum_with_content_halves_equals_gemm_form():
    case = G.CORE_CASES[3]                      # g_fpope_fp32: content 64 + position 32, GQA 4:1
    assert case.name == "g_fpope_fp32"
    inp = make_inputs(case)
    a = oracle_output(case, inp)
    b = O.cos_sum_attention(inp["q_r"], inp["k_r"], inp["v"], inp["freqs"], inp["delta"], q=inp["q"], k=inp["k"],
                            scale=case.d_qk ** -0.5)
    assert (a - b).abs().max().item() <= 2e-5
