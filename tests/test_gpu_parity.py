"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle and the golden fixtures.

Tolerances (max abs error on the attention output): 1e-4 for fp32, 2e-2 for bf16.
"""

import math
import os

import numpy as np
import pytest
import torch

from oracle import golden_cases as G
from oracle.inputs import BF16, FP32, CONFIGS, Case, make_inputs, oracle_output

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def core(golden_dir):
    return np.load(os.path.join(golden_dir, "core.npz"))


@pytest.mark.parametrize("case", G.CORE_CASES, ids=lambda c: c.name)
def test_matches_oracle_and_reference_fixture(core, case):
    from tests.gpu_util import case_error

    err, got, _ = case_error(case)
    assert err <= TOL[case.dtype], f"vs oracle: {err}"
    if case.dtype == torch.bfloat16:
        want = torch.from_numpy(core[f"{case.name}/out_bf16_bits"]).view(torch.bfloat16).float()
    else:
        want = torch.from_numpy(core[f"{case.name}/out"])
    assert (got - want).abs().max().item() <= TOL[case.dtype], "vs the reference's own output"


@pytest.mark.parametrize("case,stride", G.FULL_CASES, ids=lambda c: getattr(c, "name", str(c)))
def test_config1_full_size(core, case, stride):
    from tests.gpu_util import case_error

    err, got, _ = case_error(case)
    assert err <= 1e-4
    want = torch.from_numpy(core[f"{case.name}/out_rows"])
    assert (got[:, ::stride] - want).abs().max().item() <= 1e-4


EDGE_CASES = [
    Case("e_s1_fp32", "pope", FP32, 1, 2, 2, 1, 32, 16, 32, seed=41),
    Case("e_s17_fp32", "rotary", FP32, 1, 2, 1, 17, 64, 0, 64, seed=42),
    Case("e_s1_bf16", "pope", BF16, 1, 2, 2, 1, 64, 32, 64, seed=43),
    Case("e_s17_bf16", "rotary", BF16, 2, 4, 2, 17, 64, 0, 64, seed=44),
    Case("e_s127_bf16", "nope", BF16, 1, 2, 2, 127, 128, 0, 128, seed=45),
    Case("e_s129_bf16", "pope", BF16, 1, 4, 1, 129, 128, 32, 128, seed=46, pope_kind="pope_floor",
         training_length=64),
    Case("e_s257_bf16", "alibi", BF16, 1, 6, 2, 257, 128, 0, 128, seed=47),
    Case("e_s513_gqa4_bf16", "pope", BF16, 2, 8, 2, 513, 64, 32, 64, seed=48, pope_kind="fpope",
         training_length=128, n_fourier=16, fourier_sigma=0.4),
    Case("e_s640_pos0_bf16", "pope", BF16, 1, 2, 2, 640, 128, 64, 128, seed=49, pos0=1000, pope_kind="fpope",
         training_length=2048),
    Case("e_posonly32_bf16", "pope", BF16, 1, 2, 2, 300, 0, 32, 64, seed=50),
    Case("e_posonly64_bf16", "pope", BF16, 1, 2, 1, 300, 0, 64, 128, seed=51),
    Case("e_yarn_bf16", "rotary", BF16, 1, 4, 4, 384, 64, 0, 64, seed=52, rope_kind="yarn", rope_scale=4.0),
    Case("e_rope_pos0_bf16", "rotary", BF16, 1, 2, 2, 200, 128, 0, 128, seed=53, pos0=4000, qk_norm=True),
    Case("e_nope_plain_bf16", "nope", BF16, 2, 4, 2, 700, 64, 0, 64, seed=54),
    Case("e_alibi_noqk_bf16", "alibi", BF16, 1, 4, 4, 330, 64, 0, 64, seed=55),
]


@pytest.mark.parametrize("case", EDGE_CASES, ids=lambda c: c.name)
def test_edge_shapes(case):
    from tests.gpu_util import case_error

    err, _, _ = case_error(case)
    assert err <= TOL[case.dtype], err


MID_CASES = [
    Case("mid_cfg2_rope", "rotary", BF16, 2, 12, 12, 2048, 64, 0, 64, seed=61),
    Case("mid_cfg2_ntk4", "rotary", BF16, 1, 12, 12, 2048, 64, 0, 64, seed=62, rope_kind="ntk", rope_scale=4.0),
    Case("mid_cfg3_fope", "rotary", BF16, 1, 4, 4, 4096, 128, 0, 128, seed=63, rope_kind="fope",
         training_length=4096),
    Case("mid_cfg4_fpope", "pope", BF16, 1, 2, 2, 4096, 128, 64, 128, seed=64, pope_kind="fpope",
         training_length=16384),
]


@pytest.mark.parametrize("case", MID_CASES, ids=lambda c: c.name)
def test_benchmark_shapes_reduced_batch(case):
    """The benchmark configurations at their head dims and (up to) sequence length, fewer batch x heads."""
    from tests.gpu_util import case_error

    err, _, _ = case_error(case)
    assert err <= TOL[case.dtype], err


def test_ffma_kernel_cross_checks_tensor_core_kernel():
    """The bf16 FFMA instantiation and the tcgen05 kernel agree on the same device tensors."""
    from tests.gpu_util import run_case_on_gpu

    case = Case("x_fpope", "pope", BF16, 1, 4, 2, 900, 128, 64, 128, seed=71, pope_kind="fpope", training_length=512)
    inp = make_inputs(case)
    a = run_case_on_gpu(case, inp, simt_check=False)
    b = run_case_on_gpu(case, inp, simt_check=True)
    assert (a - b).abs().max().item() <= 2e-2


@pytest.mark.parametrize("case", [
    Case("x_pair_fpope", "pope", BF16, 1, 4, 2, 1500, 128, 64, 128, seed=81, pope_kind="fpope", training_length=1024),
    Case("x_pair_rope_qkn", "rotary", BF16, 2, 2, 2, 1100, 128, 0, 128, seed=82, qk_norm=True),
    Case("x_pair_alibi", "alibi", BF16, 1, 4, 4, 777, 128, 0, 128, seed=83),
    Case("x_pair_nope_gqa", "nope", BF16, 1, 8, 2, 1030, 128, 0, 128, seed=84),
    Case("x_pair_pope_dr32", "pope", BF16, 1, 2, 2, 900, 128, 32, 128, seed=85, pos0=300),
    Case("x_pair_posonly", "pope", BF16, 1, 2, 1, 700, 0, 64, 128, seed=86),
], ids=lambda c: c.name)
def test_cta_pair_and_single_cta_kernels_agree(case):
    """Both tcgen05 kernels on the same tensors, each against the oracle and against each other."""
    from tests.gpu_util import run_case_on_gpu

    inp = make_inputs(case)
    want = oracle_output(case, inp).float()
    pair = run_case_on_gpu(case, inp)
    single = run_case_on_gpu(case, inp, single_cta=True)
    assert (pair - want).abs().max().item() <= 2e-2
    assert (single - want).abs().max().item() <= 2e-2
    assert (pair - single).abs().max().item() <= 2e-2


@pytest.mark.parametrize("case", [
    Case("split_fpope", "pope", BF16, 1, 2, 2, 4096, 128, 64, 128, seed=201, pope_kind="fpope", training_length=4096),
    Case("split_pope_ragged", "pope", BF16, 1, 3, 3, 3000, 128, 32, 128, seed=202, pos0=70),
    Case("split_rope_qkn_gqa", "rotary", BF16, 1, 4, 2, 2500, 128, 0, 128, seed=203, qk_norm=True),
    Case("split_alibi", "alibi", BF16, 2, 2, 2, 2100, 128, 0, 128, seed=204),
], ids=lambda c: c.name)
def test_few_wave_launches_split_their_longest_blocks(case):
    """A launch with few (batch, head) problems: the CTA-pair kernel cuts the longest query blocks
    in two along the keys and merges the halves (needs the forward workspace, which the Python
    wrapper provides).  Output and logsumexp against the oracle, and against the unsplit
    single-CTA kernel."""
    import ctypes as C

    from pe_ablations_b200 import _lib as L
    from pe_ablations_b200 import check_device_status, pe_attention
    from oracle import pe_attention_oracle as O
    from tests.gpu_util import run_case_on_gpu

    inp = make_inputs(case)
    # the planner does ask for a workspace at this size
    a = L.PeAttnArgs()
    a.struct_size = C.sizeof(L.PeAttnArgs)
    a.variant = {"pope": L.POPE, "rotary": L.ROTARY, "alibi": L.ALIBI}[case.variant]
    a.dtype = L.BF16
    a.B, a.H, a.Hkv, a.Sq, a.Sk, a.d_c, a.d_r, a.d_v = case.B, case.H, case.Hkv, case.S, case.S, case.d_c, case.d_r, case.d_v
    a.scale = case.d_qk ** -0.5
    for name in ("q", "k", "v", "out", "q_r", "k_r", "freqs", "rotary_table", "alibi_slopes"):
        setattr(a, name, 0x10000)
    a.table_rows = case.pos0 + case.S
    for sname, d, hh in (("q_stride", case.d_c, case.H), ("k_stride", case.d_c, case.Hkv), ("v_stride", case.d_v, case.Hkv),
                         ("out_stride", case.d_v, case.H), ("qr_stride", max(case.d_r, 8), case.H),
                         ("kr_stride", max(case.d_r, 8), case.Hkv)):
        getattr(a, sname)[:] = (case.S * hh * d, d, hh * d)
    assert L.lib.pe_attn_forward_workspace_bytes(C.byref(a)) > 0, L.lib.pe_attn_last_error()

    want = oracle_output(case, inp).float()
    pair = run_case_on_gpu(case, inp)
    single = run_case_on_gpu(case, inp, single_cta=True)
    assert (pair - want).abs().max().item() <= 2e-2
    assert (pair - single).abs().max().item() <= 2e-2

    if case.variant == "pope":     # the merged logsumexp too
        dev = torch.device("cuda", 0)
        c = lambda t: t.to(dev, torch.bfloat16)
        lse = torch.full((case.B, case.H, case.S), float("nan"), device=dev)
        kw = dict(freqs=inp["base_freqs"], fourier_coeffs=inp["fourier_coeffs"],
                  floor_freq=2 * torch.pi / case.training_length) if case.pope_kind == "fpope" else dict(freqs=inp["freqs"])
        pe_attention("pope", c(inp["q"]), c(inp["k"]), c(inp["v"]), q_r=c(inp["q_r"]), k_r=c(inp["k_r"]),
                     delta=inp["delta"], start_pos=case.pos0, lse=lse, **kw)
        torch.cuda.synchronize()
        check_device_status()
        _, want_lse = O.attention_core("pope", inp["q"], inp["k"], inp["v"], dtype=torch.bfloat16, q_r=inp["q_r"],
                                       k_r=inp["k_r"], freqs=inp["freqs"], delta=inp["delta"], pos0=case.pos0,
                                       return_lse=True)
        assert (lse.cpu() - want_lse).abs().max().item() <= 2e-2


def test_fused_fourier_mix_equals_host_mix():
    from tests.gpu_util import run_case_on_gpu

    case = Case("x_fmix", "pope", FP32, 1, 2, 2, 96, 32, 16, 32, seed=72, pope_kind="fpope", training_length=32,
                n_fourier=16, fourier_sigma=0.5)
    inp = make_inputs(case)
    a = run_case_on_gpu(case, inp, fused_fourier=True)
    b = run_case_on_gpu(case, inp, fused_fourier=False)
    assert (a - b).abs().max().item() <= 2e-5


def test_determinism_and_unwritten_rows():
    """Same inputs give bit-identical outputs; a NaN-poisoned output buffer is fully overwritten."""
    from pe_ablations_b200 import pe_attention

    case = Case("x_det", "pope", BF16, 1, 2, 2, 777, 128, 64, 128, seed=73, pope_kind="fpope", training_length=512)
    inp = make_inputs(case)
    dev = torch.device("cuda", 0)
    c = lambda t: t.to(dev, torch.bfloat16)
    outs = []
    for _ in range(2):
        out = torch.full((1, 777, 2, 128), float("nan"), dtype=torch.bfloat16, device=dev)
        pe_attention("pope", c(inp["q"]), c(inp["k"]), c(inp["v"]), q_r=c(inp["q_r"]), k_r=c(inp["k_r"]),
                     freqs=inp["freqs"], delta=inp["delta"], out=out)
        torch.cuda.synchronize()
        outs.append(out)
    assert not torch.isnan(outs[0]).any()
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("name,variant,shape,extra", [
    ("pair_rotary_qknorm_gqa", "rotary", (2, 4096, 16, 4, 128, 0, 128), dict(qk_norm=True)),
    ("pair_rotary", "rotary", (2, 4096, 8, 8, 128, 0, 128), {}),
    ("tile4_rotary", "rotary", (4, 2048, 12, 12, 64, 0, 64), {}),
    ("tile2_nope", "nope", (4, 2048, 12, 12, 64, 0, 64), {}),
])
def test_repeated_launches_are_bitwise_identical(name, variant, shape, extra):
    """Many SMs' worth of blocks, twenty launches: every launch gives the first one's bits.  The
    hand-offs between warps and between the CTAs of a pair (K rows built in shared memory, P
    handed over in parts, relaxed arrivals) leave no room for a race to show up as noise."""
    from pe_ablations_b200 import check_device_status, pe_attention
    from pe_ablations_b200 import pe as PE

    B, S, H, Hkv, dc, dr, dv = shape
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(91)
    mk = lambda h, d: torch.randn(B, S, h, d, generator=g).to(torch.bfloat16).to(dev)
    q, k, v = mk(H, dc), mk(Hkv, dc), mk(Hkv, dv)
    kw = dict(extra)
    if variant == "rotary":
        kw["rotary_table"] = PE.RotaryEmbedding(dc, S, 10000.0).to(dev).freqs_cis
    first = pe_attention(variant, q, k, v, **kw).clone()
    for _ in range(20):
        assert torch.equal(pe_attention(variant, q, k, v, **kw), first)
    check_device_status()


def test_full_size_config4_properties():
    """BASELINE configuration 4 at full size: size-independent properties instead of a CPU oracle.

    (a) V = 1 gives an output of exactly-ish 1 (softmax rows sum to one);
    (b) the first 512 query rows depend only on the first 512 keys, so they must equal the
        output of the same call on the 512-row prefix (checked against the oracle there);
    (c) linearity in V: out(V1 + V2) = out(V1) + out(V2) within bf16 rounding.
    """
    from pe_ablations_b200 import check_device_status, pe_attention

    case = CONFIGS["cfg4_fpope_bf16"]
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(5)
    B, S, H = case.B, case.S, case.H
    mk = lambda d: torch.randn(B, S, H, d, generator=g, dtype=torch.float32).to(dev, torch.bfloat16)
    q, k, qr, kr, v1, v2 = mk(128), mk(128), mk(64), mk(64), mk(128), mk(128)
    small = make_inputs(Case("tmp", "pope", BF16, 1, 1, 1, 8, 128, 64, 128, seed=9, pope_kind="fpope",
                             training_length=16384))
    kw = dict(q_r=qr, k_r=kr, freqs=small["base_freqs"], fourier_coeffs=small["fourier_coeffs"],
              floor_freq=2 * torch.pi / 16384, delta=small["delta"])
    ones = torch.ones_like(v1)
    o1 = pe_attention("pope", q, k, ones, **kw)
    assert (o1.float() - 1.0).abs().max().item() <= 1e-2
    oa = pe_attention("pope", q, k, v1, **kw)
    ob = pe_attention("pope", q, k, v2, **kw)
    oab = pe_attention("pope", q, k, (v1.float() + v2.float()).to(torch.bfloat16), **kw)
    assert (oab.float() - (oa.float() + ob.float())).abs().max().item() <= 6e-2
    kw512 = dict(kw, q_r=qr[:, :512], k_r=kr[:, :512])
    op = pe_attention("pope", q[:, :512], k[:, :512], v1[:, :512], **kw512)
    torch.cuda.synchronize()
    check_device_status()
    assert (op.float() - oa[:, :512].float()).abs().max().item() <= 1e-2
    want = oracle_output(
        Case("pfx", "pope", BF16, B, H, H, 512, 128, 64, 128, pope_kind="fpope", training_length=16384),
        dict(q=q[:, :512].float().cpu(), k=k[:, :512].float().cpu(), q_r=qr[:, :512].float().cpu(),
             k_r=kr[:, :512].float().cpu(), v=v1[:, :512].float().cpu(), freqs=small["freqs"], delta=small["delta"]))
    assert (op.float().cpu() - want).abs().max().item() <= 2e-2


@pytest.mark.parametrize("single_cta", [False, True], ids=["cta_pair", "single_cta"])
def test_config4_last_rows_match_oracle(single_cta):
    """BASELINE configuration 4's LAST 512 query rows (positions 15872..16383) against all 16384
    keys: where phases reach 16k * omega and the tile-base rotations of the K transform matter
    most.  Four (batch, head) slices, FoPE mix inside the kernel, delta ~ U(-pi, pi)."""
    from pe_ablations_b200 import check_device_status, pe_attention
    from oracle import pe_attention_oracle as O

    B, H, S, Sq, dc, dr, dv = 2, 2, 16384, 512, 128, 64, 128
    g = torch.Generator().manual_seed(401)
    mk = lambda s, d: torch.randn(B, s, H, d, generator=g).to(torch.bfloat16)
    q, q_r, k, k_r, v = mk(Sq, dc), mk(Sq, dr), mk(S, dc), mk(S, dr), mk(S, dv)
    delta = (torch.rand(dr, generator=g) * 2 - 1) * torch.pi
    coeffs = torch.randn(dr, 16, generator=g) * 0.3
    base = O.pope_base_freqs(dr)
    eff = O.fope_effective_freqs(base, coeffs, training_length=S)
    want = O.attention_core("pope", q.float(), k.float(), v.float(), dtype=torch.bfloat16, q_r=q_r.float(),
                            k_r=k_r.float(), freqs=eff, delta=delta, pos0=S - Sq, k_pos0=0).float()
    dev = torch.device("cuda", 0)
    got = pe_attention("pope", q.to(dev), k.to(dev), v.to(dev), q_r=q_r.to(dev), k_r=k_r.to(dev), freqs=base,
                       fourier_coeffs=coeffs, floor_freq=2 * torch.pi / S, delta=delta, start_pos=S - Sq,
                       k_start_pos=0, single_cta=single_cta)
    torch.cuda.synchronize()
    check_device_status()
    assert (got.float().cpu() - want).abs().max().item() <= 2e-2


@pytest.mark.parametrize("single_cta", [False, True], ids=["cta_pair", "single_cta"])
def test_config3_last_rows_match_oracle(single_cta):
    """BASELINE configuration 3 (FoPE frequencies through the rotary table, head_dim 128): the last
    512 query rows of a 4096-token sequence against all keys."""
    from pe_ablations_b200 import check_device_status, pe_attention
    from oracle import pe_attention_oracle as O

    B, H, S, Sq, D = 1, 4, 4096, 512, 128
    g = torch.Generator().manual_seed(402)
    mk = lambda s: torch.randn(B, s, H, D, generator=g).to(torch.bfloat16)
    q, k, v = mk(Sq), mk(S), mk(S)
    coeffs = torch.randn(D // 2, 16, generator=g) * 0.3
    table = O.rotary_table(O.fope_effective_freqs(O.pope_base_freqs(D // 2), coeffs, training_length=S), S)
    want = O.attention_core("rotary", q.float(), k.float(), v.float(), dtype=torch.bfloat16, table=table,
                            table_pos0=0, pos0=S - Sq, k_pos0=0).float()
    dev = torch.device("cuda", 0)
    got = pe_attention("rotary", q.to(dev), k.to(dev), v.to(dev), rotary_table=table, table_pos0=0,
                       start_pos=S - Sq, k_start_pos=0, single_cta=single_cta)
    torch.cuda.synchronize()
    check_device_status()
    assert (got.float().cpu() - want).abs().max().item() <= 2e-2


@pytest.mark.parametrize("case", G.COS_SUM_CASES, ids=lambda c: c.name)
def test_fp32_kernel_matches_cos_sum_reference(golden_dir, case):
    """The fp32 kernel (cos/sin expansion + dense product) against the reference's explicit
    cosine-sum attention, a formulation it shares nothing with; and against its restatement."""
    from oracle import pe_attention_oracle as O
    from pe_ablations_b200 import pe_attention

    ref = np.load(os.path.join(golden_dir, "cos_sum.npz"))
    inp = make_inputs(case)
    dev = torch.device("cuda", 0)
    kw = dict(freqs=inp["freqs"], delta=inp["delta"], start_pos=case.pos0, scale=case.d_r ** -0.5)
    got = pe_attention("pope", None, None, inp["v"].to(dev), q_r=inp["q_r"].to(dev), k_r=inp["k_r"].to(dev), **kw)
    torch.cuda.synchronize()
    got = got.cpu()
    assert (got - torch.from_numpy(ref[f"{case.name}/out"])).abs().max().item() <= 1e-4
    again = O.cos_sum_attention(inp["q_r"], inp["k_r"], inp["v"], inp["freqs"], inp["delta"], pos0=case.pos0)
    assert (got - again).abs().max().item() <= 1e-4


def test_abi_rejects_bad_arguments_on_gpu():
    from pe_ablations_b200 import pe_attention
    from pe_ablations_b200._lib import PeAttnError

    dev = torch.device("cuda", 0)
    q = torch.zeros(1, 8, 2, 48, dtype=torch.bfloat16, device=dev)
    with pytest.raises(PeAttnError):
        pe_attention("nope", q, q, q)  # head dim 48 is not supported by the bf16 path
    with pytest.raises(NotImplementedError):
        pe_attention("nope", q, q, q, mask=torch.ones(1))
    with pytest.raises(RuntimeError):
        pe_attention("nope", q.cpu(), q.cpu(), q.cpu())


def test_expired_wait_is_reported_and_context_survives():
    """A bounded wait that runs out sets the status word; nothing hangs, the next launch works."""
    import ctypes as C

    from pe_ablations_b200 import _lib as L
    from pe_ablations_b200 import check_device_status
    from pe_ablations_b200.ops import device_status
    from tests.gpu_util import case_error

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    word = device_status(dev)
    word.zero_()
    stream = torch.cuda.current_stream().cuda_stream
    assert L.lib.pe_attn_selftest_wait_expiry(word.data_ptr(), 2_000_000, C.c_void_p(stream)) == 0  # ~1 ms
    torch.cuda.synchronize()
    assert int(word.item()) == 0x40000000
    with pytest.raises(RuntimeError, match="expired waits"):
        check_device_status()
    assert int(word.item()) == 0          # the wrapper clears the word after reporting
    err, _, _ = case_error(Case("after_expiry", "pope", BF16, 1, 2, 2, 300, 128, 64, 128, seed=91))
    assert err <= 2e-2
    assert L.lib.pe_attn_selftest_wait_expiry(None, 2_000_000, None) == 1
    assert L.lib.pe_attn_selftest_wait_expiry(word.data_ptr(), 10, None) == 3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_bhsd_layout_and_strided_views(dtype):
    """[B, H, S, d] storage and sliced (non-contiguous batch / head) views are read in place."""
    from pe_ablations_b200 import check_device_status, pe_attention
    from oracle import pe_attention_oracle as O

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(7)
    B, H, Hkv, S, dc, dr, dv = 2, 4, 2, 330, 128, 64, 128
    mk = lambda h, d: torch.randn(B, S, h, d, generator=g)
    q, k, q_r, k_r, v = mk(H, dc), mk(Hkv, dc), mk(H, dr), mk(Hkv, dr), mk(Hkv, dv)
    freqs = O.pope_base_freqs(dr)
    delta = -torch.rand(dr, generator=g) * 3
    want = O.attention_core("pope", q, k, v, dtype=dtype, q_r=q_r, k_r=k_r, freqs=freqs, delta=delta).float()
    tol = TOL[dtype]
    c = lambda t: t.to(dev, dtype)
    # (a) [B, H, S, d] contiguous storage
    t = lambda x: c(x).transpose(1, 2).contiguous()
    out = pe_attention("pope", t(q), t(k), t(v), q_r=t(q_r), k_r=t(k_r), freqs=freqs, delta=delta, layout="bhsd")
    assert out.shape == (B, H, S, dv)
    assert (out.transpose(1, 2).float().cpu() - want).abs().max().item() <= tol
    # (b) views into wider buffers: padded batch and a fused [q | k | v]-style last dimension
    big = torch.zeros(B + 1, S, H, dc + 64, dtype=dtype, device=dev)
    big[1:, :, :, :dc] = c(q)
    qv = big[1:, :, :, :dc]
    assert not qv.is_contiguous()
    out2 = pe_attention("pope", qv, c(k), c(v), q_r=c(q_r), k_r=c(k_r), freqs=freqs, delta=delta)
    torch.cuda.synchronize()
    check_device_status()
    assert (out2.float().cpu() - want).abs().max().item() <= tol


@pytest.mark.parametrize("chunks", [1, 4])
def test_host_streamed_call_equals_the_device_call(chunks):
    """Pinned host tensors in, pinned host tensor out, copies pipelined over sequence blocks:
    the one-shot call's result on device copies (to a bf16 ulp), and within tolerance of the oracle."""
    from pe_ablations_b200 import HostStreamedAttention, check_device_status, pe_attention
    from oracle import pe_attention_oracle as O

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(11)
    B, H, Hkv, S, dc, dr, dv = 2, 4, 2, 2048, 128, 64, 128
    mk = lambda h, d: torch.randn(B, S, h, d, generator=g).to(torch.bfloat16).pin_memory()
    host = dict(q=mk(H, dc), k=mk(Hkv, dc), q_r=mk(H, dr), k_r=mk(Hkv, dr), v=mk(Hkv, dv))
    freqs = O.pope_base_freqs(dr)
    delta = -torch.rand(dr, generator=g) * 3
    call = HostStreamedAttention("pope", B=B, S=S, H=H, Hkv=Hkv, d_c=dc, d_r=dr, d_v=dv, dtype=torch.bfloat16,
                                 device=dev, chunks=chunks, freqs=freqs, delta=delta)
    out_host = torch.full((B, S, H, dv), float("nan"), dtype=torch.bfloat16).pin_memory()
    for _ in range(3):                      # the third call reuses the first staging set
        call(host, out_host)
    torch.cuda.synchronize()
    check_device_status()
    d = {n: t.to(dev) for n, t in host.items()}
    one_shot = pe_attention("pope", d["q"], d["k"], d["v"], q_r=d["q_r"], k_r=d["k_r"], freqs=freqs, delta=delta)
    # same kernel, same tiles; a few-wave launch may cut its longest blocks in two along the keys,
    # whose merge rounds differently: at most a bf16 ulp apart
    assert (out_host.float() - one_shot.cpu().float()).abs().max().item() <= 2 ** -7
    f = lambda t: t.float()
    want = O.attention_core("pope", f(host["q"]), f(host["k"]), f(host["v"]), dtype=torch.bfloat16,
                            q_r=f(host["q_r"]), k_r=f(host["k_r"]), freqs=freqs, delta=delta).float()
    assert (out_host.float() - want).abs().max().item() <= TOL[torch.bfloat16]
    with pytest.raises(ValueError):
        call({**host, "q": host["q"].clone()}, out_host)      # not pinned

@pytest.mark.parametrize("variant", ["pope", "fpope", "rotary_qknorm", "nope_qknorm"])
def test_fp32_keys_transformed_once_give_identical_results(monkeypatch, variant):
    """fp32 calls transform their keys once into scratch (the wrapper allocates it); without
    scratch every query block builds its own K tiles.  Same code, same values: bitwise equal."""
    from pe_ablations_b200 import _lib, check_device_status, pe_attention
    from oracle import pe_attention_oracle as O

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(99)
    B, H, Hkv, Sq, Sk, d, dr = 2, 4, 2, 300, 437, 64, 32
    mk = lambda s, h, dd: torch.randn(B, s, h, dd, generator=g).to(dev)
    q, k, v = mk(Sq, H, d), mk(Sk, Hkv, d), mk(Sk, Hkv, d)
    kw = dict(start_pos=Sk - Sq, k_start_pos=0)
    name = "nope"
    if variant in ("pope", "fpope"):
        name = "pope"
        kw.update(q_r=mk(Sq, H, dr), k_r=mk(Sk, Hkv, dr), freqs=O.pope_base_freqs(dr), delta=-torch.rand(dr, generator=g) * 3)
        if variant == "fpope":
            kw.update(fourier_coeffs=torch.randn(dr, 8, generator=g) * 0.3, floor_freq=2 * math.pi / 512)
    elif variant == "rotary_qknorm":
        name = "rotary"
        kw.update(rotary_table=O.rotary_table(O.pope_base_freqs(d // 2), Sk), table_pos0=0, qk_norm=True)
    else:
        kw.update(qk_norm=True)
    with_scratch = pe_attention(name, q, k, v, **kw)
    asked = []
    real = _lib.lib.pe_attn_forward_workspace_bytes
    monkeypatch.setattr(_lib.lib, "pe_attn_forward_workspace_bytes", lambda a: asked.append(real(a)) or 0)
    without = pe_attention(name, q, k, v, **kw)
    torch.cuda.synchronize()
    check_device_status()
    assert asked and asked[0] == B * Hkv * Sk * (d + (2 * dr if name == "pope" else 0)) * 4
    assert torch.equal(with_scratch, without)
