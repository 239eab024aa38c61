"""Helpers shared by the GPU parity tests: run a seeded case through the C ABI."""

import torch

from oracle.inputs import Case, make_inputs, oracle_output


def run_case_on_gpu(case: Case, inp: dict, simt_check: bool = False, fused_fourier: bool = True,
                    single_cta: bool = False) -> torch.Tensor:
    from pe_ablations_b200 import check_device_status, pe_attention

    dev = torch.device("cuda", 0)
    cast = lambda t: None if t is None else t.to(device=dev, dtype=case.dtype)
    kw = {}
    if case.variant == "pope":
        kw["q_r"], kw["k_r"] = cast(inp["q_r"]), cast(inp["k_r"])
        kw["delta"] = inp["delta"]
        if case.pope_kind == "fpope" and fused_fourier:
            kw["freqs"] = inp["base_freqs"]
            kw["fourier_coeffs"] = inp["fourier_coeffs"]
            kw["floor_freq"] = 2 * torch.pi / case.training_length
        else:
            kw["freqs"] = inp["freqs"]
    elif case.variant == "rotary":
        kw["rotary_table"] = inp["table"]
        kw["table_pos0"] = case.pos0
        kw["mscale"] = inp["mscale"]
    elif case.variant == "alibi":
        kw["alibi_slopes"] = inp["slopes"]
    out = pe_attention(case.variant, cast(inp["q"]), cast(inp["k"]), cast(inp["v"]), start_pos=case.pos0,
                       qk_norm=case.qk_norm, simt_check=simt_check, single_cta=single_cta, **kw)
    torch.cuda.synchronize()
    check_device_status()
    return out.float().cpu()


def case_error(case: Case, simt_check: bool = False):
    inp = make_inputs(case)
    want = oracle_output(case, inp)
    got = run_case_on_gpu(case, inp, simt_check=simt_check)
    return (got - want.float()).abs().max().item(), got, want
