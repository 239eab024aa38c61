"""The C-ABI library loads, exports what include/pe_attn.h declares, and validates arguments.

No compute call is made here: ``pe_attn_validate`` touches no GPU.
"""

import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from pe_ablations_b200 import _lib
    return _lib


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "pe_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pe_[a-z_]+)\s*\(", text)))


def test_exports_every_declared_symbol(L):
    names = _declared_functions()
    assert {"pe_attn_forward", "pe_attn_backward", "pe_ce_loss_sums", "pe_pope_expand_backward",
            "pe_rotary_norm_expand"} <= set(names) and len(names) >= 18
    for n in names:
        assert hasattr(L.lib, n), n
    assert L.lib.pe_attn_version() == 4


def _valid_args(L, **over):
    a = L.PeAttnArgs()
    a.struct_size = C.sizeof(L.PeAttnArgs)
    a.variant, a.dtype = L.POPE, L.BF16
    a.B, a.H, a.Hkv, a.Sq, a.Sk = 2, 16, 16, 1024, 1024
    a.d_c, a.d_r, a.d_v = 128, 64, 128
    a.scale = 256 ** -0.5
    for name in ("q", "k", "v", "out", "q_r", "k_r", "freqs"):
        setattr(a, name, 0x10000)
    for s, d in (("q_stride", 128), ("k_stride", 128), ("v_stride", 128), ("out_stride", 128),
                 ("qr_stride", 64), ("kr_stride", 64)):
        getattr(a, s)[:] = (1024 * 16 * d, d, 16 * d)
    for k, v in over.items():
        if k.endswith("_stride"):
            getattr(a, k)[:] = v
        else:
            setattr(a, k, v)
    return a


def test_struct_layout_matches_and_valid_args_pass(L):
    a = _valid_args(L)
    assert L.lib.pe_attn_validate(C.byref(a)) == 0, L.lib.pe_attn_last_error()
    assert L.lib.pe_attn_kernel_name(C.byref(a)) == b"tcgen05-pair"
    assert L.lib.pe_attn_kernel_name(C.byref(_valid_args(L, flags=L.SINGLE_CTA))) == b"tcgen05"
    assert L.lib.pe_attn_kernel_name(C.byref(_valid_args(L, Sq=200, Sk=200))) == b"tcgen05"
    assert L.lib.pe_attn_kernel_name(C.byref(_valid_args(L, d_c=64, d_r=32, d_v=64))) == b"tcgen05-four-tile"
    assert L.lib.pe_attn_kernel_name(C.byref(_valid_args(L, d_c=64, d_r=32, d_v=64, flags=L.SINGLE_CTA))) == b"tcgen05"
    # too few query rows to fill four tiles: the two-tile kernel keeps the call
    assert L.lib.pe_attn_kernel_name(C.byref(_valid_args(L, d_c=64, d_r=32, d_v=64, Sq=200, Sk=200))) == b"tcgen05"
    a = _valid_args(L, dtype=L.FP32)
    assert L.lib.pe_attn_kernel_name(C.byref(a)) == b"ffma"
    fl = L.lib.pe_attn_flops(C.byref(a))
    assert abs(fl - 2 * 16 * (1024 * 1025 / 2) * 2 * 384) < 1e-3 * fl


def test_forward_workspace_is_only_asked_for_few_wave_pair_launches(L):
    # 2 x 16 heads x 2 blocks of 512 rows: plenty of blocks per CTA-pair slot, no split planned
    assert L.lib.pe_attn_forward_workspace_bytes(C.byref(_valid_args(L))) == 0
    # one (batch, head) pair of problems over a long sequence: the longest blocks get split
    few = _valid_args(L, B=1, H=2, Hkv=2, Sq=8192, Sk=8192)
    n = L.lib.pe_attn_forward_workspace_bytes(C.byref(few))
    assert n > 0 and n % (2 * 512 * 129 * 4) == 0          # whole items of 2 x 512 x (128 + 1) floats
    # other kernels never use it
    assert L.lib.pe_attn_forward_workspace_bytes(C.byref(_valid_args(L, B=1, H=2, Hkv=2, Sq=8192, Sk=8192,
                                                                  flags=L.SINGLE_CTA))) == 0
    # fp32: the keys transformed once, [B][Hkv][Sk][d_qk] fp32 -- where there is a transform to repeat
    assert L.lib.pe_attn_forward_workspace_bytes(C.byref(_valid_args(L, B=1, H=2, Hkv=2, Sq=8192, Sk=8192,
                                                                  dtype=L.FP32))) == 1 * 2 * 8192 * 256 * 4
    assert L.lib.pe_attn_forward_workspace_bytes(C.byref(_valid_args(L, B=1, H=2, Hkv=2, Sq=64, Sk=8192,
                                                                  dtype=L.FP32))) == 0      # one query block
    # a misaligned workspace is refused
    bad = _valid_args(L, B=1, H=2, Hkv=2, Sq=8192, Sk=8192, workspace=0x10004, workspace_bytes=n)
    assert L.lib.pe_attn_validate(C.byref(bad)) == 4


@pytest.mark.parametrize("over,code", [
    (dict(struct_size=8), 2),
    (dict(variant=9), 2),
    (dict(dtype=5), 2),
    (dict(H=15), 3),                      # not a multiple of Hkv
    (dict(Sk=512), 3),                    # Sk < Sq
    (dict(d_v=256), 3),
    (dict(d_c=192, d_r=64), 3),           # d_qk > 256
    (dict(d_c=96, d_r=0, variant=0), 3),  # bf16 path needs 64 / 128
    (dict(q=0), 1),
    (dict(q_r=0), 1),
    (dict(freqs=0), 1),
    (dict(v=0x10008), 4),                 # not 16-byte aligned
    (dict(q_stride=(7, 128, 2048)), 4),   # stride not a multiple of 8 elements
    (dict(variant=1, d_r=0, d_c=128), 1),  # rotary without a table
    (dict(variant=2, d_r=0, d_c=128), 1),  # alibi without slopes
    (dict(flags=1), 2),                   # QK_NORM with POPE
    (dict(flags=2), 1),                   # FOURIER_MIX without coefficients
])
def test_validation_codes(L, over, code):
    a = _valid_args(L, **over)
    assert L.lib.pe_attn_validate(C.byref(a)) == code
    assert L.lib.pe_attn_last_error() != b""
    assert L.lib.pe_attn_status_string(code) not in (b"ok", b"unknown status")


def test_rotary_table_must_cover_positions(L):
    a = _valid_args(L, variant=1, d_r=0, d_c=128, rotary_table=0x20000, table_rows=1000, table_pos0=0)
    assert L.lib.pe_attn_validate(C.byref(a)) == 3
    a = _valid_args(L, variant=1, d_r=0, d_c=128, rotary_table=0x20000, table_rows=2048, table_pos0=0, q_pos0=1024,
                    k_pos0=1024)
    assert L.lib.pe_attn_validate(C.byref(a)) == 0


def test_null_args(L):
    assert L.lib.pe_attn_validate(None) == 1


def test_python_wrapper_refuses_cpu_tensors_and_masks():
    import torch
    from pe_ablations_b200 import pe_attention

    q = torch.zeros(1, 4, 2, 64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pe_attention("nope", q, q, q)
    with pytest.raises(NotImplementedError):
        pe_attention("nope", q, q, q, mask=torch.ones(1))
    with pytest.raises(ValueError):
        pe_attention("rope", q, q, q)


def _bwd_args(L, **over):
    a = L.PeAttnBwdArgs()
    a.struct_size = C.sizeof(L.PeAttnBwdArgs)
    a.B, a.H, a.Hkv, a.Sq, a.Sk, a.d_qk, a.d_v = 2, 8, 4, 512, 512, 128, 64
    a.scale = 128 ** -0.5
    for name in ("q", "k", "v", "out", "dout", "dk", "dv", "lse", "dq_accum", "dvec"):
        setattr(a, name, 0x10000)
    for s_, h, d in (("q_stride", 8, 128), ("k_stride", 4, 128), ("v_stride", 4, 64), ("out_stride", 8, 64),
                     ("dout_stride", 8, 64), ("dk_stride", 4, 128), ("dv_stride", 4, 64)):
        getattr(a, s_)[:] = (512 * h * d, d, h * d)
    for k, v in over.items():
        if k.endswith("_stride"):
            getattr(a, k)[:] = v
        else:
            setattr(a, k, v)
    return a


def test_backward_entry_rejects_bad_arguments_before_touching_the_gpu(L):
    """Only calls that fail validation: a call that validates would launch on these fake pointers."""
    bwd = L.lib.pe_attn_backward
    assert bwd(None, None) == 1
    assert bwd(C.byref(_bwd_args(L, struct_size=8)), None) == 2
    assert bwd(C.byref(_bwd_args(L, Sq=600)), None) == 3                      # Sk < Sq
    assert bwd(C.byref(_bwd_args(L, H=6)), None) == 3                         # H % Hkv
    assert bwd(C.byref(_bwd_args(L, d_qk=264)), None) == 3                    # beyond every backward kernel
    assert b"(64,64), (128,64), (128,128)" in L.lib.pe_attn_last_error()
    assert bwd(C.byref(_bwd_args(L, d_qk=100)), None) == 3                    # not a multiple of 8
    assert bwd(C.byref(_bwd_args(L, dtype=7)), None) == 2                     # unknown dtype
    assert bwd(C.byref(_bwd_args(L, dtype=1, d_qk=264)), None) == 3           # fp32: the same head dims
    assert bwd(C.byref(_bwd_args(L, dout=None)), None) == 1
    assert bwd(C.byref(_bwd_args(L, dk=0x10008)), None) == 4
    assert bwd(C.byref(_bwd_args(L, q_stride=(512 * 8 * 128, 130, 8 * 128))), None) == 4
    assert bwd(C.byref(_bwd_args(L, lse=None)), None) == 1


def test_transform_entries_reject_bad_shapes(L):
    s3 = (C.c_int64 * 3)(512 * 8 * 32, 32, 8 * 32)
    rc = L.lib.pe_pope_expand(None, s3, 0x10000, s3, 0x10000, s3, 1, 512, 8, 0, 48, 0, 0x10000, None, None)
    assert rc == 3 and b"d_r must be 32 or 64" in L.lib.pe_attn_last_error()
    rc = L.lib.pe_pope_expand(None, s3, None, s3, 0x10000, s3, 1, 512, 8, 0, 32, 0, 0x10000, None, None)
    assert rc == 1
    rc = L.lib.pe_rotary_norm_expand(0x10000, s3, 0x10000, s3, 1, 512, 8, 96, None, 0, 0, 1.0, 1, 1e-6, None)
    assert rc == 3
    rc = L.lib.pe_rotary_norm_expand(0x10000, s3, 0x10000, s3, 1, 512, 8, 64, 0x10000, 10, 100, 1.0, 1, 1e-6, None)
    assert rc == 3 and b"do not cover" in L.lib.pe_attn_last_error()


def test_decode_entry_plans_and_rejects_without_touching_the_gpu(L):
    """``pe_attn_decode_workspace_bytes`` is host arithmetic; ``pe_attn_decode`` refuses a null
    workspace and calls that are not decode steps before any launch."""
    one_token = _valid_args(L, Sq=1, Sk=16384)
    n = L.lib.pe_attn_decode_workspace_bytes(C.byref(one_token))
    rows = 2 * 16
    assert n > 0 and n % (rows * (128 + 2) * 4) == 0           # rows x splits x (d_v + max + sum) floats
    splits = n // (rows * (128 + 2) * 4)
    assert 1 <= splits <= 64 and splits * 2 * 16 <= 296        # about two CTAs per SM
    assert L.lib.pe_attn_decode_workspace_bytes(C.byref(_valid_args(L, Sq=1, Sk=1))) == rows * 130 * 4
    # too many rows per K/V head, fp32, invalid arguments
    assert L.lib.pe_attn_decode_workspace_bytes(C.byref(_valid_args(L, Sq=9, Sk=1024))) == 0
    assert b"at most 8 query rows" in L.lib.pe_attn_last_error()
    assert L.lib.pe_attn_decode_workspace_bytes(C.byref(_valid_args(L, Sq=1, dtype=L.FP32))) == 0
    assert L.lib.pe_attn_decode_workspace_bytes(C.byref(_valid_args(L, Sq=1, Hkv=3))) == 0
    assert L.lib.pe_attn_decode_workspace_bytes(None) == 0
    assert L.lib.pe_attn_decode(C.byref(one_token), None, 0, None) == 1            # null workspace
    assert L.lib.pe_attn_decode(C.byref(_valid_args(L, Sq=9)), None, 0, None) == 3  # shape
    assert L.lib.pe_attn_decode(None, None, 0, None) == 1


def test_fused_gemm_entries_plan_and_reject_without_touching_the_gpu(L):
    """The head + cross-entropy workspace is host arithmetic; all three GEMM entry points check
    pointers, shapes and alignment before any CUDA call."""
    ws = L.lib.pe_lm_head_ce_workspace_bytes
    # counter block + row losses + target logits + (max, sum) per row and 256 vocabulary entries
    assert ws(16383, 32000) == 256 + 2 * 16384 * 4 + 125 * 16384 * 8
    assert ws(1, 1) == 256 + 2 * 1024 + 256 * 8 and ws(0, 32000) == 0 and ws(16, 0) == 0
    head = L.lib.pe_lm_head_ce_loss_sums
    ok = dict(h=0x10000, hs=2048, w=0x20000, wsd=2048, t=0x30000, n=512, k=2048, v=32000, ig=-100, buf=0x40000,
              nbytes=ws(512, 32000), out=0x50000)

    def call(**over):
        a = dict(ok, **over)
        return head(a["h"], a["hs"], a["w"], a["wsd"], a["t"], a["n"], a["k"], a["v"], a["ig"], a["buf"], a["nbytes"],
                    a["out"], None, None)

    assert call(t=None) == 1 and call(buf=None) == 1 and call(out=None) == 1 and call(h=None) == 1
    assert call(n=0) == 3 and call(k=100) == 3 and call(k=56, hs=56, wsd=56) == 3 and call(v=0) == 3
    assert call(hs=2044) == 4 and call(h=0x10008) == 4 and call(buf=0x40010) == 4 and call(hs=1024) == 4
    assert call(nbytes=ws(512, 32000) - 1) == 3 and b"smaller than" in L.lib.pe_attn_last_error()
    sw = L.lib.pe_swiglu_gemm
    assert sw(0x10000, 2048, 0x20000, 0x30000, 2048, None, 5632, 256, 2048, 5632, None, None) == 1
    assert sw(0x10000, 2048, 0x20000, None, 2048, 0x40000, 5632, 256, 2048, 5632, None, None) == 1
    assert sw(0x10000, 2048, 0x20000, 0x30000, 2048, 0x40000, 5632, 0, 2048, 5632, None, None) == 3
    assert sw(0x10000, 2048, 0x20000, 0x30000, 2048, 0x40000, 5630, 256, 2048, 5632, None, None) == 4
    nt = L.lib.pe_gemm_nt
    assert nt(0x10000, 2048, 0x20000, 2048, None, 512, None, 0, 256, 512, 2048, None, None) == 1
    assert nt(0x10000, 2048, 0x20000, 2048, 0x30000, 512, None, 0, 256, 500, 2048, None, None) == 3
    assert nt(0x10004, 2048, 0x20000, 2048, 0x30000, 512, None, 0, 256, 512, 2048, None, None) == 4
    assert nt(0x10000, 2048, 0x20000, 2048, 0x30000, 512, 0x40000, 510, 256, 512, 2048, None, None) == 4   # residual stride
