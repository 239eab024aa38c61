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
    return sorted(set(re.findall(r"\b(pe_attn_[a-z_]+)\s*\(", text)))


def test_exports_every_declared_symbol(L):
    names = _declared_functions()
    assert "pe_attn_forward" in names and len(names) >= 7
    for n in names:
        assert hasattr(L.lib, n), n
    assert L.lib.pe_attn_version() == 2


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
    assert L.lib.pe_attn_kernel_name(C.byref(_valid_args(L, d_c=64, d_r=32, d_v=64))) == b"tcgen05"
    a = _valid_args(L, dtype=L.FP32)
    assert L.lib.pe_attn_kernel_name(C.byref(a)) == b"ffma"
    fl = L.lib.pe_attn_flops(C.byref(a))
    assert abs(fl - 2 * 16 * (1024 * 1025 / 2) * 2 * 384) < 1e-3 * fl


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
