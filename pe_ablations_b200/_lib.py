"""ctypes binding of the C ABI declared in include/pe_attn.h.

The library is loaded from the package directory (built in-tree by
``pe_ablations_b200.build_ext``).  There is no fallback: if the shared library
is missing or a symbol is absent, importing this module raises.
"""

from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libpe_attn.so")

# enums (include/pe_attn.h)
NOPE, ROTARY, ALIBI, POPE = 0, 1, 2, 3
BF16, FP32 = 0, 1
QK_NORM = 1 << 0
FOURIER_MIX = 1 << 1
FOURIER_NORMALIZE = 1 << 2
FOURIER_CEILING = 1 << 3
TABLE_GEOMETRIC = 1 << 4
SIMT_CHECK = 1 << 8
SINGLE_CTA = 1 << 9

EXPORTS = (
    "pe_attn_version", "pe_attn_forward", "pe_attn_validate", "pe_attn_kernel_name",
    "pe_attn_last_error", "pe_attn_status_string", "pe_attn_flops",
    "pe_ce_scratch_bytes", "pe_ce_loss_sums", "pe_ce_static_max_rows", "pe_ce_loss_sums_static",
    "pe_rmsnorm_forward", "pe_swiglu_forward", "pe_attn_selftest_wait_expiry", "pe_attn_backward",
    "pe_pope_expand", "pe_pope_expand_backward", "pe_rotary_norm_expand", "pe_rotary_norm_expand_backward",
    "pe_fope_effective_freqs", "pe_fope_effective_freqs_backward",
    "pe_attn_decode_workspace_bytes", "pe_attn_decode", "pe_attn_forward_workspace_bytes",
    "pe_lm_head_ce_workspace_bytes", "pe_lm_head_ce_loss_sums", "pe_swiglu_gemm", "pe_gemm_nt",
)


class PeAttnArgs(C.Structure):
    """Mirror of ``struct pe_attn_args``."""

    _fields_ = [
        ("struct_size", C.c_uint32), ("variant", C.c_int32), ("dtype", C.c_int32), ("flags", C.c_uint32),
        ("B", C.c_int32), ("H", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32), ("Sk", C.c_int32),
        ("d_c", C.c_int32), ("d_r", C.c_int32), ("d_v", C.c_int32), ("q_pos0", C.c_int32), ("k_pos0", C.c_int32),
        ("scale", C.c_float), ("qk_norm_eps", C.c_float), ("mscale", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("q_r", C.c_void_p), ("k_r", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("out_stride", C.c_int64 * 3), ("qr_stride", C.c_int64 * 3), ("kr_stride", C.c_int64 * 3),
        ("rotary_table", C.c_void_p), ("table_pos0", C.c_int32), ("table_rows", C.c_int32),
        ("alibi_slopes", C.c_void_p), ("freqs", C.c_void_p), ("delta", C.c_void_p),
        ("fourier_coeffs", C.c_void_p), ("n_fourier", C.c_int32), ("floor_freq", C.c_float),
        ("ceil_freq", C.c_float), ("device_status", C.c_void_p), ("lse", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_uint64),
    ]


class PeAttnBwdArgs(C.Structure):
    """Mirror of ``struct pe_attn_bwd_args``."""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("B", C.c_int32), ("H", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32), ("Sk", C.c_int32),
        ("d_qk", C.c_int32), ("d_v", C.c_int32), ("scale", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("dout", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("out_stride", C.c_int64 * 3), ("dout_stride", C.c_int64 * 3),
        ("lse", C.c_void_p), ("alibi_slopes", C.c_void_p), ("dq_accum", C.c_void_p),
        ("dk", C.c_void_p), ("dv", C.c_void_p), ("dk_stride", C.c_int64 * 3), ("dv_stride", C.c_int64 * 3),
        ("dvec", C.c_void_p), ("device_status", C.c_void_p), ("dtype", C.c_int32),
    ]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m pe_ablations_b200.build_ext` "
            "(there is no fallback implementation)")
    lib = C.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(lib, name):
            raise ImportError(f"{LIB_PATH} does not export {name}")
    lib.pe_attn_version.restype = C.c_int
    lib.pe_attn_forward.restype = C.c_int
    lib.pe_attn_forward.argtypes = [C.POINTER(PeAttnArgs), C.c_void_p]
    lib.pe_attn_forward_workspace_bytes.restype = C.c_size_t
    lib.pe_attn_forward_workspace_bytes.argtypes = [C.POINTER(PeAttnArgs)]
    lib.pe_attn_decode_workspace_bytes.restype = C.c_size_t
    lib.pe_attn_decode_workspace_bytes.argtypes = [C.POINTER(PeAttnArgs)]
    lib.pe_attn_decode.restype = C.c_int
    lib.pe_attn_decode.argtypes = [C.POINTER(PeAttnArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.pe_attn_validate.restype = C.c_int
    lib.pe_attn_validate.argtypes = [C.POINTER(PeAttnArgs)]
    lib.pe_attn_kernel_name.restype = C.c_char_p
    lib.pe_attn_kernel_name.argtypes = [C.POINTER(PeAttnArgs)]
    lib.pe_attn_last_error.restype = C.c_char_p
    lib.pe_attn_status_string.restype = C.c_char_p
    lib.pe_attn_status_string.argtypes = [C.c_int]
    lib.pe_attn_flops.restype = C.c_double
    lib.pe_attn_flops.argtypes = [C.POINTER(PeAttnArgs)]
    lib.pe_ce_scratch_bytes.restype = C.c_size_t
    lib.pe_ce_scratch_bytes.argtypes = [C.c_int]
    lib.pe_ce_loss_sums.restype = C.c_int
    lib.pe_ce_loss_sums.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                    C.c_void_p, C.c_void_p, C.c_void_p]
    lib.pe_rmsnorm_forward.restype = C.c_int
    lib.pe_rmsnorm_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64,
                                       C.c_int64, C.c_float, C.c_void_p]
    lib.pe_swiglu_forward.restype = C.c_int
    lib.pe_swiglu_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_void_p]
    lib.pe_attn_selftest_wait_expiry.restype = C.c_int
    lib.pe_attn_selftest_wait_expiry.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
    lib.pe_attn_backward.restype = C.c_int
    lib.pe_attn_backward.argtypes = [C.POINTER(PeAttnBwdArgs), C.c_void_p]
    S3 = C.POINTER(C.c_int64)
    lib.pe_pope_expand.restype = C.c_int
    lib.pe_pope_expand.argtypes = [C.c_void_p, S3, C.c_void_p, S3, C.c_void_p, S3, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.pe_pope_expand_backward.restype = C.c_int
    lib.pe_pope_expand_backward.argtypes = [C.c_void_p, C.c_int, S3, C.c_void_p, S3, C.c_void_p, S3, C.c_void_p, S3,
                                            C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.pe_fope_effective_freqs.restype = C.c_int
    lib.pe_fope_effective_freqs.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_uint, C.c_float, C.c_float,
                                            C.c_void_p, C.c_void_p]
    lib.pe_fope_effective_freqs_backward.restype = C.c_int
    lib.pe_fope_effective_freqs_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_uint, C.c_float,
                                                     C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.pe_rotary_norm_expand.restype = C.c_int
    lib.pe_rotary_norm_expand.argtypes = [C.c_void_p, S3, C.c_void_p, S3, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.c_float, C.c_void_p]
    lib.pe_rotary_norm_expand_backward.restype = C.c_int
    lib.pe_rotary_norm_expand_backward.argtypes = [C.c_void_p, C.c_int, S3, C.c_void_p, S3, C.c_void_p, S3, C.c_int,
                                                   C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_float,
                                                   C.c_int, C.c_float, C.c_void_p]
    lib.pe_lm_head_ce_workspace_bytes.restype = C.c_size_t
    lib.pe_lm_head_ce_workspace_bytes.argtypes = [C.c_int, C.c_int]
    lib.pe_lm_head_ce_loss_sums.restype = C.c_int
    lib.pe_lm_head_ce_loss_sums.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int,
                                            C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p,
                                            C.c_void_p]
    lib.pe_swiglu_gemm.restype = C.c_int
    lib.pe_swiglu_gemm.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                   C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    lib.pe_gemm_nt.restype = C.c_int
    lib.pe_gemm_nt.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                               C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    lib.pe_ce_static_max_rows.restype = C.c_int
    lib.pe_ce_loss_sums_static.restype = C.c_int
    lib.pe_ce_loss_sums_static.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                           C.c_void_p, C.c_void_p]
    return lib


lib = _load()


class PeAttnError(RuntimeError):
    """A non-zero status from the C ABI."""

    def __init__(self, status: int):
        self.status = status
        name = lib.pe_attn_status_string(status).decode()
        msg = lib.pe_attn_last_error().decode()
        super().__init__(f"pe_attn status {status} ({name}): {msg}")
