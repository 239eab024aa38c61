"""Python entry point of the fused PE-attention forward (calls the C ABI).

``pe_attention`` takes the projected tensors exactly as the reference's
attention modules hold them before their positional transform -- layout
[B, S, H, d] (or [B, H, S, d] with ``layout="bhsd"``), any strides with a
contiguous last dimension -- and returns the attention output in the same
layout.  It replaces, per variant, the eager code listed in include/pe_attn.h.

There is no CPU or eager fallback: CPU tensors, a mask, or tensors that need
gradients raise.
"""

from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib

_VARIANTS = {"nope": _lib.NOPE, "rotary": _lib.ROTARY, "alibi": _lib.ALIBI, "pope": _lib.POPE}
_status_words: dict[int, torch.Tensor] = {}      # one int32 word per device, for all streams


_raw_stream_fn = getattr(torch._C, "_cuda_getCurrentRawStream", None)


class _on_device:
    """``with _on_device(dev) as stream``: makes ``dev`` the current CUDA device for the C call if
    it is not already (the library launches on the current device) and yields the raw handle of
    torch's current stream there.  The host side of a call is a few microseconds this way; the
    generic ``torch.cuda.device`` / ``current_stream`` objects cost several times that, which a
    training step of small kernels (CPU-bound at the reference's shape) pays per launch.

    Temporaries created inside a wrapper (fp32 copies of parameters, workspaces) are allocated on
    the same current stream the kernel is launched on, so the caching allocator already orders
    their reuse behind the kernel: no ``record_stream`` is needed for them."""

    __slots__ = ("idx", "prev")

    def __init__(self, device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self) -> int:
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        if _raw_stream_fn is not None:
            return _raw_stream_fn(self.idx)
        return torch.cuda.current_stream(self.idx).cuda_stream

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def device_status(device: torch.device) -> torch.Tensor:
    """The int32 word of ``device`` that the tensor-core kernels OR a code into when a bounded
    wait runs out.  One word per device serves every stream (the kernels only ever OR into it).

    It is created, zeroed and waited for on first use; that first use must not happen during
    CUDA-graph capture (the zeroing would be recorded and every replay would wipe the previous
    replay's report), so capture raises until one eager call has been made on the device.
    """
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the first pe_attn call on a device creates its status word and cannot be captured "
                               "into a CUDA graph: run one eager call on this device before capturing")
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        torch.cuda.current_stream(idx).synchronize()      # visible to every stream from here on
        _status_words[idx] = w
    return w


def poll_device_status(device: torch.device | None = None) -> int:
    """Synchronise ``device`` (default: every device used so far) and return the OR of the status
    words, leaving them as they are.  0 means that no kernel reported an expired wait."""
    code = 0
    for idx, w in list(_status_words.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        torch.cuda.synchronize(idx)
        code |= int(w.item()) & 0xFFFFFFFF
    return code


def check_device_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if any kernel on ``device`` reported an expired wait.

    A non-zero word makes every later tensor-core launch on the device return without writing
    its output, so results produced after the expiry are garbage until this is called: it
    clears the word and raises.  The library calls it wherever it synchronises with the host
    anyway (``eval.reduce_loss_sums``, ``HostStreamedAttention.synchronize``); code that calls
    ``pe_attention`` or the modules directly calls it once per step, where it reads its result.
    """
    code = poll_device_status(device)
    if code != 0:
        for idx, w in list(_status_words.items()):
            if device is None or torch.device(device).index in (None, idx):
                w.zero_()
        raise RuntimeError(f"pe_attn tensor-core kernel reported expired waits, code 0x{code:x}; every output "
                           "produced on this device since the last check is invalid")


def _strides(t: torch.Tensor, layout: str) -> tuple[int, int, int]:
    sb, s1, s2, s3 = t.stride()
    if s3 != 1:
        raise ValueError("the last dimension must be contiguous")
    return (sb, s2, s1) if layout == "bshd" else (sb, s1, s2)


def _dims(t: torch.Tensor, layout: str) -> tuple[int, int, int, int]:
    B, a, b, d = t.shape
    return (B, b, a, d) if layout == "bshd" else (B, a, b, d)  # B, H, S, d


def _f32(t: torch.Tensor | None, device) -> torch.Tensor | None:
    if t is None:
        return None
    if t.dtype == torch.float32 and t.device == device and t.is_contiguous():
        return t.detach() if t.requires_grad else t
    return t.detach().to(device=device, dtype=torch.float32).contiguous()


def pe_attention(
    variant: str,
    q: torch.Tensor | None,
    k: torch.Tensor | None,
    v: torch.Tensor,
    *,
    q_r: torch.Tensor | None = None,
    k_r: torch.Tensor | None = None,
    layout: str = "bshd",
    start_pos: int = 0,
    k_start_pos: int | None = None,
    scale: float | None = None,
    qk_norm: bool = False,
    qk_norm_eps: float = 1e-6,
    rotary_table: torch.Tensor | None = None,
    table_pos0: int = 0,
    table_geometric: bool = False,
    mscale: float = 1.0,
    alibi_slopes: torch.Tensor | None = None,
    freqs: torch.Tensor | None = None,
    delta: torch.Tensor | None = None,
    fourier_coeffs: torch.Tensor | None = None,
    floor_freq: float = 0.0,
    normalize_coeffs: bool = True,
    ceil_freq: float | None = None,
    out: torch.Tensor | None = None,
    mask: torch.Tensor | None = None,
    simt_check: bool = False,
    single_cta: bool = False,
    lse: torch.Tensor | None = None,
    split_kv: bool | None = None,
    split_blocks: bool = True,
) -> torch.Tensor:
    """Fused causal attention forward with the positional transform applied in-kernel.

    variant: ``nope`` | ``rotary`` | ``alibi`` | ``pope``.
      rotary: ``rotary_table`` is [rows, d/2, 2] fp32 (cos, sin), row i = position
              ``table_pos0 + i`` (``torch.view_as_real`` of the reference's ``freqs_cis``);
              ``table_geometric`` says that row i holds the angles i * angle_c (true for every
              table the reference builds), which lets the decode kernel advance a key's rotation
              from tile to tile instead of reading the table row of every key.
      alibi:  ``alibi_slopes`` is [H].
      pope:   ``q``/``k`` are the content halves (or None), ``q_r``/``k_r`` the position
              halves before softplus; ``freqs`` [d_r] effective frequencies, or base
              frequencies together with ``fourier_coeffs`` [d_r, D_f] (the FoPE mix and the
              ``floor_freq`` clip then run inside the kernel); ``delta`` [d_r] raw phase bias.
    lse: optional fp32 [B, H, Sq] tensor that receives each row's logsumexp (natural log of the
         sum of exp(scaled logit + bias) over the visible keys), for a later backward.
    split_kv: decode steps (bf16, at most 8 query rows per K/V head, i.e. H / Hkv * Sq <= 8) go to
         the split-KV kernel, which streams the cached keys with the whole GPU instead of one
         CTA per head.  None picks it for such calls when Sk >= 256; True requires it (raises
         if the call is not of that shape); False keeps the query-tiled kernels.
    split_blocks: let a launch with few (batch, head) problems cut its longest query blocks in two
         along the keys (a scratch tensor for the partial results is allocated for the call).
    """
    if mask is not None:
        raise NotImplementedError("pe_attention is causal-only: an explicit mask is not supported (no fallback)")
    kwargs = dict(layout=layout, start_pos=start_pos, k_start_pos=k_start_pos, scale=scale, qk_norm=qk_norm,
                  qk_norm_eps=qk_norm_eps, rotary_table=rotary_table, table_pos0=table_pos0,
                  table_geometric=table_geometric, mscale=mscale,
                  alibi_slopes=alibi_slopes, floor_freq=floor_freq, normalize_coeffs=normalize_coeffs,
                  ceil_freq=ceil_freq, out=out, simt_check=simt_check, single_cta=single_cta, split_kv=split_kv,
                  split_blocks=split_blocks)
    diff = (q, k, v, q_r, k_r, freqs, delta, fourier_coeffs)
    if torch.is_grad_enabled() and any(isinstance(t, torch.Tensor) and t.requires_grad for t in diff):
        return _training_call(variant, q, k, v, q_r, k_r, freqs, delta, fourier_coeffs, lse, kwargs)
    return _forward_impl(variant, q, k, v, q_r=q_r, k_r=k_r, freqs=freqs, delta=delta, fourier_coeffs=fourier_coeffs,
                         lse=lse, **kwargs)


def _training_call(variant, q, k, v, q_r, k_r, freqs, delta, fourier_coeffs, lse, kw):
    """Route a call that needs gradients through ``autograd.FusedAttentionFunction``."""
    from .autograd import FusedAttentionFunction

    if variant not in _VARIANTS:
        raise ValueError(f"unknown variant {variant!r}")
    if v.dtype not in (torch.bfloat16, torch.float32) or not v.is_cuda:
        raise NotImplementedError("gradients are implemented for bf16 and fp32 CUDA tensors; there is no eager "
                                  "fallback")
    if kw["layout"] != "bshd" or kw["out"] is not None or lse is not None or kw["simt_check"]:
        raise NotImplementedError("a call that needs gradients takes [B, S, H, d] tensors and owns its outputs")
    d_qk = (q.shape[-1] if q is not None else 0) + (2 * q_r.shape[-1] if q_r is not None else 0)
    if v.dtype == torch.bfloat16 and (d_qk not in (64, 128, 192, 256) or v.shape[-1] not in (64, 128)):
        raise NotImplementedError(f"gradients need d_qk in (64, 128, 192, 256) and d_v in (64, 128) -- the bf16 forward's "
                                  f"head dims; got ({d_qk}, {v.shape[-1]})")
    if v.dtype == torch.float32 and (d_qk % 8 or v.shape[-1] % 8 or d_qk > 256 or v.shape[-1] > 128):
        raise NotImplementedError(f"fp32 gradients need d_qk <= 256 and d_v <= 128 in steps of 8; got ({d_qk}, {v.shape[-1]})")
    dev = v.device
    k_start = kw["start_pos"] if kw["k_start_pos"] is None else kw["k_start_pos"]
    tab = kw["rotary_table"]
    if tab is not None:
        tab = _f32(torch.view_as_real(tab) if tab.is_complex() else tab, dev)
    o = dict(forward_kwargs={n: kw[n] for n in kw if n not in ("out",)}, start_pos=int(kw["start_pos"]),
             k_start_pos=int(k_start), table_pos0=int(kw["table_pos0"]), mscale=float(kw["mscale"]),
             qk_norm=bool(kw["qk_norm"]), qk_norm_eps=float(kw["qk_norm_eps"]), rotary_table=tab,
             normalize_coeffs=bool(kw["normalize_coeffs"]), floor_freq=float(kw["floor_freq"]),
             ceil_freq=kw["ceil_freq"], scale=float(kw["scale"]) if kw["scale"] is not None else d_qk ** -0.5,
             alibi_slopes=kw["alibi_slopes"] if variant == "alibi" else None)
    on_dev = lambda t: None if t is None else (t if t.device == dev else t.to(dev))
    return FusedAttentionFunction.apply(variant, o, q, k, v, q_r, k_r, on_dev(freqs), on_dev(delta),
                                        on_dev(fourier_coeffs))


def _forward_impl(
    variant: str,
    q: torch.Tensor | None,
    k: torch.Tensor | None,
    v: torch.Tensor,
    *,
    q_r: torch.Tensor | None = None,
    k_r: torch.Tensor | None = None,
    layout: str = "bshd",
    start_pos: int = 0,
    k_start_pos: int | None = None,
    scale: float | None = None,
    qk_norm: bool = False,
    qk_norm_eps: float = 1e-6,
    rotary_table: torch.Tensor | None = None,
    table_pos0: int = 0,
    table_geometric: bool = False,
    mscale: float = 1.0,
    alibi_slopes: torch.Tensor | None = None,
    freqs: torch.Tensor | None = None,
    delta: torch.Tensor | None = None,
    fourier_coeffs: torch.Tensor | None = None,
    floor_freq: float = 0.0,
    normalize_coeffs: bool = True,
    ceil_freq: float | None = None,
    out: torch.Tensor | None = None,
    simt_check: bool = False,
    single_cta: bool = False,
    lse: torch.Tensor | None = None,
    split_kv: bool | None = None,
    split_blocks: bool = True,
) -> torch.Tensor:
    """The forward kernel call behind ``pe_attention`` (no autograd bookkeeping)."""
    if variant not in _VARIANTS:
        raise ValueError(f"unknown variant {variant!r}")
    if layout not in ("bshd", "bhsd"):
        raise ValueError("layout must be 'bshd' or 'bhsd'")
    ref = v
    if not ref.is_cuda:
        raise RuntimeError("pe_attention needs CUDA tensors: there is no CPU path")
    if ref.dtype == torch.bfloat16:
        dtype = _lib.BF16
    elif ref.dtype == torch.float32:
        dtype = _lib.FP32
    else:
        raise TypeError(f"unsupported dtype {ref.dtype}")
    for t in (q, k, q_r, k_r):
        if t is not None and (t.dtype != ref.dtype or t.device != ref.device):
            raise TypeError("all tensors must share dtype and device")

    a = _lib.PeAttnArgs()
    a.struct_size = C.sizeof(_lib.PeAttnArgs)
    a.variant = _VARIANTS[variant]
    a.dtype = dtype
    flags = 0
    B, Hkv, Sk, d_v = _dims(v, layout)
    qq = q if q is not None else q_r
    if qq is None:
        raise ValueError("q or q_r is required")
    _, H, Sq, _ = _dims(qq, layout)
    a.B, a.H, a.Hkv, a.Sq, a.Sk = B, H, Hkv, Sq, Sk
    a.d_c = q.shape[-1] if q is not None else 0
    a.d_r = q_r.shape[-1] if q_r is not None else 0
    a.d_v = d_v
    a.q_pos0 = int(start_pos)
    a.k_pos0 = int(start_pos if k_start_pos is None else k_start_pos)
    d_qk = a.d_c + 2 * a.d_r
    a.scale = float(scale) if scale is not None else d_qk ** -0.5
    a.qk_norm_eps = float(qk_norm_eps)
    a.mscale = float(mscale)
    if qk_norm:
        flags |= _lib.QK_NORM

    if out is None:
        shape = (B, Sq, H, d_v) if layout == "bshd" else (B, H, Sq, d_v)
        out = torch.empty(shape, dtype=ref.dtype, device=ref.device)
    keep = [out]

    if q is not None:
        a.q, a.q_stride[:] = q.data_ptr(), _strides(q, layout)
    if k is not None:
        a.k, a.k_stride[:] = k.data_ptr(), _strides(k, layout)
    a.v, a.v_stride[:] = v.data_ptr(), _strides(v, layout)
    a.out, a.out_stride[:] = out.data_ptr(), _strides(out, layout)
    if q_r is not None:
        a.q_r, a.qr_stride[:] = q_r.data_ptr(), _strides(q_r, layout)
    if k_r is not None:
        a.k_r, a.kr_stride[:] = k_r.data_ptr(), _strides(k_r, layout)
    if lse is not None:
        if lse.dtype != torch.float32 or lse.shape != (B, H, Sq) or not lse.is_contiguous() or lse.device != ref.device:
            raise ValueError("lse must be a contiguous fp32 [B, H, Sq] tensor on the inputs' device")
        a.lse = lse.data_ptr()

    dev = ref.device
    if variant == "rotary":
        if rotary_table is None:
            raise ValueError("rotary needs rotary_table")
        tab = rotary_table
        if tab.is_complex():
            tab = torch.view_as_real(tab)
        tab = _f32(tab, dev)
        keep.append(tab)
        a.rotary_table = tab.data_ptr()
        a.table_pos0 = int(table_pos0)
        a.table_rows = tab.shape[0]
        if table_geometric:
            flags |= _lib.TABLE_GEOMETRIC
    if variant == "alibi":
        sl = _f32(alibi_slopes.reshape(-1), dev)
        keep.append(sl)
        a.alibi_slopes = sl.data_ptr()
    if variant == "pope":
        fr = _f32(freqs, dev)
        keep.append(fr)
        a.freqs = fr.data_ptr()
        if delta is not None:
            dl = _f32(delta, dev)
            keep.append(dl)
            a.delta = dl.data_ptr()
        if fourier_coeffs is not None:
            co = _f32(fourier_coeffs, dev)
            keep.append(co)
            a.fourier_coeffs = co.data_ptr()
            a.n_fourier = co.shape[1]
            flags |= _lib.FOURIER_MIX
            if normalize_coeffs:
                flags |= _lib.FOURIER_NORMALIZE
            a.floor_freq = float(floor_freq)
            if ceil_freq is not None:
                flags |= _lib.FOURIER_CEILING
                a.ceil_freq = float(ceil_freq)
    if simt_check:
        flags |= _lib.SIMT_CHECK
    if single_cta:
        flags |= _lib.SINGLE_CTA
    a.flags = flags
    with _on_device(dev) as stream:
        if dtype == _lib.BF16 and not simt_check:
            a.device_status = device_status(dev).data_ptr()
        use_split = False
        if split_kv or (split_kv is None and dtype == _lib.BF16 and not simt_check and not single_cta
                        and (H // max(Hkv, 1)) * Sq <= 8 and Sk >= 256):
            ws_bytes = _lib.lib.pe_attn_decode_workspace_bytes(C.byref(a))
            use_split = ws_bytes > 0
            if split_kv and not use_split:
                raise _lib.PeAttnError(_lib.lib.pe_attn_decode(C.byref(a), None, 0, C.c_void_p(stream)))
        if use_split:
            # partial outputs of the key splits; a fresh block from the caching allocator is
            # ordered after its previous use on this stream
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            rc = _lib.lib.pe_attn_decode(C.byref(a), C.c_void_p(ws.data_ptr()), C.c_size_t(ws_bytes), C.c_void_p(stream))
        else:
            # few-wave launches of the CTA-pair kernel split their longest query blocks along the
            # keys when given scratch for the partial results; fp32 calls transform their keys once
            # into scratch instead of once per query block (stream-ordered, from the allocator)
            fwd_ws = (_lib.lib.pe_attn_forward_workspace_bytes(C.byref(a))
                      if ((dtype == _lib.BF16 and split_blocks) or dtype == _lib.FP32) else 0)
            if fwd_ws > 0:
                ws = torch.empty(fwd_ws, dtype=torch.uint8, device=dev)
                a.workspace, a.workspace_bytes = ws.data_ptr(), fwd_ws
            rc = _lib.lib.pe_attn_forward(C.byref(a), C.c_void_p(stream))
    if rc != 0:
        raise _lib.PeAttnError(rc)
    del keep   # parameter copies created here were allocated on the launch stream (see _on_device)
    return out


def attention_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, dout: torch.Tensor,
                       lse: torch.Tensor, *, scale: float, alibi_slopes: torch.Tensor | None = None
                       ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of ``softmax_causal(scale q k^T + bias) v`` for transformed operands.

    bf16 with (d_qk, d_v) in {(64,64), (128,64), (128,128)} runs on the tensor cores; any other
    multiples of 8 up to (256, 128) -- the 1B shape's (256, 128) -- and every fp32 call on the CUDA
    cores (FFMA kernels).

    q [B,Sq,H,d_qk], k [B,Sk,Hkv,d_qk], v [B,Sk,Hkv,d_v], out / dout [B,Sq,H,d_v] (all bf16 or all
    fp32, last dimension contiguous), ``lse`` the forward's [B,H,Sq] logsumexp.  Returns
    ``(dq fp32 [B,Sq,H,d_qk], dk like k, dv like v)``; dq is the accumulation buffer the kernel
    adds into.
    """
    dtype = q.dtype
    if dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"attention_backward needs bf16 or fp32 tensors (got {dtype})")
    for t in (q, k, v, out, dout):
        if not t.is_cuda or t.dtype != dtype:
            raise TypeError("attention_backward needs CUDA tensors of one dtype (there is no other path)")
    B, Sq, H, d_qk = q.shape
    _, Sk, Hkv, d_v = v.shape
    dev = q.device
    if lse.dtype != torch.float32 or lse.shape != (B, H, Sq) or not lse.is_contiguous():
        raise ValueError("lse must be a contiguous fp32 [B, H, Sq] tensor")
    # TMA wants a 16-byte aligned base and strides that are multiples of 16 bytes
    tma_ok = lambda t: (t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:-1]))
    q, k, v, out, dout = (t if tma_ok(t) else t.contiguous() for t in (q, k, v, out, dout))
    a = _lib.PeAttnBwdArgs()
    a.struct_size = C.sizeof(_lib.PeAttnBwdArgs)
    a.B, a.H, a.Hkv, a.Sq, a.Sk, a.d_qk, a.d_v = B, H, Hkv, Sq, Sk, d_qk, d_v
    a.scale = float(scale)
    dq_accum = torch.empty(B, Sq, H, d_qk, dtype=torch.float32, device=dev)
    dvec = torch.empty(B, H, Sq, dtype=torch.float32, device=dev)
    dk = torch.empty(B, Sk, Hkv, d_qk, dtype=dtype, device=dev)
    dv = torch.empty(B, Sk, Hkv, d_v, dtype=dtype, device=dev)
    a.dtype = _lib.BF16 if dtype == torch.bfloat16 else _lib.FP32
    for name, sname, t in (("q", "q_stride", q), ("k", "k_stride", k), ("v", "v_stride", v), ("out", "out_stride", out),
                           ("dout", "dout_stride", dout), ("dk", "dk_stride", dk), ("dv", "dv_stride", dv)):
        setattr(a, name, t.data_ptr())
        getattr(a, sname)[:] = _strides(t, "bshd")
    a.lse, a.dq_accum, a.dvec = lse.data_ptr(), dq_accum.data_ptr(), dvec.data_ptr()
    keep = []
    if alibi_slopes is not None:
        sl = _f32(alibi_slopes.reshape(-1), dev)
        keep.append(sl)
        a.alibi_slopes = sl.data_ptr()
    with _on_device(dev) as stream:
        a.device_status = device_status(dev).data_ptr()
        rc = _lib.lib.pe_attn_backward(C.byref(a), C.c_void_p(stream))
    if rc != 0:
        raise _lib.PeAttnError(rc)
    return dq_accum, dk, dv


def _s3(t: torch.Tensor | None):
    arr = (C.c_int64 * 3)()
    if t is not None:
        arr[:] = _strides(t, "bshd")
    return arr


def pope_expand(x_c: torch.Tensor | None, x_r: torch.Tensor, pos0: int, omega: torch.Tensor,
                delta: torch.Tensor | None) -> torch.Tensor:
    """[x_c | softplus(x_r) cos(phi) | softplus(x_r) sin(phi)] as one bf16 [B,S,H,d_c+2d_r] tensor
    (phi = pos * omega + clamp(delta, -2 pi, 0)): the operands the backward kernel reads."""
    B, S, H, d_r = x_r.shape
    d_c = 0 if x_c is None else x_c.shape[-1]
    out = torch.empty(B, S, H, d_c + 2 * d_r, dtype=torch.bfloat16, device=x_r.device)
    om, dl = _f32(omega, x_r.device), _f32(delta, x_r.device)
    with _on_device(x_r.device) as stream:
        rc = _lib.lib.pe_pope_expand(None if x_c is None else x_c.data_ptr(), _s3(x_c), x_r.data_ptr(), _s3(x_r),
                                     out.data_ptr(), _s3(out), B, S, H, d_c, d_r, int(pos0), om.data_ptr(),
                                     None if dl is None else dl.data_ptr(), C.c_void_p(stream))
    if rc != 0:
        raise _lib.PeAttnError(rc)
    return out


def pope_expand_backward(grad: torch.Tensor, x_r: torch.Tensor, d_c: int, pos0: int, omega: torch.Tensor,
                         delta: torch.Tensor | None, d_omega: torch.Tensor, d_delta: torch.Tensor | None):
    """Gradient of ``pope_expand``: returns (d x_c or None, d x_r) in bf16 and accumulates the
    frequency / phase-bias gradients into the fp64 vectors ``d_omega`` / ``d_delta`` (the latter
    with respect to the raw bias: zero where the clamp to [-2 pi, 0] is active)."""
    B, S, H, d_r = x_r.shape
    dev = x_r.device
    dx_c = torch.empty(B, S, H, d_c, dtype=torch.bfloat16, device=dev) if d_c else None
    dx_r = torch.empty(B, S, H, d_r, dtype=torch.bfloat16, device=dev)
    om, dl = _f32(omega, dev), _f32(delta, dev)
    with _on_device(dev) as stream:
        rc = _lib.lib.pe_pope_expand_backward(
            grad.data_ptr(), _dtype_code(grad), _s3(grad), x_r.data_ptr(), _s3(x_r),
            None if dx_c is None else dx_c.data_ptr(), _s3(dx_c), dx_r.data_ptr(), _s3(dx_r), B, S, H, d_c, d_r,
            int(pos0), om.data_ptr(), None if dl is None else dl.data_ptr(), d_omega.data_ptr(),
            None if d_delta is None else d_delta.data_ptr(), C.c_void_p(stream))
    if rc != 0:
        raise _lib.PeAttnError(rc)
    return dx_c, dx_r


def fope_effective_freqs(base: torch.Tensor, coeffs: torch.Tensor, normalize: bool, floor_freq: float,
                         ceil_freq: float | None, d_omega: torch.Tensor | None = None, want_d_base: bool = False):
    """FoPE's effective frequencies [d_r] from base frequencies and Fourier coefficients (fp32,
    contiguous, on the GPU); with ``d_omega`` (fp64 [d_r]) their gradient instead:
    ``(d_coeffs, d_base or None)``."""
    d_r, n_f = coeffs.shape
    flags = (_lib.FOURIER_NORMALIZE if normalize else 0) | (_lib.FOURIER_CEILING if ceil_freq is not None else 0)
    ceil = float(ceil_freq) if ceil_freq is not None else 0.0
    with _on_device(coeffs.device) as raw_stream:
        stream = C.c_void_p(raw_stream)
        if d_omega is None:
            omega = torch.empty(d_r, dtype=torch.float32, device=coeffs.device)
            rc = _lib.lib.pe_fope_effective_freqs(base.data_ptr(), coeffs.data_ptr(), d_r, n_f, flags, float(floor_freq),
                                                  ceil, omega.data_ptr(), stream)
            result = omega
        else:
            d_coeffs = torch.empty_like(coeffs)
            d_base = torch.empty_like(base) if want_d_base else None
            rc = _lib.lib.pe_fope_effective_freqs_backward(
                base.data_ptr(), coeffs.data_ptr(), d_r, n_f, flags, float(floor_freq), ceil, d_omega.data_ptr(),
                d_coeffs.data_ptr(), None if d_base is None else d_base.data_ptr(), stream)
            result = (d_coeffs, d_base)
    if rc != 0:
        raise _lib.PeAttnError(rc)
    return result


def rotary_norm_expand(x: torch.Tensor, table: torch.Tensor | None, table_row0: int, mscale: float, qk_norm: bool,
                       eps: float, grad: torch.Tensor | None = None) -> torch.Tensor:
    """normalise(mscale * rotate(x)) as a bf16 [B,S,H,D] tensor; with ``grad`` (the gradient with
    respect to that result, bf16 or fp32) the gradient with respect to ``x`` instead."""
    B, S, H, D = x.shape
    out = torch.empty(B, S, H, D, dtype=torch.bfloat16, device=x.device)
    rows = 0 if table is None else table.shape[0]
    tptr = None if table is None else table.data_ptr()
    with _on_device(x.device) as raw_stream:
        stream = C.c_void_p(raw_stream)
        if grad is None:
            rc = _lib.lib.pe_rotary_norm_expand(x.data_ptr(), _s3(x), out.data_ptr(), _s3(out), B, S, H, D, tptr,
                                                int(table_row0), rows, float(mscale), int(qk_norm), float(eps), stream)
        else:
            rc = _lib.lib.pe_rotary_norm_expand_backward(grad.data_ptr(), _dtype_code(grad), _s3(grad), x.data_ptr(),
                                                         _s3(x), out.data_ptr(), _s3(out), B, S, H, D, tptr,
                                                         int(table_row0), rows, float(mscale), int(qk_norm),
                                                         float(eps), stream)
    if rc != 0:
        raise _lib.PeAttnError(rc)
    return out


class HostStreamedAttention:
    """Causal PE-attention over pinned HOST tensors, with the copies hidden behind the kernels.

    The inputs of a long sequence take longer to cross PCIe than the kernel takes to
    consume them, so the sequence is cut into ``chunks`` row blocks.  Causality makes block
    c of the queries depend only on key/value blocks 0..c: block c is copied in on one
    stream, its attention (queries of block c against keys 0..end of c, ``start_pos`` =
    first row of c) is launched on the caller's stream as soon as the copy has landed, and
    its output rows go back on a third stream while block c+1 is still arriving.  Each
    block runs the same kernel over the same 128-key tiles as the one-shot call, so the
    result is the one ``pe_attention`` gives on device copies of the same tensors (to a bf16
    rounding: launches with few blocks split their longest ones along the keys).

    The staging tensors (device copies of every input and of the output) are allocated once
    here, in two sets that calls use in turn: the copy-in of call n + 1 may start while the last
    kernel and the copy-out of call n are still running, and waits only for the kernels of call
    n - 1, which read the set it is about to overwrite.  The caller's stream waits for the last
    output block before ``__call__`` returns control of it, so work queued afterwards -- and
    CUDA events recorded around the call -- see the whole transfer + compute.
    """

    def __init__(self, variant: str, *, B: int, S: int, H: int, Hkv: int, d_c: int, d_r: int, d_v: int,
                 dtype: torch.dtype, device, chunks: int = 8, **params):
        if variant not in _VARIANTS:
            raise ValueError(f"unknown variant {variant!r}")
        if chunks < 1 or S % chunks != 0:
            raise ValueError("chunks must divide the sequence length")
        self.variant, self.params, self.chunks = variant, params, chunks
        self.device = torch.device(device)
        self.shape = dict(B=B, S=S, H=H, Hkv=Hkv, d_c=d_c, d_r=d_r, d_v=d_v)
        mk = lambda h, d: torch.empty(B, S, h, d, dtype=dtype, device=self.device) if d else None  # noqa: E731
        self.sets = [dict(stage=dict(q=mk(H, d_c), k=mk(Hkv, d_c), q_r=mk(H, d_r), k_r=mk(Hkv, d_r), v=mk(Hkv, d_v)),
                          out=mk(H, d_v), kernels_done=None, copied_out=None) for _ in range(2)]
        self.calls = 0
        self.h2d = torch.cuda.Stream(self.device)
        self.d2h = torch.cuda.Stream(self.device)

    def __call__(self, host: dict[str, torch.Tensor], out_host: torch.Tensor) -> torch.Tensor:
        cur = self.sets[self.calls % 2]
        self.calls += 1
        st, out_dev = cur["stage"], cur["out"]
        for name, t in st.items():
            if t is None:
                continue
            h = host[name]
            if h.is_cuda or not h.is_pinned() or not h.is_contiguous() or h.shape != t.shape or h.dtype != t.dtype:
                raise ValueError(f"host[{name!r}] must be a pinned contiguous CPU tensor of shape {tuple(t.shape)}")
        if (out_host.is_cuda or not out_host.is_pinned() or not out_host.is_contiguous()
                or out_host.shape != out_dev.shape):
            raise ValueError("out_host must be a pinned CPU tensor of the output shape")
        S, rows = self.shape["S"], self.shape["S"] // self.chunks
        main = torch.cuda.current_stream(self.device)
        # this set's previous user: its kernels read the input copies, its copy-out read ``out``
        if cur["kernels_done"] is not None:
            self.h2d.wait_event(cur["kernels_done"])
            main.wait_event(cur["copied_out"])
        for c in range(self.chunks):
            s0, s1 = c * rows, (c + 1) * rows
            with torch.cuda.stream(self.h2d):
                # keys and values first: they are what the block's kernel streams through
                # one copy per batch entry: each [b, s0:s1] block is contiguous on both sides,
                # so it is a single DMA transfer with no host-side repacking
                for name in ("k", "k_r", "v", "q", "q_r"):
                    if st[name] is not None:
                        for b in range(self.shape["B"]):
                            st[name][b, s0:s1].copy_(host[name][b, s0:s1], non_blocking=True)
                landed = torch.cuda.Event()
                landed.record(self.h2d)
            main.wait_event(landed)
            sl = lambda t, a, b: None if t is None else t[:, a:b]  # noqa: E731
            pe_attention(self.variant, sl(st["q"], s0, s1), sl(st["k"], 0, s1), st["v"][:, :s1],
                         q_r=sl(st["q_r"], s0, s1), k_r=sl(st["k_r"], 0, s1),
                         start_pos=s0, k_start_pos=0, out=out_dev[:, s0:s1], **self.params)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(done)
                for b in range(self.shape["B"]):
                    out_host[b, s0:s1].copy_(out_dev[b, s0:s1], non_blocking=True)
        cur["kernels_done"] = done
        back = torch.cuda.Event()
        back.record(self.d2h)
        cur["copied_out"] = back
        main.wait_event(back)
        self._last_back = back
        return out_host

    def synchronize(self) -> None:
        """Block until the last call's output has landed in host memory, then raise if a kernel
        reported an expired wait (the output is invalid in that case)."""
        back = getattr(self, "_last_back", None)
        if back is not None:
            back.synchronize()
        check_device_status(self.device)


_ce_scratch: dict[tuple[int, int], torch.Tensor] = {}     # (device, stream) -> scratch, at most _CE_SCRATCH_MAX
_CE_SCRATCH_MAX = 16


def ce_loss_sums(logits: torch.Tensor, targets: torch.Tensor, out: torch.Tensor | None = None,
                 ignore_index: int = -100) -> torch.Tensor:
    """Accumulate (sum of next-token NLLs, scored-token count) of one logits chunk into ``out``.

    logits: CUDA [n, vocab] bf16 or fp32 (last dim contiguous); targets: CUDA int64 [n];
    out: CUDA float64 [2], created zeroed if None.  Reads every logit once in its stored type.
    """
    if not logits.is_cuda:
        raise RuntimeError("ce_loss_sums needs CUDA tensors: there is no CPU path")
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("logits must be [n, vocab] with a contiguous last dimension")
    if logits.dtype == torch.bfloat16:
        dtype = _lib.BF16
    elif logits.dtype == torch.float32:
        dtype = _lib.FP32
    else:
        raise TypeError(f"unsupported dtype {logits.dtype}")
    n, vocab = logits.shape
    targets = targets.reshape(-1).to(torch.int64).contiguous()
    if targets.numel() != n:
        raise ValueError("targets must have one entry per row of logits")
    dev = logits.device
    if out is None:
        out = torch.zeros(2, dtype=torch.float64, device=dev)
    with _on_device(dev) as stream:
        need = _lib.lib.pe_ce_scratch_bytes(n)
        key = (dev.index if dev.index is not None else torch.cuda.current_device(), stream)
        scratch = _ce_scratch.get(key)
        if scratch is None or scratch.numel() < need:
            # zeroed once: the kernel leaves the counter word at zero after every call
            scratch = torch.zeros(max(need, 1 << 16), dtype=torch.uint8, device=dev)
            _ce_scratch.pop(key, None)
            while len(_ce_scratch) >= _CE_SCRATCH_MAX:
                # oldest stream first; its block goes back to the caching allocator, which orders
                # the reuse after that stream's kernels
                _ce_scratch.pop(next(iter(_ce_scratch)))
            _ce_scratch[key] = scratch
        rc = _lib.lib.pe_ce_loss_sums(logits.data_ptr(), dtype, logits.stride(0), targets.data_ptr(), n, vocab,
                                      int(ignore_index), scratch.data_ptr(), out.data_ptr(),
                                      C.c_void_p(stream))
    if rc != 0:
        raise _lib.PeAttnError(rc)
    return out


def fused_gemm_ok(x: torch.Tensor, *weights: torch.Tensor) -> bool:
    """Inference on bf16 activations with weights already stored in bf16
    (``eval.cast_matmul_weights``): the cases the tensor-core GEMM with a fused epilogue covers.
    Everything else (training, fp32, fp32 weights under autocast) takes the library GEMM and
    the stand-alone kernels."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or torch.is_grad_enabled() and (
            x.requires_grad or any(w.requires_grad for w in weights)):
        return False
    k = x.shape[-1]
    return k >= 64 and k % 8 == 0 and all(
        w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[0] % 8 == 0 and w.shape[1] == k for w in weights)


def linear_residual(linear, y: torch.Tensor, residual: torch.Tensor | None) -> torch.Tensor:
    """``linear(y)``, plus ``residual`` when given: the output projection of a block (wo, w2) and
    the block's residual add (src/model/transformer.py:176-177).  bf16 inference with bf16 weights
    and a bf16 residual runs as one tensor-core GEMM with the add in its epilogue."""
    # long reductions stay with the library: at K = 5632, N = 2048 its GEMM + a separate add measured
    # 0.274 ms against 0.312 ms fused (K = 2048: 0.133 against 0.120)
    if residual is not None and residual.dtype == torch.bfloat16 and residual.shape[:-1] == y.shape[:-1] \
            and linear.bias is None and y.shape[-1] <= 4096 and fused_gemm_ok(y, linear.weight):
        return gemm_nt(y, linear.weight, residual=residual)
    out = linear(y)
    return out if residual is None else residual + out


def projections(owner, x: torch.Tensor, *linears) -> list[torch.Tensor]:
    """``[lin(x) for lin in linears]`` for the input projections of one attention block
    (src/model/attention.py:77-80, src/model/fpope_attention.py:128-140).

    bf16 inference with bf16 weights: ONE library GEMM against the row-wise concatenation of the
    weights; the results are column slices of its output, which the norm and attention kernels
    read in place (row stride = the concatenated width).  The concatenation is a derived copy
    kept on ``owner`` (not a parameter or buffer: the state_dict is unchanged) and rebuilt when
    any weight's storage or version changes.  Anything else: one ``nn.Linear`` call each.
    """
    weights = [lin.weight for lin in linears]
    if len(linears) < 2 or any(lin.bias is not None for lin in linears) or not fused_gemm_ok(x, *weights):
        return [lin(x) for lin in linears]
    key = tuple((w.data_ptr(), w._version) for w in weights)
    cached = owner.__dict__.get("_wcat")
    if cached is None or cached[0] != key:
        cached = (key, torch.cat([w.detach() for w in weights], dim=0))
        owner.__dict__["_wcat"] = cached
    y = torch.nn.functional.linear(x, cached[1])
    outs, col = [], 0
    for w in weights:
        outs.append(y[..., col:col + w.shape[0]])
        col += w.shape[0]
    return outs


def _bf16_matrix(name: str, t: torch.Tensor) -> torch.Tensor:
    """[rows, K] bf16 CUDA view the tensor-core GEMM can read in place (TMA: 16-byte aligned rows)."""
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: there is no CPU path")
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bf16 (got {t.dtype})")
    t = t.reshape(-1, t.shape[-1])
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


_head_ws: dict[tuple[int, int], torch.Tensor] = {}     # (device, stream) -> workspace, bounded like _ce_scratch


def lm_head_ce_loss_sums(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor,
                         out: torch.Tensor | None = None, ignore_index: int = -100) -> torch.Tensor:
    """``ce_loss_sums(hidden @ weight.T, targets)`` without the logits: the head GEMM runs on the
    tensor cores with the cross-entropy in its epilogue (src/model/transformer.py:358-371).

    hidden: CUDA bf16 [n, hidden_dim]; weight: CUDA bf16 [vocab, hidden_dim]; targets: CUDA int64 [n];
    out: CUDA float64 [2] (sum of NLLs, scored rows), accumulated, created zeroed if None.
    Logits are rounded to bf16 before the loss, as the head's autocast output is.
    """
    h = _bf16_matrix("hidden", hidden)
    w = _bf16_matrix("weight", weight)
    if h.shape[1] != w.shape[1]:
        raise ValueError("hidden and weight disagree on hidden_dim")
    n, vocab = h.shape[0], w.shape[0]
    targets = targets.reshape(-1).to(torch.int64).contiguous()
    if targets.numel() != n:
        raise ValueError("targets must have one entry per row of hidden")
    dev = h.device
    if out is None:
        out = torch.zeros(2, dtype=torch.float64, device=dev)
    with _on_device(dev) as stream:
        need = _lib.lib.pe_lm_head_ce_workspace_bytes(n, vocab)
        key = (dev.index if dev.index is not None else torch.cuda.current_device(), stream)
        ws = _head_ws.get(key)
        if ws is None or ws.numel() < need:
            ws = torch.empty(need, dtype=torch.uint8, device=dev)
            _head_ws.pop(key, None)
            while len(_head_ws) >= _CE_SCRATCH_MAX:
                _head_ws.pop(next(iter(_head_ws)))
            _head_ws[key] = ws
        rc = _lib.lib.pe_lm_head_ce_loss_sums(h.data_ptr(), h.stride(0), w.data_ptr(), w.stride(0), targets.data_ptr(),
                                              n, h.shape[1], vocab, int(ignore_index), ws.data_ptr(), ws.numel(),
                                              out.data_ptr(), device_status(dev).data_ptr(),
                                              C.c_void_p(stream))
    if rc != 0:
        raise _lib.PeAttnError(rc)
    return out


def swiglu_gemm(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """cast(cast(silu(x @ w_gate.T)) * (x @ w_up.T)) in one tensor-core kernel: the feed-forward's
    two input projections with SwiGLU in the epilogue (src/model/ffn.py:30-68), so the two
    [tokens, ffn_dim] projections are never written.  bf16; w_gate, w_up: [ffn_dim, hidden_dim]."""
    x2 = _bf16_matrix("x", x)
    wg, wu = _bf16_matrix("w_gate", w_gate), _bf16_matrix("w_up", w_up)
    if wg.shape != wu.shape or wg.stride(0) != wu.stride(0) or wg.shape[1] != x2.shape[1]:
        raise ValueError("w_gate and w_up must be [ffn_dim, hidden_dim] with equal strides")
    y = torch.empty(x2.shape[0], wg.shape[0], dtype=torch.bfloat16, device=x2.device)
    with _on_device(x2.device) as stream:
        rc = _lib.lib.pe_swiglu_gemm(x2.data_ptr(), x2.stride(0), wg.data_ptr(), wu.data_ptr(), wg.stride(0),
                                     y.data_ptr(), y.stride(0), x2.shape[0], x2.shape[1], wg.shape[0],
                                     device_status(x2.device).data_ptr(), C.c_void_p(stream))
    if rc != 0:
        raise _lib.PeAttnError(rc)
    return y.view(*x.shape[:-1], wg.shape[0])


def gemm_nt(a: torch.Tensor, b: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """a @ b.T for bf16 [.., k] and [n, k] on the same kernel with the plain store epilogue;
    with ``residual`` [.., n] the result is cast(cast(a @ b.T) + residual): an output projection
    (wo, w2) together with the block's residual add (src/model/transformer.py:176-177)."""
    a2, b2 = _bf16_matrix("a", a), _bf16_matrix("b", b)
    if a2.shape[1] != b2.shape[1]:
        raise ValueError("a and b disagree on k")
    c = torch.empty(a2.shape[0], b2.shape[0], dtype=torch.bfloat16, device=a2.device)
    r2 = None
    if residual is not None:
        r2 = _bf16_matrix("residual", residual)
        if r2.shape != c.shape:
            raise ValueError("residual must have the shape of the result")
    with _on_device(a2.device) as stream:
        rc = _lib.lib.pe_gemm_nt(a2.data_ptr(), a2.stride(0), b2.data_ptr(), b2.stride(0), c.data_ptr(), c.stride(0),
                                 None if r2 is None else r2.data_ptr(), 0 if r2 is None else r2.stride(0),
                                 a2.shape[0], b2.shape[0], a2.shape[1], device_status(a2.device).data_ptr(),
                                 C.c_void_p(stream))
    if rc != 0:
        raise _lib.PeAttnError(rc)
    return c.view(*a.shape[:-1], b2.shape[0])


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    if t.dtype == torch.float32:
        return _lib.FP32
    raise TypeError(f"unsupported dtype {t.dtype}")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """cast(cast(x * rsqrt(mean(x^2) + eps)) * weight) over the last dim, in one pass; dtype of ``x``.

    For fp32 ``x`` this is the reference's RMSNorm; for bf16 ``x`` it is RMSNorm followed by the
    bf16 cast the next linear layer applies under autocast.
    """
    if not x.is_cuda:
        raise RuntimeError("rmsnorm needs CUDA tensors: there is no CPU path")
    dim = x.shape[-1]
    x2 = x.reshape(-1, dim)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    y = torch.empty_like(x2)
    w = weight.detach()
    if w.dtype != torch.float32 or not w.is_contiguous():
        w = w.float().contiguous()
    with _on_device(x.device) as stream:
        rc = _lib.lib.pe_rmsnorm_forward(x2.data_ptr(), w.data_ptr(), y.data_ptr(), _dtype_code(x2), x2.shape[0], dim,
                                         x2.stride(0), y.stride(0), float(eps), C.c_void_p(stream))
    if rc != 0:
        raise _lib.PeAttnError(rc)
    return y.view(x.shape)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """cast(cast(silu(gate)) * up), elementwise, one pass."""
    if not gate.is_cuda:
        raise RuntimeError("swiglu needs CUDA tensors: there is no CPU path")
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("gate and up must have the same shape and dtype")
    g, u = gate.contiguous(), up.contiguous()
    y = torch.empty_like(g)
    with _on_device(g.device) as stream:
        rc = _lib.lib.pe_swiglu_forward(g.data_ptr(), u.data_ptr(), y.data_ptr(), _dtype_code(g), g.numel(),
                                        C.c_void_p(stream))
    if rc != 0:
        raise _lib.PeAttnError(rc)
    return y


def attention_flops(B: int, H: int, S: int, d_qk: int, d_v: int) -> float:
    """Algorithmic causal attention FLOPs (the benchmark's convention): B H S^2 (d_qk + d_v)."""
    return float(B) * H * S * S * (d_qk + d_v)
