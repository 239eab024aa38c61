"""B200-native fused positional-encoding attention (sm_100a) behind the reference's module API.

``pe_attention`` / ``ce_loss_sums`` / ``lm_head_ce_loss_sums`` / ``swiglu_gemm`` are the functional entry points over the C ABI in
``include/pe_attn.h``; ``modules`` holds drop-in replacements for the reference's three
attention classes, ``model`` the Transformer host, ``eval`` the sharded evaluation.

The CUDA library is loaded on first use of any of them and there is no fallback: if
``libpe_attn.so`` has not been built (``python -m pe_ablations_b200.build_ext``) or lacks a
symbol, that first use raises ImportError.  Only ``build_ext`` can be imported without it.
"""

__all__ = ["pe_attention", "HostStreamedAttention", "ce_loss_sums", "lm_head_ce_loss_sums", "swiglu_gemm",
           "check_device_status", "attention_flops"]


def __getattr__(name):
    if name in __all__:
        from . import ops

        return getattr(ops, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
