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
        # Temporary library path (same role as cuBLAS for GEMMs): Dao flash-attn 2 for the dense causal case.
        if q_positions is None and q_sequence_ids is None and not return_lse:
            try:
                from flash_attn import flash_attn_func

                return flash_attn_func(q, k, v, causal=causal, softmax_scale=scale)
            except ImportError:
                pass
        return attention_reference(q, k, v, q_positions=q_positions, k_positions=k_positions, q_sequence_ids=q_sequence_ids,
                                   k_sequence_ids=k_sequence_ids, causal=causal, scale=scale, return_lse=return_lse)
    raise NotImplementedError


def flash_block_forward(q, k, v, q_positions, k_positions, q_sequence_ids, k_sequence_ids, scale):
    """Kernel block forward returning ``(out fp32, lse)``; None when the kernel does not cover the case."""
    return None


def flash_block_backward(q, k, v, out, lse, dout, q_positions, k_positions, q_sequence_ids, k_sequence_ids, scale):
    return None
