"""Attention backend names accepted by configs and the CLI.

The reference dispatches between eager / SDPA / flash-attn (``utils/attention_backend.py:20-135``). Here there is one
implementation per device class - the sm_100a flash kernels on CUDA bf16, an fp32 eager restatement elsewhere - so
the names are accepted for compatibility and only ``eager`` changes behaviour (it forces the restatement).
"""
from __future__ import annotations

from enum import Enum

import torch

from maltos_b200.ops.attention import attention, attention_reference


class AttentionBackend(str, Enum):
    EAGER = "eager"
    SDPA_AUTO = "sdpa_auto"
    SDPA_FLASH = "sdpa_flash"
    FLASH_ATTN = "flash_attn"

    def __str__(self) -> str:
        return self.value


ATTENTION_BACKEND_CHOICES = tuple(b.value for b in AttentionBackend)


def validate_attention_backend(name) -> AttentionBackend:
    try:
        return AttentionBackend(name)
    except ValueError:
        raise ValueError(f"attention_backend must be one of {sorted(ATTENTION_BACKEND_CHOICES)}, got {name!r}") from None


def causal_attention(q, k, v, *, attention_backend: str = "sdpa_auto", warning_prefix: str = "", q_positions=None,
                     k_positions=None, q_sequence_ids=None, k_sequence_ids=None, flash_varlen_mode=None) -> torch.Tensor:
    """``[B, heads, S, D]`` convention of the reference API; K/V may have fewer heads than Q (GQA)."""
    fn = attention_reference if AttentionBackend(attention_backend) is AttentionBackend.EAGER else attention
    out = fn(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), q_positions=q_positions, k_positions=k_positions,
             q_sequence_ids=q_sequence_ids, k_sequence_ids=k_sequence_ids, causal=True)
    return out.transpose(1, 2)


def eager_causal_attention(q, k, v, *, mask=None) -> torch.Tensor:
    scale = q.size(-1) ** -0.5
    scores = torch.matmul(q, k.transpose(-2, -1)) * scale
    if mask is None:
        s = q.size(-2)
        mask = torch.ones(s, s, device=q.device, dtype=torch.bool).tril()[None, None]
    scores = scores.masked_fill(~mask, torch.finfo(scores.dtype).min)
    return torch.matmul(torch.softmax(scores, dim=-1), v)
