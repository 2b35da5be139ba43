"""Canonical per-token positions / sequence ids and the visibility mask built from them
(reference ``runtime/layers/attn_masking_utils.py:54-87``)."""
from __future__ import annotations

import torch

from maltos_b200.ops.attention import build_visibility_mask


def canonical_position_ids(position_ids, *, batch_size: int, seq_len: int, position_offset: int, device) -> torch.Tensor:
    if position_ids is None:
        return (torch.arange(seq_len, device=device, dtype=torch.long) + position_offset).unsqueeze(0).expand(batch_size, seq_len).contiguous()
    p = position_ids.to(device=device, dtype=torch.long)
    if p.dim() == 1:
        p = p.unsqueeze(0).expand(batch_size, -1)
    return p.contiguous()


def canonical_sequence_ids(sequence_ids, *, batch_size: int, seq_len: int, device) -> torch.Tensor | None:
    if sequence_ids is None:
        return None
    s = sequence_ids.to(device=device, dtype=torch.long)
    if s.dim() == 1:
        s = s.unsqueeze(0).expand(batch_size, -1)
    return s.contiguous()


def build_example_causal_mask(*, q_positions, k_positions, q_sequence_ids=None, k_sequence_ids=None) -> torch.Tensor:
    return build_visibility_mask(q_positions, k_positions, q_sequence_ids, k_sequence_ids)
