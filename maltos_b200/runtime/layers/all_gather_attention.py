"""Context-parallel attention by all-gathering K and V along the sequence (backward: reduce-scatter SUM) together with
their positions / sequence ids, then one masked attention of the local queries against all keys
(reference ``runtime/layers/all_gather_attention.py:18-71``). Layout ``[B, S, heads, D]``, K/V keep their GQA head count."""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.ops.attention import attention

from .attn_masking_utils import canonical_position_ids, canonical_sequence_ids
from .functional import all_gather


def _gather_ints(t: torch.Tensor, group) -> torch.Tensor:
    parts = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim=1)


class AllGatherKvAttentionCore(nn.Module):
    preserves_native_gqa = True
    layout = "bshd"

    def __init__(self, group, attention_backend: str = "eager") -> None:
        super().__init__()
        self.group = group
        self.attention_backend = attention_backend

    def forward(self, q, k, v, position_offset: int = 0, position_ids=None, sequence_ids=None):
        B, S = q.shape[:2]
        k_all = all_gather(k, self.group, 1, backward_reduce=dist.ReduceOp.SUM)
        v_all = all_gather(v, self.group, 1, backward_reduce=dist.ReduceOp.SUM)
        q_pos = canonical_position_ids(position_ids, batch_size=B, seq_len=S, position_offset=position_offset, device=q.device)
        q_seq = canonical_sequence_ids(sequence_ids, batch_size=B, seq_len=S, device=q.device)
        k_pos = _gather_ints(q_pos, self.group)
        k_seq = _gather_ints(q_seq, self.group) if q_seq is not None else None
        return attention(q, k_all, v_all, q_positions=q_pos, k_positions=k_pos, q_sequence_ids=q_seq, k_sequence_ids=k_seq)
